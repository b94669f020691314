"""FP32 head (csrc/head_f32.cu): the reference's default target head is a cuBLAS GEMV on FP32-promoted weights
(components/dense/src/ops.cu:120-128), whose order of summation is unspecified; the operator here is checked against
the exact (FP64) product within the FP32 bound of a K-term dot product, and for its argument errors.
Parity unpinned: no bit pattern exists to reproduce."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    entry.build()
    return entry.load_package()


@pytest.mark.parametrize("M,N,K", [(1, 4099, 5120), (3, 1000, 5120), (6, 2048, 5120), (8, 777, 4096), (2, 5, 128)])
def test_fp32_head_is_the_exact_product_within_the_fp32_bound(pkg, oracle, M, N, K):
    x = oracle.gen_normal(71, M, (M, K), 1.0)
    w = oracle.gen_normal(72, N, (N, K), 0.02)
    got = pkg.head_f32(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()).cpu().numpy()
    want = x.astype(np.float64) @ w.astype(np.float64).T
    # |error| <= (K / 32 + 6) * 2^-24 * sum |w x| for a lane's chain of K / 32 fused multiply-adds and a five-level tree
    bound = (K / 32 + 6) * 2.0 ** -24 * (np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64).T)
    assert (np.abs(got - want) <= bound + 1e-30).all(), float((np.abs(got - want) / (bound + 1e-30)).max())
    again = pkg.head_f32(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()).cpu().numpy()
    assert np.array_equal(got, again)                      # a fixed order: the same bits every time


def test_fp32_head_argument_errors(pkg):
    x = torch.zeros(2, 256, device="cuda")
    w = torch.zeros(16, 256, device="cuda")
    with pytest.raises(RuntimeError):
        pkg.head_f32(torch.zeros(9, 256, device="cuda"), w)          # M > 8
    with pytest.raises(RuntimeError):
        pkg.head_f32(torch.zeros(2, 200, device="cuda"), torch.zeros(16, 200, device="cuda"))   # K not a multiple of 128
    with pytest.raises(RuntimeError):
        pkg.head_f32(torch.zeros(8, 16384, device="cuda"), torch.zeros(4, 16384, device="cuda"))  # activations beyond shared memory
    assert pkg.head_f32(x, w).shape == (2, 16)


def test_fp32_head_full_size_rate(pkg):
    """The reference's shape: 129280 x 5120 FP32 weights (2.65 GB), one row.  Prints the achieved bandwidth."""
    N, K = 129280, 5120
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    x = torch.randn(1, K, device="cuda", generator=g)
    out = torch.empty(1, N, device="cuda")
    for _ in range(3):
        pkg.head_f32(x, w, out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(10):
        pkg.head_f32(x, w, out)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) / 10 * 1e3
    ref = (w[:64].double() @ x[0].double()).cpu().numpy()
    assert np.allclose(out[0, :64].cpu().numpy(), ref, rtol=1e-4, atol=1e-5)
    print(f"FP32 head M=1: {us:.0f} us ({N * K * 4 / us / 1e3:.0f} GB/s)")
