"""GPU parity of the BF16 head drop-in (`ds41_fuse_head_decode`) against the CPU restatement of the reference kernels'
arithmetic order (components/fuse-head/src/head_half_tree.cu:7-21): bit-exact."""
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


def bf16_bits(a):
    return (torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("N,K", [(100, 512), (1031, 5120), (64, 6656)])
def test_bf16_head_bit_exact(pkg, oracle, M, N, K):
    x = oracle.gen_normal(41, M * 1000 + N, (M, K), 1.0)
    w = oracle.gen_normal(42, N + K, (N, K), 0.02)
    w[0, :7] = 0.0
    x[0, 3] = -0.0
    bits = bf16_bits(w)
    want = oracle.head_bf16(x, bits)
    got = pkg.head_bf16(torch.from_numpy(x).cuda(), torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_decode_symbol_shape_check_and_full_size(pkg, oracle):
    """The plugin symbol accepts only the target head's shape (head_decode.cpp:6); at that shape (1.32 GB of weights)
    a sample of vocabulary rows is checked bit for bit."""
    x = torch.from_numpy(oracle.gen_normal(43, 1, (6, 5120), 1.0)).cuda()
    small = torch.zeros((128, 5120), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        pkg.head_bf16(x, small, decode_symbol=True)
    g = torch.Generator(device="cuda").manual_seed(9)
    w = (0.02 * torch.randn(129280, 5120, device="cuda", generator=g)).to(torch.bfloat16)
    out = pkg.head_bf16(x, w, decode_symbol=True)
    torch.cuda.synchronize()
    rows = np.r_[0:64, 64000:64064, 129280 - 64:129280]
    bits = w[torch.from_numpy(rows).cuda()].view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.head_bf16(x.cpu().numpy(), bits)
    assert np.array_equal(out.cpu().numpy()[:, rows].view(np.uint32), want.view(np.uint32))
