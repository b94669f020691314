"""GPU parity of the operators either side of the target head: the drafter's BF16 head (ds41_dense_head_compact), the
Markov-biased draft logits and the head's prologue (HC-pre mix -> RMSNorm -> BF16 -> FP32).

Each is compared bit for bit with this repository's CPU restatement of the reference kernel's arithmetic order and, where
the reference tree was available at build time, with the reference's own CUDA kernels compiled in place for sm_100a
(oracle/_ref): components/dense/src/compact.cu, ops.cu and components/fuse-head/src/*.  The latter also gives the
same-box timing of the reference kernels, printed for the record."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import oracle_lib

pytestmark = pytest.mark.gpu
V = 129280


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available()
    entry.build()
    return entry.load_package()


@pytest.fixture(scope="module")
def refgpu():
    r = oracle_lib.ReferenceGpu()
    if not r.available:
        pytest.skip("oracle/_ref reference GPU libraries not built (reference tree absent at build time)")
    return r


def bf16_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def timed(fn, n=5):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n * 1e3


@pytest.mark.parametrize("M", [1, 2, 3, 5, 6, 8])
@pytest.mark.parametrize("N,K", [(1003, 256), (517, 1024), (64, 5120)])
def test_compact_head_matches_restatement(pkg, oracle, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = (0.05 * torch.randn(N, K, device="cuda", generator=g)).to(torch.bfloat16)
    got = pkg.head_compact(x, w)
    torch.cuda.synchronize()
    want = oracle.head_compact(x.cpu().numpy(), bf16_bits(w))
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("M", [1, 5, 8])
def test_compact_head_equals_reference_kernel_at_full_size(pkg, refgpu, M):
    K = 5120
    g = torch.Generator(device="cuda").manual_seed(90 + M)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = (0.02 * torch.randn(V, K, device="cuda", generator=g)).to(torch.bfloat16)
    got = pkg.head_compact(x, w)
    ref = torch.empty_like(got)
    assert refgpu.dense.ds41_dense_head_compact(x.data_ptr(), w.data_ptr(), ref.data_ptr(), M, V, K, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    ours = timed(lambda: pkg.head_compact(x, w, got))
    theirs = timed(lambda: refgpu.dense.ds41_dense_head_compact(x.data_ptr(), w.data_ptr(), ref.data_ptr(), M, V, K, None))
    print(f"compact head M={M}: {ours:.0f} us ({V * K * 2 / ours / 1e3:.0f} GB/s), reference kernel on this GPU {theirs:.0f} us")


@pytest.mark.parametrize("M", [1, 3, 6])
def test_bf16_head_equals_reference_plugin_at_full_size(pkg, refgpu, M):
    """ds41_fuse_head_decode against the reference plugin's kernels (head_half_tree.cu / head_half_tune.cu), whole output."""
    K = 5120
    g = torch.Generator(device="cuda").manual_seed(190 + M)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = (0.02 * torch.randn(V, K, device="cuda", generator=g)).to(torch.bfloat16)
    got = pkg.head_bf16(x, w, decode_symbol=True)
    ref = torch.empty_like(got)
    assert refgpu.fusehead.ds41_fuse_head_decode(x.data_ptr(), w.data_ptr(), ref.data_ptr(), M, V, K, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    ours = timed(lambda: pkg.head_bf16(x, w, got, decode_symbol=True))
    theirs = timed(lambda: refgpu.fusehead.ds41_fuse_head_decode(x.data_ptr(), w.data_ptr(), ref.data_ptr(), M, V, K, None))
    print(f"BF16 head M={M}: {ours:.0f} us, reference plugin on this GPU {theirs:.0f} us")


def test_markov_logits(pkg, oracle):
    g = torch.Generator(device="cuda").manual_seed(5)
    u = 3.0 * torch.randn(V, device="cuda", generator=g)
    w = (0.1 * torch.randn(V, 256, device="cuda", generator=g)).to(torch.bfloat16)
    emb = torch.randn(256, device="cuda", generator=g).to(torch.bfloat16)
    got = pkg.markov_logits(u, w, emb)
    torch.cuda.synchronize()
    want = oracle.markov_logits(u.cpu().numpy(), bf16_bits(w), bf16_bits(emb))
    assert np.array_equal(got.cpu().numpy(), want)
    # the biased row is what the drafter samples from: same token as the oracle for the same address
    seeds, steps = torch.tensor([11], device="cuda"), torch.tensor([4], device="cuda")
    tok, st = pkg.sample_logits(got[None, :], 0.6, 0.95, seeds, steps, slot=1, purpose=1)
    wtok, _ = oracle.sample_rows(want[None, :], 0.6, 0.95, [11], [4], slot=1, purpose=1)
    assert st.item() == 0 and tok.item() == wtok[0]


@pytest.mark.parametrize("M", [1, 2, 3, 4, 6, 8])
@pytest.mark.parametrize("K", [5120, 4096, 1000])
def test_final_norm(pkg, oracle, M, K):
    g = torch.Generator(device="cuda").manual_seed(M * 10 + K)
    h = torch.randn(M, 4, K, device="cuda", generator=g).to(torch.bfloat16)
    pre = torch.rand(M, 4, device="cuda", generator=g) + 0.1
    w = (1.0 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    got = pkg.final_norm(h, pre, w)
    torch.cuda.synchronize()
    r = oracle_lib.ReferenceGpu()
    if r.available:  # the three reference kernels in a row, bit for bit
        x = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
        ref = torch.empty(M, K, device="cuda")
        assert r.dense.ds41_dense_hc_pre(h.data_ptr(), pre.data_ptr(), x.data_ptr(), M, K, None) == 0
        assert r.dense.ds41_dense_rms(x.data_ptr(), w.data_ptr(), x.data_ptr(), M, K, 1e-20, None) == 0
        assert r.dense.ds41_dense_promote(x.data_ptr(), ref.data_ptr(), M * K, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, ref)
    # CPU restatement: rsqrtf on the device against 1/sqrt here can move a BF16 result by one unit in a few entries
    want = oracle.final_norm(bf16_bits(h), pre.cpu().numpy(), bf16_bits(w))
    gotn = got.cpu().numpy()
    differ = gotn != want
    assert differ.mean() < 0.02
    assert np.all(np.abs(gotn - want)[differ] <= np.abs(want[differ]) * 2.0 ** -7)


def test_argument_checks(pkg):
    x = torch.zeros(9, 256, device="cuda")
    w = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        pkg.head_compact(x, w)                      # M > 8 (compact.cu:45)
    with pytest.raises(RuntimeError):
        pkg.head_compact(x[:2, :200].contiguous(), w[:, :200].contiguous())   # K not a multiple of 256
    with pytest.raises(RuntimeError):
        pkg.final_norm(torch.zeros(9, 4, 256, dtype=torch.bfloat16, device="cuda"), torch.zeros(9, 4, device="cuda"),
                       torch.zeros(256, dtype=torch.bfloat16, device="cuda"))
