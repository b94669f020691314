"""GPU parity of the sampler's batch path for wide nuclei (csrc/flat.cu) against the CPU oracle: flat rows are answered
by it (checked in its scratch records), rows it does not fit fall through to the other paths, and every token equals
the reference rule's."""
import ctypes as C

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
V = 129280


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    entry.build()
    return entry.load_package()


def u64(a):
    return torch.from_numpy(np.asarray(a, np.uint64).view(np.int64)).cuda()


def sample(pkg, x, t, top, seeds, steps, **kw):
    rows, vocab = x.shape
    scratch = torch.zeros(pkg.sample_scratch_bytes(rows, vocab), dtype=torch.uint8, device="cuda")
    tok, st = pkg.sample_logits(x, t, top, u64(seeds), u64(steps), scratch=scratch, **kw)
    torch.cuda.synchronize()
    return tok.cpu().numpy(), st.cpu().numpy(), scratch


def answered_by_batch_path(pkg, scratch, rows, vocab):
    """`applicable` word of the per-row records (layout of launch_flat: zeroed histograms and list counters first, then
    the window lists and the sub-region sums, then the records)."""
    lib = pkg.lib()
    lib.ds41_b200_shard_chunks.restype = C.c_int
    chunks = lib.ds41_b200_shard_chunks(vocab)
    streaming = rows * chunks * 544 + ((rows * 4 + 15) & ~15)
    info = streaming + rows * (1024 * 8 + 1024 * 4 + 16 + 1024 * 8 + 128 * 8 + 128 * 8)
    rec = scratch[info: info + rows * 32].cpu().numpy().view(np.int32).reshape(rows, 8)
    return rec[:, 3] == 1


@pytest.mark.parametrize("t,top", [(0.6, 0.95), (1.0, 0.95), (0.6, 0.5), (1.3, 0.99), (0.25, 0.9)])
def test_flat_rows_match_oracle(pkg, oracle, t, top):
    rows = 200
    x = oracle.gen_normal(11, int(t * 100), (rows, V), 1.28)
    seeds, steps = np.arange(rows) * 31 + 5, np.arange(rows) + 1000
    want, wst = oracle.sample_rows(x, t, top, seeds, steps, slot=1, purpose=0, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), t, top, seeds, steps, slot=1)
    assert (st == 0).all(), st
    assert (tok == want).all()
    used = answered_by_batch_path(pkg, scratch, rows, V)
    # T=0.25 sharpens N(0,1.28^2) into a nucleus of a few hundred ids: the other paths' case
    # (a row whose crossing falls inside the FP32-class bound goes to the cluster kernel: well under 5 %)
    assert used.mean() > 0.95 if t >= 0.6 else True


def test_mixed_batch_falls_through_per_row(pkg, oracle):
    """Flat rows, peaked rows (nucleus of a few ids) and rows with one towering logit in one batch."""
    rows = 208
    x = oracle.gen_normal(12, 0, (rows, V), 1.28)
    x[1::4] = oracle.gen_logits(77, rows // 4, V)          # Zipf + Gaussian: peaked
    x[2::8, 777] = 40.0                                     # one id holds all the mass: nucleus of one
    seeds, steps = np.arange(rows) + 3, np.arange(rows) * 7
    want, wst = oracle.sample_rows(x, 0.7, 0.9, seeds, steps, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), 0.7, 0.9, seeds, steps)
    assert (st >= 0).all() and (tok == want).all(), (tok, want, st)
    used = answered_by_batch_path(pkg, scratch, rows, V)
    flat_rows = np.ones(rows, bool); flat_rows[1::4] = False; flat_rows[2::8] = False
    assert used[flat_rows].mean() > 0.9 and not used[~flat_rows].any()


def test_nonfinite_rows_and_ragged_stride(pkg, oracle):
    rows, vocab, stride = 192, 40001, 40004
    buf = np.zeros((rows, stride), np.float32)
    buf[:, :vocab] = oracle.gen_normal(13, 0, (rows, vocab), 1.0)
    bad = [3, 17, 40]
    buf[3, 5] = np.nan; buf[17, vocab - 1] = np.inf; buf[40, 20000] = -np.inf
    seeds, steps = np.arange(rows), np.arange(rows) + 9
    good = np.setdiff1d(np.arange(rows), bad)
    want, _ = oracle.sample_rows(buf[good, :vocab].copy(), 0.8, 0.95, seeds[good], steps[good], threads=8)
    x = torch.from_numpy(buf).cuda()[:, :vocab]
    assert x.stride(0) == stride
    tok, st, scratch = sample(pkg, x, 0.8, 0.95, seeds, steps)
    assert (st[bad] == -1).all() and (tok[bad] == -1).all()
    assert (st[good] == 0).all() and (tok[good] == want).all()
    assert answered_by_batch_path(pkg, scratch, rows, vocab)[good].mean() > 0.9


def test_same_tokens_as_cluster_kernel_at_1024_rows(pkg):
    """Size-independent property at the bench's batch: both device paths certify and agree on every row."""
    rows = 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    x = 1.28 * torch.randn(rows, V, device="cuda", generator=g)
    seeds, steps = np.arange(rows) + 17, np.full(rows, 4)
    tok, st, scratch = sample(pkg, x, 0.6, 0.95, seeds, steps)
    ref, rst = pkg.sample_logits(x, 0.6, 0.95, u64(seeds), u64(steps), scratch=None)
    torch.cuda.synchronize()
    assert (st == 0).all() and (rst.cpu().numpy() == 0).all()
    assert (tok == ref.cpu().numpy()).all()
    assert answered_by_batch_path(pkg, scratch, rows, V).all()  # applicable: the window exists (the cut may still be handed on)


def test_histogram_weight_error_bound(pkg):
    """The histogram pass's fixed-point weight of an id (what the ids beyond the window enter the normaliser with):
    relative error below the 2.9e-7 the certification budgets (3.2e-7), against long double, over temperatures, logit
    offsets and ranges (weights down to 1e-30 of the maximum)."""
    lib = pkg.lib()
    lib.ds41_b200_test_hist_weight.argtypes = [C.c_void_p, C.c_float, C.c_float, C.c_double, C.c_void_p, C.c_int, C.c_void_p]
    rng = np.random.default_rng(3)
    worst = 0.0
    for t, m, span in ((0.6, 5.3125, 11.3), (1.0, -2.71875, 24.0), (0.25, 11.0, 7.5), (1.7, 0.0, 50.0), (0.6, 37.5, 12.0)):
        y = (np.float32(m) - (rng.random(2_000_000) * span).astype(np.float32)).astype(np.float32)
        y[0], y[1] = np.float32(m), np.float32(m) - np.float32(span)
        yt = torch.from_numpy(y).cuda()
        out = torch.empty(y.size, dtype=torch.float64, device="cuda")
        lo = float(np.float32(m) - np.float32(span))
        assert lib.ds41_b200_test_hist_weight(yt.data_ptr(), m, lo, t, out.data_ptr(), y.size, None) == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy().astype(np.longdouble)
        want = np.exp((y.astype(np.longdouble) - np.longdouble(np.float32(m))) / np.longdouble(t))
        ok = want > 1e-30
        rel = np.abs(got[ok] - want[ok]) / want[ok]
        worst = max(worst, float(rel.max()))
    assert worst < 2.9e-7, worst


@pytest.mark.parametrize("case", range(8))
def test_random_shapes_agree_with_cluster_kernel(pkg, case):
    """Randomised distributions (scale, offset, tails), temperatures and top-p: the batch path and the cluster kernel are
    independent implementations of the same certified rule, so wherever both certify they must give the same token."""
    rng = np.random.default_rng(100 + case)
    rows = 256
    g = torch.Generator(device="cuda").manual_seed(200 + case)
    sigma = float(rng.choice([0.3, 0.8, 1.28, 2.0, 3.5]))
    offset = float(rng.choice([0.0, -7.25, 41.5, 300.0, -1000.0]))
    x = sigma * torch.randn(rows, V, device="cuda", generator=g)
    if case % 3 == 1:   # heavier tails: product of two normals
        x = x * torch.randn(rows, V, device="cuda", generator=g).abs().clamp_(max=4.0)
    if case % 3 == 2:   # a few towering ids on top of the flat bulk
        idx = torch.randint(0, V, (rows, 5), device="cuda", generator=g)
        x.scatter_add_(1, idx, torch.full((rows, 5), 4.0 * sigma, device="cuda"))
    x = (x + offset).contiguous()
    t = float(rng.choice([0.3, 0.6, 0.8, 1.0, 1.5]))
    top = float(rng.choice([0.5, 0.8, 0.9, 0.95, 0.99, 0.999]))
    seeds, steps = np.arange(rows) * 3 + case, np.arange(rows) + 50 * case
    tok, st, scratch = sample(pkg, x, t, top, seeds, steps, slot=case % 6, purpose=case % 4)
    ref, rst = pkg.sample_logits(x, t, top, u64(seeds), u64(steps), slot=case % 6, purpose=case % 4, scratch=None)
    torch.cuda.synchronize()
    ref, rst = ref.cpu().numpy(), rst.cpu().numpy()
    assert (st >= 0).all() and (rst >= 0).all(), (st[st < 0], rst[rst < 0])
    both = (st == 0) & (rst == 0)
    assert both.mean() > 0.99
    assert (tok[both] == ref[both]).all(), (sigma, offset, t, top, np.flatnonzero(tok != ref))
