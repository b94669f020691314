"""GPU parity of the sampler's batch path (csrc/flat.cu: histogram, window, FP64 masses, resolve) against the CPU oracle:
rows cut only by top-p are answered by it at every batch size (checked in its scratch records), rows it does not fit
fall through to the other paths, and every token equals the reference rule's
(engine/third_party/spark/src/sampling.cpp:18-38)."""
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


def batch_records(pkg, scratch, rows, vocab):
    """Per-row records of the batch path (layout of launch_flat: a 16-byte header, list counters, histograms, window
    lists, sub-region sums, then the 48-byte records {max, min, argmax, applicable, w0, w1, n_before, n_window, ...})."""
    lib = pkg.lib()
    lib.ds41_b200_shard_chunks.restype = C.c_int
    chunks = lib.ds41_b200_shard_chunks(vocab)
    streaming = rows * chunks * 544 + ((rows * 4 + 15) & ~15)
    info = streaming + 16 + rows * (16 + 2048 * 8 + 1024 * 8 + 128 * 8 + 128 * 8)
    return scratch[info: info + rows * 48].cpu().numpy().view(np.int32).reshape(rows, 12)


def answered_by_batch_path(pkg, scratch, rows, vocab):
    return batch_records(pkg, scratch, rows, vocab)[:, 3] == 1


@pytest.mark.parametrize("t,top", [(0.6, 0.95), (1.0, 0.95), (0.6, 0.5), (1.3, 0.99), (0.25, 0.9), (0.8, 1.0)])
def test_flat_rows_match_oracle(pkg, oracle, t, top):
    rows = 200
    x = oracle.gen_normal(11, int(t * 100), (rows, V), 1.28)
    seeds, steps = np.arange(rows) * 31 + 5, np.arange(rows) + 1000
    want, wst = oracle.sample_rows(x, t, top, seeds, steps, slot=1, purpose=0, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), t, top, seeds, steps, slot=1)
    assert (st == 0).all(), st
    assert (tok == want).all()
    assert answered_by_batch_path(pkg, scratch, rows, V).mean() > 0.95
    rec = batch_records(pkg, scratch, rows, V)
    if top < 1:
        assert (rec[:, 7] >= 1).all() and (rec[:, 7] <= 1024).all()      # ids inside the window
        assert np.median(rec[:, 5] - rec[:, 4]) <= 1                      # the window is one or two bins


@pytest.mark.parametrize("rows", [1, 3, 8, 33, 64, 130, 520])
def test_every_batch_size_takes_the_batch_path(pkg, oracle, rows):
    """The number of CTAs per row changes with the batch (32 pieces for one row down to one piece from 1024 rows)."""
    x = oracle.gen_normal(21, rows, (rows, V), 1.28)
    seeds, steps = np.arange(rows) * 7 + 1, np.arange(rows) * 3 + 11
    want, _ = oracle.sample_rows(x, 0.6, 0.95, seeds, steps, slot=0, purpose=0, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), 0.6, 0.95, seeds, steps)
    assert (st == 0).all() and (tok == want).all(), (tok, want, st)
    assert answered_by_batch_path(pkg, scratch, rows, V).all()


def test_peaked_rows_and_mixed_batch(pkg, oracle):
    """Flat rows, peaked rows (nucleus of a few ids) and rows with one towering logit in one batch: the batch path
    answers all of them (a small nucleus only makes the window small)."""
    rows = 208
    x = oracle.gen_normal(12, 0, (rows, V), 1.28)
    x[1::4] = oracle.gen_logits(77, rows // 4, V)          # Zipf + Gaussian: peaked
    x[2::8, 777] = 40.0                                     # one id holds all the mass: nucleus of one
    seeds, steps = np.arange(rows) + 3, np.arange(rows) * 7
    want, wst = oracle.sample_rows(x, 0.7, 0.9, seeds, steps, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), 0.7, 0.9, seeds, steps)
    assert (st >= 0).all() and (tok == want).all(), (tok, want, st)
    assert answered_by_batch_path(pkg, scratch, rows, V).mean() > 0.9


def test_rows_the_batch_path_cannot_take_fall_through(pkg, oracle):
    """Constant rows, rows with thousands of equal logits at the cut, and a temperature so low that the row's range
    exceeds the path's exponent limit: answered by the other paths, same tokens as the oracle."""
    rows = 40
    x = oracle.gen_normal(14, 0, (rows, V), 1.28)
    x[5] = 0.25                                  # constant row: no range
    x[6, ::2] = 1.5; x[6, 1::2] = -1.0           # two plateaus of 64640 ids: the cut falls inside the upper one
    x[7] = np.round(x[7] * 2) / 2                # quantised logits: a few dozen distinct values, plateaus of thousands
    seeds, steps = np.arange(rows) + 9, np.arange(rows) * 5 + 2
    want, _ = oracle.sample_rows(x, 0.6, 0.9, seeds, steps, threads=8)
    tok, st, scratch = sample(pkg, torch.from_numpy(x).cuda(), 0.6, 0.9, seeds, steps)
    assert (st >= 0).all(), st
    assert (tok == want).all(), (np.flatnonzero(tok != want), tok, want)
    used = answered_by_batch_path(pkg, scratch, rows, V)
    assert not used[[5, 6, 7]].any() and used.sum() >= rows - 4
    # T = 0.002: range * log2(e) / T is far above the limit of 600
    want, _ = oracle.sample_rows(x[:4], 0.002, 0.9, seeds[:4], steps[:4], threads=4)
    tok, st, scratch = sample(pkg, torch.from_numpy(x[:4]).cuda(), 0.002, 0.9, seeds[:4], steps[:4])
    assert (st >= 0).all() and (tok == want).all()
    assert not answered_by_batch_path(pkg, scratch, 4, V).any()


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
    assert answered_by_batch_path(pkg, scratch, rows, V).all()


def test_batch_weight_error_bound(pkg):
    """The FP64 pass's weight 2^-((max - y) * log2(e) / T) (64-entry table of 2^(-j/64) times a Taylor polynomial of
    degree 4) against long double: within the 1024 * 2^-53 relative that the resolve kernel's bounds allow for, over
    temperatures, offsets and ranges up to the path's exponent limit; exactly 1 at the maximum."""
    lib = pkg.lib()
    lib.ds41_b200_test_batch_weight.argtypes = [C.c_void_p, C.c_float, C.c_double, C.c_void_p, C.c_int, C.c_void_p]
    rng = np.random.default_rng(3)
    worst = 0.0
    for t, m, span in ((0.6, 5.3125, 11.3), (1.0, -2.71875, 24.0), (0.25, 11.0, 7.5), (1.7, 0.0, 50.0),
                       (0.6, 37.5, 12.0), (0.5, 1000.0, 30.0), (1.0, -3000.0, 100.0), (0.3, 2.5, 31.0), (2.0, 0.5, 1.0),
                       (0.1, 3.0, 41.0)):
        y = (np.float32(m) - (rng.random(2_000_000) * span).astype(np.float32)).astype(np.float32)
        y[0] = np.float32(m)
        yt = torch.from_numpy(y).cuda()
        out = torch.empty(y.size, dtype=torch.float64, device="cuda")
        assert lib.ds41_b200_test_batch_weight(yt.data_ptr(), m, t, out.data_ptr(), y.size, None) == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy().astype(np.longdouble)
        arg = (y.astype(np.longdouble) - np.longdouble(np.float32(m))) / np.longdouble(t)
        want = np.exp(arg)
        rel = np.abs(got - want) / want
        worst = max(worst, float(rel.max()) / 2.0 ** -53)
        assert got[0] == 1.0
    assert worst <= 1024.0, worst
    print("worst weight error in units of 2^-53:", worst)


@pytest.mark.parametrize("M", [8, 64, 300])
def test_row_extremes_from_the_head(pkg, oracle, M):
    """ds41_b200_head_fp8_stats: the head's epilogue leaves each row's first maximum, minimum and finiteness; the sampler
    given those records skips its own first pass and returns the same tokens."""
    N, K = 129280, 1024
    g = torch.Generator(device="cuda").manual_seed(70 + M)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.04
    ws = (w.view(N // 128, 128, K // 128, 128).abs().amax(dim=(1, 3)) / 448.0).float().contiguous()
    wq = (w.view(N // 128, 128, K // 128, 128) / ws[:, None, :, None]).view(N, K).to(torch.float8_e4m3fn).view(torch.uint8)
    del w
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    a, a_scale = pkg.quantize_activations(x)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain = pkg.head_fp8(a, a_scale, wq, ws, error_flag=flag)
    ext = torch.full((M, 16), 0xAB, dtype=torch.uint8, device="cuda")  # the call clears it
    logits = pkg.head_fp8(a, a_scale, wq, ws, error_flag=flag, row_extremes=ext)
    torch.cuda.synchronize()
    assert flag.item() == 0 and torch.equal(plain, logits)
    rec = ext.cpu().numpy().view(np.uint32).reshape(M, 4)
    lg = logits.cpu().numpy()

    def unorder(o):
        o = o.astype(np.uint32)
        bits = np.where(o >> 31, o ^ np.uint32(0x80000000), ~o)
        return bits.astype(np.uint32).view(np.float32)
    assert (unorder(rec[:, 1]) == lg.max(1)).all()
    assert ((0xFFFFFFFF - rec[:, 0].astype(np.int64)) == lg.argmax(1)).all()
    assert (unorder(~rec[:, 2]) == lg.min(1)).all()
    assert (rec[:, 3] == 0).all()
    seeds, steps = np.arange(M) + 1, np.arange(M) * 2 + 5
    tok0, st0, _ = sample(pkg, logits, 0.6, 0.95, seeds, steps)
    tok1, st1, scratch = sample(pkg, logits, 0.6, 0.95, seeds, steps, row_extremes=ext)
    assert (st0 == 0).all() and (st1 == 0).all() and (tok0 == tok1).all()
    assert answered_by_batch_path(pkg, scratch, M, N).all()
    want, _ = oracle.sample_rows(lg[: min(M, 48)], 0.6, 0.95, seeds[:48], steps[:48], threads=8)
    assert (tok1[: min(M, 48)] == want).all()
    # a non-finite logit in a row is seen by the record's flag
    bad = a_scale.clone(); bad[M // 2, 0] = float("inf")
    pkg.head_fp8(a, bad, wq, ws, logits=logits, error_flag=flag, row_extremes=ext)
    tok2, st2, _ = sample(pkg, logits, 0.6, 0.95, seeds, steps, row_extremes=ext)
    assert st2[M // 2] == -1 and tok2[M // 2] == -1 and (np.delete(st2, M // 2) == 0).all()


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
