"""The replay's sums: `acc += v[i]` with every rounding of the reference's one-thread loops
(engine/third_party/spark/src/sampling.cpp:18-21,34-36), computed in parallel.  Checked bit for bit against the literal
loop (numpy's add.accumulate is that loop) on inputs built to hit every branch: binade crossings at every step, exact
half-way ties, zeros, subnormals, terms far below the accumulator's spacing, and invalid terms."""
import ctypes as C

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def run():
    pkg = entry.load_package()
    lib = pkg.lib()
    lib.ds41_b200_test_sequential.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_double, C.c_void_p, C.c_void_p]

    def call(v, mode=0, threshold=0.0):
        d = torch.from_numpy(np.ascontiguousarray(v, dtype=np.float64)).cuda()
        out = torch.zeros(3, dtype=torch.float64, device="cuda")
        rc = lib.ds41_b200_test_sequential(d.data_ptr(), d.numel(), mode, threshold, out.data_ptr(),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        found, acc, before = out.cpu().numpy()
        return int(found), acc, before
    return call


def literal(v, mode=0, threshold=0.0):
    c = np.add.accumulate(np.asarray(v, dtype=np.float64))
    if mode == 1:
        hit = np.nonzero(~(c < threshold))[0]
    elif mode == 2:
        hit = np.nonzero(threshold < c)[0]
    else:
        hit = np.zeros(0, dtype=np.int64)
    if hit.size == 0:
        return -1, c[-1], None
    i = int(hit[0])
    return i, c[i], (c[i - 1] if i else 0.0)


def cases():
    rng = np.random.default_rng(7)
    out = {}
    out["weights"] = np.exp(rng.normal(0, 2.1, 129280) - 9.0)                  # what a row's exp() weights look like
    out["sorted"] = np.sort(out["weights"])[::-1].copy()                          # the top-p loop's order
    out["wide"] = np.exp2(rng.uniform(-200, 40, 50000))                           # a crossing at almost every step
    out["tiny_then_big"] = np.concatenate([np.full(5000, 2.0 ** -60), rng.uniform(0, 1, 5000)])
    # exact ties: acc in [1, 2) has spacing 2^-52; terms (k + 1/2) * 2^-52 are half way
    ties = (rng.integers(0, 1000, 20000) + 0.5) * 2.0 ** -52
    out["ties"] = np.concatenate([[1.0], ties, rng.uniform(0, 1e-3, 3000), ties[:5000]])
    out["zeros"] = np.where(rng.uniform(size=30000) < 0.7, 0.0, rng.uniform(0, 1, 30000))
    out["leading_zeros"] = np.concatenate([np.zeros(9000), rng.uniform(0, 1e-5, 4000)])
    out["subnormal"] = np.concatenate([rng.integers(1, 1 << 40, 6000).astype(np.float64) * 5e-324,
                                       [2.2250738585072014e-308] * 50, rng.uniform(0, 1e-300, 3000)])
    out["single"] = np.array([0.3])
    out["tile_edges"] = rng.uniform(0, 1, 4096 * 3 + 1)
    out["probabilities"] = out["weights"] / out["weights"].sum()
    return out


@pytest.mark.parametrize("name", list(cases().keys()))
def test_sum_has_the_loops_roundings(run, name):
    v = cases()[name]
    _, want, _ = literal(v)
    found, got, _ = run(v)
    assert found == -1
    assert got == want, (name, got, want, (got - want) / want)


@pytest.mark.parametrize("name", ["weights", "sorted", "wide", "ties", "zeros", "probabilities", "tile_edges"])
@pytest.mark.parametrize("mode", [1, 2])
def test_stopping_rule_stops_where_the_loop_does(run, name, mode):
    v = cases()[name]
    c = np.add.accumulate(v)
    rng = np.random.default_rng(len(name) + mode)
    picks = list(rng.integers(0, len(v), 12)) + [0, len(v) - 1]
    for i in picks:
        # thresholds at, just below and just above a step of the chain: the comparisons that decide a token
        for thr in (c[i], np.nextafter(c[i], 0.0), np.nextafter(c[i], np.inf), 0.5 * (c[i] + c[max(i - 1, 0)])):
            want = literal(v, mode, thr)
            got = run(v, mode, thr)
            if want[0] < 0:
                assert got[0] == -1 and got[1] == want[1]
            else:
                assert got == want, (name, mode, i, thr, got, want)


def test_invalid_terms_take_the_literal_loop(run):
    rng = np.random.default_rng(3)
    v = rng.uniform(0, 1, 10000)
    v[1234] = -0.25
    v[7000] = -1e-9
    _, want, _ = literal(v)
    assert run(v)[1] == want
    v[8000] = np.inf
    assert run(v)[1] == np.inf
