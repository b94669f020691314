"""Pins the CPU oracle (oracle/ds41_oracle.cpp) before anything is checked against it.

1. the reference's own known answers, taken as text from engine/tests/core.cpp:22-42,50-60;
2. the committed golden fixtures made by running the reference sampler (tests/golden/make_golden.py);
3. where oracle/_ref is built: bit-for-bit equality with the reference functions on random inputs, following
   engine/tests/sampling_parallel.cpp:14-41.
"""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")
TARGET, DRAFT, ACCEPT, RESIDUAL = 0, 1, 2, 3


def test_philox_known_answers(oracle):
    # engine/tests/core.cpp:22-26
    assert oracle.word(0, 0, 0, TARGET, 0) == 0xE0481467
    assert oracle.word(0, 0, 0, TARGET, 1) == 0x8DDFD609
    assert oracle.word(0, 0, 0, TARGET, 2) == 0xB08E446F
    assert oracle.word(0, 0, 0, TARGET, 3) == 0x1852B5AB
    assert oracle.uniform(0, 0, 0, TARGET) == 0.8760998513862246
    # core.cpp:27-31: domain separation and range errors
    assert oracle.word(0, 0, 0, TARGET) != oracle.word(0, 0, 0, DRAFT)
    assert oracle.word(0, 1, 0, TARGET) != oracle.word(0, 0, 0, TARGET)
    assert oracle.word(0, 0, 1, TARGET) != oracle.word(0, 0, 0, TARGET)
    assert np.isnan(oracle.uniform(0, 0, 0, TARGET, 8589934592))
    assert oracle.word(0, 0, 6, TARGET) == 0 and "range" in oracle.error()


def test_probabilities_known_answers(oracle):
    # core.cpp:35-42
    assert oracle.probabilities([0, 0, 0, 0], 1, 1)[0] == 0.25
    assert list(oracle.probabilities([2, 1, 0], 0, 1)) == [1, 0, 0]
    assert list(oracle.probabilities([0, 0, 0, 0], 1, 0.5)) == [0.5, 0.5, 0, 0]
    a = oracle.probabilities([0, 1e-6], 1e-6, 1)
    b = oracle.probabilities([0, 1e-6], 1e-5, 1)
    assert (a == b).all()
    with pytest.raises(ValueError):
        oracle.probabilities([np.nan], 1, 1)
    with pytest.raises(ValueError):
        oracle.probabilities([0], -1, 1)
    with pytest.raises(ValueError):
        oracle.sample([0, 0], 0, 0, 0, TARGET)


def test_greedy_verify_known_answers(oracle):
    # core.cpp:48-60
    rows = np.array([[0, 0, 1, 0], [0, 1, 0, 0], [1, 0, 0, 0]], np.float64)
    for seed in (0, 1, 42, 99):
        r = oracle.verify([2, 0], None, rows, True, seed, 100)
        assert list(r.tokens[:r.emitted]) == [2, 1] and r.accepted_drafts == 1
        assert r.accepted_input_rows == 2 and r.rejected == 1
        r = oracle.verify([2], None, rows[:2], True, seed, 100)
        assert list(r.tokens[:r.emitted]) == [2, 1] and not r.rejected and r.accepted_input_rows == 2


def test_losslessness_statistics(oracle):
    # core.cpp:43-76 with fewer trials: the emitted first token follows p within 6 sigma.
    pairs = [([.1, .2, .3, .4], [.4, .3, .2, .1]), ([.2, .3, .5, 0], [0, 0, 0, 1]),
             ([.25, .25, .25, .25], [.25, .25, .25, .25]),
             ([1e-30, .5, .25, .25 - 1e-30], [.5, 1e-30, .25, .25 - 1e-30])]
    trials, pos = 20000, 0
    for p, q in pairs:
        counts = np.zeros(4)
        pp = np.array([p, p], np.float64)
        for _ in range(trials):
            d = oracle.sample(q, 0, pos, 0, DRAFT)
            r = oracle.verify([d], np.array([q], np.float64), pp, False, 0, pos)
            counts[r.tokens[0]] += 1
            pos += 1
        for j in range(4):
            expected = trials * p[j]
            sigma = np.sqrt(expected * (1 - p[j]))
            assert abs(counts[j] - expected) < 6 * sigma + 2


def test_config1_fixture(oracle):
    """Oracle reproduces the reference's tokens and MTP records on benchmark configuration 1 (1,000 steps, two settings)."""
    g = json.load(open(os.path.join(GOLD, "config1_reference.json")))
    V = g["vocab"]
    x = oracle.gen_logits(g["seed"], 1, V)[0]
    draft = oracle.gen_perturbed(g["seed"], x[None, :], 0.5)[0]
    for run in g["runs"]:
        t, top = run["temperature"], run["top_p"]
        p = oracle.probabilities(x, t, top)
        q = oracle.probabilities(draft, t, top)
        assert int((p > 0).sum()) == run["kept"]
        assert [oracle.sample(p, 0, s, 0, TARGET) for s in range(g["steps"])] == run["tokens"]
        pp = np.stack([p, p])
        for s, rec in enumerate(run["mtp"]):
            d = oracle.sample(q, 0, s, 0, DRAFT)
            r = oracle.verify([d], q[None, :], pp, False, 0, s)
            assert [d, r.accepted_drafts, r.rejected] + list(r.tokens[:r.emitted]) == rec
        # the batched entry used by the GPU parity tests agrees with the single-row calls
        rows = np.repeat(x[None, :], 16, 0)
        toks, status = oracle.sample_rows(rows, t, top, np.zeros(16, np.uint64), np.arange(16, dtype=np.uint64))
        assert list(toks) == run["tokens"][:16] and not status.any()


def test_small_cases_fixture(oracle):
    g = json.load(open(os.path.join(GOLD, "small_cases_reference.json")))
    for c in g["cases"]:
        n, t, top = c["n"], c["temperature"], c["top_p"]
        x = oracle.gen_logits(g["gen_seed"], 1, n, sigma=4.0, zipf_s=0.0, first_row=n)[0]
        if c["ties"]:
            m = float(x.max()) + 1.0
            x[n // 3] = m; x[n // 2] = m; x[n - 1] = m
        p = oracle.probabilities(x, t, top)
        assert int((p > 0).sum()) == c["kept"]
        toks = [oracle.argmax(x) if t == 0 else oracle.sample(p, g["sample_seed"], s, s % 6, TARGET) for s in range(8)]
        assert toks == c["tokens"], (n, t, top)


def test_bitwise_against_reference(oracle, reference):
    """engine/tests/sampling_parallel.cpp:14-41 restated: probability rows bit-for-bit, verify outcomes equal."""
    rng = np.random.default_rng(20261018)
    for n in (4096, 4097, 65537, 129280):
        for t, top in ((1.0, 1.0), (0.7, 1.0), (1e-7, 1.0), (2.5, 1.0), (0.7, 0.9), (1.0, 0.3)):
            x = rng.normal(0, 4, n).astype(np.float32)
            x[n // 3] = x[n // 2] = x[n - 1] = x.max() + 1
            ours, theirs = oracle.probabilities(x, t, top), reference.probabilities(x, t, top)
            assert ours.tobytes() == theirs.tobytes(), (n, t, top)
            lib = reference.spark_probabilities(x, max(t, 1e-5), top)
            assert ours.tobytes() == lib.tobytes()
            for step in range(3):
                assert oracle.sample(ours, 0x5EED, step, 1, TARGET) == reference.sample(theirs, 0x5EED, step, 1, TARGET)
                r = oracle.verify(None, None, ours[None, :], False, 0x5EED, step)
                emitted, acc, rows, rej = reference.reject_sample([], None, theirs[None, :], 0x5EED, step, t)
                assert list(r.tokens[:r.emitted]) == emitted and (r.accepted_drafts, r.accepted_input_rows, r.rejected) == (acc, rows, rej)
    # drafted verification, two positions
    n = 4097
    tl = rng.normal(0, 3, (3, n)).astype(np.float32)
    dl = (tl[:2] + rng.normal(0, 0.7, (2, n))).astype(np.float32)
    for t, top in ((1.0, 1.0), (0.8, 0.9)):
        p = np.stack([oracle.probabilities(r, t, top) for r in tl])
        q = np.stack([oracle.probabilities(r, t, top) for r in dl])
        for step in range(200):
            d = [oracle.sample(q[k], 9, step, k, DRAFT) for k in range(2)]
            r = oracle.verify(d, q, p, False, 9, step)
            emitted, acc, rows, rej = reference.reject_sample(d, q, p, 9, step, t)
            assert list(r.tokens[:r.emitted]) == emitted and (r.accepted_drafts, r.rejected) == (acc, rej)
    for x in (np.array([np.nan], np.float32),):
        with pytest.raises(ValueError):
            reference.probabilities(x, 1, 1)
    last, threw = reference.attempt_counter_take2(2**64 - 2)
    assert last == 2**64 - 1 and threw


def test_rng_against_reference(oracle, reference):
    rng = np.random.default_rng(1)
    for _ in range(2000):
        seed, step = (int(v) for v in rng.integers(0, 2**63, 2, dtype=np.int64))
        slot, purpose, draw = int(rng.integers(0, 6)), int(rng.integers(0, 4)), int(rng.integers(0, 1000))
        assert oracle.word(seed, step, slot, purpose, draw) == reference.word(seed, step, slot, purpose, draw)
        assert oracle.uniform(seed, step, slot, purpose, draw) == reference.uniform(seed, step, slot, purpose, draw)


def test_extension_rule_reduces_to_reference_rule(oracle):
    """With no penalties, mask or top-k the extension rule is the reference rule (bitwise)."""
    x = oracle.gen_logits(3, 1, 4097)[0]
    for t, top in ((1.0, 1.0), (0.8, 0.9), (0.0, 1.0)):
        assert oracle.extended_probabilities(x, t, top).tobytes() == oracle.probabilities(x, t, top).tobytes()
    # top-k by the stable order: ties at the cut keep the lower ids
    p = oracle.extended_probabilities([1, 3, 3, 3, 0], 1.0, 1.0, top_k=2)
    assert list(p > 0) == [False, True, True, False, False]
    # mask excludes ids, penalties follow the pinned FP32 formula
    mask = np.array([0b10110], np.uint32)
    p, eff = oracle.extended_probabilities([5, 1, 2, -3, 4], 1.0, 1.0, history=[2, 2, 3, 9, -1], repetition=1.5,
                                           presence=0.25, frequency=0.5, mask=mask, want_effective=True)
    f = np.float32
    assert eff[0] == -np.inf and eff[3] == -np.inf and eff[1] == f(1)
    assert eff[2] == f(f(2) / f(1.5)) - (f(0.25) + f(0.5) * f(2))
    assert eff[4] == f(4)
    assert p[0] == 0 and p[3] == 0 and abs(p.sum() - 1) < 1e-12
    with pytest.raises(ValueError):
        oracle.extended_probabilities([1, 2], 1.0, 1.0, mask=np.array([0], np.uint32))


def test_e4m3_roundtrip(oracle):
    table = oracle.e4m3_table()
    assert table[0x7E] == 448 and table[0x08] == 2.0 ** -6 and table[0x01] == 2.0 ** -9 and np.isnan(table[0x7F])
    for b in range(256):
        if np.isnan(table[b]) or b == 0x80:
            continue
        assert oracle.lib.oracle_e4m3_encode(float(table[b])) == b
    # ties go to even mantissa, values beyond the range saturate
    assert oracle.lib.oracle_e4m3_encode(1.0625) == 0x38       # halfway 1.0 / 1.125 -> 1.0 (even)
    assert oracle.lib.oracle_e4m3_encode(1.1875) == 0x3A       # halfway 1.125 / 1.25 -> 1.25 (even)
    assert oracle.lib.oracle_e4m3_encode(1e9) == 0x7E and oracle.lib.oracle_e4m3_encode(-1e9) == 0xFE


def test_score_row_restatement(oracle):
    """log_normalizer / top_order (engine/src/server.cpp:178-183, 730-737) restated: against an independent numpy
    evaluation (math.fsum for the sum, a stable sort for the order), incl. ties."""
    import math
    x = oracle.gen_logits(31, 1, 5000)[0]
    x[100:110] = x.max() + 0.5
    lse, top1, ids, lp = oracle.score_row(x, 12)
    m = float(x.max())
    want = m + math.log(math.fsum(math.exp(float(v) - m) for v in x))
    assert abs(lse - want) <= 1e-13 * abs(want)
    order = np.lexsort((np.arange(x.size), -x.astype(np.float64)))[:12]
    assert top1 == 100 and ids.tolist() == order.tolist()
    assert np.allclose(lp, x[order].astype(np.float64) - lse, rtol=0, atol=1e-12)
    with pytest.raises(ValueError):
        oracle.score_row(np.array([1.0, np.inf], np.float32), 1)
