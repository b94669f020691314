"""Operators on probability rows (csrc/prob.cu): the device form of the reference sampler's C ABI
(engine/third_party/spark/src/sampling.cpp:12-59) against the oracle.

`ds41_b200_probabilities` follows the reference rule operation by operation; only its `exp` is the device's, so a row
must have EXACTLY the reference's support (the top-p cut keeps the same ids: this is what pins the replay's chain over
the stable order) and values within a few units in the last place.  Sampling and verification take rows as given, so
on the oracle's own rows their results are the oracle's bit for bit."""
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


def rows_for(oracle, kind, rows, vocab):
    if kind == "flat":                         # what a randomly initialised head gives: nuclei of tens of thousands of ids
        return oracle.gen_normal(61, 0, (rows, vocab), 1.28)
    if kind == "zipf":                         # the benchmark's Zipf + Gaussian recipe: nuclei of a few dozen ids
        return oracle.gen_logits(62, rows, vocab)
    x = oracle.gen_normal(63, 0, (rows, vocab), 2.0)
    x = np.round(x * 4) / 4                    # heavy ties: the stable order decides which of equal logits are kept
    x[0] = 0.5                                 # all equal
    return x.astype(np.float32)


@pytest.mark.parametrize("kind", ["flat", "zipf", "ties"])
@pytest.mark.parametrize("vocab", [129280, 50000, 4097])
@pytest.mark.parametrize("t,top", [(0.6, 0.95), (1.0, 0.5), (0.8, 1.0), (0.3, 0.999)])
def test_probability_rows_have_the_references_support_and_values(pkg, oracle, kind, vocab, t, top):
    rows = 5
    x = rows_for(oracle, kind, rows, vocab)
    got, st = pkg.probabilities(torch.from_numpy(x).cuda(), t, top)
    torch.cuda.synchronize()
    assert (st.cpu().numpy() == 0).all()
    got = got.cpu().numpy()
    for r in range(rows):
        want = oracle.probabilities(x[r], t, top)
        g = got[r]
        if kind == "ties" and top < 1.0:
            # an exact tie of the running mass with top_p (whole multiples of equal weights) is decided by the last place
            # of exp(): then the support may differ by the ids of ONE tie group at the cut; otherwise it is exact
            same = np.array_equal(g > 0, want > 0)
            if not same:
                diff = np.nonzero((g > 0) != (want > 0))[0]
                assert np.unique(x[r][diff]).size == 1, (kind, vocab, t, top, r, diff[:8])
                continue
        assert np.array_equal(g > 0, want > 0), (kind, vocab, t, top, r, int((g > 0).sum()), int((want > 0).sum()))
        nz = want > 0
        rel = np.abs(g[nz] - want[nz]) / want[nz]
        assert rel.max() <= 8 * 2.0 ** -52, (kind, vocab, t, top, r, rel.max())
        assert abs(g.sum() - want.sum()) < 1e-12


def test_greedy_and_invalid_rows(pkg, oracle):
    x = oracle.gen_logits(64, 3, 1000)
    x[1, 17] = np.nan
    got, st = pkg.probabilities(torch.from_numpy(x).cuda(), 0.0, 1.0)
    got, st = got.cpu().numpy(), st.cpu().numpy()
    assert st[0] == 0 and st[2] == 0 and st[1] < 0 and np.isnan(got[1]).all()
    for r in (0, 2):
        assert got[r].sum() == 1.0 and got[r][int(np.argmax(x[r]))] == 1.0


@pytest.mark.parametrize("vocab", [129280, 4097])
def test_sampling_rows_is_the_references_draw(pkg, oracle, vocab):
    rows = 12
    x = oracle.gen_normal(65, 0, (rows, vocab), 1.28)
    p = np.stack([oracle.probabilities(x[r], 0.6, 0.95) for r in range(rows)])
    seeds, steps = np.arange(rows, dtype=np.uint64) + 7, np.arange(rows, dtype=np.uint64) * 11 + 1
    tok, st = pkg.sample_probabilities(torch.from_numpy(p).cuda(), torch.from_numpy(seeds.view(np.int64)).cuda(),
                                       torch.from_numpy(steps.view(np.int64)).cuda(), slot=3, purpose=1)
    want = [oracle.sample(p[r], int(seeds[r]), int(steps[r]), 3, 1) for r in range(rows)]
    assert (st.cpu().numpy() == 0).all() and tok.cpu().numpy().tolist() == want
    bad = p.copy()
    bad[2] *= 1.001                            # not normalised: the reference's validate() rejects it
    bad[5, 3] = -1e-9
    tok, st = pkg.sample_probabilities(torch.from_numpy(bad).cuda(), torch.from_numpy(seeds.view(np.int64)).cuda(),
                                       torch.from_numpy(steps.view(np.int64)).cuda())
    st = st.cpu().numpy()
    assert st[2] < 0 and st[5] < 0 and (np.delete(st, [2, 5]) == 0).all()


def test_verifying_rows_is_the_references_verification(pkg, oracle):
    vocab, seqs, drafts = 129280, 6, 2
    target = oracle.gen_logits(66, seqs * (drafts + 1), vocab)
    draft = oracle.gen_perturbed(66, target.reshape(seqs, drafts + 1, vocab)[:, :drafts].reshape(-1, vocab), 0.4)
    p = np.stack([oracle.probabilities(r, 0.6, 0.95) for r in target])
    q = np.stack([oracle.probabilities(r, 0.6, 0.95) for r in draft])
    seeds, steps = np.arange(seqs, dtype=np.uint64) + 2, np.arange(seqs, dtype=np.uint64) + 40
    ids = np.zeros((seqs, drafts), np.int32)
    for s in range(seqs):
        for k in range(drafts):
            ids[s, k] = oracle.sample(q[s * drafts + k], int(seeds[s]), int(steps[s]), k, 1)
    res, st = pkg.verify_probabilities(torch.from_numpy(ids.reshape(-1)).cuda(), torch.from_numpy(q).cuda(),
                                       torch.from_numpy(p).cuda(), drafts, torch.from_numpy(seeds.view(np.int64)).cuda(),
                                       torch.from_numpy(steps.view(np.int64)).cuda())
    got = pkg.results_to_numpy(res)
    assert (st.cpu().numpy() == 0).all()
    for s in range(seqs):
        want = oracle.verify(ids[s], q[s * drafts:(s + 1) * drafts], p[s * (drafts + 1):(s + 1) * (drafts + 1)], False,
                             int(seeds[s]), int(steps[s]))
        assert got["emitted"][s] == want.emitted and got["accepted_drafts"][s] == want.accepted_drafts
        assert got["rejected"][s] == want.rejected
        assert list(got["tokens"][s][:want.emitted]) == list(want.tokens[:want.emitted])
