"""GPU parity of the MTP speculative verifier (accept / residual resample / bonus) against the CPU oracle."""
import json
import os

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DRAFT = 1


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available()
    entry.build()
    return entry.load_package()


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u64(a):
    return cu(np.asarray(a, np.uint64).view(np.int64))


def run(pkg, target, draft, ids, drafts, t, top, seeds, steps):
    res, st = pkg.verify_logits(cu(target), None if draft is None else cu(draft),
                                None if ids is None else cu(np.asarray(ids, np.int32)), drafts, t, top, u64(seeds),
                                u64(steps))
    torch.cuda.synchronize()
    return pkg.results_to_numpy(res), st.cpu().numpy()


def propose(oracle, draft, drafts, t, top, seeds, steps):
    """Draft ids drawn from q with the address (seed, step, slot=k, Draft), as speculation.cpp:154 does."""
    seqs = draft.shape[0] // max(drafts, 1)
    ids = np.zeros((seqs, drafts), np.int32)
    for k in range(drafts):
        if t == 0:
            ids[:, k] = draft[k::drafts].argmax(1)
        else:
            ids[:, k], _ = oracle.sample_rows(draft[k::drafts], t, top, seeds, steps, slot=k, purpose=DRAFT, threads=8)
    return ids


def same(got, want):
    for f in ("emitted", "accepted_drafts", "accepted_input_rows", "rejected"):
        assert (got[f] == want[f]).all(), (f, got[f], want[f])
    for g, w in zip(got, want):
        assert list(g["tokens"][:g["emitted"]]) == list(w["tokens"][:w["emitted"]])


@pytest.mark.parametrize("t,top,sigma", [(0.6, 0.95, 0.30), (1.0, 1.0, 0.5), (1.0, 0.9, 1.0), (0.0, 1.0, 0.5)])
@pytest.mark.parametrize("drafts", [0, 2, 5])
def test_config3_verification(pkg, oracle, t, top, sigma, drafts):
    """benchmark configuration 3 shape: sequences x (1 target + drafts) rows, V=129280."""
    seqs, vocab = (32 if drafts == 2 else 8), 129280
    target = oracle.gen_logits(31, seqs * (drafts + 1), vocab)
    seeds, steps = np.arange(seqs) * 101 + 7, np.arange(seqs) + 1000
    draft = ids = None
    if drafts:
        base = target.reshape(seqs, drafts + 1, vocab)[:, :drafts].reshape(-1, vocab)
        draft = oracle.gen_perturbed(31, base, sigma)
        ids = propose(oracle, draft, drafts, t, top, seeds, steps)
    want, wst = oracle.verify_rows(target, None if t == 0 else draft, ids, drafts, t, top, seeds, steps, threads=8)
    got, st = run(pkg, target, None if t == 0 else draft, ids, drafts, t, top, seeds, steps)
    assert (wst == 0).all() and (st == 0).all(), st
    same(got, want)
    if drafts == 2 and t > 0:
        rate = got["accepted_drafts"].sum() / max(1, (got["accepted_drafts"] + got["rejected"]).sum())
        assert 0.3 < rate <= 1.0


def test_config1_mtp_fixture(pkg, oracle):
    """The reference's own accept/resample records on benchmark configuration 1 (first 150 steps of both settings)."""
    g = json.load(open(os.path.join(GOLD, "config1_reference.json")))
    V, n = g["vocab"], 150
    x = oracle.gen_logits(g["seed"], 1, V)[0]
    d = oracle.gen_perturbed(g["seed"], x[None, :], 0.5)[0]
    target = np.repeat(x[None, :], 2 * n, 0)
    draft = np.repeat(d[None, :], n, 0)
    for rec in g["runs"]:
        ids = np.array([m[0] for m in rec["mtp"][:n]], np.int32)
        got, st = run(pkg, target, draft, ids, 1, rec["temperature"], rec["top_p"], np.zeros(n), np.arange(n))
        assert (st >= 0).all()
        for s in range(n):
            m = rec["mtp"][s]
            assert [got[s]["accepted_drafts"], got[s]["rejected"]] + list(got[s]["tokens"][:got[s]["emitted"]]) == m[1:]


def test_small_vocab_and_errors(pkg, oracle):
    rng = np.random.default_rng(5)
    vocab, seqs, drafts = 4097, 64, 3
    target = rng.normal(0, 3, (seqs * 4, vocab)).astype(np.float32)
    draft = (target.reshape(seqs, 4, vocab)[:, :3].reshape(-1, vocab) + rng.normal(0, 0.8, (seqs * 3, vocab))).astype(np.float32)
    seeds, steps = np.arange(seqs) + 3, np.arange(seqs) * 2
    ids = propose(oracle, draft, drafts, 0.9, 0.8, seeds, steps)
    ids[5, 0] = vocab          # out of range at the first position
    ids[6, 2] = -1             # out of range, reached only if the first two are accepted
    target[7 * 4 + 3, 11] = np.nan   # a bad row anywhere rejects the transaction
    # a draft id that q excludes (outside its nucleus): impossible under q
    q9 = oracle.probabilities(draft[9 * 3], 0.9, 0.8)
    ids[9, 0] = int(np.where(q9 == 0)[0][0])
    want, wst = oracle.verify_rows(target, draft, ids, drafts, 0.9, 0.8, seeds, steps, threads=8)
    got, st = run(pkg, target, draft, ids, drafts, 0.9, 0.8, seeds, steps)
    assert ((st < 0) == (wst < 0)).all(), (st, wst)
    assert st[5] == -6 and st[7] == -1 and st[9] == -6
    ok = st >= 0
    same(got[ok], want[ok])
    assert (got["emitted"][~ok] == -1).all()


def test_argument_errors(pkg):
    x = torch.zeros(2, 64, device="cuda")
    z = torch.zeros(1, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):
        pkg.verify_logits(x, None, torch.zeros(1, dtype=torch.int32, device="cuda"), 1, 1.0, 1.0, z, z)  # q missing
    with pytest.raises(RuntimeError):
        pkg.verify_logits(x, x[:1], torch.zeros(1, dtype=torch.int32, device="cuda"), 1, 1.0, 1.0, z, z,
                          scratch=torch.empty(8, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        pkg.verify_logits(torch.zeros(3, 64, device="cuda"), None, None, 1, 0.0, 1.0, z, z)
