"""Vocabulary-sharded sampling: candidates per shard + combine give the single-GPU / oracle tokens.

The ranks are emulated on one GPU (each shard's kernel is an ordinary launch over its slice of the same logits; no
kernel waits on another), the all-gather is a copy.  The real NCCL exchange is exercised by bench.py --gpus N and
the host-side exchange logic by tests/test_sharded_cpu.py (gloo, 2 ranks)."""
import importlib

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available()
    entry.build()
    return entry.load_package()


def emulate(pkg, logits, ranks, t, top, seeds, steps):
    sh = importlib.import_module("ds41_b200.sharded")
    rows, vocab = logits.shape
    plan = sh.shard_plan(vocab, ranks)
    records = []
    for v0, vn in plan:
        s = sh.ShardedSampler(pkg, torch, logits.device, rows, v0, vn, vocab, t, top, world=ranks)
        s.candidates(logits[:, v0:v0 + vn])
        records.append(s.local.clone())
    comb = sh.ShardedSampler(pkg, torch, logits.device, rows, 0, plan[0][1], vocab, t, top, world=ranks)
    comb.gathered = torch.cat(records)
    tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
    status = torch.empty(rows, dtype=torch.int32, device=logits.device)
    comb.combine(seeds, steps, tokens, status, slot=1, purpose=0)
    torch.cuda.synchronize()
    return tokens.cpu().numpy(), status.cpu().numpy()


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("t,top", [(0.6, 0.95), (0.3, 0.9), (0.0, 1.0)])
def test_sharded_matches_single_gpu_and_oracle(pkg, oracle, ranks, t, top):
    rows, vocab = 48, 129280
    x = oracle.gen_logits(77, rows, vocab)
    seeds, steps = np.arange(rows, dtype=np.uint64) + 9, np.arange(rows, dtype=np.uint64) * 11
    want, _ = oracle.sample_rows(x, t, top, seeds, steps, slot=1, threads=8)
    xd = torch.from_numpy(x).cuda()
    sd, st = torch.from_numpy(seeds.view(np.int64)).cuda(), torch.from_numpy(steps.view(np.int64)).cuda()
    tok, status = emulate(pkg, xd, ranks, t, top, sd, st)
    # a row is either certified (status 0) and equal to the oracle, or flagged as not covered -- never guessed
    assert ((status == 0) | (status == -8)).all(), status
    ok = status == 0
    assert ok.mean() > 0.8 and (tok[ok] == want[ok]).all()
    for r in np.where(~ok)[0]:
        kept = int((oracle.probabilities(x[r], t, top) > 0).sum())
        assert kept >= 16 and tok[r] == -1   # only nuclei with many ids inside one 8192-id chunk can be uncovered
    single, _ = pkg.sample_logits(xd, t, top, sd, st, slot=1)
    assert (single.cpu().numpy() == want).all()


def test_uncovered_rows_are_flagged_not_guessed(pkg, oracle):
    """A wide nucleus (T=1, top-p 0.95: ~1-4 thousand ids) cannot be covered by 64 candidates per shard."""
    rows, vocab = 8, 129280
    x = torch.from_numpy(oracle.gen_logits(78, rows, vocab)).cuda()
    z = torch.zeros(rows, dtype=torch.int64, device="cuda")
    tok, status = emulate(pkg, x, 4, 1.0, 0.95, z, z)
    assert (status == -8).all() and (tok == -1).all()
    tok, status = emulate(pkg, x, 2, 0.6, 1.0, z, z)   # top_p = 1 is never covered for large shards
    assert (status == -8).all()


def test_small_shards_send_everything(pkg, oracle):
    """Chunks with fewer than 64 ids send all of them, so any top-p (even 1.0) is covered."""
    rows, vocab = 32, 192
    x = oracle.gen_logits(79, rows, vocab, sigma=2.0, zipf_s=0.5)
    seeds, steps = np.arange(rows, dtype=np.uint64), np.arange(rows, dtype=np.uint64)
    xd = torch.from_numpy(x).cuda()
    sd, st = torch.from_numpy(seeds.view(np.int64)).cuda(), torch.from_numpy(steps.view(np.int64)).cuda()
    for t, top in ((1.0, 1.0), (0.8, 0.7)):
        want, _ = oracle.sample_rows(x, t, top, seeds, steps, slot=1, threads=4)
        sh = importlib.import_module("ds41_b200.sharded")
        records = []
        for v0 in range(0, vocab, 48):
            s = sh.ShardedSampler(pkg, torch, xd.device, rows, v0, 48, vocab, t, top, world=4)
            s.chunks = 1
            s.local = s.local[: rows * 544]
            s.candidates(xd[:, v0:v0 + 48])
            records.append(s.local.clone())
        comb = sh.ShardedSampler(pkg, torch, xd.device, rows, 0, 48, vocab, t, top, world=4)
        comb.chunks, comb.gathered = 1, torch.cat(records)
        tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
        status = torch.empty(rows, dtype=torch.int32, device="cuda")
        comb.combine(sd, st, tokens, status, slot=1)
        torch.cuda.synchronize()
        assert (status.cpu().numpy() == 0).all() and (tokens.cpu().numpy() == want).all()
