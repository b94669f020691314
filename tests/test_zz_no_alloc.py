"""The scratch-free verification entry point (ds41_b200_verify_logits_static), called through the C ABI.

Some callers cannot allocate device memory when they verify a speculative step (fixed memory plan, foreign
allocator), so this entry point keeps its per-row statistics in an array built into the library.  It must return
exactly what ds41_b200_verify_logits returns with caller scratch: same emitted tokens, accept counts and status words.
The check runs on two calls in a row (the second smaller and on different data, so stale records of the first call
would show).  This file is collected last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C

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


def call_static(pkg, target, draft, ids, drafts, t, top, seeds, steps):
    """Raw C-ABI call: only inputs and outputs are passed, scratch stays NULL."""
    seqs = target.shape[0] // (drafts + 1)
    results = torch.zeros(seqs * C.sizeof(pkg.SparkResult), dtype=torch.uint8, device="cuda")
    status = torch.full((seqs,), 99, dtype=torch.int32, device="cuda")
    a = pkg.VerifyArgs()
    a.struct_bytes = C.sizeof(pkg.VerifyArgs)
    a.sequences, a.drafts, a.vocab = seqs, drafts, target.shape[1]
    a.target_logits, a.draft_logits, a.draft_ids = target.data_ptr(), draft.data_ptr(), ids.data_ptr()
    a.temperature, a.top_p = t, top
    a.seeds, a.steps = seeds.data_ptr(), steps.data_ptr()
    a.results, a.status = results.data_ptr(), status.data_ptr()
    a.scratch, a.scratch_bytes = None, 0
    rc = pkg.lib().ds41_b200_verify_logits_static(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, results, status


def make_inputs(oracle, seed, seqs, drafts, vocab, t, top):
    target = oracle.gen_logits(seed, seqs * (drafts + 1), vocab)
    base = target.reshape(seqs, drafts + 1, vocab)[:, :drafts].reshape(-1, vocab)
    draft = oracle.gen_perturbed(seed, base, 0.6)
    seeds = np.arange(seqs, dtype=np.uint64) + seed
    steps = np.arange(seqs, dtype=np.uint64) * 3 + 1
    ids = np.zeros((seqs, drafts), np.int32)
    for k in range(drafts):
        ids[:, k], _ = oracle.sample_rows(draft[k::drafts], t, top, seeds, steps, slot=k, purpose=1, threads=8)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return (cu(target), cu(draft), cu(ids.reshape(-1)), cu(seeds.view(np.int64)), cu(steps.view(np.int64)))


def test_static_scratch_matches_caller_scratch_twice(pkg, oracle):
    for call, (seed, seqs, drafts, vocab, t, top) in enumerate([(61, 24, 3, 32768, 0.9, 0.9), (62, 5, 2, 129280, 1.0, 1.0)]):
        target, draft, ids, seeds, steps = make_inputs(oracle, seed, seqs, drafts, vocab, t, top)
        want_res, want_st = pkg.verify_logits(target, draft, ids, drafts, t, top, seeds, steps)
        rc, got_res, got_st = call_static(pkg, target, draft, ids, drafts, t, top, seeds, steps)
        torch.cuda.synchronize()
        assert rc == 0, pkg.last_error()
        assert torch.equal(got_st, want_st) and (got_st >= 0).all(), (call, got_st, want_st)
        assert torch.equal(got_res, want_res), call
        emitted = pkg.results_to_numpy(got_res)["emitted"]
        assert (emitted >= 1).all() and (emitted <= drafts + 1).all()


@pytest.mark.parametrize("seqs,drafts,vocab,t,top", [
    (1, 2, 129280, 0.6, 0.95),    # the common decode step: five rows, the chunk + combine path inside the static array
    (1, 1, 129280, 1.0, 1.0),
    (3, 0, 129280, 0.8, 0.9),     # no drafts: the bonus sample only
    (4, 2, 129280, 0.0, 1.0),     # greedy
    (1, 5, 50000, 0.7, 0.9),
])
def test_static_scratch_small_calls(pkg, oracle, seqs, drafts, vocab, t, top):
    """Calls small enough for the streaming path keep their chunk records in the built-in array too; the results are
    those of the call with caller scratch, and a larger call right after still works (no record outlives its call)."""
    t_draw = t if t > 0 else 1.0
    target, draft, ids, seeds, steps = make_inputs(oracle, 70 + seqs + drafts, seqs, max(drafts, 1), vocab, t_draw, top)
    if drafts == 0:
        target = target[::2].contiguous()          # one target row per sequence
        draft, ids = draft[:0], ids[:0]
        draft = torch.zeros((1, vocab), device="cuda")   # never read: drafts == 0
        ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    want_res, want_st = pkg.verify_logits(target, draft, ids, drafts, t, top, seeds, steps)
    rc, got_res, got_st = call_static(pkg, target, draft, ids, drafts, t, top, seeds, steps)
    torch.cuda.synchronize()
    assert rc == 0, pkg.last_error()
    assert torch.equal(got_st, want_st) and (got_st >= 0).all(), (got_st, want_st)
    assert torch.equal(got_res, want_res)
    big = make_inputs(oracle, 91, 16, 2, 32768, 0.9, 0.9)
    want_res, want_st = pkg.verify_logits(big[0], big[1], big[2], 2, 0.9, 0.9, big[3], big[4])
    rc, got_res, got_st = call_static(pkg, big[0], big[1], big[2], 2, 0.9, 0.9, big[3], big[4])
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(got_res, want_res) and torch.equal(got_st, want_st)


def test_static_scratch_rejects_oversized_requests(pkg):
    assert pkg.lib().ds41_b200_verify_logits_static_max_rows() == 1024
    a = pkg.VerifyArgs()
    a.struct_bytes = C.sizeof(pkg.VerifyArgs)
    a.sequences, a.drafts, a.vocab = 200, 3, 1024   # 200 * 7 = 1400 records > 1024
    rc = pkg.lib().ds41_b200_verify_logits_static(C.byref(a), None)
    assert rc == 1 and "built-in limit" in pkg.last_error()
