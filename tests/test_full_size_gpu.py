"""GPU parity at the full sizes of the synthetic workloads (the bench's configurations), each compared with the CPU
oracle on a sample of rows while the GPU call runs the whole batch:
  - penalties + bitmask + top-k + top-p at 256 rows with 32768-token histories,
  - the FP8 head at 1024 rows over the whole vocabulary (the 128 x 256 tile kernel) followed by the sampler's batch path,
  - speculative verification with the draft noise frozen at the value that gives about 85 % acceptance."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
V = 129280
DRAFT_SIGMA = 0.30   # draft logits = target + N(0, sigma^2): 85 % of the proposals are accepted at T = 0.6, top-p 0.95


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    entry.build()
    return entry.load_package()


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u64(a):
    return cu(np.asarray(a, np.uint64).view(np.int64))


def test_penalties_mask_topk_at_256_rows_with_32k_histories(pkg, oracle):
    rows, hist_len = 256, 32768
    x = oracle.gen_logits(4, rows, V)
    hist = oracle.gen_history(4, rows, V, hist_len)
    mask = oracle.gen_mask(4, rows, V)
    seeds, steps = np.arange(rows) + 100, np.arange(rows) * 5
    kw = dict(top_k=50, repetition=1.1, presence=0.3, frequency=0.2)
    tok, st = pkg.sample_logits(cu(x), 0.8, 0.9, u64(seeds), u64(steps), history=cu(hist),
                                mask=cu(mask.view(np.int32)), **kw)
    torch.cuda.synchronize()
    tok, st = tok.cpu().numpy(), st.cpu().numpy()
    assert (st == 0).all(), st[st != 0]
    pick = np.arange(0, rows, 8)   # 32 rows through the oracle
    want, wst = oracle.sample_rows(x[pick], 0.8, 0.9, seeds[pick], steps[pick], history=hist[pick], mask=mask[pick],
                                   threads=8, **kw)
    assert (wst == 0).all() and (tok[pick] == want).all(), (tok[pick], want)
    for r in range(rows):   # every token is an allowed id
        assert (mask[r, tok[r] >> 5] >> (tok[r] & 31)) & 1


def test_head_and_sampler_at_1024_rows_full_vocabulary(pkg, oracle):
    B, K = 1024, 4096
    g = torch.Generator(device="cuda").manual_seed(7)
    w = torch.randn(V, K, device="cuda", generator=g) * 0.02
    ws = (w.view(V // 128, 128, K // 128, 128).abs().amax(dim=(1, 3)) / 448.0).float().contiguous()
    wq = (w.view(V // 128, 128, K // 128, 128) / ws[:, None, :, None]).view(V, K).to(torch.float8_e4m3fn).view(torch.uint8)
    del w
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    a, a_scale = pkg.quantize_activations(x)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ext = torch.empty((B, 16), dtype=torch.uint8, device="cuda")
    logits = pkg.head_fp8(a, a_scale, wq, ws, error_flag=flag, row_extremes=ext)
    torch.cuda.synchronize()
    assert flag.item() == 0 and torch.isfinite(logits).all()
    # head: FP64 dequantise-and-multiply oracle on three 128-id blocks of the vocabulary, all 1024 rows
    blocks = [0, 505, 1009]
    ids = np.concatenate([np.arange(b * 128, b * 128 + 128) for b in blocks])
    want = oracle.head_fp8(a.cpu().numpy(), a_scale.cpu().numpy(), wq[ids].cpu().numpy(), ws[blocks].cpu().numpy(), threads=8)
    got = logits[:, ids].cpu().numpy()
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max() + 1e-6
    # the records of the head's epilogue are the rows' true extremes
    rec = ext.cpu().numpy().view(np.uint32).reshape(B, 4)
    assert ((0xFFFFFFFF - rec[:, 0].astype(np.int64)) == logits.argmax(1).cpu().numpy()).all()
    # sampler: whole batch on the GPU (with and without the head's records), 64 rows through the oracle
    seeds, steps = np.arange(B) + 17, np.full(B, 3)
    scratch = torch.empty(pkg.sample_scratch_bytes(B, V), dtype=torch.uint8, device="cuda")
    tok, st = pkg.sample_logits(logits, 0.6, 0.95, u64(seeds), u64(steps), scratch=scratch)
    tok2, st2 = pkg.sample_logits(logits, 0.6, 0.95, u64(seeds), u64(steps), scratch=scratch, row_extremes=ext)
    torch.cuda.synchronize()
    tok, st = tok.cpu().numpy(), st.cpu().numpy()
    assert (st == 0).all() and (st2.cpu().numpy() == 0).all() and (tok == tok2.cpu().numpy()).all()
    pick = np.arange(0, B, 16)
    want_tok, wst = oracle.sample_rows(logits[pick].cpu().numpy(), 0.6, 0.95, seeds[pick], steps[pick], threads=8)
    assert (tok[pick] == want_tok).all(), (tok[pick], want_tok)


def test_verification_with_frozen_draft_noise(pkg, oracle):
    """32 sequences x (1 target + 2 draft) positions is the bench's shape; 128 sequences here so that the acceptance rate
    is measured on 256 proposals."""
    seqs, drafts, t, top = 128, 2, 0.6, 0.95
    target = oracle.gen_logits(31, seqs * (drafts + 1), V)
    base = target.reshape(seqs, drafts + 1, V)[:, :drafts].reshape(-1, V)
    draft = oracle.gen_perturbed(31, base, DRAFT_SIGMA)
    seeds, steps = np.arange(seqs) * 101 + 7, np.arange(seqs) + 1000
    ids = np.zeros((seqs, drafts), np.int32)
    for k in range(drafts):   # proposals drawn on the device from q at (seed, step, slot = k, Draft)
        tk, stk = pkg.sample_logits(cu(draft[k::drafts]), t, top, u64(seeds), u64(steps), slot=k, purpose=1)
        assert (stk.cpu().numpy() == 0).all()
        ids[:, k] = tk.cpu().numpy()
        wk, _ = oracle.sample_rows(draft[k::drafts], t, top, seeds, steps, slot=k, purpose=1, threads=8)
        assert (ids[:, k] == wk).all()
    res, st = pkg.verify_logits(cu(target), cu(draft), cu(ids), drafts, t, top, u64(seeds), u64(steps))
    torch.cuda.synchronize()
    got, st = pkg.results_to_numpy(res), st.cpu().numpy()
    want, wst = oracle.verify_rows(target, draft, ids, drafts, t, top, seeds, steps, threads=8)
    assert (st == 0).all() and (wst == 0).all()
    for f in ("emitted", "accepted_drafts", "accepted_input_rows", "rejected"):
        assert (got[f] == want[f]).all(), f
    for gr, wr in zip(got, want):
        assert list(gr["tokens"][:gr["emitted"]]) == list(wr["tokens"][:wr["emitted"]])
    rate = got["accepted_drafts"].sum() / (got["accepted_drafts"] + got["rejected"]).sum()
    assert 0.80 <= rate <= 0.90, rate
