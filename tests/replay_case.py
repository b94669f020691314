"""Helper of test_replay_gpu.py, run as a child process so that DS41_BOUND_SCALE (read once per process by the library)
can widen the batch path's certification bounds: most rows are then flagged as uncertified and must come back from the
exact replay with the oracle's tokens and status 0.  Prints one JSON line."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    sys.path.insert(0, p)
import __graft_entry__ as entry  # noqa: E402
import oracle_lib  # noqa: E402


def verify_case(seqs, vocab, t, top):
    """Speculative verification with widened bounds: flagged transactions come back from the replay with the oracle's
    records; prints how many transactions were flagged without the replay (status words of a scratch-limited call)."""
    pkg = entry.load_package()
    orc = oracle_lib.Oracle()
    drafts = 2
    target = orc.gen_logits(51, seqs * (drafts + 1), vocab)
    base = target.reshape(seqs, drafts + 1, vocab)[:, :drafts].reshape(-1, vocab)
    draft = orc.gen_perturbed(51, base, 0.4)
    seeds, steps = np.arange(seqs, dtype=np.uint64) + 3, np.arange(seqs, dtype=np.uint64) * 7 + 2
    ids = np.zeros((seqs, drafts), np.int32)
    for k in range(drafts):
        ids[:, k], _ = orc.sample_rows(draft[k::drafts], t, top, seeds, steps, slot=k, purpose=1, threads=8)
    want, wst = orc.verify_rows(target, draft, ids.reshape(-1), drafts, t, top, seeds, steps, threads=8)
    dev = torch.device("cuda", 0)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    args = (cu(target), cu(draft), cu(ids.reshape(-1)), drafts, t, top, cu(seeds.view(np.int64)), cu(steps.view(np.int64)))
    res, st = pkg.verify_logits(*args)
    # the same call with room for the statistics and chunk records only: no replay, the bits stay
    lib = pkg.lib()
    lib.ds41_b200_shard_chunks.restype = __import__("ctypes").c_int
    rows_all = seqs * (2 * drafts + 1)   # 48-byte statistics + 544-byte chunk records per row, rounded up to 16 bytes
    streaming_only = (rows_all * 48 + rows_all * lib.ds41_b200_shard_chunks(vocab) * 544 + 15) & ~15
    assert streaming_only < pkg.verify_scratch_bytes(seqs, drafts, vocab)
    small = torch.zeros(streaming_only, dtype=torch.uint8, device=dev)
    res0, st0 = pkg.verify_logits(*args, scratch=small)
    torch.cuda.synchronize()
    got = pkg.results_to_numpy(res)
    same = all((got[f] == want[f]).all() for f in ("tokens", "emitted", "accepted_drafts", "rejected"))
    print(json.dumps({"records_equal": bool(same), "status": np.unique(st.cpu().numpy()).tolist(),
                      "flagged_without_replay": int((st0.cpu().numpy() > 0).sum()),
                      "oracle_status": np.unique(wst).tolist(), "sequences": seqs}))


def main():
    if sys.argv[1] == "verify":
        return verify_case(int(sys.argv[2]), int(sys.argv[3]), float(sys.argv[4]), float(sys.argv[5]))
    rows, vocab = int(sys.argv[1]), int(sys.argv[2])
    t, top = float(sys.argv[3]), float(sys.argv[4])
    pkg = entry.load_package()
    orc = oracle_lib.Oracle()
    x = orc.gen_normal(41, rows, (rows, vocab), 1.28)
    x[1] = 0.75                        # a constant row: every id ties
    seeds, steps = np.arange(rows) * 13 + 1, np.arange(rows) + 77
    want, wst = orc.sample_rows(x, t, top, seeds, steps, slot=2, purpose=0, threads=8)
    dev = torch.device("cuda", 0)
    scratch = torch.zeros(pkg.sample_scratch_bytes(rows, vocab), dtype=torch.uint8, device=dev)
    u64 = lambda a: torch.from_numpy(np.asarray(a, np.uint64).view(np.int64)).to(dev)
    tok, st = pkg.sample_logits(torch.from_numpy(x).to(dev), t, top, u64(seeds), u64(steps), slot=2, scratch=scratch)
    torch.cuda.synchronize()
    lib = pkg.lib()
    lib.ds41_b200_shard_chunks.restype = __import__("ctypes").c_int
    streaming = rows * lib.ds41_b200_shard_chunks(vocab) * 544 + ((rows * 4 + 15) & ~15)
    header = scratch[streaming: streaming + 16].cpu().numpy().view(np.int32)
    print(json.dumps({"tokens_equal": bool((tok.cpu().numpy() == want).all()),
                      "mismatches": int((tok.cpu().numpy() != want).sum()),
                      "status": np.unique(st.cpu().numpy()).tolist(), "handed_on": int(header[0]),
                      "replayed": int(header[1]), "rows": rows}))


if __name__ == "__main__":
    main()
