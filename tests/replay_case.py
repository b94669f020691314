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


def main():
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
