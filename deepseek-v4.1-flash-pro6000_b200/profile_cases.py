#!/usr/bin/env python
"""Small, self-ending cases of each kernel for profiler captures (a full-size bench step holds too much device memory
and runs too long to be replayed pass after pass).

    python deepseek-v4.1-flash-pro6000_b200/profile_cases.py head    [--rows 1024] [--vocab 16384] [--hidden 4096]
    python deepseek-v4.1-flash-pro6000_b200/profile_cases.py headbf16 [--rows 6]        (the reference's BF16 plugin shape)
    python deepseek-v4.1-flash-pro6000_b200/profile_cases.py sampler [--rows 64] [--dist flat|peaked] [--stream]
    python deepseek-v4.1-flash-pro6000_b200/profile_cases.py verify  [--seqs 8] [--drafts 2]

Each case launches its kernel `--repeat` times (default 3) after one warm-up call and checks the status words.  Inputs
are larger than the 126 MB L2 only where the kernel's DRAM figures are the point (sampler: rows * 517 KB); the head case
keeps the weight slice small on purpose: its question is the tensor pipe and the epilogue, not DRAM.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
VOCAB = 129280


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["head", "headbf16", "sampler", "verify"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--dist", default="flat", choices=["flat", "peaked"])
    ap.add_argument("--stream", action="store_true", help="sampler: give it scratch, i.e. allow the streaming path")
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--drafts", type=int, default=2)
    ap.add_argument("--repeat", type=int, default=3)
    args = ap.parse_args()
    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(7)
    if args.case == "head":
        rows = args.rows or 1024
        x = torch.randn(rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(args.vocab, args.hidden, device=dev, generator=g) * 0.02)
        blocks = w.view(args.vocab // 128, 128, args.hidden // 128, 128)
        ws = (blocks.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-30)
        wq = (blocks / ws[:, None, :, None]).reshape(args.vocab, args.hidden).to(torch.float8_e4m3fn).view(torch.uint8)
        a, a_scale = pkg.quantize_activations(x)
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        logits = torch.empty((rows, args.vocab), dtype=torch.float32, device=dev)
        for _ in range(1 + args.repeat):
            pkg.head_fp8(a, a_scale, wq, ws.contiguous(), logits, flag)
        torch.cuda.synchronize()
        assert flag.item() == 0
    elif args.case == "headbf16":
        rows = args.rows or 6
        x = torch.randn(rows, 5120, device=dev, generator=g)
        w = (0.02 * torch.randn(VOCAB, 5120, device=dev, generator=g)).to(torch.bfloat16)
        for _ in range(1 + args.repeat):
            pkg.head_bf16(x, w, decode_symbol=True)
        torch.cuda.synchronize()
    elif args.case == "sampler":
        rows = args.rows or 64
        if args.dist == "flat":
            x = 1.28 * torch.randn(rows, VOCAB, device=dev, generator=g)
        else:
            base = -1.1 * torch.log(torch.arange(1, VOCAB + 1, device=dev, dtype=torch.float32))
            x = torch.stack([base[torch.randperm(VOCAB, device=dev, generator=g)] for _ in range(rows)])
            x += 3.0 * torch.randn(rows, VOCAB, device=dev, generator=g)
        seeds = torch.arange(rows, dtype=torch.int64, device=dev)
        steps = torch.zeros(rows, dtype=torch.int64, device=dev)
        for _ in range(1 + args.repeat):
            tok, st = pkg.sample_logits(x, 0.6, 0.95, seeds, steps, scratch="auto" if args.stream else None)
        torch.cuda.synchronize()
        assert (st >= 0).all()
    else:
        seqs, d = args.seqs, args.drafts
        target = 3.0 * torch.randn(seqs * (d + 1), VOCAB, device=dev, generator=g)
        draft = target.view(seqs, d + 1, VOCAB)[:, :d].reshape(-1, VOCAB) + 0.35 * torch.randn(seqs * d, VOCAB, device=dev, generator=g)
        seeds = torch.arange(seqs, dtype=torch.int64, device=dev)
        steps = torch.full((seqs,), 3, dtype=torch.int64, device=dev)
        ids = torch.stack([pkg.sample_logits(draft[k::d].contiguous(), 0.6, 0.95, seeds, steps, slot=k, purpose=1)[0]
                           for k in range(d)], dim=1).contiguous()
        for _ in range(1 + args.repeat):
            res, st = pkg.verify_logits(target, draft, ids.view(-1), d, 0.6, 0.95, seeds, steps)
        torch.cuda.synchronize()
        assert (st >= 0).all()
    print("ok")


if __name__ == "__main__":
    main()
