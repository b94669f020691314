"""Generates tests/golden/*.json by running the REFERENCE's own sampler (oracle/_ref/libds41_ref.so, compiled
from the reference sources by oracle/Makefile) on seeded synthetic inputs.  Run where the reference tree is
available:  python tests/golden/make_golden.py

The inputs come from the counter-based generators in oracle/ds41_oracle.cpp, so any machine can rebuild them;
only the outputs (token ids, accept/reject records) are stored.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
import oracle_lib  # noqa: E402

V = 129280


def config1(orc, ref, steps=1000):
    """Single sequence, V=129280, Zipf+Gaussian logits from seed 0; two sampling settings; one MTP position."""
    x = orc.gen_logits(0, 1, V)[0]
    draft = orc.gen_perturbed(0, x[None, :], 0.5)[0]
    out = {"vocab": V, "seed": 0, "steps": steps, "runs": []}
    for t, top in ((1.0, 1.0), (0.7, 0.95)):
        p = ref.probabilities(x, t, top)
        q = ref.probabilities(draft, t, top)
        tokens = [ref.sample(p, 0, s, 0, 0) for s in range(steps)]
        mtp = []
        for s in range(steps):
            d = ref.sample(q, 0, s, 0, 1)
            emitted, acc, rows, rej = ref.reject_sample([d], q[None, :], np.stack([p, p]), 0, s, t)
            mtp.append([d, acc, rej] + emitted)
        out["runs"].append({"temperature": t, "top_p": top, "kept": int((p > 0).sum()), "tokens": tokens,
                            "mtp": mtp})
    return out


def small_cases(orc, ref):
    """Assorted sizes/temperatures (the shapes engine/tests/sampling_parallel.cpp sweeps), 8 draws each."""
    cases = []
    rng_seed = 20261018
    for n in (7, 512, 4096, 4097, 65537, 129281):
        for t, top in ((1.0, 1.0), (0.7, 0.9), (1e-7, 1.0), (2.5, 0.5), (0.0, 1.0)):
            x = orc.gen_logits(rng_seed, 1, n, sigma=4.0, zipf_s=0.0, first_row=n)[0]
            if n % 2:
                m = float(x.max()) + 1.0
                x[n // 3] = m; x[n // 2] = m; x[n - 1] = m
            p = ref.probabilities(x, t, top)
            toks = [ref.argmax(x) if t == 0 else ref.sample(p, 77, s, s % 6, 0) for s in range(8)]
            cases.append({"n": n, "temperature": t, "top_p": top, "ties": bool(n % 2), "tokens": toks,
                          "kept": int((p > 0).sum())})
    return {"gen_seed": rng_seed, "sample_seed": 77, "cases": cases}


def main():
    orc, ref = oracle_lib.Oracle(), oracle_lib.Reference()
    assert ref.available, "build oracle/_ref first (make -C oracle)"
    with open(os.path.join(HERE, "config1_reference.json"), "w") as f:
        json.dump(config1(orc, ref), f)
    with open(os.path.join(HERE, "small_cases_reference.json"), "w") as f:
        json.dump(small_cases(orc, ref), f)


if __name__ == "__main__":
    main()
