"""GPU parity of the score-reporting entry point against the CPU restatement of the reference's log_normalizer /
top_order (engine/src/server.cpp:178-183, 730-737): ids bit-exact, FP64 values within 1e-13 relative."""
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


@pytest.mark.parametrize("vocab,top", [(7, 7), (1000, 5), (129280, 20), (129280, 0), (131072, 32)])
def test_score_matches_oracle(pkg, oracle, vocab, top):
    rows = 6
    x = oracle.gen_logits(21 + vocab, rows, vocab)
    x[1, : min(vocab, 50)] = x[1].max() + 1.0   # ties at the top: the lower ids come first
    x[2] = 0.5                                   # a constant row
    lse, top1, ids, lp, st = pkg.score_logits(torch.from_numpy(x).cuda(), top)
    torch.cuda.synchronize()
    lse, top1, ids, lp, st = (t.cpu().numpy() for t in (lse, top1, ids, lp, st))
    assert (st == 0).all()
    for r in range(rows):
        w_lse, w_top1, w_ids, w_lp = oracle.score_row(x[r], top)
        assert top1[r] == w_top1
        assert abs(lse[r] - w_lse) <= 1e-13 * max(1.0, abs(w_lse))
        assert ids[r].tolist() == w_ids.tolist()
        assert np.all(np.abs(lp[r] - w_lp) <= 1e-13 * np.maximum(1.0, np.abs(w_lp)))


def test_score_rejects_nonfinite_rows_and_bad_arguments(pkg, oracle):
    x = oracle.gen_logits(5, 3, 4096)
    x[1, 17] = np.nan
    lse, top1, ids, lp, st = pkg.score_logits(torch.from_numpy(x).cuda(), 4)
    torch.cuda.synchronize()
    assert st.cpu().tolist() == [0, -1, 0]
    assert np.isnan(lse.cpu().numpy()[1]) and (ids.cpu().numpy()[1] == -1).all() and top1.cpu().numpy()[1] == -1
    with pytest.raises(RuntimeError):
        pkg.score_logits(torch.from_numpy(x).cuda(), 33)


@pytest.mark.parametrize("vocab", [1, 13, 14, 15, 16, 17, 129280, 129281])
def test_logits_sha256(pkg, vocab):
    """engine/src/server.cpp:184-197: SHA-256 over the row's fp32 values in little-endian byte order (all padding cases
    of the last block: 0..15 left-over words)."""
    import hashlib
    rows = 5
    g = torch.Generator(device="cuda").manual_seed(vocab)
    buf = torch.randn(rows, vocab + 3, device="cuda", generator=g)
    x = buf[:, :vocab]
    got = pkg.logits_sha256(x)
    want = [hashlib.sha256(r.tobytes()).hexdigest() for r in x.cpu().numpy()]
    assert got == want
