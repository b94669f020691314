"""Host-side logic of the vocabulary-sharded path on CPU: two gloo ranks, the exchange and the escalation of
uncovered rows run through the real ShardedSampler code; the two CUDA kernels are replaced by a NumPy restatement of
their algorithm (checked against the oracle's tokens), because no GPU exists in this test."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REC = np.dtype([("z", np.float64), ("max", np.float32), ("argmax", np.int32), ("count", np.int32),
                ("status", np.int32), ("complete", np.int32), ("z_err", np.float32),
                ("cand", [("y", np.float32), ("id", np.int32)], 64)])


def test_shard_plan():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    plan = importlib.import_module("ds41_b200.sharded").shard_plan
    assert [n // 128 for _, n in plan(129280, 8)] == [127, 127, 126, 126, 126, 126, 126, 126]
    assert [n // 128 for _, n in plan(129280, 4)] == [253, 253, 252, 252]
    assert plan(129280, 2) == [(0, 64640), (64640, 64640)]
    for v, w in ((129280, 8), (1000, 3), (7, 2), (129281, 5)):
        p = plan(v, w)
        assert p[0][0] == 0 and sum(n for _, n in p) == v
        assert all(p[i][0] + p[i][1] == p[i + 1][0] for i in range(w - 1))
    assert REC.itemsize == 544


def numpy_candidates(x, v0, t):
    out = np.zeros(x.shape[0], REC)
    for r, row in enumerate(x):
        b = int(row.argmax())
        order = np.lexsort((np.arange(row.size), -row.astype(np.float64)))[:64]
        out[r]["max"], out[r]["argmax"] = row[b], b + v0
        out[r]["z"] = np.exp((row.astype(np.float64) - np.float64(row[b])) / t).sum()
        out[r]["count"], out[r]["complete"] = order.size, int(row.size <= 64)
        out[r]["cand"]["y"][:order.size] = row[order]
        out[r]["cand"]["id"][:order.size] = order + v0
    return out


def numpy_combine(records, ranks, t, top, seeds, steps, uniform):
    rows = records.shape[1]
    tokens, status = np.full(rows, -1, np.int32), np.zeros(rows, np.int32)
    for r in range(rows):
        h = records[:, r]
        best = max(range(ranks), key=lambda k: (h[k]["max"], -h[k]["argmax"]))
        m = np.float64(h[best]["max"])
        z = sum(h[k]["z"] * np.exp((np.float64(h[k]["max"]) - m) / t) for k in range(ranks))
        y = np.concatenate([h[k]["cand"]["y"][:h[k]["count"]] for k in range(ranks)])
        ids = np.concatenate([h[k]["cand"]["id"][:h[k]["count"]] for k in range(ranks)])
        owner = np.concatenate([np.full(h[k]["count"], k) for k in range(ranks)])
        order = np.lexsort((ids, -y.astype(np.float64)))
        e = np.exp((y[order].astype(np.float64) - m) / t)
        mass = np.cumsum(e)
        pos = int(np.argmax(mass >= top * z)) if (mass >= top * z).any() and top < 1 else -1
        covered = pos >= 0 and all(h[k]["complete"] or np.where(owner[order] == k)[0].max() > pos for k in range(ranks))
        if pos < 0 and all(h[k]["complete"] for k in range(ranks)):
            covered, pos = True, len(order) - 1
        if not covered:
            status[r] = -8
            continue
        keep = np.sort(order[:pos + 1], kind="stable")
        keep = keep[np.argsort(ids[keep], kind="stable")]
        ek = np.exp((y[keep].astype(np.float64) - m) / t)
        c = np.cumsum(ek)
        u = uniform(int(seeds[r]), int(steps[r]))
        hit = np.where(u * c[-1] < c)[0]
        tokens[r] = ids[keep][hit[0]] if hit.size else ids[keep][-1]
    return tokens, status


def worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import __graft_entry__ as entry
    import oracle_lib
    entry.load_package()
    sh = importlib.import_module("ds41_b200.sharded")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    orc = oracle_lib.Oracle()
    rows, vocab = 12, 4096 + 128
    x = orc.gen_logits(5, rows, vocab, sigma=2.5, zipf_s=1.3)
    seeds, steps = np.arange(rows, dtype=np.uint64) + 3, np.arange(rows, dtype=np.uint64) * 5
    failures = []
    for t, top in ((0.5, 0.9), (1.0, 0.97)):   # the second setting leaves some rows uncovered -> escalation path
        want, _ = orc.sample_rows(x, t, top, seeds, steps, slot=1, threads=2)
        v0, vn = sh.shard_plan(vocab, world)[rank]

        class CpuSampler(sh.ShardedSampler):
            def candidates(self, logits):
                rec = numpy_candidates(logits.numpy(), self.v0, self.t)
                self.local.copy_(torch.from_numpy(rec.view(np.uint8).reshape(-1)))

            def combine(self, seeds_t, steps_t, tokens, status, slot=0, purpose=0):
                rec = self.gathered.numpy().view(REC).reshape(self.world, self.rows)
                tok, st = numpy_combine(rec, self.world, self.t, self.top_p, seeds_t.numpy().view(np.uint64),
                                        steps_t.numpy().view(np.uint64), lambda s, p: orc.uniform(s, p, slot, purpose))
                tokens.copy_(torch.from_numpy(tok)); status.copy_(torch.from_numpy(st))

            def sample_full(self, full, seeds_t, steps_t, slot, purpose):
                tok, st = orc.sample_rows(full.numpy(), self.t, self.top_p, seeds_t.numpy().view(np.uint64),
                                          steps_t.numpy().view(np.uint64), slot=slot, purpose=purpose)
                return torch.from_numpy(tok), torch.from_numpy(st)

        s = CpuSampler(None, torch, torch.device("cpu"), rows, v0, vn, vocab, t, top)
        tokens, status = torch.empty(rows, dtype=torch.int32), torch.empty(rows, dtype=torch.int32)
        s.sample(torch.from_numpy(x[:, v0:v0 + vn].copy()), torch.from_numpy(seeds.view(np.int64)),
                 torch.from_numpy(steps.view(np.int64)), tokens, status, slot=1)
        if not (tokens.numpy() == want).all():
            failures.append(f"rank {rank} T={t} top={top}: {tokens.numpy()} != {want}")
        if (t, top) == (1.0, 0.97) and s.escalated == 0:
            failures.append("escalation path not exercised")
        gathered = [torch.empty_like(tokens) for _ in range(world)]
        dist.all_gather(gathered, tokens)
        if not all(torch.equal(g, tokens) for g in gathered):
            failures.append("ranks disagree")
    out[rank] = failures
    dist.destroy_process_group()


def test_two_rank_exchange_and_escalation_on_gloo():
    world, port = 2, 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(worker, args=(world, port, out), nprocs=world, join=True)
        assert len(out) == world
        for rank in range(world):
            assert out[rank] == [], out[rank]


def test_rows_plan_covers_every_row_once():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    sharded = importlib.import_module("ds41_b200.sharded")
    for rows in (1, 7, 64, 1000, 1024):
        for world in (1, 2, 3, 4, 8):
            per, plan = sharded.rows_plan(rows, world)
            assert per * world >= rows and len(plan) == world
            covered = [r for first, n in plan for r in range(first, first + n)]
            assert covered == list(range(rows))
            assert all(first == min(rows, r * per) for r, (first, _) in enumerate(plan))


def test_team_plan_partitions_rows_and_ranks():
    """Teams of vocab_ranks ranks: every batch row is computed by exactly one team, namely the team of the rank that
    owns (samples) it, and a team's rows are contiguous."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    sh = importlib.import_module("ds41_b200.sharded")
    for rows in (1, 7, 1000, 1024):
        for world, vocab_ranks in ((2, 1), (2, 2), (4, 2), (8, 2), (8, 4), (8, 8), (6, 3)):
            per, plan = sh.rows_plan(rows, world)
            computed = []
            for team in range(world // vocab_ranks):
                members = range(team * vocab_ranks, (team + 1) * vocab_ranks)
                got = {sh.team_plan(rows, world, r, vocab_ranks) for r in members}
                assert len(got) == 1                      # every member sees the same team
                team0, row0, n = got.pop()
                assert team0 == team * vocab_ranks
                owned = [r for m in members for r in range(plan[m][0], plan[m][0] + plan[m][1])]
                assert owned == list(range(row0, row0 + n))
                computed += owned
            assert computed == list(range(rows))
    with pytest.raises(ValueError):
        sh.team_plan(16, 8, 0, 3)


def rows_worker(rank, world, port, out, rows=7):
    """Row-sharded exchange on CPU: every rank samples its own rows (here: the oracle on full-vocabulary rows that the
    other ranks' "head slices" were written into) and publishes; everyone must end with all tokens."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import __graft_entry__ as entry
    import oracle_lib
    entry.load_package()
    sh = importlib.import_module("ds41_b200.sharded")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    orc = oracle_lib.Oracle()
    vocab = 2048                   # 7 rows over 3 ranks: 3 + 3 + 1 (ragged); 6 rows: 2 + 2 + 2 (single strided copy)
    x = orc.gen_logits(9, rows, vocab, sigma=2.0, zipf_s=1.1)
    seeds, steps = np.arange(rows, dtype=np.uint64) + 11, np.arange(rows, dtype=np.uint64) * 3
    want, wst = orc.sample_rows(x, 0.8, 0.9, seeds, steps, threads=2)
    ex = sh.RowExchange.__new__(sh.RowExchange)     # no peer memory on CPU: only the host logic is under test
    ex.world, ex.rank, ex.rows, ex.vocab, ex.group, ex.device = world, rank, rows, vocab, None, torch.device("cpu")
    ex.guard = sh.StepGuard(None)
    ex.rows_per_owner, plan = sh.rows_plan(rows, world)
    ex.row0, ex.my_rows = plan[rank]
    ex.packed = torch.full((2, ex.rows_per_owner), -1, dtype=torch.int32)
    ex.everyone = torch.empty((world, 2, ex.rows_per_owner), dtype=torch.int32)
    # the head's scatter, emulated: every rank contributes its vocabulary slice of every row to the row's owner
    full = torch.zeros((ex.rows_per_owner, vocab))
    pieces = [None] * world
    v0, vn = sh.shard_plan(vocab, world)[rank]
    dist.all_gather_object(pieces, (v0, vn, x[:, v0:v0 + vn].copy()))
    for p0, pn, block in pieces:
        full[:ex.my_rows, p0:p0 + pn] = torch.from_numpy(block[ex.row0:ex.row0 + ex.my_rows])
    if ex.my_rows:
        sl = slice(ex.row0, ex.row0 + ex.my_rows)
        tok, st = orc.sample_rows(full[:ex.my_rows].numpy(), 0.8, 0.9, seeds[sl], steps[sl], threads=1)
        ex.packed[0, :ex.my_rows] = torch.from_numpy(tok)
        ex.packed[1, :ex.my_rows] = torch.from_numpy(st)
    tokens, status = torch.empty(rows, dtype=torch.int32), torch.empty(rows, dtype=torch.int32)
    ex.publish(tokens, status)
    failures = []
    if not (tokens.numpy() == want).all():
        failures.append(f"rank {rank}: {tokens.numpy()} != {want}")
    if not (status.numpy() == wst).all():
        failures.append(f"rank {rank}: status {status.numpy()} != {wst}")
    out[rank] = failures
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [7, 6])
def test_three_rank_row_exchange_on_gloo(rows):
    world, port = 3, 31500 + (os.getpid() + rows * 37) % 2000
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(rows_worker, args=(world, port, out, rows), nprocs=world, join=True)
        assert len(out) == world
        for rank in range(world):
            assert out[rank] == [], out[rank]


def _failure_rank_setup(rank, world, port, timeout_s, check_every):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    sh = importlib.import_module("ds41_b200.sharded")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rows = 6
    guard = sh.StepGuard(None, timeout_s=timeout_s, check_every=check_every)
    ex = sh.RowExchange.__new__(sh.RowExchange)     # host logic only: no peer memory on CPU
    ex.world, ex.rank, ex.rows, ex.vocab, ex.group, ex.device = world, rank, rows, 128, None, torch.device("cpu")
    ex.guard = guard
    ex.rows_per_owner, plan = sh.rows_plan(rows, world)
    ex.row0, ex.my_rows = plan[rank]
    ex.packed = torch.full((2, ex.rows_per_owner), rank, dtype=torch.int32)
    ex.everyone = torch.empty((world, 2, ex.rows_per_owner), dtype=torch.int32)
    ex.word = torch.zeros(1, dtype=torch.int32)
    return sh, guard, ex, rows


def _one_step(guard, ex, rows):
    guard.before_step()
    ex.writers_done()
    tokens, status = torch.empty(rows, dtype=torch.int32), torch.empty(rows, dtype=torch.int32)
    ex.publish(tokens, status)
    guard.finish()
    return tokens


def never_arrives_worker(rank, world, port, out):
    """Rank 1 takes part in one step and then never enters the next one's collectives (it is stuck on the host)."""
    import time
    sh, guard, ex, rows = _failure_rank_setup(rank, world, port, timeout_s=2.0, check_every=1000)
    tokens = _one_step(guard, ex, rows)
    report = {"first_step_ok": tokens.tolist() == [0, 0, 0, 1, 1, 1]}
    if rank == 1:
        time.sleep(6.0)                     # longer than the survivor's limit; it leaves without a word
        out[rank] = report
        return
    t0 = time.monotonic()
    try:
        _one_step(guard, ex, rows)
        report["raised"] = None
    except sh.CollectiveFailure as exc:
        report["raised"], report["seconds"] = str(exc), time.monotonic() - t0
    try:                                     # the guard stays failed: nothing is launched into a broken group
        guard.before_step()
        report["stays_failed"] = False
    except sh.CollectiveFailure:
        report["stays_failed"] = True
    out[rank] = report


def test_rank_that_never_arrives_ends_in_a_clean_error_on_gloo():
    world, port = 2, 33500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(never_arrives_worker, args=(world, port, out), nprocs=world, join=True)
        survivor = out[0]
        assert survivor["first_step_ok"] and out[1]["first_step_ok"]
        assert survivor["raised"] and "writers-done all-reduce" in survivor["raised"], survivor
        assert survivor["seconds"] < 5.0, survivor       # the 2 s limit, not the process group's default 30 minutes
        assert survivor["stays_failed"]


def leaves_worker(rank, world, port, out):
    """Rank 2 leaves between steps and says so in the store; both survivors stop with the same clean error."""
    import time
    sh, guard, ex, rows = _failure_rank_setup(rank, world, port, timeout_s=2.0, check_every=1)
    _one_step(guard, ex, rows)
    if rank == 2:
        guard.leave()                        # nothing of this rank is in flight: the step above has finished
        out[rank] = {"left": True}
        time.sleep(1.0)
        return
    report = {"raised": None, "steps_after": 0}
    for _ in range(400):
        try:
            guard.before_step()              # the survivors' check before their next launch
        except sh.CollectiveFailure as exc:
            report["raised"] = str(exc)
            break
        report["steps_after"] += 1           # not yet visible: this step launches nothing here (the peer may be gone)
        time.sleep(0.005)
    out[rank] = report
    if rank == 0:
        time.sleep(1.5)                      # rank 0 hosts the store: keep it up until the others have read it


def test_rank_that_leaves_between_steps_stops_the_others_before_their_next_launch_on_gloo():
    world, port = 3, 35500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(leaves_worker, args=(world, port, out), nprocs=world, join=True)
        assert out[2] == {"left": True}
        for rank in (0, 1):
            assert out[rank]["raised"] and "left the group" in out[rank]["raised"], out[rank]


class _FakeStore:
    """Stand-in for the rendezvous store: add(key, n) returns the running count, as torch's stores do."""

    def __init__(self):
        self.counts, self.reads, self.broken = {}, 0, False

    def add(self, key, n):
        if self.broken:
            raise RuntimeError("store connection lost")
        self.reads += 1
        self.counts[key] = self.counts.get(key, 0) + n
        return self.counts[key]


def test_step_guard_host_logic_without_a_process_group():
    """The guard's bookkeeping on its own (no ranks, no GPU): the leave counter is read at the configured cadence, a
    leave or a lost store stops the step before anything is launched, a collective that raises becomes
    CollectiveFailure, and once failed the guard refuses everything."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    sh = importlib.import_module("ds41_b200.sharded")
    store = _FakeStore()
    g = sh.StepGuard(None, timeout_s=1.0, check_every=4, store=store)
    g.world = 3                                   # as if two peers existed
    for _ in range(9):
        g.before_step()
    assert store.reads == 3                       # steps 1, 5, 9
    store.counts["ds41_b200/left"] = 1            # a peer announced that it stops
    for _ in range(3):
        g.before_step()                           # steps 10-12: not a check step yet
    with pytest.raises(sh.CollectiveFailure, match="left the group"):
        g.before_step()                           # step 13
    with pytest.raises(sh.CollectiveFailure, match="earlier"):
        g.before_step()
    with pytest.raises(sh.CollectiveFailure):
        g.collective("anything", lambda: None)

    g2 = sh.StepGuard(None, timeout_s=1.0, check_every=1, store=store)
    g2.world = 2
    store.counts.clear()
    g2.before_step()
    def boom():
        raise RuntimeError("connection reset by peer")
    with pytest.raises(sh.CollectiveFailure, match="token all-gather: connection reset"):
        g2.collective("token all-gather", boom)
    assert g2.failed

    g3 = sh.StepGuard(None, timeout_s=1.0, check_every=1, store=store)
    g3.world = 2
    store.broken = True                           # the store lives on rank 0: unreachable means rank 0 is gone
    with pytest.raises(sh.CollectiveFailure, match="rendezvous store"):
        g3.before_step()
    g4 = sh.StepGuard(None, timeout_s=1.0, check_every=1, store=None)
    g4.before_step()                              # a single rank: nothing to watch
    g4.collective("none", lambda: None)
    g4.finish()
