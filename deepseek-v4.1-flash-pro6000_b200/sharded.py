"""Vocabulary-sharded decode tail across the GPUs of one node (one process per GPU, torch.distributed for the plumbing).

Rank r owns the contiguous id range produced by `shard_plan` (128-row blocks of the head's weight matrix, uneven by
at most one block).  Two exchanges are implemented:

* candidates (`ShardedSampler`): local candidates (CUDA) -> one all-gather of 544-byte records (one per 8192 ids) per
  row (NCCL on GPUs, gloo in the CPU tests) -> combine (CUDA, replicated on every rank).  Rows the combine cannot
  certify as covered are re-sampled from their full logits, gathered only for those rows.  Cheap when the nucleus is
  small (trained models: a few dozen ids); useless when it is not.
* rows (`RowExchange` + `ShardedDecodeTail`): the head kernel's epilogue stores each row's vocabulary slice straight
  into the full-vocabulary buffer of the rank that owns the row (peer stores over NVLink, overlapped with the GEMM), a
  one-word all-reduce orders readers after writers, every rank samples its rows with the single-GPU sampler, and one
  small all-gather publishes tokens and status.  Cost is independent of the distribution; this is what flat
  distributions (a randomly initialised head: nuclei of tens of thousands of ids) need.

`ShardedDecodeTail` picks between them from the coverage it observes.
"""
import math
import ctypes as C

import torch
import torch.distributed as dist

SHARD_ROW_BYTES = 544
NOT_COVERED = -8


class CollectiveFailure(RuntimeError):
    """A collective of the sharded step did not complete (a peer never arrived, left, or the communicator reported an
    error).  Raised on every surviving rank; the process group is unusable afterwards."""


class StepGuard:
    """Host-side failure detection around the collectives of the sharded decode tail.

    The reference has no collectives; what this guards is the exchange this library adds.  Three mechanisms, none of
    which touches a GPU's state:
      * every collective is issued with a work handle.  On host tensors (gloo) the handle is waited on with
        `timeout_s`; on device tensors the wait is stream-ordered (no host block) and the handle is kept until
        `finish()`, which polls a CUDA event with the same time limit instead of blocking in a synchronize that a
        dead peer would never release, and then reads the handles' recorded exceptions (the process group's
        asynchronous error state);
      * a rank that stops between steps says so in the rendezvous store (`leave()`); `before_step()` reads that
        counter every `check_every` steps, so the others stop before their next launch;
      * after any failure the guard stays failed: later calls raise at once, and `abort()` tears the communicator down
        (NCCL: abort, so that kernels already enqueued do not wait for the missing peer).
    """

    def __init__(self, group=None, timeout_s=30.0, check_every=64, store=None):
        self.group, self.timeout_s, self.check_every = group, float(timeout_s), max(1, int(check_every))
        self.failed, self.step_no, self.pending = None, 0, []
        self.store = store
        if store is None and dist.is_initialized() and dist.get_world_size(group) > 1:
            try:
                self.store = dist.distributed_c10d._get_default_store()
            except Exception:
                self.store = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def _fail(self, what, cause):
        self.failed = f"{what}: {cause}"
        self.abort()
        raise CollectiveFailure(f"rank {self.rank}: {self.failed}")

    def _check_failed(self):
        if self.failed:
            raise CollectiveFailure(f"rank {self.rank}: {self.failed} (earlier)")

    def leave(self):
        """Called by a rank that stops taking part, between steps, with none of its kernels or collectives in flight."""
        if self.store is not None:
            self.store.add("ds41_b200/left", 1)

    def before_step(self):
        self._check_failed()
        self.step_no += 1
        if self.store is not None and self.world > 1 and self.step_no % self.check_every == 1 % self.check_every:
            try:
                left = self.store.add("ds41_b200/left", 0)
            except Exception as exc:  # the store lives on rank 0: gone means rank 0 is gone
                self._fail("rendezvous store", exc)
            if left:
                self._fail("before launch", f"{left} rank(s) left the group")

    def collective(self, what, issue):
        """issue() starts the collective with async_op=True and returns its work handle."""
        import datetime
        self._check_failed()
        try:
            work = issue()
        except Exception as exc:
            self._fail(what, exc)
        if work is None:
            return
        on_device = torch.cuda.is_available() and dist.get_backend(self.group) == "nccl"
        try:
            if on_device:
                work.wait()  # orders the current stream after the collective; the host does not block
                if torch.cuda.is_current_stream_capturing():
                    return   # part of a CUDA graph: there is no per-replay handle; finish() bounds the replay's wait
                self.pending.append((what, work))
                if len(self.pending) > 64:
                    self.pending = [(w, h) for w, h in self.pending if not h.is_completed()][-64:]
            else:
                work.wait(datetime.timedelta(seconds=self.timeout_s))
        except Exception as exc:
            self._fail(what, exc)

    def finish(self):
        """Waits, with the time limit, for everything enqueued on the current stream, then surfaces recorded errors."""
        import time
        self._check_failed()
        if torch.cuda.is_available():
            done = torch.cuda.Event()
            done.record()
            deadline = time.monotonic() + self.timeout_s
            spins = 0
            while not done.query():
                spins += 1
                if spins > 2000:
                    time.sleep(0.0002)
                if time.monotonic() > deadline:
                    names = ", ".join(w for w, h in self.pending if not h.is_completed()) or "kernels"
                    self._fail("step did not finish", f"no completion within {self.timeout_s:g} s (pending: {names})")
        for what, work in self.pending:
            try:
                failed = work.is_completed() and not work.is_success()
            except Exception:   # the handle cannot be queried on this build: the event wait above is the check
                failed = False
            if failed:
                self.pending = []
                self._fail(what, "the process group recorded an error for this collective")
        self.pending = []

    def abort(self):
        if not dist.is_initialized():
            return
        try:
            if dist.get_backend(self.group) == "nccl":
                dist.distributed_c10d._abort_process_group(self.group)
        except Exception:
            pass


def shard_plan(vocab, world, block=128):
    """[(offset, length)] per rank: contiguous ranges on `block` boundaries, the first ranks take the extra blocks."""
    blocks = (vocab + block - 1) // block
    per, extra = divmod(blocks, world)
    plan, start = [], 0
    for r in range(world):
        n = (per + (1 if r < extra else 0)) * block
        n = max(0, min(n, vocab - start))
        plan.append((start, n))
        start += n
    return plan


CHUNK_IDS = 8192


def chunks_for(vocab_local):
    return (vocab_local + CHUNK_IDS - 1) // CHUNK_IDS


class ShardArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("rows", C.c_int32), ("vocab_local", C.c_int32),
                ("vocab_offset", C.c_int32), ("chunks", C.c_int32), ("logits", C.c_void_p),
                ("logits_stride", C.c_int64), ("temperature", C.c_double), ("out", C.c_void_p)]


class CombineArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("rows", C.c_int32), ("ranks", C.c_int32), ("chunks", C.c_int32),
                ("vocab", C.c_int32), ("gathered", C.c_void_p), ("temperature", C.c_double), ("top_p", C.c_double),
                ("top_k", C.c_int32), ("seeds", C.c_void_p), ("steps", C.c_void_p), ("slot", C.c_uint32),
                ("purpose", C.c_uint32), ("tokens", C.c_void_p), ("status", C.c_void_p)]


class ShardedSampler:
    launches_per_step = 2

    def __init__(self, pkg, torch_mod, device, rows, vocab_offset, vocab_local, vocab, temperature, top_p, group=None,
                 world=None, guard=None):
        self.pkg, self.device, self.rows = pkg, device, rows
        self.guard = guard or StepGuard(group)
        self.v0, self.vn, self.vocab = vocab_offset, vocab_local, vocab
        self.t, self.top_p, self.group = temperature, top_p, group
        self.world = world or (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # every rank publishes the same number of 8192-id chunk records per row (short shards pad with empty ones)
        self.chunks = max(chunks_for(n) for _, n in shard_plan(vocab, self.world))
        self.local = torch.empty(rows * self.chunks * SHARD_ROW_BYTES, dtype=torch.uint8, device=device)
        self.gathered = torch.empty(self.world * rows * self.chunks * SHARD_ROW_BYTES, dtype=torch.uint8, device=device)
        self._lib = None
        self.escalated = 0

    @property
    def lib(self):
        if self._lib is None:
            self._lib = self.pkg.lib()
            self._lib.ds41_b200_shard_candidates.argtypes = [C.POINTER(ShardArgs), C.c_void_p]
            self._lib.ds41_b200_shard_combine.argtypes = [C.POINTER(CombineArgs), C.c_void_p]
        return self._lib

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def candidates(self, logits):
        a = ShardArgs(C.sizeof(ShardArgs), self.rows, self.vn, self.v0, self.chunks, logits.data_ptr(),
                      logits.stride(0), self.t, self.local.data_ptr())
        rc = self.lib.ds41_b200_shard_candidates(C.byref(a), self._stream())
        if rc:
            raise RuntimeError(f"ds41_b200_shard_candidates: cudaError {rc} ({self.pkg.last_error()})")

    def combine(self, seeds, steps, tokens, status, slot=0, purpose=0):
        a = CombineArgs(C.sizeof(CombineArgs), self.rows, self.world, self.chunks, self.vocab,
                        self.gathered.data_ptr(), self.t, self.top_p, 0, seeds.data_ptr(), steps.data_ptr(), slot,
                        purpose, tokens.data_ptr(), status.data_ptr())
        rc = self.lib.ds41_b200_shard_combine(C.byref(a), self._stream())
        if rc:
            raise RuntimeError(f"ds41_b200_shard_combine: cudaError {rc} ({self.pkg.last_error()})")

    def sample(self, logits, seeds, steps, tokens, status, slot=0, purpose=0, escalate=True):
        """logits: this rank's [rows, vocab_local] slice.  Every rank ends with the same tokens / status."""
        self.candidates(logits)
        if self.world > 1:
            self.guard.collective("candidate all-gather", lambda: dist.all_gather_into_tensor(
                self.gathered, self.local, group=self.group, async_op=True))
        else:
            self.gathered.copy_(self.local)
        self.combine(seeds, steps, tokens, status, slot, purpose)
        if escalate:
            self.resample_uncovered(logits, seeds, steps, tokens, status, slot, purpose)
        return tokens, status

    def resample_uncovered(self, logits, seeds, steps, tokens, status, slot, purpose):
        """Rows flagged NOT_COVERED: gather their full logits on every rank and use the single-GPU sampler."""
        rows = (status == NOT_COVERED).nonzero().flatten()  # identical on every rank (the combine is replicated)
        n = int(rows.numel())
        if n == 0:
            return
        self.escalated += n
        plan = shard_plan(self.vocab, self.world)
        width = max(length for _, length in plan)
        mine = torch.zeros((n, width), dtype=torch.float32, device=self.device)
        mine[:, : self.vn] = logits[rows]
        everyone = torch.empty((self.world, n, width), dtype=torch.float32, device=self.device)
        if self.world > 1:
            self.guard.collective("uncovered-row all-gather", lambda: dist.all_gather_into_tensor(
                everyone.view(-1), mine.view(-1), group=self.group, async_op=True))
        else:
            everyone[0] = mine
        full = torch.cat([everyone[r, :, :length] for r, (_, length) in enumerate(plan)], dim=1).contiguous()
        tok, st = self.sample_full(full, seeds[rows].contiguous(), steps[rows].contiguous(), slot, purpose)
        tokens[rows] = tok
        status[rows] = st

    def sample_full(self, full, seeds, steps, slot, purpose):
        return self.pkg.sample_logits(full, self.t, self.top_p, seeds, steps, slot=slot, purpose=purpose)


class _DeviceBlock:
    """Minimal CUDA array interface over a raw device pointer, so that torch can view library-allocated memory."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


def rows_plan(rows, world):
    """Rows per owner (ceil) and [(first row, count)] per rank: contiguous blocks, the tail ranks may hold fewer."""
    per = max(1, math.ceil(rows / world))
    return per, [(min(rows, r * per), max(0, min(rows, (r + 1) * per) - min(rows, r * per))) for r in range(world)]


def team_plan(rows, world, rank, vocab_ranks):
    """(first rank of this rank's team, first batch row the team computes, number of such rows): the team is the
    vocab_ranks consecutive ranks that share one copy of the head's weights, its rows are the ones its members own."""
    if vocab_ranks < 1 or world % vocab_ranks:
        raise ValueError("vocab_ranks must divide the number of ranks")
    per, _ = rows_plan(rows, world)
    team0 = (rank // vocab_ranks) * vocab_ranks
    row0 = min(rows, team0 * per)
    return team0, row0, min(rows, (team0 + vocab_ranks) * per) - row0


class PeerMappingUnavailable(RuntimeError):
    """Raised on EVERY rank when some rank could not allocate or map the peer-visible buffers."""


class RowExchange:
    """One peer-visible full-vocabulary logits buffer [rows_per_owner, vocab] per rank, mapped into every rank."""

    def __init__(self, pkg, device, rows, vocab, group=None, guard=None, vocab_ranks=None):
        """vocab_ranks: how many ranks share one copy of the head's weights (the vocabulary is split over that many;
        default: all of them).  With fewer, the ranks form world / vocab_ranks teams that each hold a copy, and a team
        computes only the batch rows its own members sample: less data crosses NVLink (a rank sends
        (vocab_ranks - 1) / vocab_ranks of a [rows / teams, vocab / vocab_ranks] slice), more weight bytes are read."""
        self.pkg, self.device, self.rows, self.vocab, self.group = pkg, device, rows, vocab, group
        self.guard = guard or StepGuard(group)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.vocab_ranks = vocab_ranks or self.world
        self.rows_per_owner, plan = rows_plan(rows, self.world)
        self.row0, self.my_rows = plan[self.rank]
        # this rank's team: ranks [team0, team0 + vocab_ranks); its batch rows are the ones its members own (contiguous)
        self.team0, self.team_row0, self.team_rows = team_plan(rows, self.world, self.rank, self.vocab_ranks)
        lib = pkg.lib()
        lib.ds41_b200_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]
        lib.ds41_b200_peer_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        lib.ds41_b200_peer_close.argtypes = [C.c_void_p]
        lib.ds41_b200_peer_free.argtypes = [C.c_void_p]
        lib.ds41_b200_head_fp8_scatter_stats.argtypes = [C.c_void_p] * 4 + [C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                                                            C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                                                            C.c_int64, C.c_void_p, C.c_void_p]
        self._lib = lib
        # Every rank must end up with the same answer (a rank that raised alone would leave the others waiting in the
        # next collective): failures are recorded, agreed on with one all-reduce, and only then raised everywhere.
        failure = None
        handle = C.create_string_buffer(64)
        mine = C.c_void_p()
        with torch.cuda.device(device):
            # [logits rows][16-byte row records the heads of all ranks merge their slice's extremes into]
            self.stats_offset = self.rows_per_owner * vocab * 4
            rc = lib.ds41_b200_peer_alloc(self.stats_offset + self.rows_per_owner * 16, C.byref(mine), handle)
        if rc:
            failure = f"ds41_b200_peer_alloc: cudaError {rc} ({pkg.last_error()})"
            mine = C.c_void_p()
        self._mine = mine if mine.value else None
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle.raw) if not failure else None, group=group)
        else:
            handles[0] = bytes(handle.raw)
        self._opened = []
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(mine.value)
                continue
            if h is None or failure:
                failure = failure or f"rank {r} could not allocate its buffer"
                continue
            p = C.c_void_p()
            with torch.cuda.device(device):
                rc = lib.ds41_b200_peer_open(C.create_string_buffer(h, 64), C.byref(p))
            if rc:
                failure = f"ds41_b200_peer_open(rank {r}): cudaError {rc} ({pkg.last_error()})"
                continue
            self._opened.append(p)
            ptrs.append(p.value)
        if self.world > 1:
            agreed = torch.tensor([0 if failure else 1], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if agreed.item() == 0:
                failure = failure or "another rank could not map the peer buffers"
        if failure:
            self.full = None
            self.close()
            raise PeerMappingUnavailable(failure)
        self.owner_ptrs = (C.c_void_p * self.vocab_ranks)(*ptrs[self.team0:self.team0 + self.vocab_ranks])
        self.full = torch.as_tensor(_DeviceBlock(mine.value, (self.rows_per_owner, vocab), "<f4"), device=device)
        self.full.zero_()
        self.stats = torch.as_tensor(_DeviceBlock(mine.value + self.stats_offset, (self.rows_per_owner, 16), "|u1"),
                                     device=device)
        self.stats.zero_()
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.packed = torch.full((2, self.rows_per_owner), -1, dtype=torch.int32, device=device)
        # scratch enables the sampler's batch path (grid-wide kernels over this rank's rows)
        self.scratch = (torch.empty(pkg.sample_scratch_bytes(self.my_rows, vocab), dtype=torch.uint8, device=device)
                        if self.my_rows else None)
        self.everyone = torch.empty((self.world, 2, self.rows_per_owner), dtype=torch.int32, device=device)
        if self.world > 1:
            dist.barrier(group=group)  # every buffer exists and is mapped before anyone writes

    def head_scatter(self, a, a_scale, w, w_scale, vocab_offset, error_flag=None):
        """This rank's vocabulary slice of its team's rows' logits, stored into the rows' owners.  a / a_scale: the
        quantised activations of the whole batch (the team's rows are taken from it) or of the team's rows only."""
        if a.shape[0] == self.rows and self.team_rows != self.rows:
            a = a[self.team_row0:self.team_row0 + self.team_rows]
            a_scale = a_scale[self.team_row0:self.team_row0 + self.team_rows]
        M, K = a.shape
        if M != self.team_rows:
            raise ValueError(f"activations of {M} rows, the team's share is {self.team_rows}")
        with torch.cuda.device(self.device):
            rc = self._lib.ds41_b200_head_fp8_scatter_stats(
                a.data_ptr(), a_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(), self.owner_ptrs, self.vocab_ranks,
                self.rows_per_owner, self.vocab, vocab_offset, M, w.shape[0], K, self.stats_offset,
                error_flag.data_ptr() if error_flag is not None else None,
                C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc:
            raise RuntimeError(f"ds41_b200_head_fp8_scatter_stats: cudaError {rc} ({self.pkg.last_error()})")

    def writers_done(self):
        """Stream-ordered: returns (on the stream) once every rank's head kernel has finished its peer stores."""
        if self.world > 1:
            self.guard.collective("writers-done all-reduce", lambda: dist.all_reduce(self.word, group=self.group,
                                                                                      async_op=True))

    def sample_mine(self, temperature, top_p, seeds, steps, slot=0, purpose=0, **kw):
        n = self.my_rows
        kw.setdefault("scratch", self.scratch)
        if n:
            sl = slice(self.row0, self.row0 + n)
            # the row records the heads of all ranks merged into this owner's buffer save the sampler its own pass for them
            kw.setdefault("row_extremes", self.stats[:n])
            self.pkg.sample_logits(self.full[:n], temperature, top_p, seeds[sl], steps[sl], slot=slot, purpose=purpose,
                                   tokens=self.packed[0, :n], status=self.packed[1, :n], **kw)
        # read: cleared for the next step's writers (ordered before them by the token all-gather that follows)
        self.stats.zero_()

    def publish(self, tokens, status):
        """All-gather of every owner's (tokens, status); also orders the next step's writers after this step's readers."""
        if self.world > 1:
            self.guard.collective("token all-gather", lambda: dist.all_gather_into_tensor(
                self.everyone.view(-1), self.packed.view(-1), group=self.group, async_op=True))
        else:
            self.everyone[0] = self.packed
        if self.rows == self.world * self.rows_per_owner and tokens.is_contiguous() and status.is_contiguous():
            # one strided copy each, no temporary
            tokens.view(self.world, self.rows_per_owner).copy_(self.everyone[:, 0, :])
            status.view(self.world, self.rows_per_owner).copy_(self.everyone[:, 1, :])
        else:
            tokens.copy_(self.everyone[:, 0, :].reshape(-1)[: self.rows])
            status.copy_(self.everyone[:, 1, :].reshape(-1)[: self.rows])

    def close(self):
        for p in self._opened:
            self._lib.ds41_b200_peer_close(p)
        self._opened = []
        if getattr(self, "_mine", None) is not None:
            self.full = None
            self._lib.ds41_b200_peer_free(self._mine)
            self._mine = None


class ShardedDecodeTail:
    """quantised activations -> this rank's head slice -> tokens for all rows on every rank.

    strategy "rows" / "candidates" fix the exchange; "auto" starts with candidates and switches to rows for
    `probe_every` steps whenever more than a quarter of the rows of a step were not covered."""

    def __init__(self, pkg, device, rows, vocab_offset, vocab_local, vocab, temperature, top_p, strategy="auto",
                 group=None, probe_every=256, timeout_s=30.0, vocab_ranks=None):
        self.pkg, self.device, self.rows, self.v0, self.vn, self.vocab = pkg, device, rows, vocab_offset, vocab_local, vocab
        self.guard = StepGuard(group, timeout_s)
        self.t, self.top_p, self.strategy, self.probe_every = temperature, top_p, strategy, probe_every
        self.rows_mode_left = 0
        self.exchange, self.exchange_error = None, None
        if strategy != "candidates":
            try:
                self.exchange = RowExchange(pkg, device, rows, vocab, group, self.guard, vocab_ranks)
            except PeerMappingUnavailable as exc:  # the same on every rank: fall back to the NCCL-only exchange
                self.exchange_error = str(exc)
                self.strategy = strategy = "candidates"
        self.cands = None
        if strategy != "rows":
            self.cands = ShardedSampler(pkg, torch, device, rows, vocab_offset, vocab_local, vocab, temperature, top_p, group,
                                        guard=self.guard)
            self.local_logits = torch.empty((rows, vocab_local), dtype=torch.float32, device=device)
        self.steps_rows = self.steps_candidates = 0

    def mode(self):
        if self.strategy != "auto":
            return self.strategy
        return "rows" if self.rows_mode_left > 0 else "candidates"

    def step(self, a, a_scale, w, w_scale, seeds, steps, tokens, status, error_flag=None, slot=0, purpose=0):
        """Enqueues one step.  `self.guard.finish()` is the bounded wait for it (and where a failed collective
        surfaces as CollectiveFailure); call it wherever the host would otherwise synchronise."""
        self.guard.before_step()
        if self.mode() == "rows":
            ex = self.exchange
            ex.head_scatter(a, a_scale, w, w_scale, self.v0, error_flag)
            ex.writers_done()
            ex.sample_mine(self.t, self.top_p, seeds, steps, slot, purpose)
            ex.publish(tokens, status)
            self.rows_mode_left -= 1
            self.steps_rows += 1
            return "rows"
        self.pkg.head_fp8(a, a_scale, w, w_scale, self.local_logits, error_flag)
        before = self.cands.escalated
        self.cands.sample(self.local_logits, seeds, steps, tokens, status, slot, purpose)
        self.steps_candidates += 1
        if self.strategy == "auto" and (self.cands.escalated - before) * 4 > self.rows:
            self.rows_mode_left = self.probe_every
        return "candidates"
