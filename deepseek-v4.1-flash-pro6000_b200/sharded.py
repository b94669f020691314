"""Vocabulary-sharded sampling across the GPUs of one node (one process per GPU, torch.distributed for the exchange).

Rank r owns the contiguous id range produced by `shard_plan` (128-row blocks of the head's weight matrix, uneven by
at most one block).  Per step: local candidates (CUDA) -> one all-gather of 544-byte records (one per 8192 ids) per row (NCCL on GPUs,
gloo in the CPU tests) -> combine (CUDA, replicated on every rank).  Rows the combine cannot certify as covered are
re-sampled from their full logits, gathered only for those rows.
"""
import ctypes as C

import torch
import torch.distributed as dist

SHARD_ROW_BYTES = 544
NOT_COVERED = -8


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
                 world=None):
        self.pkg, self.device, self.rows = pkg, device, rows
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
            dist.all_gather_into_tensor(self.gathered, self.local, group=self.group)
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
            dist.all_gather_into_tensor(everyone.view(-1), mine.view(-1), group=self.group)
        else:
            everyone[0] = mine
        full = torch.cat([everyone[r, :, :length] for r, (_, length) in enumerate(plan)], dim=1).contiguous()
        tok, st = self.sample_full(full, seeds[rows].contiguous(), steps[rows].contiguous(), slot, purpose)
        tokens[rows] = tok
        status[rows] = st

    def sample_full(self, full, seeds, steps, slot, purpose):
        return self.pkg.sample_logits(full, self.t, self.top_p, seeds, steps, slot=slot, purpose=purpose)
