"""Host-side mirror of the decode-tail call surface on top of the C-ABI library (libds41_b200.so).

The functions follow the reference engine's sampler interface (engine/include/ds41/engine.hpp:181-227):
`Rng`, `AttemptCounter`, `Purpose`, `sample`, `argmax`, `reject_sample` -- but they take LOGITS on the device and
return decisions, because the fused device path never materialises FP64 probability rows.  Torch is used only as
the owner of device memory and streams; every computation happens inside the library's CUDA kernels.  There is no
CPU fallback: without the built library or without a CUDA device every call raises.
"""
import ctypes as C
import enum
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libds41_b200.so")
MAX_VOCAB = 131072
MAX_HISTORY = 65535

_u64, _u32, _i32, _i64, _f64, _f32, _P = C.c_uint64, C.c_uint32, C.c_int32, C.c_int64, C.c_double, C.c_float, C.c_void_p


class Purpose(enum.IntEnum):
    """engine.hpp:187-192 / spark.h:96"""
    Target = 0
    Draft = 1
    Accept = 2
    Residual = 3


class SparkResult(C.Structure):
    """ds41_spark_result, spark.h:106-108"""
    _fields_ = [("tokens", _i32 * 6), ("emitted", C.c_int), ("accepted_drafts", C.c_int),
                ("accepted_input_rows", C.c_int), ("rejected", C.c_int)]


RESULT_DTYPE = np.dtype([("tokens", np.int32, 6), ("emitted", np.int32), ("accepted_drafts", np.int32),
                         ("accepted_input_rows", np.int32), ("rejected", np.int32)])


class SampleArgs(C.Structure):
    _fields_ = [("struct_bytes", _u32), ("rows", _i32), ("vocab", _i32), ("logits", _P), ("logits_stride", _i64),
                ("temperature", _f64), ("top_p", _f64), ("top_k", _i32), ("repetition", _f32), ("presence", _f32),
                ("frequency", _f32), ("history", _P), ("history_stride", _i64), ("history_len", _P), ("mask", _P),
                ("mask_stride", _i64), ("seeds", _P), ("steps", _P), ("slot", _u32), ("purpose", _u32),
                ("tokens", _P), ("status", _P), ("scratch", _P), ("scratch_bytes", C.c_size_t),
                ("row_extremes", _P)]


class VerifyArgs(C.Structure):
    _fields_ = [("struct_bytes", _u32), ("sequences", _i32), ("drafts", _i32), ("vocab", _i32),
                ("target_logits", _P), ("draft_logits", _P), ("draft_ids", _P), ("temperature", _f64),
                ("top_p", _f64), ("seeds", _P), ("steps", _P), ("results", _P), ("status", _P), ("scratch", _P),
                ("scratch_bytes", C.c_size_t)]


class ScoreArgs(C.Structure):
    _fields_ = [("struct_bytes", _u32), ("rows", _i32), ("vocab", _i32), ("logits", _P), ("logits_stride", _i64),
                ("top_n", _i32), ("logsumexp", _P), ("top1", _P), ("top_ids", _P), ("top_logprob", _P), ("status", _P)]


_lib = None


def lib():
    """Loads the CUDA library; raises if it has not been built (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python __graft_entry__.py` (build) first")
        L = C.CDLL(LIB_PATH)
        L.ds41_spark_error.restype = C.c_char_p
        L.ds41_spark_rng_word_v2.restype = _u32
        L.ds41_spark_rng_word_v2.argtypes = [_u64, _u64, _u32, _u32, _u64]
        L.ds41_spark_uniform_v2.restype = _f64
        L.ds41_spark_uniform_v2.argtypes = [_u64, _u64, _u32, _u32, _u64]
        L.ds41_b200_sample_logits.argtypes = [C.POINTER(SampleArgs), _P]
        L.ds41_b200_sample_scratch_bytes.restype = C.c_size_t
        L.ds41_b200_sample_scratch_bytes.argtypes = [C.c_int, C.c_int]
        L.ds41_b200_verify_scratch_bytes_for.restype = C.c_size_t
        L.ds41_b200_verify_scratch_bytes_for.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ds41_b200_verify_logits.argtypes = [C.POINTER(VerifyArgs), _P]
        L.ds41_b200_verify_logits_static.argtypes = [C.POINTER(VerifyArgs), _P]
        L.ds41_b200_verify_logits_static_max_rows.restype = C.c_int
        L.ds41_b200_quantize_activations.argtypes = [_P, _P, _P, C.c_int, C.c_int, _P]
        L.ds41_b200_head_fp8.argtypes = [_P, _P, _P, _P, _P, _i64, C.c_int, C.c_int, C.c_int, _P, _P]
        L.ds41_b200_head_fp8_stats.argtypes = [_P, _P, _P, _P, _P, _i64, C.c_int, C.c_int, C.c_int, _P, _P, _P]
        L.ds41_fuse_head_fp8_workspace_bytes.restype = C.c_size_t
        L.ds41_fuse_head_fp8_workspace_bytes.argtypes = [C.c_int, C.c_int]
        L.ds41_fuse_head_fp8.argtypes = [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P, _P]
        L.ds41_b200_verify_scratch_bytes.restype = C.c_size_t
        L.ds41_b200_verify_scratch_bytes.argtypes = [C.c_int, C.c_int]
        L.ds41_b200_score_logits.argtypes = [C.POINTER(ScoreArgs), _P]
        L.ds41_b200_head_bf16.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]
        L.ds41_fuse_head_decode.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]
        L.ds41_b200_logits_sha256.argtypes = [_P, C.c_int, C.c_int, _i64, _P, _P]
        L.ds41_dense_head_compact.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]
        L.ds41_b200_markov_logits.argtypes = [_P, _P, _P, _P, C.c_int, _P]
        L.ds41_b200_final_norm.argtypes = [_P, _P, _P, _P, C.c_int, C.c_int, _f32, _P]
        _lib = L
    return _lib


def last_error():
    return lib().ds41_spark_error().decode()


def _check(rc, what):
    if rc:
        raise RuntimeError(f"{what}: cudaError {rc} ({last_error()})")


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t, dtype, name):
    if t is None:
        return None
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA tensor of {dtype}")
    return t


class Rng:
    """engine.hpp:193-199: Philox4x32-10 keyed by the request seed (spark_rng.h:23-36)."""

    def __init__(self, seed):
        self.seed = int(seed)

    def word(self, step, slot, purpose, draw=0):
        if draw // 4 > 0xFFFFFFFF or slot > 5 or int(purpose) > 3:
            raise OverflowError("Philox draw counter")
        return lib().ds41_spark_rng_word_v2(self.seed, step, slot, int(purpose), draw)

    def uniform(self, step, slot, purpose, draw=0):
        if draw > 8589934591 or slot > 5 or int(purpose) > 3:
            raise OverflowError("Philox draw counter")
        return lib().ds41_spark_uniform_v2(self.seed, step, slot, int(purpose), draw)


class AttemptCounter:
    """engine/src/sampling.cpp:111-120: one fresh monotone nonce per attempt; exhaustion is an error."""

    def __init__(self, first=0):
        self._next, self._exhausted = int(first), False

    def take(self):
        if self._exhausted:
            raise OverflowError("transaction nonce exhausted")
        out = self._next
        if self._next == 2**64 - 1:
            self._exhausted = True
        else:
            self._next += 1
        return out


def sample_scratch_bytes(rows, vocab):
    return lib().ds41_b200_sample_scratch_bytes(rows, vocab)


def sample_logits(logits, temperature, top_p, seeds, steps, slot=0, purpose=Purpose.Target, top_k=0, history=None,
                  history_len=None, repetition=1.0, presence=0.0, frequency=0.0, mask=None, tokens=None, status=None,
                  scratch="auto", row_extremes=None):
    """Batched probabilities() + sample() / argmax() on device logits [rows, vocab] (fp32).

    seeds/steps: int64 CUDA tensors holding the uint64 Philox key and attempt counter of each row.
    scratch: "auto" (allocate what the batch-parallel paths need), None (cluster kernel only) or a uint8 CUDA tensor.
    row_extremes: the uint8 [rows, 16] records head_fp8(..., row_extremes=...) wrote for these logits, or None.
    Returns (tokens int32 [rows], status int32 [rows]); see ds41_b200.h for the status words."""
    logits = _dev(logits, torch.float32, "logits") if logits.is_contiguous() else logits
    if logits.dim() != 2 or logits.stride(1) != 1 or not logits.is_cuda or logits.dtype != torch.float32:
        raise ValueError("logits must be a CUDA fp32 [rows, vocab] tensor with unit inner stride")
    rows, vocab = logits.shape
    seeds = _dev(seeds, torch.int64, "seeds")
    steps = _dev(steps, torch.int64, "steps")
    history = _dev(history, torch.int32, "history")
    history_len = _dev(history_len, torch.int32, "history_len")
    mask = _dev(mask, torch.int32, "mask")
    if tokens is None:
        tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if status is None:
        status = torch.empty(rows, dtype=torch.int32, device=logits.device)
    a = SampleArgs()
    a.struct_bytes = C.sizeof(SampleArgs)
    a.rows, a.vocab = rows, vocab
    a.logits, a.logits_stride = logits.data_ptr(), logits.stride(0)
    a.temperature, a.top_p, a.top_k = temperature, top_p, top_k
    a.repetition, a.presence, a.frequency = repetition, presence, frequency
    a.history = history.data_ptr() if history is not None else None
    a.history_stride = history.stride(0) if history is not None else 0
    a.history_len = history_len.data_ptr() if history_len is not None else None
    a.mask = mask.data_ptr() if mask is not None else None
    a.mask_stride = mask.stride(0) if mask is not None else 0
    a.seeds, a.steps = seeds.data_ptr(), steps.data_ptr()
    a.slot, a.purpose = slot, int(purpose)
    a.tokens, a.status = tokens.data_ptr(), status.data_ptr()
    if isinstance(scratch, str):
        usable = history is None and mask is None and top_k <= 64
        scratch = torch.empty(sample_scratch_bytes(rows, vocab), dtype=torch.uint8, device=logits.device) if usable else None
    a.scratch = scratch.data_ptr() if scratch is not None else None
    a.scratch_bytes = scratch.numel() if scratch is not None else 0
    a.row_extremes = row_extremes.data_ptr() if row_extremes is not None else None
    with torch.cuda.device(logits.device):
        _check(lib().ds41_b200_sample_logits(C.byref(a), _stream()), "ds41_b200_sample_logits")
    return tokens, status


def verify_scratch_bytes(sequences, drafts, vocab=MAX_VOCAB):
    return lib().ds41_b200_verify_scratch_bytes_for(sequences, drafts, vocab)


def verify_logits(target_logits, draft_logits, draft_ids, drafts, temperature, top_p, seeds, steps, scratch=None,
                  results=None, status=None):
    """Batched probabilities_rows() + reject_sample() (engine/src/speculation.cpp:179-182) on device logits.

    target_logits [sequences*(drafts+1), vocab], draft_logits [sequences*drafts, vocab] (None when greedy or no
    drafts), draft_ids int32 [sequences*drafts].  Returns (results, status): results is a uint8 CUDA tensor holding
    `sequences` ds41_spark_result records (view it with RESULT_DTYPE on the host)."""
    target_logits = _dev(target_logits, torch.float32, "target_logits")
    draft_logits = _dev(draft_logits, torch.float32, "draft_logits")
    draft_ids = _dev(draft_ids, torch.int32, "draft_ids")
    seeds = _dev(seeds, torch.int64, "seeds")
    steps = _dev(steps, torch.int64, "steps")
    rows, vocab = target_logits.shape
    if rows % (drafts + 1):
        raise ValueError("speculative row count")
    sequences = rows // (drafts + 1)
    device = target_logits.device
    need = verify_scratch_bytes(sequences, drafts, vocab)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=device)
    if results is None:
        results = torch.empty(sequences * C.sizeof(SparkResult), dtype=torch.uint8, device=device)
    if status is None:
        status = torch.empty(sequences, dtype=torch.int32, device=device)
    a = VerifyArgs()
    a.struct_bytes = C.sizeof(VerifyArgs)
    a.sequences, a.drafts, a.vocab = sequences, drafts, vocab
    a.target_logits = target_logits.data_ptr()
    a.draft_logits = draft_logits.data_ptr() if draft_logits is not None else None
    a.draft_ids = draft_ids.data_ptr() if draft_ids is not None else None
    a.temperature, a.top_p = temperature, top_p
    a.seeds, a.steps = seeds.data_ptr(), steps.data_ptr()
    a.results, a.status = results.data_ptr(), status.data_ptr()
    a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    with torch.cuda.device(device):
        _check(lib().ds41_b200_verify_logits(C.byref(a), _stream()), "ds41_b200_verify_logits")
    return results, status


def results_to_numpy(results):
    return np.frombuffer(results.cpu().numpy().tobytes(), dtype=RESULT_DTYPE)


def quantize_activations(x_bf16, a=None, a_scale=None):
    """bf16 [M,K] -> (e4m3 bytes [M,K] uint8, fp32 power-of-two scales [M,K/128]); rule of
    ds41_dense_quant (components/dense/src/dense.cu:8-16) with the group widened to 128."""
    x_bf16 = _dev(x_bf16, torch.bfloat16, "x")
    M, K = x_bf16.shape
    if a is None:
        a = torch.empty((M, K), dtype=torch.uint8, device=x_bf16.device)
    if a_scale is None:
        a_scale = torch.empty((M, K // 128), dtype=torch.float32, device=x_bf16.device)
    with torch.cuda.device(x_bf16.device):
        _check(lib().ds41_b200_quantize_activations(x_bf16.data_ptr(), a.data_ptr(), a_scale.data_ptr(), M, K, _stream()),
               "ds41_b200_quantize_activations")
    return a, a_scale


def head_fp8(a, a_scale, w, w_scale, logits=None, error_flag=None, row_extremes=None):
    """Block-scaled FP8 head GEMM: a uint8 [M,K] (e4m3), w uint8 [N,K] (e4m3) -> fp32 logits [M,N].
    row_extremes: optional uint8 CUDA tensor [M, 16]; the head then also leaves each row's first maximum, minimum and
    finiteness there (ds41_b200_head_fp8_stats) for sample_logits(row_extremes=...)."""
    a = _dev(a, torch.uint8, "a"); w = _dev(w, torch.uint8, "w")
    a_scale = _dev(a_scale, torch.float32, "a_scale"); w_scale = _dev(w_scale, torch.float32, "w_scale")
    M, K = a.shape
    N = w.shape[0]
    if logits is None:
        logits = torch.empty((M, N), dtype=torch.float32, device=a.device)
    flag = error_flag.data_ptr() if error_flag is not None else None
    with torch.cuda.device(a.device):
        if row_extremes is None:
            _check(lib().ds41_b200_head_fp8(a.data_ptr(), a_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(),
                                            logits.data_ptr(), logits.stride(0), M, N, K, flag, _stream()),
                   "ds41_b200_head_fp8")
        else:
            row_extremes = _dev(row_extremes, torch.uint8, "row_extremes")
            if row_extremes.numel() < 16 * M:
                raise ValueError("row_extremes must hold 16 bytes per row")
            _check(lib().ds41_b200_head_fp8_stats(a.data_ptr(), a_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(),
                                                  logits.data_ptr(), logits.stride(0), M, N, K,
                                                  row_extremes.data_ptr(), flag, _stream()),
                   "ds41_b200_head_fp8_stats")
    return logits


def head_bf16(x, w_bf16, out=None, decode_symbol=False):
    """The reference's BF16 head (ds41_fuse_head_decode, components/fuse-head/include/ds41/fuse_head.h:9-10): x fp32
    [M,K], weights bf16 [N,K] -> fp32 [M,N], bit-identical to the reference plugin.  decode_symbol=True calls the
    plugin's own entry point, which only accepts N == 129280 and K == 5120."""
    x = _dev(x, torch.float32, "x")
    w_bf16 = _dev(w_bf16, torch.bfloat16, "w")
    M, K = x.shape
    N = w_bf16.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    fn = lib().ds41_fuse_head_decode if decode_symbol else lib().ds41_b200_head_bf16
    with torch.cuda.device(x.device):
        _check(fn(x.data_ptr(), w_bf16.data_ptr(), out.data_ptr(), M, N, K, _stream()), "BF16 head")
    return out


def head_f32(x, w_f32, out=None):
    """FP32 head (the reference's default target head, ds41_dense_cublas(f32=1): dense/src/ops.cu:120-128): x fp32
    [M, K], w fp32 [N, K] -> fp32 [M, N]."""
    x, w_f32 = _dev(x, torch.float32, "x"), _dev(w_f32, torch.float32, "w")
    M, K = x.shape
    N = w_f32.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    L = lib()
    L.ds41_b200_head_f32.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]
    with torch.cuda.device(x.device):
        _check(L.ds41_b200_head_f32(x.data_ptr(), w_f32.data_ptr(), out.data_ptr(), M, N, K, _stream()), "ds41_b200_head_f32")
    return out


def head_compact(x, w_bf16, out=None):
    """The drafter's BF16 head (ds41_dense_head_compact, components/dense/src/compact.cu:10-24,44-50): x fp32 [M,K]
    (M <= 8), weights bf16 [N,K] -> fp32 [M,N], bit-identical to the reference kernel."""
    x = _dev(x, torch.float32, "x")
    w_bf16 = _dev(w_bf16, torch.bfloat16, "w")
    M, K = x.shape
    N = w_bf16.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().ds41_dense_head_compact(x.data_ptr(), w_bf16.data_ptr(), out.data_ptr(), M, N, K, _stream()),
               "ds41_dense_head_compact")
    return out


def markov_logits(draft_row, markov_weight, embedding, out=None):
    """Draft logits of one position: draft_row fp32 [V] + markov_weight bf16 [V,256] . embedding bf16 [256]
    (engine/third_party/spark/src/forward.cu:46,135-139)."""
    draft_row = _dev(draft_row, torch.float32, "draft_row")
    markov_weight = _dev(markov_weight, torch.bfloat16, "markov_weight")
    embedding = _dev(embedding, torch.bfloat16, "embedding")
    if markov_weight.shape != (draft_row.numel(), 256) or embedding.numel() != 256:
        raise ValueError("markov_weight must be [V,256] and embedding [256]")
    if out is None:
        out = torch.empty_like(draft_row)
    with torch.cuda.device(draft_row.device):
        _check(lib().ds41_b200_markov_logits(draft_row.data_ptr(), markov_weight.data_ptr(), embedding.data_ptr(),
                                             out.data_ptr(), draft_row.numel(), _stream()), "ds41_b200_markov_logits")
    return out


def final_norm(h, pre, norm_weight, eps=1e-20, out=None):
    """The head's prologue (engine/src/hotpath/batch.inc:487-492): h bf16 [M,4,K], pre fp32 [M,4], norm_weight bf16 [K]
    -> fp32 [M,K] (HC-pre mix, RMSNorm, rounded to bf16, promoted)."""
    h = _dev(h, torch.bfloat16, "h")
    pre = _dev(pre, torch.float32, "pre")
    norm_weight = _dev(norm_weight, torch.bfloat16, "norm_weight")
    M, four, K = h.shape
    if four != 4 or pre.shape != (M, 4) or norm_weight.numel() != K:
        raise ValueError("h must be [M,4,K], pre [M,4], norm_weight [K]")
    if out is None:
        out = torch.empty((M, K), dtype=torch.float32, device=h.device)
    with torch.cuda.device(h.device):
        _check(lib().ds41_b200_final_norm(h.data_ptr(), pre.data_ptr(), norm_weight.data_ptr(), out.data_ptr(), M, K,
                                          eps, _stream()), "ds41_b200_final_norm")
    return out


def score_logits(logits, top_n=0):
    """log_normalizer + top_order of the reference's score / logprobs events (engine/src/server.cpp:178-183,730-737)
    on device logits [rows, vocab].  Returns (logsumexp f64 [rows], top1 i32 [rows], top_ids i32 [rows, top_n],
    top_logprob f64 [rows, top_n], status i32 [rows])."""
    if logits.dim() != 2 or logits.stride(1) != 1 or not logits.is_cuda or logits.dtype != torch.float32:
        raise ValueError("logits must be a CUDA fp32 [rows, vocab] tensor with unit inner stride")
    rows, vocab = logits.shape
    dev = logits.device
    lse = torch.empty(rows, dtype=torch.float64, device=dev)
    top1 = torch.empty(rows, dtype=torch.int32, device=dev)
    ids = torch.empty((rows, top_n), dtype=torch.int32, device=dev)
    lp = torch.empty((rows, top_n), dtype=torch.float64, device=dev)
    status = torch.empty(rows, dtype=torch.int32, device=dev)
    a = ScoreArgs(C.sizeof(ScoreArgs), rows, vocab, logits.data_ptr(), logits.stride(0), top_n, lse.data_ptr(),
                  top1.data_ptr(), ids.data_ptr() if top_n else None, lp.data_ptr() if top_n else None, status.data_ptr())
    with torch.cuda.device(dev):
        _check(lib().ds41_b200_score_logits(C.byref(a), _stream()), "ds41_b200_score_logits")
    return lse, top1, ids, lp, status


class ProbArgs(C.Structure):
    _fields_ = [("struct_bytes", C.c_uint32), ("rows", C.c_int32), ("vocab", C.c_int32), ("logits", C.c_void_p),
                ("logits_stride", C.c_int64), ("temperature", C.c_double), ("top_p", C.c_double),
                ("probabilities", C.c_void_p), ("status", C.c_void_p), ("scratch", C.c_void_p),
                ("scratch_bytes", C.c_size_t)]


def probabilities(logits, temperature, top_p):
    """The reference's probability rows on the device (ds41_spark_probabilities through the adapter's temperature
    floor: engine/third_party/spark/src/sampling.cpp:30-38, engine/src/sampling.cpp:205-219).  Returns (float64
    [rows, vocab], int32 status [rows]); a row with non-finite logits is NaN with a negative status."""
    logits = _dev(logits, torch.float32, "logits")
    rows, vocab = logits.shape
    L = lib()
    L.ds41_b200_probabilities_scratch_bytes.restype = C.c_size_t
    L.ds41_b200_probabilities_scratch_bytes.argtypes = [C.c_int]
    L.ds41_b200_probabilities.argtypes = [C.POINTER(ProbArgs), _P]
    need = L.ds41_b200_probabilities_scratch_bytes(rows)
    out = torch.empty((rows, vocab), dtype=torch.float64, device=logits.device)
    status = torch.empty(rows, dtype=torch.int32, device=logits.device)
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device)
    a = ProbArgs(C.sizeof(ProbArgs), rows, vocab, logits.data_ptr(), logits.stride(0), float(temperature), float(top_p),
                 out.data_ptr(), status.data_ptr(), scratch.data_ptr(), need)
    with torch.cuda.device(logits.device):
        _check(L.ds41_b200_probabilities(C.byref(a), _stream()), "ds41_b200_probabilities")
    return out, status


def sample_probabilities(p, seeds, steps, slot=0, purpose=Purpose.Target):
    """ds41_spark_sample_v2 on device rows (sampling.cpp:12-21,59): validate, then the sequential inverse CDF.  p float64
    [rows, vocab]; returns (tokens, status)."""
    p = _dev(p, torch.float64, "p")
    rows, vocab = p.shape
    seeds, steps = _dev(seeds, torch.int64, "seeds"), _dev(steps, torch.int64, "steps")
    tokens = torch.empty(rows, dtype=torch.int32, device=p.device)
    status = torch.empty(rows, dtype=torch.int32, device=p.device)
    L = lib()
    L.ds41_b200_sample_probabilities.argtypes = [_P, C.c_int, C.c_int, _i64, _P, _P, C.c_uint32, C.c_uint32, _P, _P, _P]
    with torch.cuda.device(p.device):
        _check(L.ds41_b200_sample_probabilities(p.data_ptr(), rows, vocab, p.stride(0), seeds.data_ptr(), steps.data_ptr(),
                                                int(slot), int(purpose), tokens.data_ptr(), status.data_ptr(), _stream()),
               "ds41_b200_sample_probabilities")
    return tokens, status


def verify_probabilities(draft_ids, q, p, drafts, seeds, steps, greedy=False):
    """ds41_spark_verify_v2 on device rows (sampling.cpp:39-56).  p float64 [sequences * (drafts + 1), vocab], q float64
    [sequences * drafts, vocab] (None when greedy), draft_ids int32 [sequences * drafts].  Returns (results, status)."""
    p = _dev(p, torch.float64, "p")
    vocab = p.shape[1]
    sequences = p.shape[0] // (drafts + 1)
    q = _dev(q, torch.float64, "q") if q is not None else None
    draft_ids = _dev(draft_ids, torch.int32, "draft_ids") if drafts else None
    seeds, steps = _dev(seeds, torch.int64, "seeds"), _dev(steps, torch.int64, "steps")
    results = torch.empty(sequences * C.sizeof(SparkResult), dtype=torch.uint8, device=p.device)
    status = torch.empty(sequences, dtype=torch.int32, device=p.device)
    L = lib()
    L.ds41_b200_verify_probabilities.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P, _P]
    with torch.cuda.device(p.device):
        _check(L.ds41_b200_verify_probabilities(draft_ids.data_ptr() if draft_ids is not None else None,
                                                q.data_ptr() if q is not None else None, p.data_ptr(), sequences,
                                                drafts, vocab, 1 if greedy else 0, seeds.data_ptr(), steps.data_ptr(),
                                                results.data_ptr(), status.data_ptr(), _stream()),
               "ds41_b200_verify_probabilities")
    return results, status


def spark_sample_gpu_v2(p_f32, seed, step, slot=0, purpose=Purpose.Target):
    """The reference's GPU sampler entry point (spark.h:133; sampling.cu:24-39,71): one FP32 measure row on the device,
    normalised in FP64.  Returns the token (−1: in-band failure)."""
    p_f32 = _dev(p_f32, torch.float32, "p")
    token = torch.empty(1, dtype=torch.int32, device=p_f32.device)
    L = lib()
    L.ds41_spark_sample_gpu_v2.argtypes = [_P, C.c_int, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, _P, _P]
    with torch.cuda.device(p_f32.device):
        _check(L.ds41_spark_sample_gpu_v2(p_f32.data_ptr(), p_f32.numel(), int(seed), int(step), int(slot), int(purpose),
                                          token.data_ptr(), _stream()), "ds41_spark_sample_gpu_v2")
    return int(token.item())


SAMPLER_PHASES = ("flat_stats_kernel", "flat_hist_kernel", "flat_window_kernel", "flat_mass_kernel",
                  "flat_resolve_kernel", "row_kernel", "replay_sample_kernel")


def profile_sampler_call(call):
    """Runs call() (one sample_logits on the batch path) with the library's phase events on and returns
    {kernel name: milliseconds}, timed with CUDA events on the launching stream."""
    L = lib()
    L.ds41_b200_profile_phases.argtypes = [C.c_int]
    L.ds41_b200_profile_read.argtypes = [C.POINTER(C.c_float), C.c_int]
    _check(L.ds41_b200_profile_phases(1), "ds41_b200_profile_phases")
    try:
        call()
        ms = (C.c_float * len(SAMPLER_PHASES))()
        n = L.ds41_b200_profile_read(ms, len(SAMPLER_PHASES))
        if n < 0:
            raise RuntimeError("ds41_b200_profile_read failed")
        return {SAMPLER_PHASES[i]: float(ms[i]) for i in range(n)}
    finally:
        L.ds41_b200_profile_phases(0)


def logits_sha256(logits):
    """SHA-256 of every row's fp32 logits (the logits_sha256 of the reference's score event, server.cpp:184-197), as
    hexadecimal strings."""
    if logits.dim() != 2 or logits.stride(1) != 1 or not logits.is_cuda or logits.dtype != torch.float32:
        raise ValueError("logits must be a CUDA fp32 [rows, vocab] tensor with unit inner stride")
    rows, vocab = logits.shape
    out = torch.empty((rows, 32), dtype=torch.uint8, device=logits.device)
    with torch.cuda.device(logits.device):
        _check(lib().ds41_b200_logits_sha256(logits.data_ptr(), rows, vocab, logits.stride(0), out.data_ptr(), _stream()),
               "ds41_b200_logits_sha256")
    return [bytes(r).hex() for r in out.cpu().numpy()]


def fuse_head_fp8_workspace_bytes(M, K):
    return lib().ds41_fuse_head_fp8_workspace_bytes(M, K)


def fuse_head_fp8(x_bf16, w, w_scale, logits=None, workspace=None, error_flag=None):
    """x bf16 [M,K] -> fp32 logits [M,N]: activation quantisation + FP8 head in one call."""
    x_bf16 = _dev(x_bf16, torch.bfloat16, "x"); w = _dev(w, torch.uint8, "w")
    w_scale = _dev(w_scale, torch.float32, "w_scale")
    M, K = x_bf16.shape
    N = w.shape[0]
    if logits is None:
        logits = torch.empty((M, N), dtype=torch.float32, device=x_bf16.device)
    if workspace is None:
        workspace = torch.empty(fuse_head_fp8_workspace_bytes(M, K), dtype=torch.uint8, device=x_bf16.device)
    with torch.cuda.device(x_bf16.device):
        _check(lib().ds41_fuse_head_fp8(x_bf16.data_ptr(), w.data_ptr(), w_scale.data_ptr(), logits.data_ptr(), M, N, K,
                                        workspace.data_ptr(), workspace.numel(),
                                        error_flag.data_ptr() if error_flag is not None else None, _stream()),
               "ds41_fuse_head_fp8")
    return logits
