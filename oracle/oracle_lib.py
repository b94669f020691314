"""ctypes bindings of the CPU oracle (test infrastructure; never imported by the product package).

`Oracle` wraps oracle/libds41_oracle.so (this repository's restatement of the reference's host sampling rule)
and `Reference` wraps oracle/_ref/libds41_ref.so (the reference's own sampler sources compiled in place by
oracle/Makefile, present only where the reference tree was available at build time).
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
u64, u32, i32, f64, f32 = C.c_uint64, C.c_uint32, C.c_int32, C.c_double, C.c_float
P = C.c_void_p


def _ptr(a):
    return None if a is None else a.ctypes.data_as(P)


class SparkResult(C.Structure):
    """Layout of ds41_spark_result (engine/third_party/spark/include/ds41/spark.h:106-108)."""
    _fields_ = [("tokens", i32 * 6), ("emitted", C.c_int), ("accepted_drafts", C.c_int),
                ("accepted_input_rows", C.c_int), ("rejected", C.c_int)]


RESULT_DTYPE = np.dtype([("tokens", np.int32, 6), ("emitted", np.int32), ("accepted_drafts", np.int32),
                         ("accepted_input_rows", np.int32), ("rejected", np.int32)])


def build(force=False):
    lib = os.path.join(HERE, "libds41_oracle.so")
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(os.path.join(HERE, "ds41_oracle.cpp")):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return lib


class Oracle:
    def __init__(self):
        self.lib = L = C.CDLL(build())
        L.oracle_error.restype = C.c_char_p
        L.oracle_rng_word_v2.restype = u32
        L.oracle_rng_word_v2.argtypes = [u64, u64, u32, u32, u64]
        L.oracle_uniform_v2.restype = f64
        L.oracle_uniform_v2.argtypes = [u64, u64, u32, u32, u64]
        for name in ("oracle_probabilities", "oracle_engine_probabilities"):
            getattr(L, name).argtypes = [P, P, C.c_int, f64, f64]
        L.oracle_sample_v2.argtypes = [P, C.c_int, u64, u64, u32, u32, P]
        L.oracle_verify_v2.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, u64, u64, P]
        L.oracle_argmax.argtypes = [P, C.c_int, P]
        L.oracle_score_row.argtypes = [P, C.c_int, C.c_int, P, P, P, P]
        L.oracle_head_bf16.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int]
        L.oracle_head_compact.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int]
        L.oracle_markov_logits.argtypes = [P, P, P, P, C.c_int]
        L.oracle_final_norm.argtypes = [P, P, P, P, C.c_int, C.c_int, f32]
        L.oracle_extended_probabilities.argtypes = [P, P, C.c_int, f64, f64, C.c_int, P, C.c_int, f32, f32, f32, P, P]
        L.oracle_sample_rows.argtypes = [P, C.c_int, C.c_int, C.c_int64, f64, f64, C.c_int, P, C.c_int64, P, f32,
                                         f32, f32, P, C.c_int64, P, P, u32, u32, P, P, C.c_int]
        L.oracle_verify_rows.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, f64, f64, P, P, P, P, C.c_int]
        L.oracle_e4m3_table.argtypes = [P]
        L.oracle_e4m3_encode.restype = C.c_uint8
        L.oracle_e4m3_encode.argtypes = [f32]
        L.oracle_quantize_activations.argtypes = [P, P, P, C.c_int, C.c_int]
        L.oracle_quantize_weights.argtypes = [P, P, P, C.c_int, C.c_int]
        L.oracle_head_fp8.argtypes = [P, P, P, P, P, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_gen_logits.argtypes = [u64, u64, C.c_int, f64, f64, P]
        L.oracle_gen_perturbed.argtypes = [u64, u64, C.c_int, f64, P, P]
        L.oracle_gen_normal.argtypes = [u64, u64, C.c_int64, f64, P]
        L.oracle_gen_history.argtypes = [u64, u64, C.c_int, C.c_int, f64, P]
        L.oracle_gen_mask.argtypes = [u64, u64, C.c_int, f64, P]

    def error(self):
        return self.lib.oracle_error().decode()

    def _check(self, rc):
        if rc:
            raise ValueError(self.error())

    # --- RNG
    def word(self, seed, step, slot, purpose, draw=0):
        return self.lib.oracle_rng_word_v2(seed, step, slot, purpose, draw)

    def uniform(self, seed, step, slot, purpose, draw=0):
        return self.lib.oracle_uniform_v2(seed, step, slot, purpose, draw)

    # --- single-row rule
    def probabilities(self, x, t, top, engine=True):
        x = np.ascontiguousarray(x, np.float32)
        p = np.empty(x.size, np.float64)
        f = self.lib.oracle_engine_probabilities if engine else self.lib.oracle_probabilities
        self._check(f(_ptr(x), _ptr(p), x.size, t, top))
        return p

    def extended_probabilities(self, x, t, top, top_k=0, history=None, repetition=1.0, presence=0.0, frequency=0.0,
                               mask=None, want_effective=False):
        x = np.ascontiguousarray(x, np.float32)
        p = np.empty(x.size, np.float64)
        h = None if history is None else np.ascontiguousarray(history, np.int32)
        m = None if mask is None else np.ascontiguousarray(mask, np.uint32)
        eff = np.empty(x.size, np.float32) if want_effective else None
        self._check(self.lib.oracle_extended_probabilities(_ptr(x), _ptr(p), x.size, t, top, top_k, _ptr(h),
                                                           0 if h is None else h.size, repetition, presence,
                                                           frequency, _ptr(m), _ptr(eff)))
        return (p, eff) if want_effective else p

    def sample(self, p, seed, step, slot, purpose):
        p = np.ascontiguousarray(p, np.float64)
        out = i32(-1)
        self._check(self.lib.oracle_sample_v2(_ptr(p), p.size, seed, step, slot, purpose, C.byref(out)))
        return out.value

    def argmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = i32(-1)
        self._check(self.lib.oracle_argmax(_ptr(x), x.size, C.byref(out)))
        return out.value

    def head_bf16(self, x, w_bits):
        """out fp32 [M,N] = x fp32 [M,K] . W^T with W given as bf16 bit patterns uint16 [N,K], in the reference
        plugin's arithmetic order."""
        x = np.ascontiguousarray(x, np.float32)
        w_bits = np.ascontiguousarray(w_bits, np.uint16)
        y = np.empty((x.shape[0], w_bits.shape[0]), np.float32)
        self._check(self.lib.oracle_head_bf16(_ptr(x), _ptr(w_bits), _ptr(y), x.shape[0], w_bits.shape[0], x.shape[1]))
        return y

    def head_compact(self, x, w_bits):
        """The drafter's BF16 head (components/dense/src/compact.cu) in the reference kernel's arithmetic order."""
        x = np.ascontiguousarray(x, np.float32)
        w_bits = np.ascontiguousarray(w_bits, np.uint16)
        y = np.empty((x.shape[0], w_bits.shape[0]), np.float32)
        self._check(self.lib.oracle_head_compact(_ptr(x), _ptr(w_bits), _ptr(y), x.shape[0], w_bits.shape[0], x.shape[1]))
        return y

    def markov_logits(self, u, w_bits, emb_bits):
        u = np.ascontiguousarray(u, np.float32)
        w_bits = np.ascontiguousarray(w_bits, np.uint16)
        emb_bits = np.ascontiguousarray(emb_bits, np.uint16)
        out = np.empty(u.size, np.float32)
        self._check(self.lib.oracle_markov_logits(_ptr(u), _ptr(w_bits), _ptr(emb_bits), _ptr(out), u.size))
        return out

    def final_norm(self, h_bits, pre, w_bits, eps=1e-20):
        h_bits = np.ascontiguousarray(h_bits, np.uint16)     # [M, 4, K]
        pre = np.ascontiguousarray(pre, np.float32)           # [M, 4]
        w_bits = np.ascontiguousarray(w_bits, np.uint16)
        M, _, K = h_bits.shape
        out = np.empty((M, K), np.float32)
        self._check(self.lib.oracle_final_norm(_ptr(h_bits), _ptr(pre), _ptr(w_bits), _ptr(out), M, K, eps))
        return out

    def score_row(self, x, top):
        """(logsumexp, top1, top_ids, top_logprob) of one logits row by the reference's score rule."""
        x = np.ascontiguousarray(x, np.float32)
        lse, top1 = C.c_double(), i32(-1)
        ids, lp = np.empty(top, np.int32), np.empty(top, np.float64)
        self._check(self.lib.oracle_score_row(_ptr(x), x.size, top, C.byref(lse), C.byref(top1), _ptr(ids), _ptr(lp)))
        return lse.value, top1.value, ids, lp

    def verify(self, drafts, q, p, greedy, seed, step):
        p = np.ascontiguousarray(p, np.float64)
        n = p.shape[-1]
        d = None if drafts is None else np.ascontiguousarray(drafts, np.int32)
        count = 0 if d is None else d.size
        qq = None if q is None else np.ascontiguousarray(q, np.float64)
        r = SparkResult()
        self._check(self.lib.oracle_verify_v2(_ptr(d), _ptr(qq), _ptr(p), count, n, int(greedy), seed, step, C.byref(r)))
        return r

    # --- batched
    def sample_rows(self, logits, t, top, seeds, steps, slot=0, purpose=0, top_k=0, history=None, history_len=None,
                    repetition=1.0, presence=0.0, frequency=0.0, mask=None, threads=1):
        logits = np.ascontiguousarray(logits, np.float32)
        rows, n = logits.shape
        seeds = np.ascontiguousarray(seeds, np.uint64)
        steps = np.ascontiguousarray(steps, np.uint64)
        h = None if history is None else np.ascontiguousarray(history, np.int32)
        hl = None if history_len is None else np.ascontiguousarray(history_len, np.int32)
        m = None if mask is None else np.ascontiguousarray(mask, np.uint32)
        tokens = np.full(rows, -1, np.int32)
        status = np.zeros(rows, np.int32)
        self._check(self.lib.oracle_sample_rows(_ptr(logits), rows, n, n, t, top, top_k, _ptr(h),
                                                0 if h is None else h.shape[1], _ptr(hl), repetition, presence,
                                                frequency, _ptr(m), 0 if m is None else m.shape[1], _ptr(seeds),
                                                _ptr(steps), slot, purpose, _ptr(tokens), _ptr(status), threads))
        return tokens, status

    def verify_rows(self, target, draft, ids, drafts, t, top, seeds, steps, threads=1):
        target = np.ascontiguousarray(target, np.float32)
        n = target.shape[-1]
        seqs = target.shape[0] // (drafts + 1)
        dr = None if draft is None else np.ascontiguousarray(draft, np.float32)
        idv = None if ids is None else np.ascontiguousarray(ids, np.int32)
        seeds = np.ascontiguousarray(seeds, np.uint64)
        steps = np.ascontiguousarray(steps, np.uint64)
        out = np.zeros(seqs, RESULT_DTYPE)
        status = np.zeros(seqs, np.int32)
        self._check(self.lib.oracle_verify_rows(_ptr(target), _ptr(dr), _ptr(idv), seqs, drafts, n, t, top,
                                                _ptr(seeds), _ptr(steps), _ptr(out), _ptr(status), threads))
        return out, status

    # --- FP8 head
    def e4m3_table(self):
        t = np.empty(256, np.float32)
        self.lib.oracle_e4m3_table(_ptr(t))
        return t

    def quantize_activations(self, x_bf16_bits):
        x = np.ascontiguousarray(x_bf16_bits, np.uint16)
        M, K = x.shape
        a = np.empty((M, K), np.uint8)
        s = np.empty((M, K // 128), np.float32)
        self._check(self.lib.oracle_quantize_activations(_ptr(x), _ptr(a), _ptr(s), M, K))
        return a, s

    def quantize_weights(self, w):
        w = np.ascontiguousarray(w, np.float32)
        N, K = w.shape
        q = np.empty((N, K), np.uint8)
        s = np.empty(((N + 127) // 128, K // 128), np.float32)
        self._check(self.lib.oracle_quantize_weights(_ptr(w), _ptr(q), _ptr(s), N, K))
        return q, s

    def head_fp8(self, a, a_scale, w, w_scale, threads=1):
        a = np.ascontiguousarray(a, np.uint8)
        w = np.ascontiguousarray(w, np.uint8)
        a_scale = np.ascontiguousarray(a_scale, np.float32)
        w_scale = np.ascontiguousarray(w_scale, np.float32)
        M, K = a.shape
        N = w.shape[0]
        out = np.empty((M, N), np.float32)
        self._check(self.lib.oracle_head_fp8(_ptr(a), _ptr(a_scale), _ptr(w), _ptr(w_scale), _ptr(out), M, N, K, threads))
        return out

    # --- synthetic inputs
    def gen_logits(self, seed, rows, n, sigma=3.0, zipf_s=1.1, first_row=0):
        out = np.empty((rows, n), np.float32)
        for r in range(rows):
            self._check(self.lib.oracle_gen_logits(seed, first_row + r, n, sigma, zipf_s, out[r].ctypes.data_as(P)))
        return out

    def gen_perturbed(self, seed, base, sigma, first_row=0):
        base = np.ascontiguousarray(base, np.float32)
        out = np.empty_like(base)
        for r in range(base.shape[0]):
            self._check(self.lib.oracle_gen_perturbed(seed, first_row + r, base.shape[1], sigma,
                                                      base[r].ctypes.data_as(P), out[r].ctypes.data_as(P)))
        return out

    def gen_normal(self, seed, stream, shape, sigma=1.0):
        out = np.empty(shape, np.float32)
        self._check(self.lib.oracle_gen_normal(seed, stream, out.size, sigma, _ptr(out)))
        return out

    def gen_history(self, seed, rows, n, length, zipf_s=1.1):
        out = np.empty((rows, length), np.int32)
        for r in range(rows):
            self._check(self.lib.oracle_gen_history(seed, r, n, length, zipf_s, out[r].ctypes.data_as(P)))
        return out

    def gen_mask(self, seed, rows, n, lo=0.01, hi=0.05):
        out = np.empty((rows, (n + 31) // 32), np.uint32)
        for r in range(rows):
            frac = lo + (hi - lo) * ((r * 2654435761) % 1000) / 1000.0
            self._check(self.lib.oracle_gen_mask(seed, r, n, frac, out[r].ctypes.data_as(P)))
        return out


def float_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


class Reference:
    """The reference's own sampler, compiled from its sources (oracle/_ref); None-like when absent."""

    def __init__(self):
        path = os.path.join(HERE, "_ref", "libds41_ref.so")
        self.available = os.path.exists(path)
        if not self.available:
            return
        self.lib = L = C.CDLL(path)
        L.ref_error.restype = C.c_char_p
        L.ds41_spark_error.restype = C.c_char_p
        L.ds41_spark_rng_word_v2.restype = u32
        L.ds41_spark_rng_word_v2.argtypes = [u64, u64, u32, u32, u64]
        L.ds41_spark_uniform_v2.restype = f64
        L.ds41_spark_uniform_v2.argtypes = [u64, u64, u32, u32, u64]
        L.ds41_spark_probabilities.argtypes = [P, P, C.c_int, f64, f64]
        L.ds41_spark_sample_v2.argtypes = [P, C.c_int, u64, u64, u32, u32, P]
        L.ds41_spark_verify_v2.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, u64, u64, P]
        L.ref_probabilities.argtypes = [P, P, C.c_int, f64, f64]
        L.ref_probabilities_rows.argtypes = [P, P, C.c_int, C.c_int, f64, f64]
        L.ref_sample.argtypes = [P, C.c_int, u64, u64, u32, u32, P]
        L.ref_argmax.argtypes = [P, C.c_int, P]
        L.ref_reject_sample.argtypes = [P, P, P, C.c_int, C.c_int, u64, u64, f64, P, P, P, P, P]
        L.ref_attempt_counter_take2.restype = u64
        L.ref_attempt_counter_take2.argtypes = [u64, P]

    def _check(self, rc):
        if rc:
            raise ValueError(self.lib.ref_error().decode() or self.lib.ds41_spark_error().decode())

    def word(self, seed, step, slot, purpose, draw=0):
        return self.lib.ds41_spark_rng_word_v2(seed, step, slot, purpose, draw)

    def uniform(self, seed, step, slot, purpose, draw=0):
        return self.lib.ds41_spark_uniform_v2(seed, step, slot, purpose, draw)

    def probabilities(self, x, t, top):
        x = np.ascontiguousarray(x, np.float32)
        p = np.empty(x.size, np.float64)
        self._check(self.lib.ref_probabilities(_ptr(x), _ptr(p), x.size, t, top))
        return p

    def probabilities_rows(self, x, t, top):
        x = np.ascontiguousarray(x, np.float32)
        p = np.empty(x.shape, np.float64)
        self._check(self.lib.ref_probabilities_rows(_ptr(x), _ptr(p), x.shape[0], x.shape[1], t, top))
        return p

    def spark_probabilities(self, x, t, top):
        x = np.ascontiguousarray(x, np.float32)
        p = np.empty(x.size, np.float64)
        if self.lib.ds41_spark_probabilities(_ptr(x), _ptr(p), x.size, t, top):
            raise ValueError(self.lib.ds41_spark_error().decode())
        return p

    def sample(self, p, seed, step, slot, purpose):
        p = np.ascontiguousarray(p, np.float64)
        out = i32(-1)
        self._check(self.lib.ref_sample(_ptr(p), p.size, seed, step, slot, purpose, C.byref(out)))
        return out.value

    def argmax(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = i32(-1)
        self._check(self.lib.ref_argmax(_ptr(x), x.size, C.byref(out)))
        return out.value

    def reject_sample(self, proposals, q, p, seed, step, temperature):
        p = np.ascontiguousarray(p, np.float64)
        n = p.shape[-1]
        d = np.ascontiguousarray(proposals, np.int32)
        qq = None if q is None else np.ascontiguousarray(q, np.float64)
        emitted = (i32 * 6)()
        ne, acc, rows, rej = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        self._check(self.lib.ref_reject_sample(_ptr(d), _ptr(qq), _ptr(p), d.size, n, seed, step, temperature,
                                               emitted, C.byref(ne), C.byref(acc), C.byref(rows), C.byref(rej)))
        return list(emitted[:ne.value]), acc.value, rows.value, rej.value

    def attempt_counter_take2(self, first):
        threw = C.c_int()
        return self.lib.ref_attempt_counter_take2(first, C.byref(threw)), bool(threw.value)


class ReferenceGpu:
    """The reference's own CUDA kernels (fuse-head; dense compact head, hc_pre, rms, promote), compiled in place for
    sm_100a by oracle/Makefile into oracle/_ref.  Calls take raw device pointers (ints) and a stream."""

    def __init__(self):
        fh = os.path.join(HERE, "_ref", "libds41_ref_fusehead.so")
        de = os.path.join(HERE, "_ref", "libds41_ref_dense.so")
        self.available = os.path.exists(fh) and os.path.exists(de)
        if not self.available:
            return
        self.fusehead, self.dense = C.CDLL(fh), C.CDLL(de)
        self.fusehead.ds41_fuse_head_decode.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, P]
        self.fusehead.ds41_fuse_head_half_tree.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, P]
        self.dense.ds41_dense_head_compact.argtypes = [P, P, P, C.c_int, C.c_int, C.c_int, P]
        self.dense.ds41_dense_hc_pre.argtypes = [P, P, P, C.c_int, C.c_int, P]
        self.dense.ds41_dense_rms.argtypes = [P, P, P, C.c_int, C.c_int, f32, P]
        self.dense.ds41_dense_promote.argtypes = [P, P, C.c_int, P]
