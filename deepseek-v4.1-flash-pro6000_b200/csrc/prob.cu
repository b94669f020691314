// Operators on PROBABILITY rows: the device form of the reference sampler's C ABI, for callers that keep the
// reference's interface (logits -> probability row -> sample / verify) instead of the fused calls on logits.
//   ds41_b200_probabilities          ds41_spark_probabilities   (third_party/spark/src/sampling.cpp:30-38)
//   ds41_b200_sample_probabilities   ds41_spark_sample_v2       (:12-21,59)
//   ds41_b200_verify_probabilities   ds41_spark_verify_v2       (:39-56)
//   ds41_spark_sample_gpu_v2 / ds41_spark_verify_gpu_v2          (third_party/spark/src/sampling.cu:24-39,71-72;
//                                                                 spark.h:133-134: FP32 measures normalised in FP64)
// Every sum runs on one thread in index order, as the reference's host loops do, so that for the same probability rows
// the results are the reference's bit for bit (no exponential is involved once the rows exist; ds41_b200_probabilities
// itself can differ from the host's rows in the last place of exp()).  One CTA per row / per transaction: these are
// compatibility and reporting paths (milliseconds per full-vocabulary row), not the decode-rate path.
#include "ds41_b200.h"
#include "host_error.h"
#include "replay_core.cuh"
#include <cmath>

namespace ds41 {
namespace {

constexpr int kRowNotNormalized = DS41_B200_ROW_NOT_NORMALIZED;

// validate() of the reference (sampling.cpp:12-17): finite, non-negative, |sum - 1| <= 1e-8.  Returns 0 or a row status.
template <class T>
__device__ int validate_row(ReplaySmem &s, const T *p, int n) {
  int bad = 0;
  for (int i = threadIdx.x; i < n; i += kRT) {
    const double v = double(p[i]);
    if (!isfinite(v) || v < 0) bad = 1;
  }
  bad = __syncthreads_or(bad);
  if (bad) return DS41_B200_ROW_NONFINITE;
  const double z = sequential_sum(s, n, [p](int i) { return double(p[i]); });
  return fabs(z - 1.0) > 1e-8 ? kRowNotNormalized : 0;
}

// first maximum of a row (std::max_element / best(), sampling.cpp:22)
template <class T>
__device__ int first_max(ReplaySmem &s, const T *p, int n) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double best = -CUDART_INF;
  int best_id = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += kRT) {
    const double v = double(p[i]);
    if (v > best) { best = v; best_id = i; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
  }
  if (lane == 0) { s.stage[warp] = best; s.red_i[warp] = best_id; }
  __syncthreads();
  for (int w = 0; w < kRT / 32; ++w)
    if (s.stage[w] > best || (s.stage[w] == best && s.red_i[w] < best_id)) { best = s.stage[w]; best_id = s.red_i[w]; }
  __syncthreads();
  return best_id == 0x7fffffff ? 0 : best_id;
}

struct ProbArgs {
  const float *logits;
  long long stride;
  int rows, vocab;
  double t, top_p;
  double *out;
  int32_t *status;
  unsigned char *scratch;
};

__global__ void __launch_bounds__(kRT) probabilities_kernel(ProbArgs a) {
  __shared__ ReplaySmem s;
  extern __shared__ __align__(16) unsigned char dynamic[];
  unsigned char *mine = a.scratch + size_t(blockIdx.x) * size_t(kReplayPad) * 12;
  unsigned long long *key = reinterpret_cast<unsigned long long *>(mine);
  int *idx = reinterpret_cast<int *>(mine + size_t(kReplayPad) * 8);
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const float *x = a.logits + size_t(row) * a.stride;
    double *p = a.out + size_t(row) * a.vocab;
    int bad = 0;
    for (int i = threadIdx.x; i < a.vocab; i += kRT)
      if ((__float_as_uint(x[i]) & 0x7f800000u) == 0x7f800000u) bad = 1;
    bad = __syncthreads_or(bad);
    if (bad) {  // "nonfinite logits" (sampling.cpp:32)
      for (int i = threadIdx.x; i < a.vocab; i += kRT) p[i] = CUDART_NAN;
      if (threadIdx.x == 0) a.status[row] = DS41_B200_ROW_NONFINITE;
      __syncthreads();
      continue;
    }
    if (a.t == 0) {  // one-hot at the first maximum
      const int b = first_max(s, x, a.vocab);
      for (int i = threadIdx.x; i < a.vocab; i += kRT) p[i] = i == b ? 1.0 : 0.0;
    } else {
      replay_probabilities(s, x, a.vocab, a.t, a.top_p, p, key, idx, dynamic);
    }
    if (threadIdx.x == 0) a.status[row] = 0;
    __syncthreads();
  }
}

template <class T>
struct SampleArgs {
  const T *p;
  long long stride;
  int rows, vocab;
  const uint64_t *seeds, *steps;
  uint64_t seed, step;   // used when seeds / steps are null
  uint32_t slot, purpose;
  int32_t *tokens, *status;
};

// kMeasure: the row is an FP32 measure normalised here (the reference's GPU sampler); else a probability row that must
// already be normalised (the host rule's validate()).
template <class T, bool kMeasure>
__global__ void __launch_bounds__(kRT) sample_rows_kernel(SampleArgs<T> a) {
  __shared__ ReplaySmem s;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T *p = a.p + size_t(row) * a.stride;
    int status = 0, token = -1;
    if (kMeasure) {  // mass(): a non-finite or negative entry poisons the sum (sampling.cu:7)
      int bad = 0;
      for (int i = threadIdx.x; i < a.vocab; i += kRT) {
        const double v = double(p[i]);
        if (!isfinite(v) || v < 0) bad = 1;
      }
      if (__syncthreads_or(bad)) status = DS41_B200_ROW_NONFINITE;
    } else {
      status = validate_row(s, p, a.vocab);
    }
    if (status == 0) {
      const uint64_t seed = a.seeds ? a.seeds[row] : a.seed, step = a.steps ? a.steps[row] : a.step;
      const double u = philox_uniform(seed, step, a.slot, a.purpose);
      double margin;
      token = replay_draw(s, a.vocab, u, [p](int i) { return double(p[i]); }, &margin);
      if (token < 0) status = DS41_B200_ROW_EMPTY;
    }
    if (threadIdx.x == 0) {
      a.tokens[row] = status ? -1 : token;
      if (a.status) a.status[row] = status;
    }
    __syncthreads();
  }
}

template <class T>
struct VerifyRowsArgs {
  const int32_t *draft_ids;  // [sequences, drafts]
  const T *q, *p;            // [sequences, drafts, vocab], [sequences, drafts + 1, vocab]
  int sequences, drafts, vocab, greedy;
  const uint64_t *seeds, *steps;
  uint64_t seed, step;
  ds41_spark_result *results;
  int32_t *status;
};

// verify_impl of the reference (sampling.cpp:39-53) for one transaction per CTA.
template <class T, bool kMeasure>
__global__ void __launch_bounds__(kRT) verify_rows_kernel(VerifyRowsArgs<T> a) {
  __shared__ ReplaySmem s;
  for (int seq = blockIdx.x; seq < a.sequences; seq += gridDim.x) {
    const int n = a.vocab, count = a.drafts;
    const T *p = a.p + size_t(seq) * (count + 1) * n;
    const T *q = a.q ? a.q + size_t(seq) * count * n : nullptr;
    const int32_t *d = a.draft_ids ? a.draft_ids + size_t(seq) * count : nullptr;
    const uint64_t seed = a.seeds ? a.seeds[seq] : a.seed, step = a.steps ? a.steps[seq] : a.step;
    ds41_spark_result r{};
    int status = 0;
    // the normaliser of a measure (1 for a validated probability row)
    auto measure = [&](const T *row, double *z) -> int {
      if (!kMeasure) { *z = 1.0; return validate_row(s, row, n); }
      int bad = 0;
      for (int i = threadIdx.x; i < n; i += kRT) {
        const double v = double(row[i]);
        if (!isfinite(v) || v < 0) bad = 1;
      }
      if (__syncthreads_or(bad)) return DS41_B200_ROW_NONFINITE;
      *z = sequential_sum(s, n, [row](int i) { return double(row[i]); });
      return (*z > 0 && isfinite(*z)) ? 0 : DS41_B200_ROW_EMPTY;
    };
    // every target row is validated before the first decision (sampling.cpp:42); the measure variant checks each row
    // where it is used, as the reference kernel does
    double pz[6] = {1, 1, 1, 1, 1, 1};
    if (!kMeasure)
      for (int k = 0; k <= count && status == 0; ++k) status = measure(p + size_t(k) * n, &pz[k]);
    for (int k = 0; k < count && status == 0; ++k) {
      const T *pk = p + size_t(k) * n;
      const T *qk = q ? q + size_t(k) * n : nullptr;
      if (kMeasure) { status = measure(pk, &pz[k]); if (status) break; }
      if (d[k] < 0 || d[k] >= n) { status = DS41_B200_ROW_DRAFT; break; }
      bool accept;
      double qz = 1;
      if (a.greedy) {
        accept = d[k] == first_max(s, pk, n);
      } else {
        status = measure(qk, &qz);
        if (status) break;
        if (!(double(qk[d[k]]) > 0)) { status = DS41_B200_ROW_DRAFT; break; }
        const double u = philox_uniform(seed, step, uint32_t(k), 2u);
        const double ratio = kMeasure ? (double(pk[d[k]]) / pz[k]) / (double(qk[d[k]]) / qz)
                                      : double(pk[d[k]]) / double(qk[d[k]]);
        accept = u < fmin(1.0, ratio);
      }
      if (accept) {
        r.tokens[r.emitted++] = d[k];
        ++r.accepted_drafts;
      } else {
        int token;
        if (a.greedy) {
          token = first_max(s, pk, n);
        } else {
          const double u = philox_uniform(seed, step, uint32_t(k), 3u);
          const double pzk = pz[k];
          double margin;
          token = replay_draw(s, n, u, [pk, qk, pzk, qz](int i) {
            return kMeasure ? fmax(0.0, double(pk[i]) / pzk - double(qk[i]) / qz) : fmax(0.0, double(pk[i]) - double(qk[i]));
          }, &margin);
          if (token < 0) { status = DS41_B200_ROW_EMPTY; break; }
        }
        r.tokens[r.emitted++] = token;
        r.rejected = 1;
        break;
      }
    }
    if (status == 0 && !r.rejected) {
      const T *last = p + size_t(count) * n;
      int token;
      if (kMeasure) status = measure(last, &pz[count]);
      if (status == 0) {
        if (a.greedy) {
          token = first_max(s, last, n);
        } else {
          const double u = philox_uniform(seed, step, uint32_t(count), 0u);
          const double z = pz[count];
          double margin;
          token = replay_draw(s, n, u, [last, z](int i) { return kMeasure ? double(last[i]) / z : double(last[i]); }, &margin);
          if (token < 0) status = DS41_B200_ROW_EMPTY;
        }
        if (status == 0) r.tokens[r.emitted++] = token;
      }
    }
    if (threadIdx.x == 0) {
      if (status) { r = ds41_spark_result{}; r.emitted = -1; }   // in-band failure, as sampling.cu:29-32
      else r.accepted_input_rows = r.accepted_drafts + 1;
      a.results[seq] = r;
      if (a.status) a.status[seq] = status;
    }
    __syncthreads();
  }
}

// The transactions of ds41_b200_verify_logits whose status carries a certification bit, redone from the logits:
// probability rows by the reference's rule (replay_probabilities), then verify_impl (sampling.cpp:39-53) on them, one
// CTA per transaction, two rows in memory at a time.  A decision that is still within 16 * 2^-53 of its threshold keeps
// its bit; everything else leaves with status 0.
constexpr double kVerifyStillClose = 16.0 * kU;

__global__ void __launch_bounds__(kRT) verify_replay_kernel(VerifyReplayArgs a) {
  __shared__ ReplaySmem s;
  extern __shared__ __align__(16) unsigned char dynamic[];
  unsigned char *mine = a.scratch + size_t(blockIdx.x) * size_t(kReplayPad) * 28;
  double *pbuf = reinterpret_cast<double *>(mine), *qbuf = pbuf + kReplayPad;
  unsigned long long *key = reinterpret_cast<unsigned long long *>(mine + size_t(kReplayPad) * 16);
  int *idx = reinterpret_cast<int *>(mine + size_t(kReplayPad) * 24);
  ds41_spark_result *results = static_cast<ds41_spark_result *>(a.results);
  const int n = a.vocab, count = a.drafts;
  for (int first = 0; first < a.sequences; first += kRT) {
    const int candidate = first + threadIdx.x;
    if (!__syncthreads_or(candidate < a.sequences && a.status[candidate] > 0)) continue;
    for (int seq = first + blockIdx.x; seq < min(a.sequences, first + kRT); seq += gridDim.x) {
      if (!(a.status[seq] > 0)) continue;   // the same in every thread
      const uint64_t seed = a.seeds[seq], step = a.steps[seq];
      ds41_spark_result r{};
      int status = 0, close = 0;
      for (int k = 0; k < count && status == 0 && !r.rejected; ++k) {
        const int d = a.ids[size_t(seq) * count + k];   // in range: the first pass rejects the transaction otherwise
        const Replayed rp = replay_probabilities(s, a.target + (size_t(seq) * (count + 1) + k) * n, n, a.t, a.top_p, pbuf,
                                                 key, idx, dynamic);
        const Replayed rq = replay_probabilities(s, a.draft + (size_t(seq) * count + k) * n, n, a.t, a.top_p, qbuf, key,
                                                 idx, dynamic);
        if (rp.cut_margin < kVerifyStillClose || rq.cut_margin < kVerifyStillClose) close |= 2;
        const double pd = pbuf[d], qd = qbuf[d];
        if (!(qd > 0)) { status = DS41_B200_ROW_DRAFT; break; }
        const double u = philox_uniform(seed, step, uint32_t(k), 2u);
        const double ratio = pd / qd;
        const bool accept = u < fmin(1.0, ratio);
        if (ratio < 1.0 && fabs(u - ratio) < kVerifyStillClose * ratio) close |= 4;
        if (accept) {
          r.tokens[r.emitted++] = d;
          ++r.accepted_drafts;
        } else {
          double margin;
          const int token = replay_draw(s, n, philox_uniform(seed, step, uint32_t(k), 3u),
                                        [pbuf, qbuf](int i) { return fmax(0.0, pbuf[i] - qbuf[i]); }, &margin);
          if (token < 0) { status = DS41_B200_ROW_EMPTY; break; }
          if (margin < kVerifyStillClose) close |= 8;
          r.tokens[r.emitted++] = token;
          r.rejected = 1;
        }
      }
      if (status == 0 && !r.rejected) {
        const Replayed rp = replay_probabilities(s, a.target + (size_t(seq) * (count + 1) + count) * n, n, a.t, a.top_p,
                                                 pbuf, key, idx, dynamic);
        if (rp.cut_margin < kVerifyStillClose) close |= 2;
        double margin;
        const int token = replay_draw(s, n, philox_uniform(seed, step, uint32_t(count), 0u),
                                      [pbuf](int i) { return pbuf[i]; }, &margin);
        if (margin < kVerifyStillClose) close |= 1;
        r.tokens[r.emitted++] = token;
      }
      if (threadIdx.x == 0) {
        if (status) { r = ds41_spark_result{}; r.emitted = -1; }
        else r.accepted_input_rows = r.accepted_drafts + 1;
        results[seq] = r;
        a.status[seq] = status ? status : close;
      }
      __syncthreads();
    }
  }
}

int grid_for(int items) { return items < 592 ? items : 592; }

}  // namespace
}  // namespace ds41

namespace ds41 {
cudaError_t launch_verify_replay(const VerifyReplayArgs &a, cudaStream_t stream) {
  const cudaError_t e = cudaFuncSetAttribute(verify_replay_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             int(kReplayDynamicBytes));
  if (e != cudaSuccess) return e;
  const int ctas = a.sequences < kVerifyReplayCtas ? a.sequences : kVerifyReplayCtas;
  verify_replay_kernel<<<ctas, kRT, kReplayDynamicBytes, stream>>>(a);
  return cudaGetLastError();
}
}  // namespace ds41

using namespace ds41;

extern "C" size_t ds41_b200_probabilities_scratch_bytes(int rows) {
  if (rows < 1) return 0;
  return size_t(rows < kReplayCtas * 8 ? rows : kReplayCtas * 8) * size_t(kReplayPad) * 12;
}

extern "C" int ds41_b200_probabilities(const ds41_b200_prob_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_prob_args)) return invalid("probabilities args: struct size / ABI mismatch");
  if (p->rows < 1 || p->vocab < 1 || p->vocab > DS41_B200_MAX_VOCAB || !p->logits || p->logits_stride < p->vocab ||
      !p->probabilities || !p->status)
    return invalid("probabilities arguments");
  if (!std::isfinite(p->temperature) || p->temperature < 0 || !std::isfinite(p->top_p) || p->top_p <= 0 || p->top_p > 1)
    return invalid("temperature/top_p/logits");
  const size_t need = ds41_b200_probabilities_scratch_bytes(p->rows);
  if (!p->scratch || p->scratch_bytes < need || (reinterpret_cast<uintptr_t>(p->scratch) & 15u))
    return invalid("probabilities scratch too small or misaligned");
  ProbArgs a{p->logits, p->logits_stride, p->rows, p->vocab,
             p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0,  // engine/src/sampling.cpp:209-210
             p->top_p, p->probabilities, p->status, static_cast<unsigned char *>(p->scratch)};
  const int ctas = int(need / (size_t(kReplayPad) * 12));
  const cudaError_t e = cudaFuncSetAttribute(probabilities_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             int(kReplayDynamicBytes));
  if (e != cudaSuccess) return int(e);
  probabilities_kernel<<<ctas, kRT, kReplayDynamicBytes, stream>>>(a);
  return int(cudaGetLastError());
}

extern "C" int ds41_b200_sample_probabilities(const double *p, int rows, int vocab, int64_t stride, const uint64_t *seeds,
                                              const uint64_t *steps, uint32_t slot, uint32_t purpose, int32_t *tokens,
                                              int32_t *status, cudaStream_t stream) {
  if (!p || rows < 1 || vocab < 1 || stride < vocab || !seeds || !steps || !tokens) return invalid("sample arguments");
  if (slot > 5 || purpose > 3) return invalid("Philox v2 address out of range");
  SampleArgs<double> a{p, stride, rows, vocab, seeds, steps, 0, 0, slot, purpose, tokens, status};
  sample_rows_kernel<double, false><<<grid_for(rows), kRT, 0, stream>>>(a);
  return int(cudaGetLastError());
}

extern "C" int ds41_b200_verify_probabilities(const int32_t *draft_ids, const double *q, const double *p, int sequences,
                                              int drafts, int vocab, int greedy, const uint64_t *seeds,
                                              const uint64_t *steps, ds41_spark_result *results, int32_t *status,
                                              cudaStream_t stream) {
  if (!results || !p || sequences < 1 || drafts < 0 || drafts > 5 || vocab < 1 || !seeds || !steps ||
      (drafts && (!draft_ids || (!q && !greedy))))
    return invalid("verify arguments");
  VerifyRowsArgs<double> a{draft_ids, q, p, sequences, drafts, vocab, greedy ? 1 : 0, seeds, steps, 0, 0, results, status};
  verify_rows_kernel<double, false><<<grid_for(sequences), kRT, 0, stream>>>(a);
  return int(cudaGetLastError());
}

// The reference's device sampler ABI (spark.h:133-134): FP32 measures on the device, one row / one transaction, the
// result in caller-owned device memory, data errors in band (token -1 / emitted -1).
extern "C" int ds41_spark_sample_gpu_v2(const float *p, int vocab, uint64_t seed, uint64_t step, uint32_t slot,
                                        uint32_t purpose, int32_t *out, void *stream) {
  if (!p || !out || vocab < 1 || purpose > 3 || slot > 5) return int(cudaErrorInvalidValue);
  SampleArgs<float> a{p, vocab, 1, vocab, nullptr, nullptr, seed, step, slot, purpose, out, nullptr};
  sample_rows_kernel<float, true><<<1, kRT, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return int(cudaGetLastError());
}

extern "C" int ds41_spark_verify_gpu_v2(const int32_t *d, const float *q, const float *p, int drafts, int vocab, int greedy,
                                        uint64_t seed, uint64_t step, ds41_spark_result *out, void *stream) {
  if (!out || !p || drafts < 0 || drafts > 5 || vocab < 1 || (drafts && (!d || (!q && !greedy))))
    return int(cudaErrorInvalidValue);
  VerifyRowsArgs<float> a{d, q, p, 1, drafts, vocab, greedy ? 1 : 0, nullptr, nullptr, seed, step, out, nullptr};
  verify_rows_kernel<float, true><<<1, kRT, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return int(cudaGetLastError());
}
