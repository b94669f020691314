// Score reporting on device logits: log-normaliser, first maximum and the top-N ids with their log-probabilities, the
// caller-visible outputs the reference computes with host passes over the vocabulary (engine/src/server.cpp:178-183
// log_normalizer, :730-737 top_order, used at :450-461 and :603-612).  One CTA per row; the row is read from L2/HBM
// 2 + N times, which is what a reporting path (a few rows per request, N <= 32) needs, not a decode-rate kernel.
//   logsumexp   = m + log(sum_i exp(double(x_i) - m)), m = the row maximum (the reference sums sequentially; here the
//                 sum is a fixed-order tree, so the value agrees to a few units in the last place, not bit for bit)
//   top ids     = the first N ids in the order (logit descending, id ascending): exact
//   top_logprob = double(x_id) - logsumexp
#include "ds41_b200.h"
#include "host_error.h"
#include "row_core.cuh"

namespace ds41 {
namespace {

constexpr int kScoreThreads = 512;
constexpr int kScoreWarps = kScoreThreads / 32;

// (value, id) maximum under "larger value, then lower id" over the CTA; every thread gets the result.
__device__ __forceinline__ void score_argmax(float &v, int &id, float *sv, int *si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, id, o);
    if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
  }
  if (lane == 0) { sv[warp] = v; si[warp] = id; }
  __syncthreads();
  v = sv[0]; id = si[0];
  for (int w = 1; w < kScoreWarps; ++w)
    if (sv[w] > v || (sv[w] == v && si[w] < id)) { v = sv[w]; id = si[w]; }
  __syncthreads();
}

__global__ void __launch_bounds__(kScoreThreads) score_kernel(ds41_b200_score_args a) {
  __shared__ float sv[kScoreWarps];
  __shared__ int si[kScoreWarps];
  __shared__ double sd[kScoreWarps];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float *x = a.logits + size_t(row) * a.logits_stride;
  // first maximum and finiteness
  float best = -CUDART_INF_F;
  int best_id = 0x7fffffff, bad = 0;
  for (int i = tid; i < a.vocab; i += kScoreThreads) {
    const float v = __ldg(x + i);
    if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) bad = 1;
    if (v > best) { best = v; best_id = i; }
  }
  bad = __syncthreads_or(bad);
  if (bad) {  // the reference rejects non-finite logits (engine/src/sampling.cpp:133-139)
    if (tid == 0) {
      a.status[row] = DS41_B200_ROW_NONFINITE;
      a.logsumexp[row] = CUDART_NAN;
      if (a.top1) a.top1[row] = -1;
    }
    for (int k = tid; k < a.top_n; k += kScoreThreads) {
      a.top_ids[size_t(row) * a.top_n + k] = -1;
      a.top_logprob[size_t(row) * a.top_n + k] = CUDART_NAN;
    }
    return;
  }
  score_argmax(best, best_id, sv, si);
  // normaliser: lanes stride the row, fixed-order tree
  const double m = double(best);
  double z = 0;
  for (int i = tid; i < a.vocab; i += kScoreThreads) z += exp_nonpos(double(__ldg(x + i)) - m);
#pragma unroll
  for (int o = 16; o; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
  if (lane == 0) sd[warp] = z;
  __syncthreads();
  z = 0;
  for (int w = 0; w < kScoreWarps; ++w) z += sd[w];
  const double lse = m + log(z);
  if (tid == 0) {
    a.status[row] = 0;
    a.logsumexp[row] = lse;
    if (a.top1) a.top1[row] = best_id;
  }
  // top-N by repeated selection of the next id in the order (logit descending, id ascending)
  float prev_v = best;
  int prev_id = best_id;
  for (int k = 0; k < a.top_n; ++k) {
    float v = -CUDART_INF_F;
    int id = 0x7fffffff;
    if (k == 0) { v = best; id = best_id; }
    else {
      for (int i = tid; i < a.vocab; i += kScoreThreads) {
        const float y = __ldg(x + i);
        const bool after = y < prev_v || (y == prev_v && i > prev_id);  // strictly after the previous pick
        if (after && (y > v || (y == v && i < id))) { v = y; id = i; }
      }
      score_argmax(v, id, sv, si);
    }
    if (id == 0x7fffffff) id = -1;  // fewer than top_n ids in the row
    if (tid == 0) {
      a.top_ids[size_t(row) * a.top_n + k] = id;
      a.top_logprob[size_t(row) * a.top_n + k] = id >= 0 ? double(v) - lse : CUDART_NAN;
    }
    prev_v = v; prev_id = id;
    if (id < 0) {
      for (int k2 = k + 1 + tid; k2 < a.top_n; k2 += kScoreThreads) {
        a.top_ids[size_t(row) * a.top_n + k2] = -1;
        a.top_logprob[size_t(row) * a.top_n + k2] = CUDART_NAN;
      }
      break;
    }
  }
}

}  // namespace
}  // namespace ds41

using namespace ds41;

extern "C" int ds41_b200_score_logits(const ds41_b200_score_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_score_args)) return invalid("score args: struct size / ABI mismatch");
  if (p->rows < 1 || p->vocab < 1 || !p->logits || p->logits_stride < p->vocab || !p->logsumexp || !p->status)
    return invalid("score args: rows / vocab / buffers");
  if (p->top_n < 0 || p->top_n > DS41_B200_SCORE_MAX_TOP || (p->top_n > 0 && (!p->top_ids || !p->top_logprob)))
    return invalid("score args: top_n out of range or missing output buffers");
  score_kernel<<<p->rows, kScoreThreads, 0, stream>>>(*p);
  return int(cudaGetLastError());
}
