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

// ---------------------------------------------------------------------------------------------------------------
// logits_sha256 of the reference's score event (engine/src/server.cpp:184-197: SHA-256 over the row's FP32 values in
// little-endian byte order, i.e. over the row as it lies in device memory).  SHA-256 is a chain over 64-byte blocks, so a
// row is one thread's work (8080 blocks at the full vocabulary, a few milliseconds); rows run side by side, one per
// thread.  What leaves the device is 32 bytes per row instead of the row itself.
namespace ds41 {
namespace {

__constant__ uint32_t kSha256K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

__device__ __forceinline__ uint32_t rotr(uint32_t x, int n) { return __funnelshift_r(x, x, n); }

__device__ void sha256_block(uint32_t (&h)[8], const uint32_t (&m)[16]) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = m[i];
  uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    if (i >= 16) {
      const uint32_t w15 = w[(i + 1) & 15], w2 = w[(i + 14) & 15];
      const uint32_t s0 = rotr(w15, 7) ^ rotr(w15, 18) ^ (w15 >> 3), s1 = rotr(w2, 17) ^ rotr(w2, 19) ^ (w2 >> 10);
      w[i & 15] = w[i & 15] + s0 + w[(i + 9) & 15] + s1;
    }
    const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kSha256K[i] + w[i & 15];
    const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
    hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}

__global__ void sha256_rows_kernel(const float *logits, long long stride, int rows, int vocab, uint8_t *digests) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const uint32_t *src = reinterpret_cast<const uint32_t *>(logits + size_t(row) * stride);
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  const int words = vocab;                 // 32-bit words of message; the message length is always a multiple of 4 bytes
  int at = 0;
  uint32_t m[16];
  for (; at + 16 <= words; at += 16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = __byte_perm(__ldg(src + at + i), 0, 0x0123);  // message words are big-endian
    sha256_block(h, m);
  }
  // padding: 0x80, zeros, 64-bit big-endian bit length
  const int rest = words - at;             // 0..15 words
#pragma unroll
  for (int i = 0; i < 16; ++i) m[i] = i < rest ? __byte_perm(__ldg(src + at + i), 0, 0x0123) : (i == rest ? 0x80000000u : 0u);
  const unsigned long long bits = (unsigned long long)words * 32ull;
  if (rest >= 14) {                        // no room for the length in this block
    sha256_block(h, m);
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = 0u;
  }
  m[14] = uint32_t(bits >> 32); m[15] = uint32_t(bits);
  sha256_block(h, m);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    digests[size_t(row) * 32 + 4 * i] = uint8_t(h[i] >> 24);
    digests[size_t(row) * 32 + 4 * i + 1] = uint8_t(h[i] >> 16);
    digests[size_t(row) * 32 + 4 * i + 2] = uint8_t(h[i] >> 8);
    digests[size_t(row) * 32 + 4 * i + 3] = uint8_t(h[i]);
  }
}

}  // namespace
}  // namespace ds41

extern "C" int ds41_b200_logits_sha256(const float *logits, int rows, int vocab, int64_t logits_stride, uint8_t *digests,
                                       cudaStream_t stream) {
  if (!logits || !digests || rows < 1 || vocab < 1 || logits_stride < vocab) return ds41::invalid("sha256 arguments");
  ds41::sha256_rows_kernel<<<(rows + 31) / 32, 32, 0, stream>>>(logits, logits_stride, rows, vocab, digests);
  return int(cudaGetLastError());
}
