// The operators either side of the target head that also produce or consume logits rows:
//   ds41_dense_head_compact    the drafter's BF16 head (components/dense/src/compact.cu:10-24,44-50; called from
//                              engine/third_party/spark/src/forward.cu:132): y[m,n] = sum_k W[n,k] x[m,k], M <= 8
//   ds41_b200_markov_logits    draft logits of position k: U[k] + W_markov . emb(previous token)
//                              (third_party/spark/src/forward.cu:46,135-139: markov() + add_bias)
//   ds41_b200_final_norm       what runs in front of the target head: HC-pre mix -> RMSNorm (eps 1e-20) -> BF16 -> FP32
//                              (engine/src/hotpath/batch.inc:487-492; components/dense/src/ops.cu:17-27,45-48,102)
// Each keeps the reference kernel's FP32 order of operations, which is what fixes the bits of the result, and changes only
// how the data moves: activations staged in shared memory, several weight rows per warp so that an activation fragment
// read from shared memory is used four times, 16-byte weight loads in flight ahead of their use, one fused launch for
// the three-kernel prologue.
#include "ds41_b200.h"
#include "host_error.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ds41 {
namespace {

constexpr int kHeadThreads = 256, kHeadWarps = kHeadThreads / 32;

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Arithmetic of the reference kernel head<M, 8, 4> for one output: lane l of 32 takes k = 8 l + 256 i, i = 0, 1, ...;
// element j of its eight goes to accumulator j % 4 by fused multiply-add (so accumulator a sees k + a, k + a + 4 of every
// i, in that order); at the end (a0 + a1) + (a2 + a3), then the five-level shuffle-down tree over the lanes.
template <int M, int kRowsPerWarp>
__global__ void __launch_bounds__(kHeadThreads) head_compact_kernel(const float *__restrict__ x,
                                                                    const __nv_bfloat16 *__restrict__ w,
                                                                    float *__restrict__ y, int N, int K) {
  extern __shared__ __align__(16) float xs[];  // [M][K]
  for (int i = threadIdx.x * 4; i < M * K; i += kHeadThreads * 4)
    *reinterpret_cast<float4 *>(xs + i) = __ldg(reinterpret_cast<const float4 *>(x + i));
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = (N + kRowsPerWarp - 1) / kRowsPerWarp;
  for (int g = blockIdx.x * kHeadWarps + warp; g < groups; g += gridDim.x * kHeadWarps) {
    const int row0 = g * kRowsPerWarp;
    float acc[kRowsPerWarp][M][4];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int a = 0; a < 4; ++a) acc[r][m][a] = 0.f;
    const uint4 *wr[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
      wr[r] = reinterpret_cast<const uint4 *>(w + size_t(min(row0 + r, N - 1)) * K);  // rows beyond N repeat the last one
    // two steps of weights are in flight ahead of the one being consumed (about 32 KB per SM: what the HBM latency needs)
    uint4 cur[kRowsPerWarp], nxt[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      cur[r] = __ldg(wr[r] + lane);
      nxt[r] = 256 < K ? __ldg(wr[r] + lane + 32) : cur[r];
    }
    for (int k = lane * 8; k < K; k += 256) {
      uint4 far[kRowsPerWarp];
      const bool more = k + 512 < K;
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) far[r] = more ? __ldg(wr[r] + ((k + 512) >> 3)) : nxt[r];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 a = *reinterpret_cast<const float4 *>(xs + m * K + k);
        const float4 b = *reinterpret_cast<const float4 *>(xs + m * K + k + 4);
        const float xx[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
          const uint32_t ww[4] = {cur[r].x, cur[r].y, cur[r].z, cur[r].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float wj = bf16_bits_to_float((j & 1) ? (ww[j >> 1] >> 16) : (ww[j >> 1] & 0xffffu));
            acc[r][m][j & 3] = __fmaf_rn(wj, xx[j], acc[r][m][j & 3]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) { cur[r] = nxt[r]; nxt[r] = far[r]; }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float sum = __fadd_rn(__fadd_rn(acc[r][m][0], acc[r][m][1]), __fadd_rn(acc[r][m][2], acc[r][m][3]));
#pragma unroll
        for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
        if (lane == 0 && row0 + r < N) y[size_t(m) * N + row0 + r] = sum;
      }
  }
}

// logits[n] = U[n] + bias[n], bias[n] = W[n, 0..256) . e with e = the previous token's Markov embedding promoted to FP32.
// The reference forms the bias with a library GEMV whose order of summation is not specified; here it is the compact
// head's order for K = 256 (one step per lane), then the reference's single rounded addition (forward.cu:46).
__global__ void __launch_bounds__(256) markov_logits_kernel(const float *__restrict__ u,
                                                            const __nv_bfloat16 *__restrict__ w,
                                                            const __nv_bfloat16 *__restrict__ emb, float *__restrict__ out,
                                                            int vocab) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= vocab) return;
  const uint4 ev = __ldg(reinterpret_cast<const uint4 *>(emb) + lane);
  const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w + size_t(row) * 256) + lane);
  const uint32_t ee[4] = {ev.x, ev.y, ev.z, ev.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float wj = bf16_bits_to_float((j & 1) ? (ww[j >> 1] >> 16) : (ww[j >> 1] & 0xffffu));
    const float ej = bf16_bits_to_float((j & 1) ? (ee[j >> 1] >> 16) : (ee[j >> 1] & 0xffffu));
    acc[j & 3] = __fmaf_rn(wj, ej, acc[j & 3]);
  }
  float sum = __fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3]));
#pragma unroll
  for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
  if (lane == 0) out[row] = __fadd_rn(__ldg(u + row), sum);
}

// Launch geometry of the reference's RMS norm (ops.cu:16: it follows a PyTorch reduction and depends on the number of
// rows in the call): threads per block and the width of one reduction segment.
int rms_geometry(int M, int K, int *width) {
  int height = 1;
  while (height * 2 <= M && height * 2 <= 16) height *= 2;
  int n = 1;
  while (n * 2 <= K / 4 && n * 2 <= 512) n *= 2;
  *width = n < 512 / height ? n : 512 / height;
  return K / *width >= height * 16 ? *width * height : *width;
}

// One block per row: y = x mixed over its four hyper-connection streams (rounded to BF16), sum of squares with the
// reference's accumulation and reduction order (four strided accumulators per thread, ((v0 + v1) + v2) + v3, halving
// inside segments of `width` threads down to a warp, shuffle-down, then a halving tree over the segments), rsqrtf of
// mean + eps, x * rstd * weight rounded to BF16, stored as FP32 (the head's input type).
__global__ void final_norm_kernel(const __nv_bfloat16 *__restrict__ h, const float *__restrict__ pre,
                                  const __nv_bfloat16 *__restrict__ weight, float *__restrict__ out, int K, float eps,
                                  int width) {
  extern __shared__ __align__(16) unsigned char norm_smem[];
  float *sh = reinterpret_cast<float *>(norm_smem);                        // [512]
  __nv_bfloat16 *xrow = reinterpret_cast<__nv_bfloat16 *>(sh + 512);       // [K]
  const int tid = threadIdx.x, row = blockIdx.x;
  float p[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = pre[row * 4 + j];
  for (int k = tid; k < K; k += blockDim.x) {  // HC-pre mix (ops.cu:45-48)
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) s = __fadd_rn(s, __fmul_rn(p[j], __bfloat162float(h[(size_t(row) * 4 + j) * K + k])));
    xrow[k] = __float2bfloat16_rn(s);
  }
  __syncthreads();
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = tid * 4; i < K; i += blockDim.x * 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j < K) {
        const float z = __bfloat162float(xrow[i + j]);
        v[j] = __fadd_rn(v[j], __fmul_rn(z, z));
      }
  }
  float sum = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[1]), v[2]), v[3]);
  sh[tid] = sum;
  __syncthreads();
  for (int d = width / 2; d >= 32; d >>= 1) {
    if (tid % width < d) { sum = __fadd_rn(sum, sh[tid + d]); sh[tid] = sum; }
    __syncthreads();
  }
  for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
  if (tid % width == 0) sh[tid] = sum;
  __syncthreads();
  for (int d = (blockDim.x / width) / 2; d; d >>= 1) {
    if (tid % width == 0 && tid / width < d) { sum = __fadd_rn(sum, sh[tid + d * width]); sh[tid] = sum; }
    __syncthreads();
  }
  const float total = sh[0];
  __syncthreads();
  if (tid == 0) sh[0] = rsqrtf(__fadd_rn(__fmul_rn(total, 1.f / K), eps));
  __syncthreads();
  const float rstd = sh[0];
  for (int k = tid; k < K; k += blockDim.x) {
    const __nv_bfloat16 yb =
        __float2bfloat16_rn(__fmul_rn(__fmul_rn(__bfloat162float(xrow[k]), rstd), __bfloat162float(weight[k])));
    out[size_t(row) * K + k] = __bfloat162float(yb);
  }
}

template <int M>
cudaError_t launch_compact(const float *x, const void *w, float *y, int N, int K, cudaStream_t stream) {
  // weight rows that share one read of an activation fragment; at one or two batch rows the kernel only streams
  // weights and more resident CTAs (fewer registers each) keep more loads in flight
  constexpr int kRowsPerWarp = M <= 2 ? 2 : M <= 6 ? 4 : 2;
  const size_t smem = size_t(M) * K * sizeof(float);
  static thread_local int configured = -1;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  if (configured != dev) {
    e = cudaFuncSetAttribute(head_compact_kernel<M, kRowsPerWarp>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured = dev;
  }
  const int per_sm = smem <= 48 * 1024 ? 4 : smem <= 100 * 1024 ? 2 : 1;
  const int groups = (N + kRowsPerWarp - 1) / kRowsPerWarp;
  int grid = sms * per_sm;
  if (grid > (groups + kHeadWarps - 1) / kHeadWarps) grid = (groups + kHeadWarps - 1) / kHeadWarps;
  head_compact_kernel<M, kRowsPerWarp><<<grid, kHeadThreads, smem, stream>>>(x, static_cast<const __nv_bfloat16 *>(w), y, N, K);
  return cudaGetLastError();
}

}  // namespace
}  // namespace ds41

using namespace ds41;

extern "C" int ds41_dense_head_compact(const float *x, const void *w, float *y, int M, int N, int K, cudaStream_t stream) {
  // the reference's argument check (compact.cu:45), plus what this kernel needs on top: the activations in shared memory
  if (!x || !w || !y || M < 1 || M > 8 || N < 1 || K < 256 || K % 256) return invalid("compact head arguments");
  if (size_t(M) * K * sizeof(float) > 224 * 1024) return invalid("compact head: M * K * 4 bytes must fit 224 KB of shared memory");
  if ((reinterpret_cast<uintptr_t>(w) & 15u) || (reinterpret_cast<uintptr_t>(x) & 15u)) return invalid("compact head operands must be 16-byte aligned");
  cudaError_t e;
  switch (M) {
    case 1: e = launch_compact<1>(x, w, y, N, K, stream); break;
    case 2: e = launch_compact<2>(x, w, y, N, K, stream); break;
    case 3: e = launch_compact<3>(x, w, y, N, K, stream); break;
    case 4: e = launch_compact<4>(x, w, y, N, K, stream); break;
    case 5: e = launch_compact<5>(x, w, y, N, K, stream); break;
    case 6: e = launch_compact<6>(x, w, y, N, K, stream); break;
    case 7: e = launch_compact<7>(x, w, y, N, K, stream); break;
    default: e = launch_compact<8>(x, w, y, N, K, stream); break;
  }
  return int(e);
}

extern "C" int ds41_b200_markov_logits(const float *draft_row, const void *markov_weight_bf16, const void *embedding_bf16,
                                       float *logits, int vocab, cudaStream_t stream) {
  if (!draft_row || !markov_weight_bf16 || !embedding_bf16 || !logits || vocab < 1 ||
      (reinterpret_cast<uintptr_t>(markov_weight_bf16) & 15u) || (reinterpret_cast<uintptr_t>(embedding_bf16) & 15u))
    return invalid("Markov logits arguments");
  const long long threads = (long long)vocab * 32;
  markov_logits_kernel<<<unsigned((threads + 255) / 256), 256, 0, stream>>>(
      draft_row, static_cast<const __nv_bfloat16 *>(markov_weight_bf16), static_cast<const __nv_bfloat16 *>(embedding_bf16),
      logits, vocab);
  return int(cudaGetLastError());
}

extern "C" int ds41_b200_final_norm(const void *h_bf16, const float *pre, const void *norm_weight_bf16, float *x_f32, int M,
                                    int K, float eps, cudaStream_t stream) {
  // M and K as ds41_dense_rms accepts them (ops.cu:110)
  if (!h_bf16 || !pre || !norm_weight_bf16 || !x_f32 || M < 1 || M > 8 || K < 128 || K % 4 || K > 16384)
    return invalid("final norm arguments");
  int width = 0;
  const int threads = rms_geometry(M, K, &width);
  final_norm_kernel<<<M, threads, 512 * sizeof(float) + size_t(K) * 2, stream>>>(
      static_cast<const __nv_bfloat16 *>(h_bf16), pre, static_cast<const __nv_bfloat16 *>(norm_weight_bf16), x_f32, K, eps,
      width);
  return int(cudaGetLastError());
}
