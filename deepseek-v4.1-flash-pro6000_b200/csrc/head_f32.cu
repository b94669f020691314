// FP32 head: y[m, n] = sum over k of w[n, k] * x[m, k], weights and activations in FP32.
//
// The reference's default target head promotes the BF16 weights to FP32 once (2.65 GB) and calls cuBLAS
// (ds41_dense_cublas(f32 = 1): components/dense/src/ops.cu:120-128, called from engine/src/forward.cu:1306-1318, TF32
// off), once per row.  cuBLAS does not specify its order of summation, so there is no bit pattern to reproduce: this
// kernel defines its own fixed order (per lane: fused multiply-adds over k = 4 l + 128 i + j in ascending i, j; then the
// five-level shuffle-down tree) and is checked against an FP64 product within the FP32 bound.  Weight streaming with
// 16-byte loads, activations in shared memory, all rows of the (small) batch per pass over the weights.
#include "ds41_b200.h"
#include "host_error.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace ds41 {
namespace {

constexpr int kF32Threads = 256, kF32Warps = kF32Threads / 32, kF32RowsPerWarp = 2;

template <int M>
__global__ void __launch_bounds__(kF32Threads) head_f32_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                               float *__restrict__ y, int N, int K) {
  extern __shared__ __align__(16) float xs[];  // [M][K]
  for (int i = threadIdx.x * 4; i < M * K; i += kF32Threads * 4)
    *reinterpret_cast<float4 *>(xs + i) = __ldg(reinterpret_cast<const float4 *>(x + i));
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = (N + kF32RowsPerWarp - 1) / kF32RowsPerWarp;
  for (int g = blockIdx.x * kF32Warps + warp; g < groups; g += gridDim.x * kF32Warps) {
    const int row0 = g * kF32RowsPerWarp;
    float acc[kF32RowsPerWarp][M];
#pragma unroll
    for (int r = 0; r < kF32RowsPerWarp; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    const float4 *wr[kF32RowsPerWarp];
#pragma unroll
    for (int r = 0; r < kF32RowsPerWarp; ++r)
      wr[r] = reinterpret_cast<const float4 *>(w + size_t(min(row0 + r, N - 1)) * K);  // rows beyond N repeat the last one
    // two 16-byte loads per row in flight ahead of the one being consumed
    float4 cur[kF32RowsPerWarp], nxt[kF32RowsPerWarp];
#pragma unroll
    for (int r = 0; r < kF32RowsPerWarp; ++r) {
      cur[r] = __ldg(wr[r] + lane);
      nxt[r] = 128 < K ? __ldg(wr[r] + lane + 32) : cur[r];
    }
    for (int k = lane * 4; k < K; k += 128) {
      float4 far[kF32RowsPerWarp];
      const bool more = k + 256 < K;
#pragma unroll
      for (int r = 0; r < kF32RowsPerWarp; ++r) far[r] = more ? __ldg(wr[r] + ((k + 256) >> 2)) : nxt[r];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 a = *reinterpret_cast<const float4 *>(xs + m * K + k);
#pragma unroll
        for (int r = 0; r < kF32RowsPerWarp; ++r) {
          acc[r][m] = __fmaf_rn(cur[r].x, a.x, acc[r][m]);
          acc[r][m] = __fmaf_rn(cur[r].y, a.y, acc[r][m]);
          acc[r][m] = __fmaf_rn(cur[r].z, a.z, acc[r][m]);
          acc[r][m] = __fmaf_rn(cur[r].w, a.w, acc[r][m]);
        }
      }
#pragma unroll
      for (int r = 0; r < kF32RowsPerWarp; ++r) { cur[r] = nxt[r]; nxt[r] = far[r]; }
    }
#pragma unroll
    for (int r = 0; r < kF32RowsPerWarp; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float sum = acc[r][m];
#pragma unroll
        for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
        if (lane == 0 && row0 + r < N) y[size_t(m) * N + row0 + r] = sum;
      }
  }
}

template <int M>
cudaError_t launch_f32(const float *x, const float *w, float *y, int N, int K, cudaStream_t stream) {
  const size_t smem = size_t(M) * K * sizeof(float);
  static thread_local int configured = -1;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  if (configured != dev) {
    e = cudaFuncSetAttribute(head_f32_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured = dev;
  }
  const int per_sm = smem <= 56 * 1024 ? 4 : smem <= 100 * 1024 ? 2 : 1;
  const int groups = (N + kF32RowsPerWarp - 1) / kF32RowsPerWarp;
  int grid = sms * per_sm;
  if (grid > (groups + kF32Warps - 1) / kF32Warps) grid = (groups + kF32Warps - 1) / kF32Warps;
  head_f32_kernel<M><<<grid, kF32Threads, smem, stream>>>(x, w, y, N, K);
  return cudaGetLastError();
}

}  // namespace
}  // namespace ds41

using namespace ds41;

extern "C" int ds41_b200_head_f32(const float *x, const float *w, float *y, int M, int N, int K, cudaStream_t stream) {
  // M as the reference's own FP32 operators accept it (ds41_dense_f32: ops.cu:114); K in runs of 128 for the 16-byte loads
  if (!x || !w || !y || M < 1 || M > 8 || N < 1 || K < 128 || K % 128) return invalid("FP32 head arguments");
  if (size_t(M) * K * sizeof(float) > 224 * 1024) return invalid("FP32 head: M * K * 4 bytes must fit 224 KB of shared memory");
  if ((reinterpret_cast<uintptr_t>(w) & 15u) || (reinterpret_cast<uintptr_t>(x) & 15u))
    return invalid("FP32 head operands must be 16-byte aligned");
  cudaError_t e;
  switch (M) {
    case 1: e = launch_f32<1>(x, w, y, N, K, stream); break;
    case 2: e = launch_f32<2>(x, w, y, N, K, stream); break;
    case 3: e = launch_f32<3>(x, w, y, N, K, stream); break;
    case 4: e = launch_f32<4>(x, w, y, N, K, stream); break;
    case 5: e = launch_f32<5>(x, w, y, N, K, stream); break;
    case 6: e = launch_f32<6>(x, w, y, N, K, stream); break;
    case 7: e = launch_f32<7>(x, w, y, N, K, stream); break;
    default: e = launch_f32<8>(x, w, y, N, K, stream); break;
  }
  return int(e);
}
