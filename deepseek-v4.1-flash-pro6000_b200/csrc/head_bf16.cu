// ds41_fuse_head_decode for B200: the reference engine's BF16 head plugin symbol, same signature, same results bit for
// bit.  The reference kernels (components/fuse-head/src/head_half_tree.cu:7-21, head_half_tune.cu:7-22) fix the FP32
// arithmetic of out[m,n] = sum_k W[n,k] * x[m,k]: sixteen chains per output, chain l takes k = l, l+16, l+32, ... in
// ascending order with one fused multiply-add per term, then the chains are added by a four-level tree (distance 8, 4,
// 2, 1 over the chain index) and +0.f canonicalises a negative zero.  This kernel keeps exactly that order — every
// intermediate is the same FP32 number — and changes only how the bytes move: a persistent CTA keeps the M activation
// rows in shared memory, streams 64 weight rows x 256 K at a time through a double buffer with 16-byte cp.async copies
// (512 bytes contiguous per weight row and copy, against 32 bytes per half-warp step in the reference), and each thread runs
// the chains of two weight rows so that every activation load feeds two fused multiply-adds.
// HBM-bound: the BF16 weights, 2*N*K bytes (1.32 GB at N=129280, K=5120), are read exactly once.
#include "ds41_b200.h"
#include "host_error.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ds41 {
namespace {

constexpr int kRowsPerCta = 64, kChunkK = 256, kHeadBf16Threads = 16 * kRowsPerCta / 2;  // 512: two rows per thread
constexpr int kRowPitch = kChunkK * 2 + 32;  // bytes; the 32-byte skew keeps the two rows of a warp on different banks

template <int M>
__global__ void __launch_bounds__(kHeadBf16Threads) head_bf16_kernel(const float *x, const __nv_bfloat16 *w, float *y,
                                                                     int N, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  // activations chain-major: x[m][l + 16 j] at sx[(m * 16 + l) * pitch + j], so that a chain reads four consecutive
  // terms with one 16-byte load (the pitch of K/16 + 4 floats spreads the sixteen chains over the banks)
  float *sx = reinterpret_cast<float *>(smem);
  const int pitch = K / 16 + 4;
  unsigned char *sw = smem + size_t(M) * 16 * pitch * sizeof(float);             // [2][kRowsPerCta][kRowPitch]
  const int tid = threadIdx.x, lane = tid & 15, pair = tid >> 4;                 // rows pair and pair + 32 of the block
  for (int i = tid; i < M * K; i += kHeadBf16Threads) {
    const int m = i / K, k = i - m * K;
    sx[(m * 16 + (k & 15)) * pitch + (k >> 4)] = __ldg(x + i);
  }
  const int blocks = (N + kRowsPerCta - 1) / kRowsPerCta, chunks = K / kChunkK;
  auto stage = [&](int block, int chunk, int buf) {  // 64 rows x 512 bytes, 16 bytes per copy
    unsigned char *dst = sw + size_t(buf) * kRowsPerCta * kRowPitch;
    for (int i = tid; i < kRowsPerCta * (kChunkK * 2 / 16); i += kHeadBf16Threads) {
      const int r = i / (kChunkK * 2 / 16), c = i % (kChunkK * 2 / 16);
      const int row = block * kRowsPerCta + r;
      const uint32_t d = uint32_t(__cvta_generic_to_shared(dst + r * kRowPitch + c * 16));
      if (row < N) {
        const void *src = reinterpret_cast<const unsigned char *>(w + size_t(row) * K + size_t(chunk) * kChunkK) + c * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
      } else {
        *reinterpret_cast<uint4 *>(dst + r * kRowPitch + c * 16) = make_uint4(0u, 0u, 0u, 0u);  // the reference uses weight 0
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int buf = 0;
  if (int(blockIdx.x) < blocks) stage(blockIdx.x, 0, 0);
  for (int block = blockIdx.x; block < blocks; block += gridDim.x) {
    float acc0[M], acc1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
    for (int chunk = 0; chunk < chunks; ++chunk) {
      // next copy in flight while this chunk is consumed
      int nb = block, nc = chunk + 1;
      if (nc == chunks) { nb = block + gridDim.x; nc = 0; }
      if (nb < blocks) stage(nb, nc, buf ^ 1); else asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");
      __syncthreads();
      const unsigned char *rows = sw + size_t(buf) * kRowsPerCta * kRowPitch;
      const __nv_bfloat16 *w0 = reinterpret_cast<const __nv_bfloat16 *>(rows + pair * kRowPitch);
      const __nv_bfloat16 *w1 = reinterpret_cast<const __nv_bfloat16 *>(rows + (pair + kRowsPerCta / 2) * kRowPitch);
      const float *xs = sx + lane * pitch + chunk * (kChunkK / 16);  // this chain's terms of the chunk, row m at + m*16*pitch
#pragma unroll
      for (int q = 0; q < kChunkK / 64; ++q) {  // four terms of the chain per round, in ascending k
        float4 xv[M];
#pragma unroll
        for (int m = 0; m < M; ++m) xv[m] = *reinterpret_cast<const float4 *>(xs + size_t(m) * 16 * pitch + 4 * q);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int k = lane + 16 * (4 * q + t);
          const float a0 = __bfloat162float(w0[k]), a1 = __bfloat162float(w1[k]);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const float xt = t == 0 ? xv[m].x : t == 1 ? xv[m].y : t == 2 ? xv[m].z : xv[m].w;
            acc0[m] = __fmaf_rn(a0, xt, acc0[m]);
            acc1[m] = __fmaf_rn(a1, xt, acc1[m]);
          }
        }
      }
      __syncthreads();
      buf ^= 1;
    }
    const int row0 = block * kRowsPerCta + pair, row1 = row0 + kRowsPerCta / 2;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      for (int d = 8; d; d >>= 1) {
        acc0[m] = __fadd_rn(acc0[m], __shfl_down_sync(0xffffffffu, acc0[m], d, 16));
        acc1[m] = __fadd_rn(acc1[m], __shfl_down_sync(0xffffffffu, acc1[m], d, 16));
      }
      if (lane == 0 && row0 < N) y[size_t(m) * N + row0] = __fadd_rn(acc0[m], 0.f);
      if (lane == 0 && row1 < N) y[size_t(m) * N + row1] = __fadd_rn(acc1[m], 0.f);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int M>
cudaError_t launch_head_bf16(const float *x, const void *w, float *y, int N, int K, cudaStream_t stream) {
  const size_t smem = size_t(M) * (K + 64) * sizeof(float) + 2 * size_t(kRowsPerCta) * kRowPitch;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  static thread_local int configured = -1;
  if (configured != dev) {
    e = cudaFuncSetAttribute(head_bf16_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured = dev;
  }
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  const int blocks = (N + kRowsPerCta - 1) / kRowsPerCta;
  head_bf16_kernel<M><<<blocks < sms ? blocks : sms, kHeadBf16Threads, smem, stream>>>(
      x, static_cast<const __nv_bfloat16 *>(w), y, N, K);
  return cudaGetLastError();
}

}  // namespace
}  // namespace ds41

using namespace ds41;

// General shapes (the tests use small N); ds41_fuse_head_decode below is the reference's restricted entry point.
extern "C" int ds41_b200_head_bf16(const float *x, const void *weights_bf16, float *out, int M, int N, int K,
                                   cudaStream_t stream) {
  if (!x || !weights_bf16 || !out || M < 1 || M > 6 || N < 1 || K < kChunkK || K % kChunkK ||
      size_t(M) * (K + 64) * sizeof(float) + 2 * size_t(kRowsPerCta) * kRowPitch > 227 * 1024)
    return invalid("BF16 head arguments (1 <= M <= 6, K a multiple of 256, M*K*4 bytes of activations + 68 KB within 227 KB)");
  if ((reinterpret_cast<uintptr_t>(weights_bf16) & 15u)) return invalid("BF16 head: weights must be 16-byte aligned");
  cudaError_t e;
  switch (M) {
    case 1: e = launch_head_bf16<1>(x, weights_bf16, out, N, K, stream); break;
    case 2: e = launch_head_bf16<2>(x, weights_bf16, out, N, K, stream); break;
    case 3: e = launch_head_bf16<3>(x, weights_bf16, out, N, K, stream); break;
    case 4: e = launch_head_bf16<4>(x, weights_bf16, out, N, K, stream); break;
    case 5: e = launch_head_bf16<5>(x, weights_bf16, out, N, K, stream); break;
    default: e = launch_head_bf16<6>(x, weights_bf16, out, N, K, stream); break;
  }
  return int(e);
}

extern "C" int ds41_fuse_head_decode(const float *x, const void *weights_bf16, float *out, int M, int N, int K,
                                     cudaStream_t stream) {
  // the reference's own argument check (components/fuse-head/src/head_decode.cpp:6)
  if (!x || !weights_bf16 || !out || M < 1 || M > 6 || N != 129280 || K != 5120) return int(cudaErrorInvalidValue);
  return ds41_b200_head_bf16(x, weights_bf16, out, M, N, K, stream);
}
