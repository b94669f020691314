// FP8 LM head for sm_100a: logits[m, n] = sum over 128-wide K blocks of a_scale[m, kb] * w_scale[n/128, kb] *
// dot(a_e4m3[m, kb], w_e4m3[n, kb]).
//
// The reference's head is a BF16 GEMV (components/fuse-head/src/head_half_tune.cu:7-21) and its only FP8 GEMM is
// ds41_dense_fp8 for the dense projections (components/dense/src/dense.cu:25-91, UE8M0 scales per 32x32 block).
// This operator is new: e4m3 weights with one fp32 scale per 128x128 block, activations quantised per (row, 128-K
// group) by the reference's power-of-two rule (dense.cu:8-16) widened to the weight block.  It keeps the plugin
// conventions of fuse_head.h:8 (caller-owned buffers, stream-ordered, no allocation, no synchronisation).
//
// Kernel shape: an output tile is kRows batch rows x 128 vocabulary ids.  The batch rows are the M dimension of
// tcgen05.mma (one TMEM lane per batch row; M is always 128, the activation tile holds kRows = 16..128 real rows and
// the lanes beyond them are never read), the 128 vocabulary rows of a weight tile are its N dimension (128 TMEM
// columns).  With this orientation the combined scale a_scale[m,kb] * w_scale[n/128,kb] of a K block is ONE number
// per epilogue thread (its batch row; the weight block is the whole tile), so the fp32 promotion of a K block is a
// register-only loop of fused multiply-adds.  Per CTA: warp 0 streams W and A tiles with TMA (128-byte swizzle) into
// a ring of shared-memory stages, warp 1 issues four K=32 tcgen05.mma per 128-wide K block into one of four TMEM
// accumulators, sixteen epilogue warps (lane quadrant x 32-column group) pull each finished K block out of TMEM
// (tcgen05.ld), hand the accumulator back at once, scale and add in fp32 registers.
// Every wait is bounded; on expiry the kernel raises *error_flag, frees its TMEM and returns.
#include "ds41_b200.h"
#include "flat.cuh"
#include "host_error.h"
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdlib.h>

namespace ds41 {
namespace {

constexpr int kTmemColumns = 512;  // all of an SM's tensor memory: 4 accumulators of 128 columns or 2 of 256
constexpr int kTileK = 128;   // K elements per block = one 128-byte swizzle row of e4m3
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

struct Abort {  // shared flag: once set every later wait returns immediately
  volatile int *flag;
  __device__ __forceinline__ bool set() const { return *flag != 0; }
};

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait on a phase parity.  Returns false (and raises the abort flag) if the phase never completed.  The first
// probe carries no other work: the single threads that issue the copies and the MMAs call this once or twice per K
// block, and every instruction on their path delays the tensor pipe.
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, volatile int *flag) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 255u) == 255u && *flag != 0) return false;
  }
  *flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, const Abort &ab) {
  if (mbar_try(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ab.flag);
}

// Box {128 bytes, rows, K blocks} of the operand seen as [K/128][rows][128 bytes] (see make_map).
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int row, int kb) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
          "r"(smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(x), "r"(row), "r"(kb)
      : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows are 128 bytes apart, groups of 8 rows 1024 bytes
// apart (stride byte offset), leading byte offset unused (1), descriptor version 1 for sm_100.
constexpr uint64_t kDescFixed = (uint64_t(1) << 16)              // leading byte offset (>>4), bits [16,30)
                                | (uint64_t(1024 >> 4) << 32)    // stride byte offset (>>4), bits [32,46)
                                | (uint64_t(1) << 46)            // version, bits [46,48)
                                | (uint64_t(2) << 61);           // layout type SWIZZLE_128B, bits [61,64)
// addr16 = shared-memory byte address >> 4 (start address field, bits [0,14); shared memory ends below 2^18 bytes)
__device__ __forceinline__ uint64_t umma_desc16(uint32_t addr16) { return kDescFixed | uint64_t(addr16); }
// Instruction descriptor for kind::f8f6f4, E4M3 x E4M3 -> F32, both operands K-major, M=128, N=n_cols.
__host__ __device__ constexpr uint32_t umma_idesc(int n_cols) {
  return (1u << 4) | (uint32_t(n_cols >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}
template <bool kAccumulate>
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Two fp32 fused multiply-adds in one instruction (fma.rn.f32x2: each half is the same correctly rounded FMA as
// fmaf): the promotion of a K block is 32 or 64 of them per thread, and the epilogue warps' issue slots are what the
// tensor pipe ends up waiting for.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void fma2_acc(float &s0, float &s1, uint32_t d0, uint32_t d1, unsigned long long scale2) {
  unsigned long long d, c, out;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(d0), "r"(d1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(s0), "f"(s1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(out) : "l"(d), "l"(scale2), "l"(c));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(out));
}

// kRows batch rows x kVocab vocabulary ids per output tile (kVocab = UMMA N: 128, or 256 to halve the activation
// traffic per output element when the batch is large and the kernel is bound by L2 -> shared-memory copies)
template <int kRows, int kVocab>
struct HeadSmem {
  static constexpr int kAccBufs = kTmemColumns / kVocab;
  static constexpr int kStageBytes = kVocab * kTileK + kRows * kTileK;
  // the MMA reads 128 activation rows from every stage; with kRows < 128 the rows beyond the tile belong to the next
  // stage (or to the pad after the last one) and only feed TMEM lanes nobody reads
  static constexpr int kPadBytes = (128 - kRows) * kTileK;
  static constexpr int kMaxStages = 12;
  // bytes beside the stages: alignment slack, pad, scale table [K/128][kRows], barriers and flags
  static constexpr size_t fixed_bytes(int kblocks) {
    return 1024 + kPadBytes + size_t(kblocks) * kRows * 4 + (2 * kMaxStages + 2 * kAccBufs) * 8 + 16;
  }
  // a stage holds `group` consecutive K blocks (one TMA box per operand)
  static constexpr int stages(int kblocks, int group) {
    const long long room = 226 * 1024 - (long long)fixed_bytes(kblocks);
    const int n = room < 0 ? 0 : int(room / (kStageBytes * group));
    return n > kMaxStages ? kMaxStages : n;
  }
};

constexpr int kMaxOwners = 8;
constexpr int kEpiWarps = 16, kHeadThreads = 64 + 32 * kEpiWarps;
struct HeadArgs {
  const float *a_scale;  // [M, K/128]
  const float *w_scale;  // [ceil(N/128), K/128]
  float *logits;         // [M, ldl]
  long long ldl;
  int M, N, K;
  int *error_flag;       // device word, raised on a wait timeout (may be null)
  // Row-scattered output (vocabulary-sharded head): batch row m goes to owner m / rows_per_owner, into
  // owner_base[owner] + (m % rows_per_owner) * ldl + col_offset + n.  The bases may be peer GPUs' memory; the epilogue
  // writes them with plain stores, so the vocabulary-to-row transposition rides on the GEMM.  rows_per_owner == 0: off.
  float *owner_base[kMaxOwners];
  int rows_per_owner, col_offset;
  // Optional per-row statistics for the sampler (zero-initialised by the host): every epilogue thread keeps the first
  // maximum, the minimum and a finiteness flag of the logits it produces for its batch row and merges them with atomic
  // maxima when it leaves the row, so the sampler's own pass over the logits for these three numbers can be skipped.
  HeadRowStats *row_stats;
  // The same records in the row-scattered variant: row m's record lies owner_stats_offset bytes behind owner_base[owner]
  // at index m % rows_per_owner (0: none).  Several GPUs merge into one record, so those atomics have system scope.
  long long owner_stats_offset;
  int stages;            // shared-memory stages of the TMA ring (host: HeadSmem::stages)
  int group;             // K blocks per stage: every row of a weight tile is fetched as group*128 contiguous bytes
};

template <int kRows, int kVocab>
__global__ void __launch_bounds__(kHeadThreads, 1)
head_fp8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, HeadArgs p) {
  using Smem = HeadSmem<kRows, kVocab>;
  constexpr int kTileN = kVocab, kAccBufs = Smem::kAccBufs;
  constexpr int kStageBytes = Smem::kStageBytes;
  constexpr int kMaxStages = Smem::kMaxStages;
  const int kStages = p.stages, group = p.group;
  const int stage_bytes = kStageBytes * group, w_bytes = kTileN * kTileK * group;  // [W g0..][A g0..]
  constexpr uint32_t kTmemCols = kTmemColumns;
  constexpr int kQuads = (kRows + 31) / 32;          // lane quadrants that hold real batch rows
  constexpr int kGroups = 4, kMyCols = kTileN / kGroups;  // 32- or 64-column groups: warp (quadrant q, group g)
  constexpr int kEpiActive = 32 * kQuads * kGroups;  // epilogue threads that take part
  extern __shared__ __align__(1024) unsigned char smem[];
  // carve: [stages][W tile 16 KB | A tile kRows*128 B], pad, then the activation-scale table, then barriers
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  float *sa = reinterpret_cast<float *>(tiles + size_t(kStages) * stage_bytes + Smem::kPadBytes);  // [K/128][kRows]
  const int kblocks = p.K / kTileK;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sa + size_t(kblocks) * kRows);
  uint64_t *full = bars, *empty = bars + kMaxStages, *acc_full = bars + 2 * kMaxStages, *acc_empty = acc_full + kAccBufs;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + kAccBufs);
  int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + kTileN - 1) / kTileN, b_tiles = (p.M + kRows - 1) / kRows;
  const int total_tiles = n_tiles * b_tiles;  // tile t = (vocabulary tile t / b_tiles, batch tile t % b_tiles)
  Abort ab{abort_word};

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < kAccBufs; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kQuads * kGroups); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM allocation by one full warp; the address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !ab.set(); tile += gridDim.x) {
        const int nt = tile / b_tiles, bt = tile % b_tiles;
        for (int kb = 0; kb < kblocks; kb += group) {
          if (!mbar_wait(&empty[stage], phase ^ 1, ab)) break;
          unsigned char *w_dst = tiles + size_t(stage) * stage_bytes, *a_dst = w_dst + w_bytes;
          mbar_expect_tx(&full[stage], uint32_t(stage_bytes));
          tma_load_3d(w_dst, &map_w, &full[stage], 0, nt * kTileN, kb);
          tma_load_3d(a_dst, &map_a, &full[stage], 0, bt * kRows, kb);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kTileN);
      const uint32_t tiles16 = smem_addr(tiles) >> 4, stage16 = uint32_t(stage_bytes) >> 4;
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !ab.set(); tile += gridDim.x) {
        bool ok = true;
        for (int kb = 0; kb < kblocks && ok; kb += group) {
          if (!mbar_wait(&full[stage], phase, ab)) break;
          uint32_t w16 = tiles16 + stage * stage16, a16 = w16 + (w_bytes >> 4);  // addresses >> 4
          for (int g = 0; g < group; ++g) {
            if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, ab)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d_addr = tmem_base + acc * kTileN;
            // D[batch row, vocabulary id] (+)= A[batch row, k] * W[vocabulary id, k], K = 32 bytes per instruction
            umma_f8<false>(d_addr, umma_desc16(a16), umma_desc16(w16), idesc);
            umma_f8<true>(d_addr, umma_desc16(a16 + 2), umma_desc16(w16 + 2), idesc);
            umma_f8<true>(d_addr, umma_desc16(a16 + 4), umma_desc16(w16 + 4), idesc);
            umma_f8<true>(d_addr, umma_desc16(a16 + 6), umma_desc16(w16 + 6), idesc);
            umma_commit(&acc_full[acc]);   // accumulator of this K block is complete
            if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
            w16 += (kTileN * kTileK) >> 4; a16 += (kRows * kTileK) >> 4;
          }
          if (ok) umma_commit(&empty[stage]);  // the stage may be refilled once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if ((warp & 3) < kQuads) {
    // ------------------------------------------------------------------ epilogue: warp = (lane quadrant, column group)
    const int quad = warp & 3;          // TMEM lanes [32*quad, 32*quad+32) are readable by this warp: batch rows
    const int group = (warp - 2) >> 2;  // vocabulary ids [32*group, 32*group+32) of the tile
    const int row = quad * 32 + lane;   // batch row inside the tile
    const int et = (group * kQuads + quad) * 32 + lane;  // 0..kEpiActive-1
    const uint32_t lane_base = tmem_base + group * kMyCols + (uint32_t(quad * 32) << 16);
    uint32_t acc = 0, acc_phase = 0;
    int table_bt = -1;
    bool alive = true;  // warp-uniform; once false the remaining tiles are walked without waiting or computing,
                        // so that all epilogue threads still meet at every named barrier
    // running statistics of this thread's batch row over the tiles of one batch tile (vocabulary tiles come in
    // ascending order, so a strict comparison keeps the first maximum)
    float st_best = -CUDART_INF_F, st_low = CUDART_INF_F, st_bad = 0.f;
    int st_id = 0x7fffffff;
    const bool stats_on = p.row_stats != nullptr || p.owner_stats_offset != 0;
    auto flush_stats = [&](int bt_of) {
      const int m = bt_of * kRows + row;
      if (stats_on && st_id != 0x7fffffff && row < kRows && m < p.M) {
        auto ordered = [](float v) {
          const uint32_t bits = __float_as_uint(v == 0.f ? 0.f : v);  // -0 and +0 are the same logit
          return bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
        };
        const unsigned long long key = (unsigned long long)(ordered(st_best)) << 32 |
                                       (0xffffffffu - uint32_t(st_id + p.col_offset));
        if (p.owner_stats_offset) {
          const int owner = m / p.rows_per_owner;
          HeadRowStats *rs = reinterpret_cast<HeadRowStats *>(reinterpret_cast<unsigned char *>(p.owner_base[owner]) +
                                                              p.owner_stats_offset) + (m - owner * p.rows_per_owner);
          atomicMax_system(&rs->max_key, key);
          atomicMax_system(&rs->min_key, ~ordered(st_low));
          if (st_bad != st_bad) atomicOr_system(&rs->flags, 1u);
        } else {
          HeadRowStats *rs = p.row_stats + m;
          atomicMax(&rs->max_key, key);
          atomicMax(&rs->min_key, ~ordered(st_low));
          if (st_bad != st_bad) atomicOr(&rs->flags, 1u);
        }
      }
      st_best = -CUDART_INF_F; st_low = CUDART_INF_F; st_bad = 0.f; st_id = 0x7fffffff;
    };
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int nt = tile / b_tiles, bt = tile % b_tiles;
      if (bt != table_bt) {  // activation scales of this batch tile: sa[kb][row] (a grid that is a multiple of b_tiles
                             // keeps bt fixed per CTA, so this normally happens once)
        if (table_bt >= 0) flush_stats(table_bt);
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiActive) : "memory");  // readers of the previous table are done
        for (int i = et; i < kblocks * kRows; i += kEpiActive) {
          const int r = i / kblocks, kb = i % kblocks, m = bt * kRows + r;
          sa[kb * kRows + r] = m < p.M ? __ldg(p.a_scale + size_t(m) * kblocks + kb) : 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiActive) : "memory");
        table_bt = bt;
      }
      // fp32 scale of the 128-row weight block this warp's columns belong to (a 256-wide tile spans two blocks)
      const int w_block = min((nt * kTileN + group * kMyCols) / 128, (p.N + 127) / 128 - 1);
      const float *wsc = p.w_scale + size_t(w_block) * kblocks;
      float sum[kMyCols];
#pragma unroll
      for (int c = 0; c < kMyCols; ++c) sum[c] = 0.f;
      float w_next = __ldg(wsc);
      for (int kb = 0; kb < kblocks && alive; ++kb) {
        alive = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], acc_phase, ab));
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float scale = sa[kb * kRows + (row < kRows ? row : 0)] * w_next;
        const unsigned long long scale2 = pack2(scale, scale);
        if (kb + 1 < kblocks) w_next = __ldg(wsc + kb + 1);
        if constexpr (kMyCols == 32) {
          uint32_t r[32];
          tmem_ld32(lane_base + acc * kTileN, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          // the values are in registers: the accumulator can be refilled while they are scaled and added
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[acc]);
#pragma unroll
          for (int c = 0; c < 32; c += 2) fma2_acc(sum[c], sum[c + 1], r[c], r[c + 1], scale2);
        } else {
          // 64 columns per thread: four 16-column loads, one in flight at a time (what the registers of 576 threads leave room for)
#pragma unroll
          for (int c0 = 0; c0 < kMyCols; c0 += 16) {
            uint32_t r[32];
            tmem_ld16(lane_base + acc * kTileN + c0, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (c0 + 16 == kMyCols) {
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[acc]);
            }
#pragma unroll
            for (int c = 0; c < 16; c += 2) fma2_acc(sum[c0 + c], sum[c0 + c + 1], r[c], r[c + 1], scale2);
          }
        }
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
      }
      // Output.  Lane l holds row l of the warp's 32 x 32 block.  Written as it is, one store instruction would touch
      // 32 rows with 16 bytes each; an 8 x 8 transpose of the 16-byte column groups across the lanes that share
      // l % 4 (butterflies at lane distances 4, 8, 16) turns that into 4 rows with 128 contiguous bytes each, which is
      // what a peer GPU's memory wants to be written with (and the local L2 as well).
      if (alive && stats_on) {
        const int n0 = nt * kTileN + group * kMyCols;
        if (n0 + kMyCols <= p.N) {
#pragma unroll
          for (int c = 0; c < kMyCols; ++c) {
            const float v = sum[c];
            st_bad = fmaf(v, 0.f, st_bad);  // NaN once any logit is NaN or infinite
            if (v > st_best) { st_best = v; st_id = n0 + c; }
            st_low = fminf(st_low, v);
          }
        } else {
#pragma unroll
          for (int c = 0; c < kMyCols; ++c) {
            const float v = sum[c];
            if (n0 + c < p.N) {
              st_bad = fmaf(v, 0.f, st_bad);
              if (v > st_best) { st_best = v; st_id = n0 + c; }
              st_low = fminf(st_low, v);
            }
          }
        }
      }
      if (alive) {
#pragma unroll
       for (int half = 0; half < kMyCols / 32; ++half) {
        float4 x[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          x[c] = make_float4(sum[32 * half + 4 * c], sum[32 * half + 4 * c + 1], sum[32 * half + 4 * c + 2], sum[32 * half + 4 * c + 3]);
#pragma unroll
        for (int s3 = 0; s3 < 3; ++s3) {
          const int dist = 4 << s3;
          const bool upper = (lane >> (2 + s3)) & 1;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if ((c >> s3) & 1) continue;
            const int c2 = c | (1 << s3);
            const float4 give = upper ? x[c] : x[c2];
            float4 take;
            take.x = __shfl_xor_sync(0xffffffffu, give.x, dist);
            take.y = __shfl_xor_sync(0xffffffffu, give.y, dist);
            take.z = __shfl_xor_sync(0xffffffffu, give.z, dist);
            take.w = __shfl_xor_sync(0xffffffffu, give.w, dist);
            if (upper) x[c] = take; else x[c2] = take;
          }
        }
        // now x[a] = columns [4*(lane/4), +4) of block row 4*a + lane%4
        const int n = nt * kTileN + group * kMyCols + 32 * half + 4 * (lane >> 2);
#pragma unroll
        for (int a8 = 0; a8 < 8; ++a8) {
          const int r = quad * 32 + 4 * a8 + (lane & 3), m = bt * kRows + r;
          if (r >= kRows || m >= p.M || n >= p.N) continue;
          float *dst;
          if (p.rows_per_owner == 0) {
            dst = p.logits + size_t(m) * p.ldl + n;
          } else {
            const int owner = m / p.rows_per_owner;
            dst = p.owner_base[owner] + size_t(m - owner * p.rows_per_owner) * p.ldl + p.col_offset + n;
          }
          if (n + 4 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<float4 *>(dst) = x[a8];
          } else {
            const float v[4] = {x[a8].x, x[a8].y, x[a8].z, x[a8].w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (n + k < p.N) dst[k] = v[k];
          }
        }
       }
      }
    }
    if (alive && table_bt >= 0) flush_stats(table_bt);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
  if (threadIdx.x == 0 && *abort_word && p.error_flag) atomicExch(p.error_flag, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// Activation quantisation: per (row, 128-wide K group) scale = 2^ceil(log2(max(amax,1e-4)/448)), e4m3 round to
// nearest even with saturation (components/dense/src/dense.cu:8-16 with the group widened from 32 to 128).
__global__ void quantize_kernel(const __nv_bfloat16 *x, uint8_t *a, float *scale, int groups) {
  const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (g >= groups) return;
  const uint2 raw = *reinterpret_cast<const uint2 *>(x + size_t(g) * 128 + lane * 4);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
  float v[4] = {__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const uint32_t bits = __float_as_uint(__fmul_rn(fmaxf(amax, 1e-4f), 1.f / 448.f));
  const uint32_t exponent = (bits >> 23) + ((bits & 0x7fffffu) != 0);
  const float s = __uint_as_float(exponent << 23);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float q = fminf(448.f, fmaxf(-448.f, __fdiv_rn(v[i], s)));
    packed |= uint32_t(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  }
  *reinterpret_cast<uint32_t *>(a + size_t(g) * 128 + lane * 4) = packed;
  if (lane == 0) scale[g] = s;
}

// ---------------------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encoder() {
  static EncodeFn fn = [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}
// uint8 matrix [rows, cols] row-major seen as a 3-D tensor [cols/128][rows][128 bytes] (strides 128 and cols bytes),
// box {128 bytes, box_rows, group}: one copy brings `group` consecutive K blocks of box_rows rows, laid out in shared
// memory as `group` K-major tiles of box_rows x 128 bytes with the 128-byte swizzle, and reads every row of the matrix
// in runs of group*128 contiguous bytes.  Zero fill outside.
bool make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t group) {
  EncodeFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {uint64_t(kTileK), rows, cols / kTileK};
  const cuuint64_t strides[2] = {cols, uint64_t(kTileK)};
  const cuuint32_t box[3] = {uint32_t(kTileK), box_rows, group};
  const cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int kRows, int kVocab>
cudaError_t launch_head(const CUtensorMap &mw, const CUtensorMap &ma, const HeadArgs &p, int sms, cudaStream_t stream) {
  using Smem = HeadSmem<kRows, kVocab>;
  const int stages = Smem::stages(p.K / kTileK, p.group);
  if (stages < 2) return cudaErrorInvalidValue;
  const size_t smem = Smem::fixed_bytes(p.K / kTileK) + size_t(stages) * Smem::kStageBytes * p.group;
  HeadArgs q = p;
  q.stages = stages;
  static thread_local int configured = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (configured != dev) {
    e = cudaFuncSetAttribute(head_fp8_kernel<kRows, kVocab>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured = dev;
  }
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  const int b_tiles = (p.M + kRows - 1) / kRows;
  const int tiles = ((p.N + kVocab - 1) / kVocab) * b_tiles;
  int grid = tiles < sms ? tiles : sms;
  if (b_tiles <= grid) grid -= grid % b_tiles;  // every CTA then keeps one batch tile (and its scale table) for good
  head_fp8_kernel<kRows, kVocab><<<grid, kHeadThreads, smem, stream>>>(mw, ma, q);
  return cudaGetLastError();
}

}  // namespace
}  // namespace ds41

using namespace ds41;

extern "C" int ds41_b200_quantize_activations(const void *x_bf16, void *a_e4m3, float *a_scale, int M, int K,
                                              cudaStream_t stream) {
  if (!x_bf16 || !a_e4m3 || !a_scale || M < 1 || K < 128 || K % 128) return invalid("quantize arguments");
  const int groups = M * (K / 128);
  quantize_kernel<<<(groups * 32 + 255) / 256, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x_bf16),
                                                                 static_cast<uint8_t *>(a_e4m3), a_scale, groups);
  return int(cudaGetLastError());
}

namespace {
int run_head(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale, HeadArgs p,
             cudaStream_t stream);
}

extern "C" int ds41_b200_head_fp8(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                                  float *logits, int64_t logits_stride, int M, int N, int K, int *error_flag,
                                  cudaStream_t stream) {
  if (!a_e4m3 || !a_scale || !w_e4m3 || !w_scale || !logits || M < 1 || N < 1 || K < 128 || K % 128 || K > 16384 ||
      logits_stride < N)
    return invalid("head arguments");
  HeadArgs p{};
  p.a_scale = a_scale; p.w_scale = w_scale; p.logits = logits; p.ldl = logits_stride;
  p.M = M; p.N = N; p.K = K; p.error_flag = error_flag;
  return run_head(a_e4m3, a_scale, w_e4m3, w_scale, p, stream);
}

extern "C" int ds41_b200_head_fp8_stats(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                                        float *logits, int64_t logits_stride, int M, int N, int K, void *row_extremes,
                                        int *error_flag, cudaStream_t stream) {
  if (!a_e4m3 || !a_scale || !w_e4m3 || !w_scale || !logits || M < 1 || N < 1 || K < 128 || K % 128 || K > 16384 ||
      logits_stride < N || !row_extremes || (reinterpret_cast<uintptr_t>(row_extremes) & 15u))
    return invalid("head arguments");
  static_assert(sizeof(HeadRowStats) == DS41_B200_ROW_EXTREMES_BYTES, "row record size");
  cudaError_t e = cudaMemsetAsync(row_extremes, 0, size_t(M) * sizeof(HeadRowStats), stream);
  if (e != cudaSuccess) return int(e);
  HeadArgs p{};
  p.a_scale = a_scale; p.w_scale = w_scale; p.logits = logits; p.ldl = logits_stride;
  p.M = M; p.N = N; p.K = K; p.error_flag = error_flag;
  p.row_stats = static_cast<HeadRowStats *>(row_extremes);
  return run_head(a_e4m3, a_scale, w_e4m3, w_scale, p, stream);
}

extern "C" int ds41_b200_head_fp8_scatter_stats(const void *a_e4m3, const float *a_scale, const void *w_e4m3,
                                                const float *w_scale, float *const *owner_logits, int owners,
                                                int rows_per_owner, int64_t logits_stride, int vocab_offset, int M,
                                                int N, int K, int64_t stats_offset_bytes, int *error_flag,
                                                cudaStream_t stream);

extern "C" int ds41_b200_head_fp8_scatter(const void *a_e4m3, const float *a_scale, const void *w_e4m3,
                                          const float *w_scale, float *const *owner_logits, int owners,
                                          int rows_per_owner, int64_t logits_stride, int vocab_offset, int M, int N,
                                          int K, int *error_flag, cudaStream_t stream) {
  return ds41_b200_head_fp8_scatter_stats(a_e4m3, a_scale, w_e4m3, w_scale, owner_logits, owners, rows_per_owner,
                                          logits_stride, vocab_offset, M, N, K, 0, error_flag, stream);
}

extern "C" int ds41_b200_head_fp8_scatter_stats(const void *a_e4m3, const float *a_scale, const void *w_e4m3,
                                                const float *w_scale, float *const *owner_logits, int owners,
                                                int rows_per_owner, int64_t logits_stride, int vocab_offset, int M,
                                                int N, int K, int64_t stats_offset_bytes, int *error_flag,
                                                cudaStream_t stream) {
  if (stats_offset_bytes < 0 || (stats_offset_bytes & 15) ||
      (stats_offset_bytes && stats_offset_bytes < int64_t(rows_per_owner) * logits_stride * 4))
    return invalid("scattered head: the row records must lie behind the owner's logits, 16-byte aligned");
  if (!a_e4m3 || !a_scale || !w_e4m3 || !w_scale || !owner_logits || M < 1 || N < 1 || K < 128 || K % 128 ||
      K > 16384 || owners < 1 || owners > kMaxOwners || rows_per_owner < 1 || vocab_offset < 0 ||
      logits_stride < int64_t(vocab_offset) + N || int64_t(owners) * rows_per_owner < M)
    return invalid("scattered head arguments");
  HeadArgs p{};
  p.a_scale = a_scale; p.w_scale = w_scale; p.logits = nullptr; p.ldl = logits_stride;
  p.M = M; p.N = N; p.K = K; p.error_flag = error_flag;
  p.rows_per_owner = rows_per_owner; p.col_offset = vocab_offset;
  p.owner_stats_offset = stats_offset_bytes;
  for (int r = 0; r < owners; ++r) {
    if (!owner_logits[r] && int64_t(r) * rows_per_owner < M) return invalid("scattered head: null owner buffer");
    p.owner_base[r] = owner_logits[r];
  }
  return run_head(a_e4m3, a_scale, w_e4m3, w_scale, p, stream);
}

namespace {
int run_head(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale, HeadArgs p,
             cudaStream_t stream) {
  (void)a_scale; (void)w_scale;
  const int M = p.M, N = p.N, K = p.K;
  if ((reinterpret_cast<uintptr_t>(a_e4m3) & 15u) || (reinterpret_cast<uintptr_t>(w_e4m3) & 15u))
    return invalid("head operands must be 16-byte aligned");
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return int(e);
  const int cols = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  // Vocabulary tile: 256 wide once the batch spans several tiles (then the kernel is bound by L2 -> shared-memory
  // copies and a wider tile re-reads the activations half as often), else 128.
  const int vocab_tile = (M > 128 && N >= 256) ? 256 : 128;
  // K blocks per stage: the largest of 4, 2, 1 that divides K/128 and still leaves a ring of at least 2 stages
  // (measured: longer contiguous runs per weight row beat a deeper ring of shorter ones)
  const int kblocks = K / kTileK;
  auto ring = [&](int g) {
    return vocab_tile == 256 ? HeadSmem<128, 256>::stages(kblocks, g)
         : cols == 16 ? HeadSmem<16, 128>::stages(kblocks, g) : cols == 32 ? HeadSmem<32, 128>::stages(kblocks, g)
         : cols == 64 ? HeadSmem<64, 128>::stages(kblocks, g) : HeadSmem<128, 128>::stages(kblocks, g);
  };
  int group = 1;
  for (int g = 4; g > 1; g >>= 1)
    if (kblocks % g == 0 && ring(g) >= 2) { group = g; break; }
  if (const char *forced = getenv("DS41_HEAD_GROUP")) {
    const int g = atoi(forced);
    if ((g == 1 || g == 2 || g == 4) && kblocks % g == 0 && ring(g) >= 2) group = g;
  }
  p.group = group;
  CUtensorMap mw, ma;
  if (!make_map(&mw, w_e4m3, uint64_t(N), uint64_t(K), uint32_t(vocab_tile), uint32_t(group)) ||
      !make_map(&ma, a_e4m3, uint64_t(M), uint64_t(K), uint32_t(cols), uint32_t(group)))
    return invalid("cuTensorMapEncodeTiled failed");
  if (vocab_tile == 256) return int(launch_head<128, 256>(mw, ma, p, sms, stream));
  switch (cols) {
    case 16: e = launch_head<16, 128>(mw, ma, p, sms, stream); break;
    case 32: e = launch_head<32, 128>(mw, ma, p, sms, stream); break;
    case 64: e = launch_head<64, 128>(mw, ma, p, sms, stream); break;
    default: e = launch_head<128, 128>(mw, ma, p, sms, stream); break;
  }
  return int(e);
}
}  // namespace

extern "C" size_t ds41_fuse_head_fp8_workspace_bytes(int M, int K) {
  if (M < 1 || K < 128 || K % 128) return 0;
  return ((size_t(M) * K + 255) & ~size_t(255)) + size_t(M) * (K / 128) * sizeof(float);
}

extern "C" int ds41_fuse_head_fp8(const void *x_bf16, const void *w_e4m3, const float *w_scale, float *logits, int M,
                                  int N, int K, void *workspace, size_t workspace_bytes, int *error_flag,
                                  cudaStream_t stream) {
  const size_t need = ds41_fuse_head_fp8_workspace_bytes(M, K);
  if (!need || !workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return invalid("head workspace too small or misaligned");
  uint8_t *a = static_cast<uint8_t *>(workspace);
  float *a_scale = reinterpret_cast<float *>(a + ((size_t(M) * K + 255) & ~size_t(255)));
  int rc = ds41_b200_quantize_activations(x_bf16, a, a_scale, M, K, stream);
  if (rc) return rc;
  return ds41_b200_head_fp8(a, a_scale, w_e4m3, w_scale, logits, N, M, N, K, error_flag, stream);
}
