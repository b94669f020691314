// Row machinery shared by the sampler and the speculative verifier.
//
// One thread-block CLUSTER owns one logits row.  Each CTA of the cluster stages a contiguous slice of the row in
// shared memory with a single bulk asynchronous copy (TMA 1-D), so HBM is read exactly once and every later pass
// (penalties/mask, maximum, sum of exponentials, top-k / top-p cut search, inverse-CDF draw) runs out of shared
// memory.  CTAs exchange their partial results through distributed shared memory.
//
// What is reproduced is the reference's host rule (engine/third_party/spark/src/sampling.cpp:18-21,30-38 behind
// engine/src/sampling.cpp:205-226): first-maximum argmax, p_i = exp((double(x_i)-double(x_b))/T), normaliser in
// FP64, top-p = minimal prefix of the stable descending order (ties keep the lower id), inverse CDF in id order.
// The reference sums sequentially; a parallel sum differs in the low bits, so every DECISION made here (is this id
// inside the nucleus, which id does the uniform select, accept or reject) is taken together with a rigorous bound
// on the difference, and the row's status word says whether the decision is certified (see ds41_b200.h).
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace ds41 {

namespace cg = cooperative_groups;

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kSliceCap = 16384;   // fp32 logits staged per CTA
constexpr int kMaxCluster = 8;     // portable cluster size
constexpr int kBins = 1024;        // histogram bins per search level
constexpr int kListCap = 1024;     // candidates resolved exactly (sorted) at the cut
constexpr int kMaxLevels = 6;
constexpr double kU = 1.1102230246251565e-16;  // 2^-53, unit roundoff of FP64
constexpr double kFix = 70368744177664.0;      // 2^46: fixed-point scale of the histogram masses

// ---------------------------------------------------------------------------------------------------------------
// Philox4x32-10 with the reference's v2 address layout (third_party/spark/include/ds41/spark_rng.h:23-36).
__host__ __device__ inline uint32_t philox_word(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose,
                                                uint64_t draw) {
  uint32_t c0 = uint32_t(step), c1 = uint32_t(step >> 32), c2 = uint32_t(draw >> 2),
           c3 = 0x53500000u | (purpose << 3) | slot;
  uint32_t k0 = uint32_t(seed), k1 = uint32_t(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t a = uint64_t(0xD2511F53u) * c0, b = uint64_t(0xCD9E8D57u) * c2;
    const uint32_t n0 = uint32_t(b >> 32) ^ c1 ^ k0, n1 = uint32_t(b), n2 = uint32_t(a >> 32) ^ c3 ^ k1, n3 = uint32_t(a);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  const uint32_t w = uint32_t(draw & 3);
  return w == 0 ? c0 : w == 1 ? c1 : w == 2 ? c2 : c3;
}
__host__ __device__ inline double philox_uniform(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose,
                                                 uint64_t draw = 0) {
  const uint64_t hi = philox_word(seed, step, slot, purpose, 2 * draw) >> 5;
  const uint64_t lo = philox_word(seed, step, slot, purpose, 2 * draw + 1) >> 6;
  return double((hi << 26) | lo) * 0x1p-53;
}

// ---------------------------------------------------------------------------------------------------------------
struct Cut {  // ids "at or before" the cut in the order (logit descending, id ascending) survive
  float y;
  int id;
};
__device__ __forceinline__ bool survives(float y, int id, Cut c) { return y > c.y || (y == c.y && id <= c.id); }

// Per-row summary written by the statistics pass and consumed by the verifier.
struct RowStats {
  double z;        // sum of exp over the ids that enter the softmax
  double e_kept;   // sum of exp over the ids that survive top-k/top-p (equals z without a cut)
  float max_logit; // y_b
  int argmax;      // b, first maximum
  Cut cut;         // survivors: survives(y, id, cut)
  int kept;        // number of survivors
  int entered;     // number of ids that entered the softmax
  int status;      // 0, certification bits, or a negative row error
  int pad;
};

struct Slot {  // one CTA's contribution to a cluster-wide exchange
  double d[4];
  unsigned long long q[2];
  float f[2];
  int i[6];
};

// exp(x) for x <= 0, the only arguments the samplers have ((logit - row maximum) / T).  Table-driven:
// x = (64 k + j) ln2/64 + r with |r| <= ln2/128, exp(x) = 2^k * 2^(j/64) * exp(r), exp(r) - 1 from a degree-6 Taylor
// polynomial (truncation < 3e-20), the reduction with ln2/64 split into a 32-bit head and a tail so that n * head is
// exact.  Error: half an ulp from the table entry, half an ulp from the final fused multiply-add, < 0.01 ulp from the
// rest: below 1.01 ulp, i.e. a relative error < 2.1 * 2^-53, which the decision bounds of every caller allow for
// (they allow tens of units per weight).  Results below the normal range (x < -708) are returned as 0: such a weight
// is < 1e-307 of the row's largest, which no comparison made on the sums can see.  12 FP64 instructions against the
// library routine's ~47.
static __device__ const double kExp2Table[64] = {
    0x1.0000000000000p+0, 0x1.02c9a3e778061p+0, 0x1.059b0d3158574p+0, 0x1.0874518759bc8p+0,
    0x1.0b5586cf9890fp+0, 0x1.0e3ec32d3d1a2p+0, 0x1.11301d0125b51p+0, 0x1.1429aaea92de0p+0,
    0x1.172b83c7d517bp+0, 0x1.1a35beb6fcb75p+0, 0x1.1d4873168b9aap+0, 0x1.2063b88628cd6p+0,
    0x1.2387a6e756238p+0, 0x1.26b4565e27cddp+0, 0x1.29e9df51fdee1p+0, 0x1.2d285a6e4030bp+0,
    0x1.306fe0a31b715p+0, 0x1.33c08b26416ffp+0, 0x1.371a7373aa9cbp+0, 0x1.3a7db34e59ff7p+0,
    0x1.3dea64c123422p+0, 0x1.4160a21f72e2ap+0, 0x1.44e086061892dp+0, 0x1.486a2b5c13cd0p+0,
    0x1.4bfdad5362a27p+0, 0x1.4f9b2769d2ca7p+0, 0x1.5342b569d4f82p+0, 0x1.56f4736b527dap+0,
    0x1.5ab07dd485429p+0, 0x1.5e76f15ad2148p+0, 0x1.6247eb03a5585p+0, 0x1.6623882552225p+0,
    0x1.6a09e667f3bcdp+0, 0x1.6dfb23c651a2fp+0, 0x1.71f75e8ec5f74p+0, 0x1.75feb564267c9p+0,
    0x1.7a11473eb0187p+0, 0x1.7e2f336cf4e62p+0, 0x1.82589994cce13p+0, 0x1.868d99b4492edp+0,
    0x1.8ace5422aa0dbp+0, 0x1.8f1ae99157736p+0, 0x1.93737b0cdc5e5p+0, 0x1.97d829fde4e50p+0,
    0x1.9c49182a3f090p+0, 0x1.a0c667b5de565p+0, 0x1.a5503b23e255dp+0, 0x1.a9e6b5579fdbfp+0,
    0x1.ae89f995ad3adp+0, 0x1.b33a2b84f15fbp+0, 0x1.b7f76f2fb5e47p+0, 0x1.bcc1e904bc1d2p+0,
    0x1.c199bdd85529cp+0, 0x1.c67f12e57d14bp+0, 0x1.cb720dcef9069p+0, 0x1.d072d4a07897cp+0,
    0x1.d5818dcfba487p+0, 0x1.da9e603db3285p+0, 0x1.dfc97337b9b5fp+0, 0x1.e502ee78b3ff6p+0,
    0x1.ea4afa2a490dap+0, 0x1.efa1bee615a27p+0, 0x1.f50765b6e4540p+0, 0x1.fa7c1819e90d8p+0};

__device__ __forceinline__ double exp_nonpos(double x) {
  constexpr double kInvL = 0x1.71547652b82fep+6;    // 64 / ln 2
  constexpr double kLHead = 0x1.62e42fee00000p-7;   // ln 2 / 64, upper 32 bits
  constexpr double kLTail = 0x1.a39ef35793c76p-39;  // and the rest
  constexpr double kMagic = 6755399441055744.0;     // 1.5 * 2^52: adding it leaves round(x * kInvL) in the low word
  const bool tiny = !(x >= -708.0);  // also NaN, which the callers have excluded (non-finite rows are rejected)
  x = tiny ? -708.0 : x;               // branch free: independent calls can overlap
  const double t = fma(x, kInvL, kMagic);
  const int n = __double2loint(t);
  const double nd = t - kMagic;
  double r = fma(nd, -kLHead, x);
  r = fma(nd, -kLTail, r);
  double q = fma(r, 1.0 / 720.0, 1.0 / 120.0);
  q = fma(q, r, 1.0 / 24.0);
  q = fma(q, r, 1.0 / 6.0);
  q = fma(q, r, 0.5);
  q = fma(q, r, 1.0);
  q *= r;  // exp(r) - 1
  const double table = __ldg(&kExp2Table[n & 63]);
  const double v = fma(table, q, table);
  const double scaled = __hiloint2double(__double2hiint(v) + (n >> 6) * 1048576, __double2loint(v));
  return tiny ? 0.0 : scaled;
}

struct __align__(128) RowSmem {
  float y[kSliceCap];  // staged logits, rewritten in place as effective logits (-inf = excluded)
  union {              // 32 KB: history counters first, cut-search work space afterwards
    uint32_t count_pairs[kSliceCap / 2];
    struct {
      unsigned long long total_mass[kBins];
      int total_count[kBins];
      float list_y[kListCap];
      int list_id[kListCap];
      float sorted_y[kListCap];
      int sorted_id[kListCap];
    } w;
  } u;
  unsigned long long bin_mass[kBins];  // also holds the sorted candidates' exp values (doubles) while resolving
  int bin_count[kBins];
  uint32_t mask_words[kSliceCap / 32];
  Slot exch[2][kMaxCluster];
  double warp_sum[kWarps];
  double red_d[kWarps];
  float red_f[kWarps];
  int red_i[kWarps];
  int red_j[kWarps];
  unsigned long long red_q[kWarps];
  Slot outcome;
  unsigned long long mbar;
  unsigned long long bcast_q;
  int list_count;
  int bcast_i[3];
};
static_assert(kListCap * sizeof(double) <= kBins * sizeof(unsigned long long), "sorted_e aliases bin_mass");
static_assert(sizeof(RowSmem) <= 113 * 1024, "two CTAs must fit in one SM's shared memory");

struct RowCtx {
  cg::cluster_group cluster;
  RowSmem *s;
  int rank, nranks, tid, lane, warp;
  int vocab, stride_ids;  // ids per CTA slice (multiple of 32)
  int begin, len;         // this CTA's slice [begin, begin+len)
  int region;             // ids per warp region (multiple of 32): warp w owns local [w*region, (w+1)*region)
  int xphase;
  int timed_out;          // a staging copy of the row just processed did not land (the same in every CTA of the cluster)
};

__device__ __forceinline__ RowCtx make_ctx(RowSmem *s, int vocab) {
  RowCtx c{cg::this_cluster(), s};
  c.rank = int(c.cluster.block_rank());
  c.nranks = int(c.cluster.num_blocks());
  c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5;
  c.vocab = vocab;
  c.stride_ids = (((vocab + c.nranks - 1) / c.nranks) + 31) & ~31;
  c.begin = min(vocab, c.rank * c.stride_ids);
  c.len = min(vocab, c.begin + c.stride_ids) - c.begin;
  c.region = (((c.stride_ids + kWarps - 1) / kWarps) + 31) & ~31;
  c.xphase = 0;
  c.timed_out = 0;
  return c;
}

// All-gather of one Slot per CTA.  Every thread of the CTA must pass the same `mine`.  Two buffers alternate, so a
// fast CTA's next exchange cannot overwrite values a slower CTA is still reading (a third exchange can only start
// after the second one's cluster barrier, which every CTA reaches after it has finished reading the first).
__device__ __forceinline__ const Slot *exchange(RowCtx &c, const Slot &mine) {
  Slot *buf = c.s->exch[c.xphase & 1];
  ++c.xphase;
  if (c.tid < c.nranks) *c.cluster.map_shared_rank(&buf[c.rank], c.tid) = mine;
  c.cluster.sync();
  return buf;
}

// Block-wide reductions in a fixed order (bitwise reproducible run to run).  Result returned to every thread.
__device__ __forceinline__ double block_sum(RowCtx &c, double v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (c.lane == 0) c.s->red_d[c.warp] = v;
  __syncthreads();
  double t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += c.s->red_d[w];
  __syncthreads();
  return t;
}
__device__ __forceinline__ int block_sum(RowCtx &c, int v) {
  v = __reduce_add_sync(0xffffffffu, v);
  if (c.lane == 0) c.s->red_i[c.warp] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += c.s->red_i[w];
  __syncthreads();
  return t;
}
__device__ __forceinline__ unsigned long long block_sum(RowCtx &c, unsigned long long v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (c.lane == 0) c.s->red_q[c.warp] = v;
  __syncthreads();
  unsigned long long t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += c.s->red_q[w];
  __syncthreads();
  return t;
}
__device__ __forceinline__ int block_max(RowCtx &c, int v) {
  v = __reduce_max_sync(0xffffffffu, v);
  if (c.lane == 0) c.s->red_i[c.warp] = v;
  __syncthreads();
  int t = c.s->red_i[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) t = max(t, c.s->red_i[w]);
  __syncthreads();
  return t;
}
__device__ __forceinline__ int block_or(RowCtx &c, int v) {
  v = __reduce_or_sync(0xffffffffu, unsigned(v));
  if (c.lane == 0) c.s->red_i[c.warp] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t |= c.s->red_i[w];
  __syncthreads();
  return t;
}
// (value, id) maximum under "larger value, then lower id".
__device__ __forceinline__ void block_argmax(RowCtx &c, float &v, int &id) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, id, o);
    if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
  }
  if (c.lane == 0) { c.s->red_f[c.warp] = v; c.s->red_j[c.warp] = id; }
  __syncthreads();
  v = c.s->red_f[0]; id = c.s->red_j[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) {
    const float ov = c.s->red_f[w];
    const int oi = c.s->red_j[w];
    if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------------
// Stage the slice.  16-byte aligned slices go through one mbarrier-tracked bulk copy; anything else is loaded with
// plain coalesced loads.  The wait is bounded: on expiry the row is reported as DS41_B200_ROW_TIMEOUT.
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void stage_begin(RowCtx &c, const float *row, bool &used_tma) {
  const float *src = row + c.begin;
  const uint32_t bytes = uint32_t(c.len) * 4u;
  used_tma = c.len > 0 && (bytes & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  if (c.tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&c.s->mbar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (used_tma) {
    if (c.tid == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&c.s->mbar)), "r"(bytes)
                   : "memory");
      for (uint32_t off = 0; off < bytes; off += 16384u) {
        const uint32_t n = min(16384u, bytes - off);
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_u32(reinterpret_cast<const char *>(c.s->y) + off)),
            "l"(reinterpret_cast<const char *>(src) + off), "r"(n), "r"(smem_u32(&c.s->mbar))
            : "memory");
      }
    }
  } else {
    for (int j = c.tid; j < c.len; j += kThreads) c.s->y[j] = __ldg(src + j);
  }
}
// Returns false if the copy did not land within the bound.
__device__ __forceinline__ bool stage_wait(RowCtx &c, bool used_tma) {
  bool ok = true;
  if (used_tma) {
    uint32_t done = 0;
    for (int spin = 0; spin < (1 << 22) && !done; ++spin) {
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
          : "=r"(done)
          : "r"(smem_u32(&c.s->mbar))
          : "memory");
    }
    ok = done != 0;
  }
  __syncthreads();
  // the barrier object is initialised again for the cluster's next row (not after a timeout: the copy may still
  // signal it, and the cluster then takes no further row)
  if (c.tid == 0 && used_tma && ok) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&c.s->mbar)) : "memory");
  return ok;
}

// ---------------------------------------------------------------------------------------------------------------
// Cut search: the k-th id (COUNT) or the id at which the cumulated mass reaches top_p * z (MASS) in the order
// (logit descending, id ascending), found without sorting the row.
//   1. ids are histogrammed by d = max - y into kBins bins per level (counts exact; masses in 2^-46 fixed point,
//      so the histogram does not depend on the order of the atomic additions);
//   2. the crossing bin is located from cluster-wide totals; a bin holding more than kListCap ids is refined
//      (kBins sub-bins), a crossing beyond the range descends into the overflow bin with wider bins;
//   3. the ids of the crossing bin are gathered into rank 0's shared memory, ranked exactly by counting, and
//      walked SEQUENTIALLY in that order, as the reference walks its sorted prefix (sampling.cpp:36).
// The MASS search also produces the normaliser z (its level-0 pass visits every id that enters the softmax).
struct Levels {
  int n;
  float lo[kMaxLevels], inv_w[kMaxLevels];
  int pick[kMaxLevels];      // chosen bin of each finished level (kBins = its overflow bin)
  bool bounded[kMaxLevels];  // refined levels have no overflow bin
};
constexpr int kBefore = -1, kAfter = -2;
// Position of distance d relative to the chain: kBefore / kAfter, or the bin index at the deepest level
// (kBins = overflow).  Monotone in d because every operation (FP32 subtract, multiply, truncation, clamp) is.
__device__ __forceinline__ int classify(const Levels &L, float d) {
  int j = 0;
  for (int l = 0; l < L.n; ++l) {
    const float rel = (d - L.lo[l]) * L.inv_w[l];
    j = rel < 0.f ? 0 : (rel >= float(kBins) ? kBins : int(rel));
    if (L.bounded[l] && j == kBins) j = kBins - 1;
    if (l + 1 < L.n) {
      if (j < L.pick[l]) return kBefore;
      if (j > L.pick[l]) return kAfter;
    }
  }
  return j;
}

struct CutResult {
  Cut cut;        // {-inf,-1}: every active id survives
  int kept;       // survivors
  double z;       // MASS: sum of exp over every active id (fixed parallel order)
  double e_kept;  // MASS: sum of exp over survivors
  int ambiguous;  // MASS: the crossing lies inside the error bound of the parallel sums
  int error;      // 0 or a negative row status
};

// active(y,id): the id takes part.  weight(y): exp((double(y)-double(max))/T).  n_active: number of active ids.
template <bool kMass, class Active, class Weight>
__device__ CutResult find_cut(RowCtx &c, float max_logit, float first_width, int target_count, double top_p,
                              int n_active, Active active, Weight weight) {
  RowSmem *s = c.s;
  Levels L;
  L.n = 1; L.lo[0] = 0.f; L.inv_w[0] = 1.f / first_width; L.bounded[0] = false; L.pick[0] = 0;
  CutResult out{};
  out.cut.y = -CUDART_INF_F; out.cut.id = -1;
  const double rel_bound = 2.0 * (double(n_active) + 256.0) * kU;
  int count_before_level = 0;                // ids before the current level's range (exact)
  unsigned long long mass_before_level = 0;  // their fixed-point mass
  unsigned long long target_fix = 0;
  double target_mass = 0;
  int chosen = -1;  // bin to resolve; -2 = every active id survives
  bool plateau = false;  // the bin to resolve holds more than kListCap ids, all with the logit plateau_y
  float plateau_y = 0.f;
  int plateau_n = 0;
  for (int level = 0;; ++level) {
    for (int j = c.tid; j < kBins; j += kThreads) { s->bin_count[j] = 0; s->bin_mass[j] = 0; }
    __syncthreads();
    int ovf_count = 0;
    unsigned long long ovf_mass = 0;
    double lane_sum = 0;
    for (int it = 0; it < c.region; it += 32) {
      const int j = c.warp * c.region + it + c.lane;
      if (j >= c.len) continue;
      const float y = s->y[j];
      if (!active(y, c.begin + j)) continue;
      const int b = classify(L, max_logit - y);
      if (b < 0) continue;
      unsigned long long m = 0;
      if (kMass) {
        const double e = weight(y);
        lane_sum += e;
        m = (unsigned long long)(e * kFix);
      }
      if (b == kBins) { ++ovf_count; ovf_mass += m; }
      else {
        atomicAdd(&s->bin_count[b], 1);
        if (kMass) atomicAdd(&s->bin_mass[b], m);
      }
    }
    Slot mine{};
    mine.i[0] = block_sum(c, ovf_count);
    if (kMass) {
      mine.q[0] = block_sum(c, ovf_mass);
      if (level == 0) mine.d[0] = block_sum(c, lane_sum);
    }
    c.cluster.sync();  // every CTA's local histogram is complete
    {                  // each CTA totals a share of the bins over all ranks (rank order) and sends them to every CTA
      const int share = kBins / c.nranks;  // nranks is a power of two <= 8
      for (int j = c.tid; j < share; j += kThreads) {
        const int b = c.rank * share + j;
        int tc = 0;
        unsigned long long tm = 0;
        for (int r = 0; r < c.nranks; ++r) {
          tc += *c.cluster.map_shared_rank(&s->bin_count[b], r);
          if (kMass) tm += *c.cluster.map_shared_rank(&s->bin_mass[b], r);
        }
        for (int r = 0; r < c.nranks; ++r) {
          *c.cluster.map_shared_rank(&s->u.w.total_count[b], r) = tc;
          if (kMass) *c.cluster.map_shared_rank(&s->u.w.total_mass[b], r) = tm;
        }
      }
    }
    const Slot *all = exchange(c, mine);  // its barrier also orders the totals before the scan below
    int ovf_total = 0;
    for (int r = 0; r < c.nranks; ++r) ovf_total += all[r].i[0];
    if (kMass && level == 0) {
      double z = 0;
      for (int r = 0; r < c.nranks; ++r) z += all[r].d[0];
      out.z = z;
      target_mass = top_p * z;
      target_fix = (unsigned long long)(target_mass * kFix);
    }
    // ---- locate the crossing bin (warp 0, 32 bins per step)
    if (c.warp == 0) {
      int found = -1;
      int run_c = count_before_level;
      unsigned long long run_m = mass_before_level;
      for (int base = 0; base < kBins && found < 0; base += 32) {
        const int vc = s->u.w.total_count[base + c.lane];
        const unsigned long long vm = kMass ? s->u.w.total_mass[base + c.lane] : 0ull;
        int sc = vc;
        unsigned long long sm = vm;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int tc = __shfl_up_sync(0xffffffffu, sc, o);
          const unsigned long long tm = __shfl_up_sync(0xffffffffu, sm, o);
          if (c.lane >= o) { sc += tc; sm += tm; }
        }
        const bool hit = vc > 0 && (kMass ? (run_m + sm >= target_fix) : (run_c + sc >= target_count));
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (ballot) {
          const int l = __ffs(ballot) - 1;
          found = base + l;
          run_c += __shfl_sync(0xffffffffu, sc - vc, l);
          run_m += __shfl_sync(0xffffffffu, sm - vm, l);
        } else {
          run_c += __shfl_sync(0xffffffffu, sc, 31);
          run_m += __shfl_sync(0xffffffffu, sm, 31);
        }
      }
      if (c.lane == 0) { s->bcast_i[0] = found; s->bcast_i[1] = run_c; s->bcast_q = run_m; }
    }
    __syncthreads();
    const int found = s->bcast_i[0];
    const int before_c = s->bcast_i[1];  // ids before the found bin (or before the overflow bin if none found)
    const unsigned long long before_m = s->bcast_q;
    const int in_bin = found >= 0 ? s->u.w.total_count[found] : 0;
    __syncthreads();
    if (found < 0) {  // the crossing is not inside this level's range
      if (L.bounded[L.n - 1] || ovf_total == 0) { chosen = -2; break; }
      if (L.n == kMaxLevels) { out.error = -4; return out; }
      L.pick[L.n - 1] = kBins;  // descend into the overflow bin, bins 64 times wider
      L.lo[L.n] = L.lo[L.n - 1] + float(kBins) / L.inv_w[L.n - 1];
      L.inv_w[L.n] = L.inv_w[L.n - 1] * (1.f / 64.f);
      L.bounded[L.n] = false;
      ++L.n;
      count_before_level = before_c; mass_before_level = before_m;
      continue;
    }
    if (in_bin > kListCap) {  // refine the crossing bin -- unless all of its ids share one logit (a plateau of ties)
      float lo_y = CUDART_INF_F, hi_y = -CUDART_INF_F;
      for (int it = 0; it < c.region; it += 32) {
        const int j = c.warp * c.region + it + c.lane;
        if (j >= c.len) continue;
        const float y = s->y[j];
        if (!active(y, c.begin + j) || classify(L, max_logit - y) != found) continue;
        lo_y = fminf(lo_y, y); hi_y = fmaxf(hi_y, y);
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        lo_y = fminf(lo_y, __shfl_xor_sync(0xffffffffu, lo_y, o));
        hi_y = fmaxf(hi_y, __shfl_xor_sync(0xffffffffu, hi_y, o));
      }
      if (c.lane == 0) { s->red_f[c.warp] = lo_y; s->red_d[c.warp] = double(hi_y); }
      __syncthreads();
      for (int w = 0; w < kWarps; ++w) { lo_y = fminf(lo_y, s->red_f[w]); hi_y = fmaxf(hi_y, float(s->red_d[w])); }
      __syncthreads();
      Slot span{};
      span.f[0] = lo_y; span.f[1] = hi_y;
      const Slot *spans = exchange(c, span);
      for (int r = 0; r < c.nranks; ++r) { lo_y = fminf(lo_y, spans[r].f[0]); hi_y = fmaxf(hi_y, spans[r].f[1]); }
      if (lo_y == hi_y) {  // equal logits have equal weights: the cut inside the plateau follows from arithmetic
        plateau = true; plateau_y = lo_y; plateau_n = in_bin;
        chosen = found;
        break;
      }
      if (L.n == kMaxLevels) { out.error = -4; return out; }
      L.pick[L.n - 1] = found;
      L.lo[L.n] = L.lo[L.n - 1] + float(found) / L.inv_w[L.n - 1];
      L.inv_w[L.n] = L.inv_w[L.n - 1] * float(kBins);
      L.bounded[L.n] = true;
      ++L.n;
      count_before_level = before_c; mass_before_level = before_m;
      continue;
    }
    chosen = found;
    break;
  }

  // ---- resolve.  (MASS) the fixed-point histogram can pick a neighbour of the true crossing bin when the target
  // lies within n*2^-46 of a bin edge; the exact sums below detect that and the search moves one bin over.
  for (int attempt = 0; attempt < 4; ++attempt) {
    if (c.tid == 0) s->list_count = 0;
    c.cluster.sync();  // reset visible before any remote push; everyone is done with the previous attempt's list
    double before_mass = 0;
    int before_count = 0, after_count = 0;
    int *list_count0 = c.cluster.map_shared_rank(&s->list_count, 0);
    float *list_y0 = c.cluster.map_shared_rank(s->u.w.list_y, 0);
    int *list_id0 = c.cluster.map_shared_rank(s->u.w.list_id, 0);
    for (int it = 0; it < c.region; it += 32) {
      const int j = c.warp * c.region + it + c.lane;
      if (j >= c.len) continue;
      const float y = s->y[j];
      const int id = c.begin + j;
      if (!active(y, id)) continue;
      const int b = chosen == -2 ? kBefore : classify(L, max_logit - y);
      if (b == kBefore || (b >= 0 && b < chosen)) {
        ++before_count;
        if (kMass) before_mass += weight(y);
      } else if (b == chosen) {
        if (!plateau) {
          const int slot = atomicAdd(list_count0, 1);
          if (slot < kListCap) { list_y0[slot] = y; list_id0[slot] = id; }
        }
      } else {
        ++after_count;
      }
    }
    Slot mine{};
    if (kMass) mine.d[0] = block_sum(c, before_mass);
    mine.i[0] = block_sum(c, before_count);
    mine.i[1] = block_sum(c, after_count);
    const Slot *all = exchange(c, mine);  // cluster barrier: the gathered list is complete
    double mass_before = 0;
    int n_before = 0, n_after = 0;
    for (int r = 0; r < c.nranks; ++r) { mass_before += all[r].d[0]; n_before += all[r].i[0]; n_after += all[r].i[1]; }

    if (plateau) {
      // ---- the cut inside a plateau of plateau_n equal logits (reference: stable order, ties keep the lower id, one
      // weight added per kept id: sampling.cpp:34-36).  Every thread of the cluster computes the same numbers.
      long long k = 0;  // ids of the plateau that are kept
      int direction = 0, amb = 0;
      double mass = mass_before;
      if constexpr (!kMass) {
        k = (long long)target_count - n_before;
        if (k < 1) direction = -1; else if (k > plateau_n) direction = 1;
      } else {
        const double w = weight(plateau_y);
        const double lo = target_mass * (1.0 - rel_bound), hi = target_mass * (1.0 + rel_bound);
        if (n_before > 0 && mass_before >= target_mass) direction = -1;
        else {
          const double need = (target_mass - mass_before) / w;
          k = need > double(plateau_n) + 2.0 ? (long long)plateau_n + 1 : (long long)need;
          if (k < 1) k = 1;
          while (k <= plateau_n && mass_before + double(k) * w < target_mass) ++k;
          while (k > 1 && mass_before + double(k - 1) * w >= target_mass) --k;
          if (k > plateau_n) {
            if (n_after > 0) direction = 1;
            else { k = plateau_n; mass = mass_before + double(k) * w; amb = !(mass < lo); }  // every id kept
          } else {
            mass = mass_before + double(k) * w;
            const double prev = mass_before + double(k - 1) * w;
            amb = (mass < hi) || (prev >= lo);
          }
        }
      }
      if (direction != 0) { out.error = -4; return out; }  // the histogram mis-picked a crowded bin's neighbour: not handled
      // the k-th id of the plateau in ascending id order: counts per warp region, per CTA, then a walk of one region
      int mine = 0;
      for (int it = 0; it < c.region; it += 32) {
        const int j = c.warp * c.region + it + c.lane;
        if (j < c.len && s->y[j] == plateau_y && active(s->y[j], c.begin + j)) ++mine;
      }
      mine = __reduce_add_sync(0xffffffffu, mine);
      if (c.lane == 0) s->red_i[c.warp] = mine;
      __syncthreads();
      int cta_total = 0;
      for (int w2 = 0; w2 < kWarps; ++w2) cta_total += s->red_i[w2];
      Slot cnt{};
      cnt.i[0] = cta_total;
      const Slot *cnts = exchange(c, cnt);
      long long skip = k - 1;  // tied ids before the wanted one
      int owner = -1;
      for (int r = 0; r < c.nranks; ++r) {
        if (owner < 0 && skip < cnts[r].i[0]) owner = r;
        if (owner < 0) skip -= cnts[r].i[0];
      }
      Slot pick{};
      pick.i[0] = -1;
      if (owner == c.rank) {
        int ow = -1;
        long long left = skip;
        for (int w2 = 0; w2 < kWarps; ++w2) {
          if (ow < 0 && left < s->red_i[w2]) ow = w2;
          if (ow < 0) left -= s->red_i[w2];
        }
        if (c.warp == ow) {
          int found_id = -1;
          int remaining = int(left);
          for (int it = 0; it < c.region && found_id < 0; it += 32) {
            const int j = ow * c.region + it + c.lane;
            const bool tied = j < c.len && s->y[j] == plateau_y && active(s->y[j], c.begin + j);
            const unsigned ballot = __ballot_sync(0xffffffffu, tied);
            const int here = __popc(ballot);
            if (remaining < here) {
              unsigned m = ballot;
              for (int q = 0; q < remaining; ++q) m &= m - 1;  // drop the lowest `remaining` set bits
              found_id = c.begin + ow * c.region + it + (__ffs(m) - 1);
            } else {
              remaining -= here;
            }
          }
          if (c.lane == 0) s->bcast_i[0] = found_id;
        }
        __syncthreads();
        pick.i[0] = s->bcast_i[0];
        __syncthreads();
      }
      const Slot *picks = exchange(c, pick);
      int cut_id = -1;
      for (int r = 0; r < c.nranks; ++r) cut_id = max(cut_id, picks[r].i[0]);
      if (cut_id < 0) { out.error = -4; return out; }
      const bool all_kept = k == plateau_n && n_after == 0;
      out.cut.y = all_kept ? -CUDART_INF_F : plateau_y;
      out.cut.id = all_kept ? -1 : cut_id;
      out.kept = n_before + int(k);
      out.e_kept = mass;
      out.ambiguous = amb;
      return out;
    }
    Slot outcome{};
    double *sorted_e = reinterpret_cast<double *>(s->bin_mass);  // local bins are dead once the totals exist
    if (c.rank == 0) {
      const int n = chosen == -2 ? 0 : min(s->list_count, kListCap);
      for (int i = c.tid; i < n; i += kThreads) {  // exact rank by counting (strict total order)
        const float yi = s->u.w.list_y[i];
        const int idi = s->u.w.list_id[i];
        int r = 0;
        for (int k = 0; k < n; ++k) {
          const float yk = s->u.w.list_y[k];
          const int idk = s->u.w.list_id[k];
          r += (yk > yi || (yk == yi && idk < idi)) ? 1 : 0;
        }
        s->u.w.sorted_y[r] = yi;
        s->u.w.sorted_id[r] = idi;
        if (kMass) sorted_e[r] = weight(yi);
      }
      __syncthreads();
      if (c.tid == 0) {
        int direction = 0, pos = -1, amb = 0;
        double mass = mass_before;
        if (!kMass) {
          pos = target_count - n_before - 1;
          if (pos < 0) direction = -1;
          else if (pos >= n) direction = 1;
        } else {
          const double lo = target_mass * (1.0 - rel_bound), hi = target_mass * (1.0 + rel_bound);
          if (chosen == -2) {
            amb = !(mass < lo);  // reference keeps every id only if its own sum stays below top_p
          } else if (n_before > 0 && mass >= target_mass) {
            direction = -1;  // the prefix before this bin already reaches the target
          } else {
            for (int r = 0; r < n; ++r) {
              const double prev = mass;
              mass += sorted_e[r];
              if (mass >= target_mass) {
                pos = r;
                amb = (mass < hi) || (prev >= lo);
                break;
              }
            }
            if (pos < 0) {
              if (n_after > 0) direction = 1;  // the crossing lies in a later bin
              else { pos = n - 1; amb = !(mass < lo); }  // every id kept
            }
          }
        }
        outcome.i[0] = direction;
        outcome.i[1] = amb;
        if (direction == 0) {
          const bool all_kept = chosen == -2 || pos < 0 || (pos == n - 1 && n_after == 0);
          outcome.f[0] = all_kept ? -CUDART_INF_F : s->u.w.sorted_y[pos];
          outcome.i[2] = all_kept ? -1 : s->u.w.sorted_id[pos];
          outcome.i[3] = all_kept ? n_before + n : n_before + pos + 1;
          outcome.d[0] = mass;
        }
        s->outcome = outcome;
      }
      __syncthreads();
      outcome = s->outcome;
      __syncthreads();
    }
    const Slot v = exchange(c, outcome)[0];
    if (v.i[0] == 0) {
      out.cut.y = v.f[0]; out.cut.id = v.i[2]; out.kept = v.i[3]; out.e_kept = v.d[0]; out.ambiguous = v.i[1];
      return out;
    }
    const int next = chosen + v.i[0];  // one bin over at the deepest level; it must fit the list as well
    if (chosen < 0 || next < 0 || next >= kBins || s->u.w.total_count[next] > kListCap) { out.error = -4; return out; }
    chosen = next;
  }
  out.error = -4;
  return out;
}

}  // namespace ds41
