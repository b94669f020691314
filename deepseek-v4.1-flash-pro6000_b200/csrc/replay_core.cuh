// Device routines that follow the reference's host arithmetic literally: sums on one thread in index order, the stable
// order of the probabilities, the sequential inverse CDF (engine/third_party/spark/src/sampling.cpp:12-38).  Shared by
// the replay of uncertified rows (replay.cu) and by the operators on probability rows (prob.cu).  One CTA of
// kReplayThreads threads works on one row.
#pragma once
#include "replay.cuh"
#include "row_core.cuh"

namespace ds41 {
namespace {

constexpr int kRT = kReplayThreads;
constexpr int kTile = 2048;   // elements sorted / summed out of shared memory at a time

struct ReplaySmem {
  double stage[kTile];
  unsigned long long key[kTile];
  int idx[kTile];
  unsigned long long scan[kRT / 32];
  unsigned long long quick[2][kRT / 32];
  float red_f[kRT / 32];
  int red_i[kRT / 32];
  double bcast_d[4];
  int bcast_i[4];
};

__device__ __forceinline__ bool key_less(unsigned long long ka, int ia, unsigned long long kb, int ib) {
  return ka < kb || (ka == kb && ia < ib);
}

// Ascending bitonic sort of (key, idx) pairs, kReplayPad of them, in global memory.  Tiles of kTile elements are first
// sorted out of shared memory; after that every merge step runs its wide strides on global memory and its strides below
// kTile again out of shared memory.
__device__ void sort_pairs(ReplaySmem &s, unsigned long long *key, int *idx) {
  const int tid = threadIdx.x;
  auto local_stages = [&](int base, int k, int j_first) {  // strides j_first, j_first / 2 ... 1 of merge step k
    for (int jj = j_first; jj > 0; jj >>= 1) {
      for (int i = tid; i < kTile / 2; i += kRT) {
        const int lo = ((i & ~(jj - 1)) << 1) | (i & (jj - 1)), hi = lo + jj;   // jj is a power of two
        const bool up = ((base + lo) & k) == 0;
        const unsigned long long ka = s.key[lo], kb = s.key[hi];
        const int ia = s.idx[lo], ib = s.idx[hi];
        if (key_less(kb, ib, ka, ia) == up) { s.key[lo] = kb; s.key[hi] = ka; s.idx[lo] = ib; s.idx[hi] = ia; }
      }
      __syncthreads();
    }
  };
  for (int base = 0; base < kReplayPad; base += kTile) {
    for (int i = tid; i < kTile; i += kRT) { s.key[i] = key[base + i]; s.idx[i] = idx[base + i]; }
    __syncthreads();
    for (int k = 2; k <= kTile; k <<= 1) local_stages(base, k, k >> 1);
    for (int i = tid; i < kTile; i += kRT) { key[base + i] = s.key[i]; idx[base + i] = s.idx[i]; }
    __syncthreads();
  }
  for (int k = 2 * kTile; k <= kReplayPad; k <<= 1) {
    for (int j = k >> 1; j >= kTile; j >>= 1) {  // partners further apart than a tile
      for (int i = tid; i < kReplayPad / 2; i += kRT) {
        const int lo = ((i & ~(j - 1)) << 1) | (i & (j - 1)), hi = lo + j;
        const bool up = (lo & k) == 0;
        const unsigned long long ka = key[lo], kb = key[hi];
        const int ia = idx[lo], ib = idx[hi];
        if (key_less(kb, ib, ka, ia) == up) { key[lo] = kb; key[hi] = ka; idx[lo] = ib; idx[hi] = ia; }
      }
      __syncthreads();
    }
    for (int base = 0; base < kReplayPad; base += kTile) {
      for (int i = tid; i < kTile; i += kRT) { s.key[i] = key[base + i]; s.idx[i] = idx[base + i]; }
      __syncthreads();
      local_stages(base, k, kTile >> 1);
      for (int i = tid; i < kTile; i += kRT) { key[base + i] = s.key[i]; idx[base + i] = s.idx[i]; }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The reference's loops `acc += v[i]` run on one host thread; what has to be reproduced is every rounding of that
// chain.  For non-negative terms the chain can be followed exactly in parallel.  While acc stays inside one binade
// [2^e, 2^(e+1)) its grid has the fixed spacing U = 2^(e-52), acc = S * U with an integer S, and
//     fl(acc + x) = (S + rn(x / U)) * U
// where rn rounds to the nearest integer: the rounding of the sum does not depend on S, except when x / U lies exactly
// half way between two integers (the tie goes to the even S + ...).  So inside a binade the chain is an INTEGER prefix
// sum of rn(x_i / U), which a block scan computes exactly, and every intermediate acc is known exactly.  The two events
// that end such a stretch are found by the same scan: the first term whose sum reaches 2^(e+1) (the spacing changes) and
// the first tie.  That one term is added with a real FP64 addition to the exactly known acc before it (this IS the
// reference's operation), and the scan restarts behind it with the new acc.  A whole pass costs one block scan per tile
// plus one per binade crossed (a few dozen), instead of one dependent addition per term on a single thread.
// Terms that are negative, NaN or infinite (rows a caller passed in without validation) take the literal loop.
constexpr int kSeqHead = 256;               // terms of a chain from zero that one thread adds literally
constexpr int kSumPer = 4;                 // consecutive terms a thread holds in registers
constexpr int kSumTile = kSumPer * kRT;    // terms scanned at a time
constexpr unsigned long long kTwo52 = 1ull << 52, kTwo53 = 1ull << 53;

struct SeqResult {
  int found;            // index of the term after which stop(acc) first held; -1: the loop ran through
  double acc, before;   // acc after that term (or after the last one) and just before it
};

// x = m * 2^(be - 1075), be >= 1 (subnormals: be = 1 without the implicit bit)
__device__ __forceinline__ void split_double(double x, int &be, unsigned long long &m) {
  const unsigned long long b = (unsigned long long)__double_as_longlong(x);
  be = int(b >> 52) & 0x7ff;
  m = b & (kTwo52 - 1);
  if (be) m |= kTwo52; else be = 1;
}

// units * 2^(be - 1075) for units < 2^53 (below 2^52 only in the subnormal range, be == 1)
__device__ __forceinline__ double join_double(unsigned long long units, int be) {
  return __longlong_as_double((long long)(units >= kTwo52 ? ((unsigned long long)be << 52) + (units - kTwo52) : units));
}

// rn(x / U) for U = 2^(be_acc - 1075), x >= 0 finite; *tie: x / U is exactly half way (the floor is returned).  Values
// that certainly carry acc out of its binade are returned as 2^53.
__device__ __forceinline__ unsigned long long to_units(double x, int be_acc, bool *tie) {
  int bx;
  unsigned long long mx;
  split_double(x, bx, mx);
  *tie = false;
  const int shift = be_acc - bx;
  if (shift <= 0) return shift == 0 ? mx : (mx ? kTwo53 : 0ull);
  if (shift >= 64) return 0ull;
  const unsigned long long q = mx >> shift, rem = mx & ((1ull << shift) - 1), half = 1ull << (shift - 1);
  if (rem == half) *tie = true;
  return q + (rem > half ? 1ull : 0ull);
}

// exclusive prefix of one value per thread over the block, in thread order; *total = the block's sum (mod 2^64)
__device__ __forceinline__ unsigned long long block_exclusive_u64(ReplaySmem &s, unsigned long long v,
                                                                  unsigned long long *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  if (lane == 31) s.scan[warp] = inc;
  __syncthreads();
  unsigned long long w = lane < kRT / 32 ? s.scan[lane] : 0ull, winc = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += up;
  }
  *total = __shfl_sync(0xffffffffu, winc, 31);
  const unsigned long long before_warp = __shfl_sync(0xffffffffu, winc - w, warp);
  __syncthreads();   // scan[] may be rewritten by the next call
  return before_warp + inc - v;
}

// acc = 0; for i in [0, n): acc += value(i); if (stop(acc)) return i   -- with every rounding of that chain.
// stop must be monotone (once true it stays true as acc grows) and may be false throughout.
// (first, acc0): the loop resumed at term `first` with the acc the earlier terms left.
template <class Value, class Stop>
__device__ SeqResult exact_sequential(ReplaySmem &s, int n, Value value, Stop stop, int first = 0, double acc0 = 0.0) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double acc = acc0;         // the same in every thread
  int start = first;
  if (first == 0 && acc0 == 0.0) {
    // A chain that starts from zero leaves a binade with almost every one of its first terms: those are added as the
    // reference adds them, by one thread, out of shared memory.
    const int head = min(n, kSeqHead);
    if (tid < head) s.stage[tid] = value(tid);
    __syncthreads();
    if (tid == 0) {
      int found = -1;
      double a = 0.0, before = 0.0;
      for (int i = 0; i < head; ++i) {
        before = a;
        a += s.stage[i];
        if (stop(a)) { found = i; break; }
      }
      s.bcast_i[0] = found; s.bcast_d[0] = a; s.bcast_d[1] = before;
    }
    __syncthreads();
    const int found = s.bcast_i[0];
    acc = s.bcast_d[0];
    const double before = s.bcast_d[1];
    __syncthreads();
    if (found >= 0) return SeqResult{found, acc, before};
    start = head;
  }
  int parity = 0;
  for (int base = start; base < n; base += kSumTile) {
    const int m = min(kSumTile, n - base);
    // every thread keeps kSumPer consecutive terms in registers
    double v[kSumPer];
    int bad = 0;
    {
      // A first look at the tile as a whole: if no term is invalid or ties, and the chain neither leaves its binade nor
      // stops by the tile's end, the tile is one integer sum (one barrier).
      int be0;
      unsigned long long s00, quick = 0;
      split_double(acc, be0, s00);
      int tied = 0;
#pragma unroll
      for (int r = 0; r < kSumPer; ++r) {
        const int i = tid * kSumPer + r;
        v[r] = i < m ? value(base + i) : 0.0;
        bad |= !(v[r] >= 0.0 && v[r] < CUDART_INF);
        bool tie;
        quick += to_units(v[r], be0, &tie);
        tied |= tie ? 1 : 0;
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) quick += __shfl_xor_sync(0xffffffffu, quick, o);
      if (lane == 0) s.quick[parity][warp] = quick;
      if (tid == 0) { s.bcast_i[0] = 0x7fffffff; s.bcast_i[1] = 0x7fffffff; }
      const int any = __syncthreads_or(bad | tied);
      unsigned long long total = 0;
#pragma unroll
      for (int w = 0; w < kRT / 32; ++w) total += s.quick[parity][w];
      parity ^= 1;
      const unsigned long long through = s00 + total;
      if (!any && through < kTwo53 && !stop(join_double(through, be0))) {
        acc = join_double(through, be0);
        continue;
      }
      if (any) bad = __syncthreads_or(bad);   // (uniform: `any` is the same in every thread)
    }
    if (bad) {   // the literal loop, one thread
      if (tid == 0) {
        int found = -1;
        double before = acc;
        for (int i = 0; i < m; ++i) {
          before = acc;
          acc += value(base + i);
          if (stop(acc)) { found = base + i; break; }
        }
        s.bcast_i[0] = found; s.bcast_d[0] = acc; s.bcast_d[1] = before;
      }
      __syncthreads();
      const int found = s.bcast_i[0];
      acc = s.bcast_d[0];
      const double before = s.bcast_d[1];
      __syncthreads();
      if (found >= 0) return SeqResult{found, acc, before};
      continue;
    }
    int pos = 0;
    while (pos < m) {   // uniform: one pass per stretch of the chain inside one binade
      int be;
      unsigned long long s0;
      split_double(acc, be, s0);
      unsigned long long t[kSumPer], sum = 0;
      unsigned ties = 0;
#pragma unroll
      for (int r = 0; r < kSumPer; ++r) {
        const int i = tid * kSumPer + r;
        bool tie = false;
        t[r] = (i >= pos && i < m) ? to_units(v[r], be, &tie) : 0ull;
        ties |= tie ? (1u << r) : 0u;
        sum += t[r];
      }
      unsigned long long total;
      unsigned long long running = s0 + block_exclusive_u64(s, sum, &total);
      int special = 0x7fffffff, stop_at = 0x7fffffff;
      double at_acc = 0.0, at_before = 0.0, special_term = 0.0;
      unsigned long long special_before = 0;
      // the chain is monotone: only a thread whose last term crosses a line has to look at its terms one by one
      const unsigned long long after_mine = running + sum;
      const bool look = ties != 0 || after_mine >= kTwo53 || (tid * kSumPer < m && stop(join_double(after_mine, be)));
      if (look) {
#pragma unroll
        for (int r = 0; r < kSumPer; ++r) {
          const int i = tid * kSumPer + r;
          if (i < pos || i >= m || special != 0x7fffffff || stop_at != 0x7fffffff) continue;
          const unsigned long long units_before = running;
          running += t[r];
          if (((ties >> r) & 1u) || running >= kTwo53) {
            special = i; special_before = units_before; special_term = v[r];
          } else {
            const double a = join_double(running, be);
            if (stop(a)) { stop_at = i; at_acc = a; at_before = join_double(units_before, be); }
          }
        }
      }
      if (special != 0x7fffffff) atomicMin(&s.bcast_i[0], special);
      if (stop_at != 0x7fffffff) atomicMin(&s.bcast_i[1], stop_at);
      __syncthreads();
      const int js = s.bcast_i[0], jt = s.bcast_i[1];
      if (jt < js) {   // the loop stops inside this stretch
        if (stop_at == jt) { s.bcast_d[0] = at_acc; s.bcast_d[1] = at_before; }
        __syncthreads();
        const SeqResult out{base + jt, s.bcast_d[0], s.bcast_d[1]};
        __syncthreads();
        return out;
      }
      if (js == 0x7fffffff) {   // the rest of the tile stays inside the binade
        acc = join_double(s0 + total, be);
        break;
      }
      if (special == js) {      // the term that leaves the binade (or ties): the reference's own addition
        const double before = join_double(special_before, be);
        s.bcast_d[1] = before;
        s.bcast_d[0] = __dadd_rn(before, special_term);
      }
      __syncthreads();
      acc = s.bcast_d[0];
      const double before = s.bcast_d[1];
      if (tid == 0) { s.bcast_i[0] = 0x7fffffff; s.bcast_i[1] = 0x7fffffff; }
      __syncthreads();   // (also orders the reset before the next round's minima, which follow the scan's barriers)
      if (stop(acc)) return SeqResult{base + js, acc, before};
      pos = js + 1;
    }
    __syncthreads();
  }
  return SeqResult{-1, acc, acc};
}

template <class Value>
__device__ double sequential_sum(ReplaySmem &s, int n, Value value) {
  return exact_sequential(s, n, value, [](double) { return false; }).acc;
}

// ---------------------------------------------------------------------------------------------------------------
// Order of the probabilities (p descending, id ascending) without a full sort: the ids are distributed over kBuckets
// ranges of the upper key word (counted while the row is normalised, one pass of scattering), and the buckets are put
// in order only as far as the top-p loop gets: a warp takes the buckets that begin within one run of kChunk positions
// and sorts them together out of its own shared-memory area (buckets are ranges of the key, so whole buckets sorted
// jointly are in their final order).  The loop normally stops long before the tail, so most buckets are never ordered.
constexpr int kBuckets = 4096;
constexpr int kWarpSort = 256;                       // entries a warp orders out of its own area
constexpr int kChunk = 128;                          // positions per chunk; a chunk holds at most kChunk - 1 + its last bucket
constexpr int kSpanCap = 96 << 20;                   // binades (2^20 upper-word steps each) the bucket grid covers
constexpr size_t kReplayDynamicBytes = size_t(kRT / 32) * kWarpSort * 12 + size_t(kBuckets + 1) * 4;

struct BucketOrder {
  int *starts;                 // [kBuckets + 1] first position of each bucket (dynamic shared memory); counts before the scan
  unsigned long long *wkey;    // [warps][kWarpSort]
  int *widx;
  uint32_t hi_min;             // upper key word of the largest p
  float scale;                 // buckets per upper-word step
  int n;                       // entries
  __device__ __forceinline__ int bucket_of(unsigned long long k) const {
    const uint32_t hi = uint32_t(k >> 32), d = hi > hi_min ? hi - hi_min : 0u;
    const float f = __uint2float_rz(d) * scale;   // monotone in the key
    return f >= float(kBuckets - 1) ? kBuckets - 1 : int(f);
  }
  // first bucket whose first position is >= v (kBuckets when there is none)
  __device__ __forceinline__ int bucket_from(int v) const {
    int lo = 0, hi = kBuckets;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (starts[mid] >= v) hi = mid; else lo = mid + 1;
    }
    return lo;
  }
};

__device__ __forceinline__ unsigned long long order_key(double p) { return ~(unsigned long long)__double_as_longlong(p); }

// The bucket grid for probabilities between p_max and p_low (or kSpanCap below p_max; the rest shares the last bucket);
// clears the counters.  Every thread gets the same record.
__device__ BucketOrder bucket_begin(unsigned char *dynamic, int n, double p_max, double p_low) {
  BucketOrder b;
  b.wkey = reinterpret_cast<unsigned long long *>(dynamic);
  b.widx = reinterpret_cast<int *>(dynamic + size_t(kRT / 32) * kWarpSort * 8);
  b.starts = reinterpret_cast<int *>(dynamic + size_t(kRT / 32) * kWarpSort * 12);
  b.n = n;
  b.hi_min = uint32_t(order_key(p_max) >> 32);
  const uint32_t hi_low = uint32_t(order_key(p_low) >> 32);
  uint32_t span = p_low > 0 ? (hi_low >= b.hi_min ? hi_low - b.hi_min + 1 : 1) : uint32_t(kSpanCap);
  if (span > uint32_t(kSpanCap)) span = kSpanCap;
  b.scale = float(kBuckets - 1) / float(span);
  for (int i = threadIdx.x; i <= kBuckets; i += kRT) b.starts[i] = 0;
  __syncthreads();
  return b;
}
__device__ __forceinline__ void bucket_count(const BucketOrder &b, double p) { atomicAdd(&b.starts[b.bucket_of(order_key(p))], 1); }

// After every p has been counted: first positions from the counts, then (key, id) of p[0..n) into key[] / idx[] by bucket.
__device__ void bucket_scatter(ReplaySmem &s, BucketOrder &b, const double *p, unsigned long long *key, int *idx) {
  const int tid = threadIdx.x, n = b.n;
  int *count = b.starts, *cursor = reinterpret_cast<int *>(s.stage);
  __syncthreads();
  constexpr int kPerThread = kBuckets / kRT;
  int mine[kPerThread], sum = 0;
#pragma unroll
  for (int r = 0; r < kPerThread; ++r) { mine[r] = count[tid * kPerThread + r]; sum += mine[r]; }
  unsigned long long total;
  int at = int(block_exclusive_u64(s, (unsigned long long)sum, &total));
#pragma unroll
  for (int r = 0; r < kPerThread; ++r) { count[tid * kPerThread + r] = at; cursor[tid * kPerThread + r] = at; at += mine[r]; }
  if (tid == 0) count[kBuckets] = n;
  __syncthreads();
  for (int i0 = tid; i0 < n; i0 += 4 * kRT) {   // four independent loads in flight per thread
    double v[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) v[r] = i0 + r * kRT < n ? p[i0 + r * kRT] : 0.0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + r * kRT;
      if (i >= n) continue;
      const unsigned long long k = order_key(v[r]);
      const int pos = atomicAdd(&cursor[b.bucket_of(k)], 1);
      key[pos] = k; idx[pos] = i;
    }
  }
  __syncthreads();
}

// One chunk (the buckets that begin within positions [c * kChunk, (c + 1) * kChunk)): first position and length.
__device__ __forceinline__ void chunk_range(const BucketOrder &b, int c, int *st, int *m) {
  const int q0 = b.bucket_from(c * kChunk), q1 = b.bucket_from((c + 1) * kChunk);
  *st = b.starts[q0];
  *m = b.starts[q1] - *st;   // (starts[kBuckets] = n)
}

// Puts positions [st, st + m) of key[] / idx[] in order: warp 0 out of its shared-memory area, or the whole CTA for up
// to kTile entries.  Called by every thread; false when the range is too large (long runs of equal logits).
__device__ bool order_range(ReplaySmem &s, const BucketOrder &b, int st, int m, unsigned long long *key, int *idx) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (m > kTile) return false;
  if (m <= 1) return true;
  int padded = 2;
  while (padded < m) padded <<= 1;
  if (m <= kWarpSort) {
    if (warp == 0) {
      unsigned long long *wk = b.wkey;
      int *wi = b.widx;
      for (int i = lane; i < padded; i += 32) { wk[i] = i < m ? key[st + i] : ~0ull; wi[i] = i < m ? idx[st + i] : 0x7fffffff; }
      __syncwarp();
      for (int k = 2; k <= padded; k <<= 1)
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
          for (int i = lane; i < padded / 2; i += 32) {
            const int lo = ((i & ~(jj - 1)) << 1) | (i & (jj - 1)), hi = lo + jj;   // jj is a power of two
            const bool up = (lo & k) == 0;
            const unsigned long long ka = wk[lo], kb = wk[hi];
            const int ia = wi[lo], ib = wi[hi];
            if (key_less(kb, ib, ka, ia) == up) { wk[lo] = kb; wk[hi] = ka; wi[lo] = ib; wi[hi] = ia; }
          }
          __syncwarp();
        }
      for (int i = lane; i < m; i += 32) { key[st + i] = wk[i]; idx[st + i] = wi[i]; }
    }
    __syncthreads();
    return true;
  }
  for (int i = tid; i < padded; i += kRT) { s.key[i] = i < m ? key[st + i] : ~0ull; s.idx[i] = i < m ? idx[st + i] : 0x7fffffff; }
  __syncthreads();
  for (int k = 2; k <= padded; k <<= 1)
    for (int jj = k >> 1; jj > 0; jj >>= 1) {
      for (int i = tid; i < padded / 2; i += kRT) {
        const int lo = ((i & ~(jj - 1)) << 1) | (i & (jj - 1)), hi = lo + jj;
        const bool up = (lo & k) == 0;
        const unsigned long long ka = s.key[lo], kb = s.key[hi];
        const int ia = s.idx[lo], ib = s.idx[hi];
        if (key_less(kb, ib, ka, ia) == up) { s.key[lo] = kb; s.key[hi] = ka; s.idx[lo] = ib; s.idx[hi] = ia; }
      }
      __syncthreads();
    }
  for (int i = tid; i < m; i += kRT) { key[st + i] = s.key[i]; idx[st + i] = s.idx[i]; }
  __syncthreads();
  return true;
}

// The reference's loop `mass += p[idx[k++]] while k < n && mass < top` over the stable order, without putting the order
// together first.  Inside one binade of the accumulator (and without exact ties) the chain adds rn(x / U) per term
// whatever the order of the terms, so a chunk -- whole buckets, i.e. a range of the key, unordered inside -- is consumed
// by one integer sum as long as the chain neither leaves the binade nor stops inside it; the warps take 32 chunks at a
// time.  Only a chunk in which that happens (a few dozen per row, and the one where the loop stops) is put in order and
// walked term by term.  found = the loop's k - 1 (a position of the order); key[found] / idx[found] are then in place.
// ok = false: a chunk was too large to order here.
template <class Stop>
__device__ SeqResult chain_over_chunks(ReplaySmem &s, const BucketOrder &b, const double *p, unsigned long long *key,
                                       int *idx, Stop stop, bool *ok) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kW = kRT / 32;
  const int chunks = (b.n + kChunk - 1) / kChunk;
  double acc = 0.0;
  *ok = true;
  int c = 0;
  while (c < chunks) {
    int be;
    unsigned long long s0;
    split_double(acc, be, s0);
    // one chunk per warp: integer sum of its terms at the accumulator's spacing, and whether any of them ties
    unsigned long long sum = 0;
    int tie = 0;
    if (c + warp < chunks) {
      int st, m;
      chunk_range(b, c + warp, &st, &m);
      for (int j = lane; j < m; j += 32) {
        bool t;
        sum += to_units(p[idx[st + j]], be, &t);
        tie |= t ? 1 : 0;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      tie |= __shfl_xor_sync(0xffffffffu, tie, o);
    }
    if (lane == 0) { s.scan[warp] = sum; s.red_i[warp] = tie; }
    __syncthreads();
    // every thread walks the (at most 32) chunk sums: the first chunk that needs its terms one by one
    unsigned long long units = s0;
    int special = -1;
    for (int w = 0; w < kW && c + w < chunks; ++w) {
      const unsigned long long through = units + s.scan[w];
      if (s.red_i[w] || through >= kTwo53 || stop(join_double(through, be))) { special = w; break; }
      units = through;
    }
    __syncthreads();   // scan[] / red_i[] are rewritten by the next round (and by the walk below)
    acc = join_double(units, be);   // the chunks before the special one are consumed
    if (special < 0) { c += kW; continue; }
    int st, m;
    chunk_range(b, c + special, &st, &m);
    if (!order_range(s, b, st, m, key, idx)) { *ok = false; return SeqResult{-1, acc, acc}; }
    const SeqResult r = exact_sequential(s, st + m, [p, idx](int i) { return p[idx[i]]; }, stop, st, acc);
    if (r.found >= 0) return r;
    acc = r.acc;
    c += special + 1;
  }
  return SeqResult{-1, acc, acc};
}

// largest value over the block, to every thread
__device__ float flat_like_max(ReplaySmem &s, float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) s.red_f[threadIdx.x >> 5] = v;
  __syncthreads();
  for (int w = 0; w < kRT / 32; ++w) v = fmaxf(v, s.red_f[w]);
  __syncthreads();
  return v;
}

struct Replayed {
  int first_max;
  double cut_margin;   // relative distance of the top-p crossing from its threshold (inf without a cut)
};

// p[0..n) = the reference's probability row of x; key / idx are work space of kReplayPad entries.
// dynamic: kReplayDynamicBytes of dynamic shared memory for the bucket order (nullptr: the whole row is sorted).
__device__ Replayed replay_probabilities(ReplaySmem &s, const float *x, int n, double t, double top, double *p,
                                         unsigned long long *key, int *idx, unsigned char *dynamic = nullptr) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // first maximum (and the minimum: where the bucket grid of the order ends)
  float best = -CUDART_INF_F, low = CUDART_INF_F;
  int best_id = 0x7fffffff;
  for (int i = tid; i < n; i += kRT) {
    const float v = x[i];
    if (v > best) { best = v; best_id = i; }
    low = fminf(low, v);
  }
  low = -flat_like_max(s, -low);
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
  }
  if (lane == 0) { s.red_f[warp] = best; s.red_i[warp] = best_id; }
  __syncthreads();
  for (int w = 0; w < kRT / 32; ++w)
    if (s.red_f[w] > best || (s.red_f[w] == best && s.red_i[w] < best_id)) { best = s.red_f[w]; best_id = s.red_i[w]; }
  __syncthreads();
  Replayed out{best_id, CUDART_INF};
  const double xb = double(best);
  for (int i = tid; i < n; i += kRT) p[i] = exp_nonpos((double(x[i]) - xb) / t);
  __syncthreads();
  const double z = sequential_sum(s, n, [p](int i) { return p[i]; });
  bool bucketed = dynamic != nullptr && top < 1.0;
  BucketOrder b{};
  if (bucketed) b = bucket_begin(dynamic, n, 1.0 / z, exp_nonpos((double(low) - xb) / t) / z);
  for (int i = tid; i < n; i += kRT) {
    const double v = p[i] / z;
    p[i] = v;
    if (bucketed) bucket_count(b, v);
  }
  __syncthreads();
  if (top < 1.0) {
    // order: p descending, id ascending (positive doubles order like their bit patterns); mass += p[idx[k++]] while
    // k < n and mass < top
    SeqResult c{-1, 0.0, 0.0};
    if (bucketed) {
      bucket_scatter(s, b, p, key, idx);
      bool fits;
      c = chain_over_chunks(s, b, p, key, idx, [top](double mass) { return !(mass < top); }, &fits);
      if (!fits) bucketed = false;
    }
    if (!bucketed) {
      for (int i = tid; i < kReplayPad; i += kRT) {
        key[i] = i < n ? ~(unsigned long long)__double_as_longlong(p[i]) : ~0ull;
        idx[i] = i < n ? i : 0x7fffffff;
      }
      __syncthreads();
      sort_pairs(s, key, idx);
      c = exact_sequential(s, n, [p, idx](int i) { return p[idx[i]]; }, [top](double mass) { return !(mass < top); });
    }
    const int k = c.found >= 0 ? c.found + 1 : n;
    const double mass = c.acc, prev = c.before;
    // how far the crossing is from flipping: the kept prefix reached top by (mass - top), the one before missed it by (top - prev)
    out.cut_margin = k >= n && mass < top ? (top - mass) / top : fmin(mass - top, top - prev) / top;
    // the rest is zeroed and every p divided by the kept mass; kept = the order's first k = everything up to the k-th pair
    // (the loop ran through without reaching top: everything is kept)
    const unsigned long long cut_key = c.found >= 0 ? key[k - 1] : ~0ull;
    const int cut_id = c.found >= 0 ? idx[k - 1] : 0x7fffffff;
    __syncthreads();
    for (int i = tid; i < n; i += kRT) {
      const double v = p[i];
      const unsigned long long kk = ~(unsigned long long)__double_as_longlong(v);
      p[i] = (kk < cut_key || (kk == cut_key && i <= cut_id)) ? v / mass : 0.0;
    }
    __syncthreads();
  }
  return out;
}

// draw(p, n, u) of the reference over the values value(0) .. value(n-1); *margin = relative distance of u * z from the two
// CDF steps around the chosen id; *total = z.  Returns -1 when z is not positive (the reference throws "empty residual
// support").
template <class Value>
__device__ int replay_draw(ReplaySmem &s, int n, double u, Value value, double *margin, double *total = nullptr) {
  const double z = sequential_sum(s, n, value);
  if (total) *total = z;
  if (!(z > 0)) { *margin = 0.0; return -1; }
  const double target = u * z;
  const SeqResult c = exact_sequential(s, n, value, [target](double acc) { return target < acc; });
  const int found = c.found;
  const double c_at = c.acc, c_before = c.before;
  int last = -1;
  if (found < 0) {   // the last index with a positive value
    for (int i = threadIdx.x; i < n; i += kRT)
      if (value(i) > 0) last = i;
    if (threadIdx.x == 0) s.bcast_i[0] = -1;
    __syncthreads();
    if (last >= 0) atomicMax(&s.bcast_i[0], last);
    __syncthreads();
    last = s.bcast_i[0];
    __syncthreads();
  }
  if (found < 0) { *margin = 0.0; return last; }  // rounding left the target past the last step: the reference returns `last`
  *margin = fmin(c_at - target, target - c_before) / z;
  return found;
}

}  // namespace
}  // namespace ds41
