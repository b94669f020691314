// Batch path of the sampler for WIDE nuclei (flat distributions) at batch sizes where a thread-block cluster per row
// leaves the GPU idle most of the time: the wide-nucleus algorithm of row_wide.cuh restated as five grid-wide kernels
// over the whole batch, so that every pass runs at full occupancy.
//   flat_stats_kernel   (row, 1/4 or 1/8 row)  maximum (first), minimum, finiteness                         -> FlatPartial
//   flat_hist_kernel    (row, 1/4 or 1/8 row) 1024-bin histogram over the row's range: exact counts and fixed-point
//                                           FP32-class masses, shared memory first, then global integer atomics
//   flat_window_kernel  (row)               error-bracketed running mass -> the window of bins that holds the top-p
//                                           crossing; rows this path does not fit get status -8 (the caller sends
//                                           them to the other paths), non-finite rows -1
//   flat_mass_kernel    (row, 1/4 or 1/8 row) the one FP64 pass: per 1024-id sub-region the normaliser part, the mass
//                                           and count of the ids before the window; the window's ids to a per-row list
//   flat_resolve_kernel (row)               sorts the list exactly, FP64 prefix sums -> certified cut; kept mass per
//                                           sub-region -> the sub-region that holds u * total -> walks its 1024 ids
// Rule, error bounds and status words are those of the cluster kernel (row_kernel.cuh, row_wide.cuh); the reference
// rule is engine/third_party/spark/src/sampling.cpp:18-38.
#include "flat.cuh"

#include "row_core.cuh"

namespace ds41 {
namespace {

constexpr int kFT = kFlatThreads;
constexpr int kFW = kFT / 32;

__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct FlatRed {  // per-CTA scratch for block reductions / prefix sums
  double d[kFW], e[kFW];
  float f[kFW], g[kFW];
  int i[kFW], j[kFW];
};

// Inclusive prefix over 2 * kFT values, two consecutive per thread; returns the prefix through v0.
__device__ __forceinline__ double flat_prefix2(FlatRed &r, double v0, double v1) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double scan = v0 + v1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(0xffffffffu, scan, o);
    if (lane >= o) scan += up;
  }
  if (lane == 31) r.d[warp] = scan;
  __syncthreads();
  double base = 0;
  for (int w = 0; w < warp; ++w) base += r.d[w];
  __syncthreads();
  return base + scan - v1;
}
__device__ __forceinline__ int flat_sum(FlatRed &r, int v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = __reduce_add_sync(0xffffffffu, v);
  if (lane == 0) r.i[warp] = v;
  __syncthreads();
  int t = 0;
  for (int w = 0; w < kFW; ++w) t += r.i[w];
  __syncthreads();
  return t;
}
__device__ __forceinline__ double flat_sum(FlatRed &r, double v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) r.d[warp] = v;
  __syncthreads();
  double t = 0;
  for (int w = 0; w < kFW; ++w) t += r.d[w];
  __syncthreads();
  return t;
}

// ids [begin, end) of this CTA's quarter row
__device__ __forceinline__ void quarter(const FlatArgs &a, int chunk, int *begin, int *end) {
  const int ids = kFlatSub * (kFlatSubs / a.chunks);
  *begin = min(a.vocab, chunk * ids);
  *end = min(a.vocab, *begin + ids);
}

__global__ void __launch_bounds__(kFT) flat_stats_kernel(FlatArgs a) {
  __shared__ FlatRed red;
  const int row = blockIdx.x / a.chunks, chunk = blockIdx.x % a.chunks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int begin, end;
  quarter(a, chunk, &begin, &end);
  const float *x = a.logits + size_t(row) * a.stride;
  float best = -CUDART_INF_F, lowest = CUDART_INF_F;
  int best_id = 0x7fffffff, flags = 0;
  auto take = [&](float v, int id) {
    if ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) flags = 1;
    if (v > best) { best = v; best_id = id; }
    lowest = fminf(lowest, v);
  };
  const int vec_end = begin + ((end - begin) & ~3);  // begin is a multiple of 4, rows are 16-byte aligned
  for (int i = begin + 4 * threadIdx.x; i < vec_end; i += 4 * kFT) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + i));
    take(v.x, i); take(v.y, i + 1); take(v.z, i + 2); take(v.w, i + 3);
  }
  for (int i = vec_end + threadIdx.x; i < end; i += kFT) take(__ldg(x + i), i);
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
    lowest = fminf(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
  }
  flags = int(__reduce_or_sync(0xffffffffu, unsigned(flags)));
  if (lane == 0) { red.f[warp] = best; red.i[warp] = best_id; red.g[warp] = lowest; red.j[warp] = flags; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kFW; ++w) {
      if (red.f[w] > best || (red.f[w] == best && red.i[w] < best_id)) { best = red.f[w]; best_id = red.i[w]; }
      lowest = fminf(lowest, red.g[w]);
      flags |= red.j[w];
    }
    a.s.partial[row * kFlatMaxChunks + chunk] = FlatPartial{best, lowest, best_id, flags};
  }
}

// Row maximum (first), minimum and flags from the quarter rows' partial results; the same in every thread.
__device__ __forceinline__ FlatPartial row_extremes(const FlatArgs &a, int row) {
  FlatPartial r = a.s.partial[row * kFlatMaxChunks];
  for (int c = 1; c < a.chunks; ++c) {
    const FlatPartial p = a.s.partial[row * kFlatMaxChunks + c];
    if (p.max > r.max || (p.max == r.max && p.argmax < r.argmax)) { r.max = p.max; r.argmax = p.argmax; }
    r.min = fminf(r.min, p.min);
    r.flags |= p.flags;
  }
  return r;
}

struct FlatBins {  // binning of one row: bin = min(1023, int((max - y) * inv_w))
  float m, range, inv_w, c32, step;
  float c_lo;  // log2(e)/T = c32 + c_lo to 2^-48
};
__device__ __forceinline__ FlatBins make_bins(const FlatPartial &e, double t) {
  FlatBins b;
  b.m = e.max;
  const double c64 = 1.4426950408889634074 / t;
  b.c32 = float(c64);
  b.c_lo = float(c64 - double(b.c32));
  b.range = (e.max - e.min) * 1.0001f + 1e-30f;
  b.inv_w = float(kFlatBins) / b.range;
  b.step = b.range / float(kFlatBins) * b.c32;  // bin width in units of the exponent of 2
  return b;
}

// Histogram mass of an id of bin k, in fixed point relative to the weight at the bin's near edge:
// Q = round(2^24 * w / 2^-(k*step)), w = 2^-X, X = (m - y) * log2(e)/T.  X is formed in double-float (the difference by
// TwoSum, the product with the constant split in two floats: good to 3 * 2^-47 relative), the exponent k*step - X of
// the quotient with one fused multiply-add from its head (|quotient exponent| <= step, so the rounding there is below
// 2^-29 absolute), ex2.approx is within 2^-22, the product by 2^24 within 2^-24 and the rounding to an integer within
// 2^-25 of a value above 0.94 * 2^24.  Relative error of Q * 2^-24 * 2^-(k*step) as a weight: below 2.9e-7 (test:
// against long double); integer accumulation adds nothing.  The two halves of Q go to two 32-bit shared-memory words
// (a CTA sees at most 32768 ids: 32768 * 65535 and 32768 * 512 both fit), i.e. two integer atomics per id.
constexpr double kHistRel = 3.2e-7;  // 2.9e-7 rounded up
__device__ __forceinline__ unsigned fixed_weight(float y, const FlatBins &b, int *bin) {
  const float s = __fsub_rn(b.m, y);
  const float bb = __fsub_rn(s, b.m);
  const float ed = __fadd_rn(__fsub_rn(b.m, __fsub_rn(s, bb)), __fsub_rn(-y, bb));  // m - y = s + ed exactly
  const float p = __fmul_rn(s, b.c32);
  const float pe = __fmaf_rn(s, b.c32, -p);                                         // s * c32 = p + pe exactly
  const float q = __fmaf_rn(s, b.c_lo, __fmaf_rn(ed, b.c32, pe));                   // X = p + q
  const int k = min(kFlatBins - 1, int(__fmul_rn(s, b.inv_w)));
  *bin = k;
  const float r = __fsub_rn(__fmaf_rn(float(k), b.step, -p), q);                    // k*step - X, in [-step, 0] but for the last bin
  // (the bin index comes from a differently rounded quotient than the edge k*step, so r can exceed 0 by a few 1e-5:
  // the quotient is allowed above 1; the cap only guards the 32-bit sums against a wild value)
  return min(33554431u, __float2uint_rn(__fmul_rn(16777216.f, ex2_approx(r))));
}

__global__ void __launch_bounds__(kFT) flat_hist_kernel(FlatArgs a) {
  __shared__ unsigned lo16[kFlatBins], hi8[kFlatBins];
  const int row = blockIdx.x / a.chunks, chunk = blockIdx.x % a.chunks;
  const FlatPartial ext = row_extremes(a, row);
  if (ext.flags || !(ext.min < ext.max)) return;  // the window kernel reports the row
  const FlatBins b = make_bins(ext, a.t);
  for (int j = threadIdx.x; j < kFlatBins; j += kFT) { lo16[j] = 0u; hi8[j] = 0u; }
  __syncthreads();
  int begin, end;
  quarter(a, chunk, &begin, &end);
  const float *x = a.logits + size_t(row) * a.stride;
  auto take = [&](float y) {
    int k;
    const unsigned q = fixed_weight(y, b, &k);
    atomicAdd(&lo16[k], q & 0xffffu);
    atomicAdd(&hi8[k], q >> 16);
  };
  const int vec_end = begin + ((end - begin) & ~3);
  for (int i = begin + 4 * threadIdx.x; i < vec_end; i += 4 * kFT) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + i));
    take(v.x); take(v.y); take(v.z); take(v.w);
  }
  for (int i = vec_end + threadIdx.x; i < end; i += kFT) take(__ldg(x + i));
  __syncthreads();
  for (int j = threadIdx.x; j < kFlatBins; j += kFT) {
    const unsigned long long q = ((unsigned long long)hi8[j] << 16) + lo16[j];
    if (q) atomicAdd(&a.s.hmass[size_t(row) * kFlatBins + j], q);
  }
}

__global__ void __launch_bounds__(kFT) flat_window_kernel(FlatArgs a) {
  __shared__ FlatRed red;
  __shared__ int first[2];
  __shared__ double totals[2];
  const int row = blockIdx.x;
  const FlatPartial ext = row_extremes(a, row);
  FlatInfo info{};
  info.max = ext.max; info.min = ext.min; info.argmax = ext.argmax;
  if (ext.flags) {  // same answer in every thread
    if (threadIdx.x == 0) {
      a.s.info[row] = info;
      a.tokens[row] = -1;
      a.status[row] = -1;
    }
    return;
  }
  const FlatBins b = make_bins(ext, a.t);
  // ids of a bin, bracketed from its fixed-point mass (every id adds between 0.94 * 2^24 and 2^24): enough to tell a
  // wide nucleus from a small one and whether the window fits the list; the exact counts come from the FP64 pass
  int cnt_lo[2] = {0, 0}, cnt_hi[2] = {0, 0};
  double lo[2] = {0, 0}, hi[2] = {0, 0}, mid[2] = {0, 0};
  if (ext.min < ext.max) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = 2 * threadIdx.x + i;
      const unsigned long long q = a.s.hmass[size_t(row) * kFlatBins + k];
      const double mass = double(q) * 5.9604644775390625e-8 * exp2(-double(k) * double(b.step));
      mid[i] = mass;
      lo[i] = mass * (1.0 - kHistRel); hi[i] = mass * (1.0 + kHistRel);
      cnt_lo[i] = int(double(q) * 5.9604644775390625e-8 / 1.001);                // every id adds at most 1.001 * 2^24
      cnt_hi[i] = int((double(q) * 5.9604644775390625e-8) / 0.94) + (q ? 1 : 0);  // and at least 0.94 * 2^24 (step <= 0.08)
    }
  }
  const double lo0 = flat_prefix2(red, lo[0], lo[1]), hi0 = flat_prefix2(red, hi[0], hi[1]);
  if (threadIdx.x == kFT - 1) { totals[0] = lo0 + lo[1]; totals[1] = hi0 + hi[1]; }
  if (threadIdx.x == 0) { first[0] = 0x7fffffff; first[1] = 0x7fffffff; }
  __syncthreads();
  const double t_lo = a.top_p * totals[0] * (1.0 - 1e-12), t_hi = a.top_p * totals[1] * (1.0 + 1e-12);
  // w0: first bin through which the running mass MAY reach the target; w1: first through which it SURELY does
  if (hi0 >= t_lo) atomicMin(&first[0], 2 * threadIdx.x); else if (hi0 + hi[1] >= t_lo) atomicMin(&first[0], 2 * threadIdx.x + 1);
  if (lo0 >= t_hi) atomicMin(&first[1], 2 * threadIdx.x); else if (lo0 + lo[1] >= t_hi) atomicMin(&first[1], 2 * threadIdx.x + 1);
  __syncthreads();
  const int w0 = first[0], w1 = first[1];
  const bool found = w0 != 0x7fffffff && w1 != 0x7fffffff && w1 >= w0;
  int through = 0, inside = 0;
  if (found) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = 2 * threadIdx.x + i;
      if (k <= w1) { through += cnt_lo[i]; if (k >= w0) inside += cnt_hi[i]; }
    }
  }
  through = flat_sum(red, through);
  inside = flat_sum(red, inside);
  // this path's case: a window exists, the nucleus is wide (a small one is the other paths' case), the window fits
  // the list, and the bins are narrow enough for the count bracket above (step <= 0.08: any row whose range times
  // 1.44/T is below 82)
  const bool ok = found && through > kFlatMinNucleus && inside <= kFlatList && b.step <= 0.08f;
  // mass of the ids beyond the window, as the histogram has it: their only use is as part of the normaliser
  double beyond = 0;
  if (found) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (2 * threadIdx.x + i > w1) beyond += mid[i];
  }
  beyond = flat_sum(red, beyond);
  if (threadIdx.x == 0) {
    info.applicable = ok ? 1 : 0; info.w0 = w0; info.w1 = w1; info.tail = beyond;
    a.s.info[row] = info;
    if (!ok) { a.tokens[row] = -1; a.status[row] = -8; }
  }
}

// The ids beyond the window only enter the normaliser, hold less than 1 - top_p of it, and the histogram pass already
// has their mass to kHistRel: the FP64 pass skips them.
__global__ void __launch_bounds__(kFT, 2) flat_mass_kernel(FlatArgs a) {
  // per-warp queue of the ids that need an FP64 weight (before or inside the window): position in the sub-region
  __shared__ float queue_y[kFW][256];
  __shared__ unsigned short queue_at[kFW][256];
  const int row = blockIdx.x / a.chunks, chunk = blockIdx.x % a.chunks;
  const FlatInfo info = a.s.info[row];
  if (!info.applicable) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  FlatPartial ext{info.max, info.min, info.argmax, 0};
  const FlatBins b = make_bins(ext, a.t);
  const float edge0 = float(info.w0), edge1 = info.w1 >= kFlatBins - 1 ? CUDART_INF_F : float(info.w1 + 1);
  const double inv_t = 1.0 / a.t, m64 = double(info.max);
  const float *x = a.logits + size_t(row) * a.stride;
  const int subs_per_warp = kFlatSubs / a.chunks / kFW;  // 2 or 1
#pragma unroll 1
  for (int s = 0; s < subs_per_warp; ++s) {
    const int sub = chunk * (kFlatSubs / a.chunks) + warp * subs_per_warp + s;
    const int base = sub * kFlatSub;
    double z = 0, sure_mass = 0;
    int sure_count = 0;
    int head = 0, count = 0;                // queue state, warp-uniform
    // FP64 weights of up to 32 queued ids (lane i takes entry head + i)
    auto drain = [&](int take) {
      const bool mine = lane < take;
      const int slot = (head + lane) & 255;
      const float y = mine ? queue_y[warp][slot] : 0.f;
      const int id = base + (mine ? int(queue_at[warp][slot]) : 0);
      bool inside = false;
      if (mine) {
        const double e = exp_nonpos((double(y) - m64) * inv_t);
        z += e;
        // bin(y) < w0 without forming the bin: int(v) < k is v < k for v >= 0
        const bool sure = (b.m - y) * b.inv_w < edge0;
        if (sure) { sure_mass += e; ++sure_count; }
        inside = !sure;
      }
      const unsigned ballot = __ballot_sync(0xffffffffu, inside);
      if (ballot) {
        int slot0 = 0;
        if (lane == 0) slot0 = atomicAdd(&a.s.lcount[row * 4], __popc(ballot));
        slot0 = __shfl_sync(0xffffffffu, slot0, 0);
        if (inside) {
          const int at = slot0 + __popc(ballot & ((1u << lane) - 1u));
          // ascending 64-bit key = (logit descending, id ascending); +0 and -0 compare equal as logits: both map to +0
          const float yy = y == 0.f ? 0.f : y;
          const uint32_t bits = __float_as_uint(yy), ordered = bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
          if (at < kFlatList) a.s.lkeys[size_t(row) * kFlatList + at] = (unsigned long long)(~ordered) << 32 | uint32_t(id);
        }
      }
      head = (head + take) & 255;
      count -= take;
      __syncwarp();  // the drained slots may be written again
    };
    // 128 ids per round (one 16-byte load per lane), the next round's load in flight while this one is processed
    auto fetch = [&](int j) {
      const int id = base + (j * 32 + lane) * 4;
      float4 v;
      if (id + 3 < a.vocab) {
        v = __ldg(reinterpret_cast<const float4 *>(x + id));
      } else {
        v.x = id < a.vocab ? __ldg(x + id) : 0.f;
        v.y = id + 1 < a.vocab ? __ldg(x + id + 1) : 0.f;
        v.z = id + 2 < a.vocab ? __ldg(x + id + 2) : 0.f;
        v.w = 0.f;
      }
      return v;
    };
    float4 cur = fetch(0);
#pragma unroll 1
    for (int j = 0; j < kFlatSub / 128; ++j) {
      const float4 nxt = j + 1 < kFlatSub / 128 ? fetch(j + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float ys4[4] = {cur.x, cur.y, cur.z, cur.w};
      const int at0 = (j * 32 + lane) * 4;
      // ids up to the window's far edge go to the FP64 queue, the others are skipped; the lane's (up to four) queue
      // entries are placed with one warp-wide prefix of the lanes' counts (three votes on the bits of the count)
      int mine = 0;
      bool near[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float y = ys4[q4];
        const bool valid = base + at0 + q4 < a.vocab;
        near[q4] = valid && (b.m - y) * b.inv_w < edge1;
        mine += near[q4] ? 1 : 0;
      }
      const unsigned below = (1u << lane) - 1u;
      const unsigned v1 = __ballot_sync(0xffffffffu, mine & 1), v2 = __ballot_sync(0xffffffffu, mine & 2),
                     v4 = __ballot_sync(0xffffffffu, mine & 4);
      int slot = head + count + __popc(v1 & below) + 2 * __popc(v2 & below) + 4 * __popc(v4 & below);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        if (near[q4]) {
          queue_y[warp][slot & 255] = ys4[q4];
          queue_at[warp][slot & 255] = (unsigned short)(at0 + q4);
          ++slot;
        }
      }
      count += __popc(v1) + 2 * __popc(v2) + 4 * __popc(v4);
      __syncwarp();
      while (count >= 32) drain(32);
      cur = nxt;
    }
    if (count > 0) drain(count);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      z += __shfl_xor_sync(0xffffffffu, z, o);
      sure_mass += __shfl_xor_sync(0xffffffffu, sure_mass, o);
    }
    sure_count = __reduce_add_sync(0xffffffffu, sure_count);
    if (lane == 0) {
      a.s.subz[size_t(row) * kFlatSubs + sub] = z;
      a.s.subsure[size_t(row) * kFlatSubs + sub] = sure_mass;
      a.s.subcnt[size_t(row) * kFlatSubs + sub] = sure_count;
    }
  }
}

__global__ void __launch_bounds__(kFT) flat_resolve_kernel(FlatArgs a) {
  __shared__ FlatRed red;
  __shared__ unsigned long long keys[kFlatList];
  __shared__ double ksum[kFlatSubs];
  __shared__ int found_at;
  __shared__ double cut_mass[2];
  __shared__ float cut_y;
  __shared__ int cut_id, cut_amb;
  const int row = blockIdx.x;
  const FlatInfo info = a.s.info[row];
  if (!info.applicable) return;
  const int tid = threadIdx.x, lane = tid & 31;
  const double inv_t = 1.0 / a.t, m64 = double(info.max);
  const float *x = a.logits + size_t(row) * a.stride;
  const int listed = a.s.lcount[row * 4];
  // normaliser, mass and count before the window: fixed order (sub-regions across threads, then the block tree)
  double z = 0, mass_before = 0;
  const double tail = info.tail;  // ids beyond the window, from the histogram pass (relative error kHistRel)
  int n_before = 0;
  if (tid < kFlatSubs) {
    z = a.s.subz[size_t(row) * kFlatSubs + tid];
    mass_before = a.s.subsure[size_t(row) * kFlatSubs + tid];
    n_before = a.s.subcnt[size_t(row) * kFlatSubs + tid];
    ksum[tid] = mass_before;
  }
  z = flat_sum(red, z) + tail;
  mass_before = flat_sum(red, mass_before);
  n_before = flat_sum(red, n_before);
  bool ok = listed >= 1 && listed <= kFlatList;
  const int n = ok ? listed : 0;
  int padded = 64;
  while (padded < n) padded <<= 1;
  for (int i = tid; i < padded; i += kFT) keys[i] = i < n ? a.s.lkeys[size_t(row) * kFlatList + i] : ~0ull;
  __syncthreads();
  if (padded <= kFT) {
    // bitonic network, one key per thread: partners closer than a warp exchange by shuffle, the others through
    // shared memory
    unsigned long long key = tid < padded ? keys[tid] : ~0ull;
    for (int k = 2; k <= padded; k <<= 1) {
      for (int jj = k >> 1; jj > 0; jj >>= 1) {
        unsigned long long other;
        if (jj < 32) {
          other = __shfl_xor_sync(0xffffffffu, key, jj);
        } else {
          keys[tid] = key;
          __syncthreads();
          other = keys[tid ^ jj];
          __syncthreads();
        }
        const bool keep_min = ((tid & jj) == 0) == ((tid & k) == 0);
        key = keep_min ? (key < other ? key : other) : (key < other ? other : key);
      }
    }
    keys[tid] = key;
    __syncthreads();
  } else {
    for (int k = 2; k <= padded; k <<= 1) {
      for (int jj = k >> 1; jj > 0; jj >>= 1) {
        for (int i = tid; i < padded / 2; i += kFT) {
          const int lo_i = ((i / jj) * 2 * jj) + (i % jj), hi_i = lo_i + jj;
          const bool up = (lo_i & k) == 0;
          const unsigned long long p = keys[lo_i], q = keys[hi_i];
          if ((p > q) == up) { keys[lo_i] = q; keys[hi_i] = p; }
        }
        __syncthreads();
      }
    }
  }
  // FP64 weights in sorted order and their prefix sums from the mass before the window
  double e[2];
  float ys[2];
  int ids[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = 2 * tid + i;
    const unsigned long long key = r < n ? keys[r] : 0ull;
    const uint32_t ordered = r < n ? ~uint32_t(key >> 32) : 0x80000000u;
    ys[i] = __uint_as_float(ordered ^ ((ordered >> 31) ? 0x80000000u : 0xffffffffu));
    ids[i] = int(uint32_t(key));
    e[i] = r < n ? exp_nonpos((double(ys[i]) - m64) * inv_t) : 0.0;
  }
  const double through0 = mass_before + flat_prefix2(red, e[0], e[1]), through1 = through0 + e[1];
  const double rel = 2.0 * (double(a.vocab) + 256.0) * kU;
  // Two attempts at the crossing.  First with the normaliser as the earlier passes left it: the ids beyond the window
  // enter it with the histogram's FP32-class masses, so their share of z carries a relative error kHistRel.  If the crossing falls inside
  // that wider bound (about one row in a hundred), this CTA recomputes the tail of its row with FP64 weights and
  // decides again with the FP64 bound alone.
  const FlatBins b = make_bins(FlatPartial{info.max, info.min, info.argmax, 0}, a.t);
  const float edge1 = info.w1 >= kFlatBins - 1 ? CUDART_INF_F : float(info.w1 + 1);
  double tail_abs = a.top_p * (kHistRel * tail + 1e-30);
  int pos = 0x7fffffff;
  for (int attempt = 0; attempt < 2; ++attempt) {
    const double target_p = a.top_p * z, lo = target_p * (1.0 - rel) - tail_abs, hi = target_p * (1.0 + rel) + tail_abs;
    if (tid == 0) { found_at = 0x7fffffff; cut_amb = 0; }
    __syncthreads();
    {
      int mine = -1;
      if (2 * tid < n && through0 >= target_p) mine = 2 * tid;
      else if (2 * tid + 1 < n && through1 >= target_p) mine = 2 * tid + 1;
      if (mine >= 0) atomicMin(&found_at, mine);
    }
    __syncthreads();
    pos = found_at;
    // mass_before >= lo: the crossing is (or may be) before the window; pos unset: not reached inside it
    if (!(ok && mass_before < lo && pos != 0x7fffffff)) { ok = false; break; }
    if ((pos >> 1) == tid) {
      const int i = pos & 1;
      const double mass_at = i ? through1 : through0, prev_at = mass_at - e[i];
      cut_amb = ((mass_at < hi) || (prev_at >= lo)) ? 1 : 0;
      cut_y = ys[i]; cut_id = ids[i];
      cut_mass[0] = mass_at;
    }
    __syncthreads();
    if (!cut_amb || attempt == 1) break;
    // FP64 weights of the ids beyond the window (the same predicate as the mass pass)
    double exact = 0;
    auto add_tail = [&](float y) {
      const double w = exp_nonpos((double(y) - m64) * inv_t);  // unconditional: independent calls overlap
      exact += ((b.m - y) * b.inv_w < edge1) ? 0.0 : w;
    };
    const int vec_end = a.vocab & ~3;  // rows are 16-byte aligned
    for (int id0 = 4 * tid; id0 < vec_end; id0 += 16 * kFT) {  // four 16-byte loads in flight per thread
      float4 v[4];
#pragma unroll
      for (int u4 = 0; u4 < 4; ++u4) {
        const int id = id0 + u4 * 4 * kFT;
        v[u4] = id < vec_end ? __ldg(reinterpret_cast<const float4 *>(x + id))
                             : make_float4(CUDART_INF_F, CUDART_INF_F, CUDART_INF_F, CUDART_INF_F);  // +inf: not tail
      }
#pragma unroll
      for (int u4 = 0; u4 < 4; ++u4) { add_tail(v[u4].x); add_tail(v[u4].y); add_tail(v[u4].z); add_tail(v[u4].w); }
    }
    for (int id = vec_end + tid; id < a.vocab; id += kFT) add_tail(__ldg(x + id));
    exact = flat_sum(red, exact);
    z = (z - tail) + exact;
    tail_abs = 0;
  }
  if (!ok) {  // uniform in the CTA: the cluster kernel redoes the row (the nucleus is wide: no candidate set covers it)
    if (tid == 0) { a.tokens[row] = -1; a.status[row] = kNeedsCluster; }
    return;
  }
  const int uncertified_cut = cut_amb;  // still inside the FP64 bound: decided, flagged like every other path does
  // kept mass per sub-region: the ids before the window plus the window's ids up to the cut
#pragma unroll
  for (int i = 0; i < 2; ++i)
    if (2 * tid + i <= pos) atomicAdd(&ksum[ids[i] / kFlatSub], e[i]);
  __syncthreads();
  const Cut cut{cut_y, cut_id};
  const int kept = n_before + pos + 1;
  int status = uncertified_cut ? 2 : 0;
  // ---- inverse CDF in id order (sampling.cpp:18-21): sub-region that holds u * total, then its ids one by one
  const double k0 = tid < kFlatSubs / 2 ? ksum[2 * tid] : 0.0, k1 = tid < kFlatSubs / 2 ? ksum[2 * tid + 1] : 0.0;
  const double pre0 = flat_prefix2(red, k0, k1), pre1 = pre0 + k1;  // kept mass through sub-region 2*tid (and 2*tid+1)
  if (tid == kFT - 1) cut_mass[1] = pre1;  // total (threads beyond the sub-regions add zeros)
  if (tid == 0) found_at = 0x7fffffff;
  __syncthreads();
  const double total = cut_mass[1];
  const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
  const double target = u * total, slack = (2.0 * kept + 512.0) * kU * total;
  if (tid < kFlatSubs / 2) {
    int mine = -1;
    if (k0 > 0 && target < pre0) mine = 2 * tid;
    else if (k1 > 0 && target < pre1) mine = 2 * tid + 1;
    if (mine >= 0) atomicMin(&found_at, mine);
  }
  __syncthreads();
  int sub = found_at;
  bool amb = false;
  if (sub == 0x7fffffff) {  // target >= total by rounding: the last sub-region with kept mass, flagged
    amb = true;
    if (tid == 0) found_at = -1;
    __syncthreads();
    if (tid < kFlatSubs && ksum[tid] > 0) atomicMax(&found_at, tid);
    __syncthreads();
    sub = found_at;
  }
  if (sub < 0) {  // cannot happen (the maximum has weight 1): leave the row to the other paths
    if (tid == 0) { a.tokens[row] = -1; a.status[row] = -8; }
    return;
  }
  // kept mass before the sub-region, as the prefix above saw it
  __syncthreads();
  if ((sub >> 1) == tid) cut_mass[0] = (sub & 1) ? pre0 : pre0 - k0;
  if (tid == 0) found_at = 0x7fffffff;
  __syncthreads();
  const double carry = cut_mass[0];
  double v[2];
  int vid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    vid[i] = sub * kFlatSub + 2 * tid + i;
    const bool in = vid[i] < a.vocab;
    const float y = in ? __ldg(x + vid[i]) : -CUDART_INF_F;
    const double w = exp_nonpos((double(y) - m64) * inv_t);
    v[i] = (in && survives(y, vid[i], cut)) ? w : 0.0;
  }
  const double c0 = carry + flat_prefix2(red, v[0], v[1]), c1 = c0 + v[1];
  {
    int mine = -1;
    if (v[0] > 0 && target < c0) mine = 2 * tid;
    else if (v[1] > 0 && target < c1) mine = 2 * tid + 1;
    if (mine >= 0) atomicMin(&found_at, mine);
  }
  __syncthreads();
  const int hit = found_at;
  if (hit == 0x7fffffff) {
    // rounding left the target past the sub-region's last step: its last kept id, flagged (as the cluster kernel)
    if (tid == 0) found_at = -1;
    __syncthreads();
    if (v[1] > 0) atomicMax(&found_at, 2 * tid + 1); else if (v[0] > 0) atomicMax(&found_at, 2 * tid);
    __syncthreads();
    if (tid == 0) {
      a.tokens[row] = found_at >= 0 ? sub * kFlatSub + found_at : -1;
      a.status[row] = found_at >= 0 ? (status | 1) : -8;
    }
    return;
  }
  if ((hit >> 1) == tid) {
    const int i = hit & 1;
    const double cum = i ? c1 : c0, below = cum - v[i];
    if ((cum - target < slack) || (below > 0 && target - below < slack)) amb = true;
    a.tokens[row] = vid[i];
    a.status[row] = status | (amb ? 1 : 0);
  }
  (void)lane;
}

__global__ void hist_probe_kernel(const float *y, FlatBins b, double *out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int k;
  const unsigned q = fixed_weight(y[i], b, &k);
  out[i] = double(q) * 5.9604644775390625e-8 * exp2(-double(k) * double(b.step));
}

}  // namespace

cudaError_t launch_hist_probe(const float *y, float max_logit, float min_logit, double t, double *out, int n,
                              cudaStream_t stream) {
  FlatBins b;
  {  // make_bins is device code; the same arithmetic on the host (FP32 operations are IEEE on both sides)
    const double c64 = 1.4426950408889634074 / t;
    b.m = max_logit;
    b.c32 = float(c64);
    b.c_lo = float(c64 - double(b.c32));
    b.range = (max_logit - min_logit) * 1.0001f + 1e-30f;
    b.inv_w = float(kFlatBins) / b.range;
    b.step = b.range / float(kFlatBins) * b.c32;
  }
  hist_probe_kernel<<<(n + 255) / 256, 256, 0, stream>>>(y, b, out, n);
  return cudaGetLastError();
}

size_t flat_scratch_bytes(int rows) {
  size_t per_row = kFlatMaxChunks * sizeof(FlatPartial) + kFlatBins * (sizeof(unsigned) + sizeof(unsigned long long)) +
                   sizeof(FlatInfo) + kFlatSubs * (2 * sizeof(double) + sizeof(int)) + 4 * sizeof(int) +
                   kFlatList * sizeof(unsigned long long);
  return size_t(rows) * per_row + 256;
}

cudaError_t launch_flat(FlatArgs a, void *scratch, cudaStream_t stream) {
  // carve (every array is a multiple of 16 bytes per row; the zeroed ones come first, in one block)
  unsigned char *p = static_cast<unsigned char *>(scratch);
  const size_t rows = size_t(a.rows);
  a.s.hmass = reinterpret_cast<unsigned long long *>(p); p += rows * kFlatBins * sizeof(unsigned long long);
  p += rows * kFlatBins * sizeof(unsigned);  // (spare)
  a.s.lcount = reinterpret_cast<int *>(p); p += rows * 4 * sizeof(int);
  const size_t zeroed = size_t(p - static_cast<unsigned char *>(scratch));
  a.s.lkeys = reinterpret_cast<unsigned long long *>(p); p += rows * kFlatList * sizeof(unsigned long long);
  a.s.subz = reinterpret_cast<double *>(p); p += rows * kFlatSubs * sizeof(double);
  a.s.subsure = reinterpret_cast<double *>(p); p += rows * kFlatSubs * sizeof(double);
  a.s.info = reinterpret_cast<FlatInfo *>(p); p += rows * sizeof(FlatInfo);
  a.s.partial = reinterpret_cast<FlatPartial *>(p); p += rows * kFlatMaxChunks * sizeof(FlatPartial);
  a.s.subcnt = reinterpret_cast<int *>(p);
  cudaError_t e = cudaMemsetAsync(scratch, 0, zeroed, stream);
  if (e != cudaSuccess) return e;
  a.chunks = a.rows >= 512 ? 4 : 8;  // fewer rows: more, shorter CTAs per row
  flat_stats_kernel<<<a.rows * a.chunks, kFT, 0, stream>>>(a);
  flat_hist_kernel<<<a.rows * a.chunks, kFT, 0, stream>>>(a);
  flat_window_kernel<<<a.rows, kFT, 0, stream>>>(a);
  flat_mass_kernel<<<a.rows * a.chunks, kFT, 0, stream>>>(a);
  flat_resolve_kernel<<<a.rows, kFT, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ds41
