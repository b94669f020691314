// Batch path of the sampler: top-p rows (no penalties, bitmask or top-k) decided by grid-wide kernels over the whole
// batch, every pass at full occupancy, the logits read twice.
//   flat_stats_kernel   (row, part)  maximum (first), minimum, finiteness -> FlatPartial.  Skipped when the FP8 head's
//                                    epilogue already delivered them (HeadRowStats).
//   flat_hist_kernel    (row, part)  2048-bin histogram over the row's range.  Per id ONE shared-memory integer atomic
//                                    that adds 1 to the bin's count and the id's place inside the bin (0..127) to the
//                                    bin's place sum.  Count and first moment bracket the bin's mass from both sides
//                                    (Jensen below, the chord above) to a few 1e-5.
//   flat_window_kernel  (row)        bracketed running mass -> the window of bins that provably holds the top-p crossing,
//                                    exact id counts before and inside it.  Rows this path does not fit get status -8
//                                    (the caller sends them to the other paths), non-finite rows -1.
//   flat_mass_kernel    (row, part)  the FP64 pass, dense and branch free: every id's weight 2^-((max-y)*log2(e)/T) from a
//                                    256-entry table and a degree-4 polynomial (12 FP64 instructions per id); per 1024-id
//                                    sub-region the sum over all ids and over the ids before the window; the window's
//                                    ids go to a per-row list.
//   flat_resolve_kernel (row)        sorts the list exactly, FP64 prefix sums -> certified cut; kept mass per sub-region
//                                    -> the sub-region that holds u * total -> walks its 1024 ids.
// Rule, error bounds and status words are those of the cluster kernel (row_kernel.cuh); the reference rule is
// engine/third_party/spark/src/sampling.cpp:18-38.
#include "flat.cuh"

#include "row_core.cuh"
#include "phase_events.h"

namespace ds41 {
namespace {

constexpr int kFT = kFlatThreads;
constexpr int kFW = kFT / 32;

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
// Exclusive prefix of one value per thread, and the total.
__device__ __forceinline__ double flat_exclusive(FlatRed &r, double v, double *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double scan = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(0xffffffffu, scan, o);
    if (lane >= o) scan += up;
  }
  if (lane == 31) r.e[warp] = scan;
  __syncthreads();
  double base = 0, all = 0;
  for (int w = 0; w < kFW; ++w) {
    if (w < warp) base += r.e[w];
    all += r.e[w];
  }
  __syncthreads();
  *total = all;
  return base + scan - v;
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

// ids [begin, end) of one of the row's `parts` pieces (whole sub-regions)
__device__ __forceinline__ void piece(const FlatArgs &a, int part, int *begin, int *end) {
  const int ids = kFlatSub * (kFlatSubs / a.parts);
  *begin = min(a.vocab, part * ids);
  *end = min(a.vocab, *begin + ids);
}

__device__ __forceinline__ float unorder(uint32_t o) {
  return __uint_as_float(o ^ ((o >> 31) ? 0x80000000u : 0xffffffffu));
}

// Row maximum (first), minimum and flags: from the head's record, or from the pieces' partial results.  The same in
// every thread.
__device__ __forceinline__ FlatPartial row_extremes(const FlatArgs &a, int row) {
  if (a.head_stats) {
    const HeadRowStats h = a.head_stats[row];
    FlatPartial r;
    r.max = unorder(uint32_t(h.max_key >> 32));
    r.argmax = int(0xffffffffu - uint32_t(h.max_key));
    r.min = unorder(~h.min_key);
    r.flags = int(h.flags & 1u);
    return r;
  }
  FlatPartial r = a.s.partial[row * kFlatMaxParts];
  for (int c = 1; c < a.parts; ++c) {
    const FlatPartial p = a.s.partial[row * kFlatMaxParts + c];
    if (p.max > r.max || (p.max == r.max && p.argmax < r.argmax)) { r.max = p.max; r.argmax = p.argmax; }
    r.min = fminf(r.min, p.min);
    r.flags |= p.flags;
  }
  return r;
}

__global__ void __launch_bounds__(kFT) flat_stats_kernel(FlatArgs a) {
  __shared__ FlatRed red;
  const int row = blockIdx.x / a.parts, part = blockIdx.x % a.parts;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int begin, end;
  piece(a, part, &begin, &end);
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
    a.s.partial[row * kFlatMaxParts + part] = FlatPartial{best, lowest, best_id, flags};
  }
}

// Placement of the ids of one row.  place(y) = fl(fl(max - y) * scale) in FP32 (two roundings, monotone in y) runs over
// [0, kFlatQMax + 1); q = int(place) is the id's position, q / kFlatFrac its bin.  The same expression is evaluated by
// the histogram pass and by the mass pass, so both see every id in the same bin.  In real numbers
// (max - y) * scale lies within 3 * 2^-24 relative of place(y), and the weight's exponent is
// X = (max - y) * log2(e)/T = (max - y) * scale * kappa.
struct FlatMap {
  float m, scale;
  double kappa;  // exponent (base 2) per unit of position
  bool ok;       // the row has a usable range
};
constexpr double kLog2e = 1.4426950408889634074;
constexpr double kPlaceRel = 1.8e-7;  // 3 * 2^-24, rounded up
__device__ __forceinline__ FlatMap make_map(const FlatPartial &e, double t) {
  FlatMap b;
  b.m = e.max;
  const float range = __fsub_rn(e.max, e.min);
  b.ok = e.min < e.max && range >= 1e-30f && range <= 3e38f;
  // 0.999998: the largest place, fl(range * scale), stays below kFlatQMax + 1 after its two roundings
  b.scale = __fdiv_rn(float(kFlatQMax + 1) * 0.999998f, b.ok ? range : 1.f);
  b.kappa = (kLog2e / t) / double(b.scale);
  b.ok = b.ok && double(range) * (kLog2e / t) <= kFlatMaxExponent;
  return b;
}
__device__ __forceinline__ float place(float y, const FlatMap &b) { return __fmul_rn(__fsub_rn(b.m, y), b.scale); }

// One shared-memory word per bin: count in the upper 14 bits, sum of the places inside the bin in the lower 18.  A
// field that overflows (more than 16383 ids of one CTA in one bin, or a place sum above 2^18) makes the sum of the
// count fields differ from the number of ids the CTA has seen; the row is then left to the other paths.
__global__ void __launch_bounds__(kFT) flat_hist_kernel(FlatArgs a) {
  __shared__ unsigned bins[kFlatBins];
  __shared__ FlatRed red;
  const int row = blockIdx.x / a.parts, part = blockIdx.x % a.parts;
  const FlatPartial ext = row_extremes(a, row);
  const FlatMap b = make_map(ext, a.t);
  if (ext.flags || !b.ok) return;  // the window kernel reports the row
  for (int j = threadIdx.x; j < kFlatBins; j += kFT) bins[j] = 0u;
  __syncthreads();
  int begin, end;
  piece(a, part, &begin, &end);
  const float *x = a.logits + size_t(row) * a.stride;
  auto take = [&](float y) {
    // (the conversion saturates: a logit above the recorded maximum, or a NaN, lands in bin 0 instead of outside the array)
    const int q = int(min(unsigned(kFlatQMax), __float2uint_rz(place(y, b))));
    atomicAdd(&bins[q >> 7], 0x40000u | unsigned(q & (kFlatFrac - 1)));
  };
  const int vec_end = begin + ((end - begin) & ~3);
  int i = begin + 4 * threadIdx.x;
  for (; i + 12 * kFT < vec_end; i += 16 * kFT) {  // four 16-byte loads in flight per thread
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __ldg(reinterpret_cast<const float4 *>(x + i + 4 * kFT * k));
#pragma unroll
    for (int k = 0; k < 4; ++k) { take(v[k].x); take(v[k].y); take(v[k].z); take(v[k].w); }
  }
  for (; i < vec_end; i += 4 * kFT) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + i));
    take(v.x); take(v.y); take(v.z); take(v.w);
  }
  for (int k = vec_end + threadIdx.x; k < end; k += kFT) take(__ldg(x + k));
  __syncthreads();
  int seen = 0;
  unsigned long long *out = a.s.hist + size_t(row) * kFlatBins;
  for (int j = threadIdx.x; j < kFlatBins; j += kFT) {
    const unsigned v = bins[j];
    seen += int(v >> 18);
    const unsigned long long add = (unsigned long long)(v >> 18) << 32 | (v & 0x3ffffu);
    if (a.parts == 1) out[j] = add;
    else if (v) atomicAdd(&out[j], add);
  }
  seen = flat_sum(red, seen);
  if (threadIdx.x == 0 && seen != end - begin) atomicOr(&a.s.lcount[row * 4 + 1], 1);
}

// 2^-x for x >= 0 in FP64 (a few ulp; the brackets below allow 1e-12)
__device__ __forceinline__ double pow2_neg(double x) { return exp_nonpos(-0.69314718055994530942 * x); }

// The bracket of a bin's mass.  The ids of bin k have positions q = 128 k + f, f = 0..127, exponents X in
// [q (1 - r) kappa, (q + 1)(1 + r) kappa] (r = kPlaceRel) and weights 2^-X.  With n ids and S = sum of their f:
//   above: sum 2^-(q (1-r) kappa) = 2^-(128 k kl) * sum 2^-(f kl) <= 2^-(128 k kl) * (n - S * (1 - 2^-(127 kl)) / 127)
//          (2^-(f kl) is convex in f: it lies below its chord over [0, 127]),  kl = (1 - r) kappa
//   below: sum 2^-((q+1)(1+r) kappa) = 2^-((128 k + 1) kh) * sum 2^-(f kh) >= 2^-((128 k + 1) kh) * n * 2^-(S/n * kh)
//          (Jensen),  kh = (1 + r) kappa
// The two differ by about kappa * ln 2 (one position) plus (128 kappa ln 2)^2 / 8 (the curvature over a bin) relative.
__global__ void __launch_bounds__(kFT) flat_window_kernel(FlatArgs a) {
  __shared__ FlatRed red;
  __shared__ int first[2];
  const int row = blockIdx.x, tid = threadIdx.x;
  const FlatPartial ext = row_extremes(a, row);
  FlatInfo info{};
  info.max = ext.max; info.min = ext.min; info.argmax = ext.argmax;
  if (ext.flags) {  // same answer in every thread
    if (tid == 0) {
      a.s.info[row] = info;
      a.tokens[row] = -1;
      a.status[row] = -1;
    }
    return;
  }
  const FlatMap b = make_map(ext, a.t);
  const bool full = a.top_p >= 1.0;  // no cut: every id is kept, the histogram pass did not run
  bool usable = b.ok && (full || a.s.lcount[row * 4 + 1] == 0);
  if (!usable || full) {
    if (tid == 0) {
      info.applicable = usable ? 1 : 0;
      info.w0 = kFlatBins; info.w1 = kFlatBins - 1; info.n_before = a.vocab; info.n_window = 0;
      info.y_sure = -CUDART_INF_F; info.y_tail = -CUDART_INF_F;  // every (finite) logit is before the window
      a.s.info[row] = info;
      if (!usable) { a.tokens[row] = -1; a.status[row] = -8; atomicAdd(a.s.pending, 1); }
    }
    return;
  }
  constexpr int kPer = kFlatBins / kFT;  // 4 consecutive bins per thread
  const double kl = b.kappa * (1.0 - kPlaceRel), kh = b.kappa * (1.0 + kPlaceRel);
  const double chord = (1.0 - pow2_neg(double(kFlatFrac - 1) * kl)) / double(kFlatFrac - 1);
  double lo[kPer], hi[kPer];
  int cnt[kPer];
  double lo_sum = 0, hi_sum = 0;
  // prefactors of the thread's first bin, then one multiplication per bin (three steps: within the 1e-12 allowance)
  const double ratio_l = pow2_neg(double(kFlatFrac) * kl), ratio_h = pow2_neg(double(kFlatFrac) * kh);
  double above = pow2_neg(double(kFlatFrac * kPer * tid) * kl), below = pow2_neg(double(kFlatFrac * kPer * tid + 1) * kh);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int k = kPer * tid + i;
    const unsigned long long v = a.s.hist[size_t(row) * kFlatBins + k];
    const double n = double(uint32_t(v >> 32)), s = double(uint32_t(v));
    cnt[i] = int(uint32_t(v >> 32));
    lo[i] = hi[i] = 0;
    if (cnt[i] > 0) {
      hi[i] = above * (n - s * chord) * (1.0 + 1e-12);
      // 2^-(S/n * kh) = e^-x >= 1 - x + x^2/2 - x^3/6 for x >= 0 (x is at most the width of a bin, below 0.06)
      const double x = (s / n) * kh * 0.69314718055994530942;
      const double jensen = fma(x, fma(x, fma(x, -1.0 / 6.0, 0.5), -1.0), 1.0);
      lo[i] = below * jensen * n * (1.0 - 1e-12);
    }
    above *= ratio_l; below *= ratio_h;
    lo_sum += lo[i]; hi_sum += hi[i];
  }
  double z_lo, z_hi;
  const double lo0 = flat_exclusive(red, lo_sum, &z_lo), hi0 = flat_exclusive(red, hi_sum, &z_hi);
  if (tid == 0) { first[0] = 0x7fffffff; first[1] = 0x7fffffff; }
  __syncthreads();
  // the reference's own sums carry a relative rounding error of about vocab * 2^-53 (1.5e-11): 1e-9 covers it
  const double t_lo = a.top_p * z_lo * (1.0 - 1e-9), t_hi = a.top_p * z_hi * (1.0 + 1e-9);
  {  // w0: first bin through which the running mass MAY reach the target; w1: first through which it SURELY has
    double run_lo = lo0, run_hi = hi0;
    int f0 = 0x7fffffff, f1 = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      run_lo += lo[i]; run_hi += hi[i];
      if (f0 == 0x7fffffff && run_hi >= t_lo) f0 = kPer * tid + i;
      if (f1 == 0x7fffffff && run_lo >= t_hi) f1 = kPer * tid + i;
    }
    if (f0 != 0x7fffffff) atomicMin(&first[0], f0);
    if (f1 != 0x7fffffff) atomicMin(&first[1], f1);
  }
  __syncthreads();
  const int w0 = first[0];
  const int w1 = first[1] == 0x7fffffff ? kFlatBins - 1 : first[1];  // never surely reached: the window runs to the end
  const bool found = w0 != 0x7fffffff && w1 >= w0;
  // the mass pass draws the window a quarter of a bin wider on both sides, so its list holds at most the ids of the
  // bins w0 - 1 .. w1 + 1
  int before = 0, inside = 0, listed_most = 0;
  if (found) {
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int k = kPer * tid + i;
      if (k < w0) before += cnt[i];
      else if (k <= w1) inside += cnt[i];
      if (k >= w0 - 1 && k <= w1 + 1) listed_most += cnt[i];
    }
  }
  before = flat_sum(red, before);
  inside = flat_sum(red, inside);
  listed_most = flat_sum(red, listed_most);
  const bool ok = found && inside >= 1 && listed_most <= kFlatList;
  if (tid == 0) {
    info.applicable = ok ? 1 : 0; info.w0 = w0; info.w1 = w1; info.n_before = before; info.n_window = inside;
    if (ok) {
      const double quarter = double(kFlatFrac / 4);
      info.y_sure = float(double(b.m) - (double(kFlatFrac) * w0 - quarter) / double(b.scale));
      info.y_tail = float(double(b.m) - (double(kFlatFrac) * (w1 + 1) + quarter) / double(b.scale));
    }
    a.s.info[row] = info;
    if (!ok) { a.tokens[row] = -1; a.status[row] = -8; atomicAdd(a.s.pending, 1); }
  }
}

// 2^(-j/64), j = 0..63, correctly rounded
static __device__ const double kPow2Neg64[64] = {
#include "pow2neg64.inc"
};

// Weight of one id in the FP64 pass: 2^-X, X = (max - y) * log2(e)/T >= 0, as 2^-(n >> 6) * table[n & 63] * 2^(-r/64)
// with n = round(64 X) and r = 64 X - n.  n comes from FP32 arithmetic (it only chooses the expansion point: its
// error, below 0.002, widens |r| to 0.502), r from one FP64 fused multiply-add of the exact difference max - y, the last
// factor from its Taylor polynomial of degree 4 (|r ln 2 / 64| <= 5.44e-3: truncation below 4e-14 relative).  The table
// has 64 entries (512 bytes, four rows of shared memory) so that a warp's 32 lookups cost few wavefronts.  Error of a
// weight: 360 * 2^-53 from the truncation, 2 X ln 2 * 2^-53 from the roundings of max - y and of the product, 1.5 ulp from
// the table entry and the polynomial's arithmetic: below kFlatWeightUlps * 2^-53 for X <= kFlatMaxExponent, which the
// resolve kernel's bounds allow for.  Ten FP64 instructions with the two accumulations, none of them a branch.
constexpr double kFlatWeightUlps = 1024.0;
struct WeightRow {     // per-row constants of the weight routine
  float m, k32;        // maximum; 64 * log2(e)/T
  double m64, k64;
  const double *table; // shared-memory copy of kPow2Neg64
};
__device__ __forceinline__ double row_weight(float y, const WeightRow &w) {
  const float kf = fmaf(__fsub_rn(w.m, y), w.k32, 12582912.f);  // 1.5 * 2^23 + round(64 X)
  const int n = __float_as_int(kf) & 0x3fffff;
  const double nd = double(__fsub_rn(kf, 12582912.f));           // the same integer, exactly
  const double d = w.m64 - double(y);
  const double r = fma(d, w.k64, -nd);
  constexpr double b1 = -0x1.62e42fefa39efp-7, b2 = 0x1.ebfbdff82c58fp-15, b3 = -0x1.c6b08d704a0c0p-23,
                   b4 = 0x1.3b2ab6fba4e77p-31;  // (-ln 2 / 64)^k / k!
  double q = fma(r, b4, b3);
  q = fma(q, r, b2);
  q = fma(q, r, b1);
  q *= r;
  const double tb = w.table[n & 63];
  const double v = fma(tb, q, tb);
  return __hiloint2double(__double2hiint(v) - ((n >> 6) << 20), __double2loint(v));
}

// Window ids met by one warp in one sub-region wait in a small shared-memory buffer (a sub-region of 1024 ids holds
// about three of them) and go to the row's list at the end of the sub-region with one global atomic per warp.
constexpr int kWarpWindowCap = 96;
struct WarpWindow {
  int count;
  float y[kWarpWindowCap];
  int id[kWarpWindowCap];
};

template <bool kWhole>
__device__ __forceinline__ void mass_sub_region(const FlatArgs &a, const FlatInfo &info, const WeightRow &w, const float *x,
                                                int row, int base, int lane, WarpWindow *mine, double *z_out,
                                                double *sure_out) {
  double zc[2] = {0, 0}, sc[2] = {0, 0};
  const float y_sure = info.y_sure, y_tail = info.y_tail;
  // a lane's j-th 16-byte load of the sub-region: ids base + (32 j + lane) * 4 .. + 3, j = 0..7
  auto fetch = [&](int j) {
    const int id = base + (j * 32 + lane) * 4;
    float4 v;
    if (kWhole) {
      v = __ldg(reinterpret_cast<const float4 *>(x + id));
    } else {  // the row's last, partial sub-region: ids beyond the vocabulary read as the maximum and are masked below
      v.x = id < a.vocab ? __ldg(x + id) : info.max;
      v.y = id + 1 < a.vocab ? __ldg(x + id + 1) : info.max;
      v.z = id + 2 < a.vocab ? __ldg(x + id + 2) : info.max;
      v.w = id + 3 < a.vocab ? __ldg(x + id + 3) : info.max;
    }
    return v;
  };
  auto consume = [&](const float4 &v, int j) {
    const float ys[4] = {v.x, v.y, v.z, v.w};
    const int id0 = base + (j * 32 + lane) * 4;
    unsigned outside = 1u;  // 0 once one of the four ids is neither before nor beyond the window
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float y = ys[k];
      double e = row_weight(y, w);
      if (!kWhole) e = id0 + k < a.vocab ? e : 0.0;   // (an id beyond the vocabulary reads as the maximum: weight 0 here)
      zc[k & 1] += e;
      // sc += e for the ids before the window, as one predicated addition (no select of e against 0)
      asm("{\n .reg .pred p;\n setp.gt.f32 p, %2, %3;\n @p add.f64 %0, %0, %1;\n}" : "+d"(sc[k & 1]) : "d"(e), "f"(y), "f"(y_sure));
      outside &= unsigned(y > y_sure) | unsigned(y < y_tail);
    }
    if (!outside) {  // a handful of the row's ids: the window's
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if ((kWhole || id0 + k < a.vocab) && !(ys[k] > y_sure) && !(ys[k] < y_tail)) {
          const int at = atomicAdd(&mine->count, 1);
          if (at < kWarpWindowCap) { mine->y[at] = ys[k]; mine->id[at] = id0 + k; }
        }
      }
    }
  };
  // two loads are consumed while the next two are in flight; the loop stays rolled (two rounds per trip, so that the
  // two register sets alternate without copies) and its body fits the instruction cache
  float4 a0 = fetch(0), a1 = fetch(1), b0, b1;
#pragma unroll 1
  for (int j = 0; j < 8; j += 4) {
    b0 = fetch(j + 2); b1 = fetch(j + 3);
    consume(a0, j); consume(a1, j + 1);
    if (j + 4 < 8) { a0 = fetch(j + 4); a1 = fetch(j + 5); }
    consume(b0, j + 2); consume(b1, j + 3);
  }
  *z_out = zc[0] + zc[1];
  *sure_out = sc[0] + sc[1];
  // hand the buffered window ids to the row's list
  __syncwarp();
  const int n = mine->count;
  if (n > 0) {
    int slot0 = 0;
    if (lane == 0) slot0 = atomicAdd(&a.s.lcount[row * 4], n);
    slot0 = __shfl_sync(0xffffffffu, slot0, 0);
    if (n > kWarpWindowCap) {  // more window ids in one sub-region than the buffer holds: the row goes to another path
      if (lane == 0) atomicOr(&a.s.lcount[row * 4 + 1], 2);
    } else {
      unsigned long long *keys = a.s.lkeys + size_t(row) * kFlatList;
      for (int i = lane; i < n; i += 32) {
        // ascending 64-bit key = (logit descending, id ascending); +0 and -0 compare equal as logits: both map to +0
        const float yy = mine->y[i] == 0.f ? 0.f : mine->y[i];
        const uint32_t bits = __float_as_uint(yy), ordered = bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
        if (slot0 + i < kFlatList) keys[slot0 + i] = (unsigned long long)(~ordered) << 32 | uint32_t(mine->id[i]);
      }
    }
    __syncwarp();
    if (lane == 0) mine->count = 0;
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kFlatMassThreads, 5) flat_mass_kernel(FlatArgs a) {
  __shared__ double table[64];
  __shared__ WarpWindow windows[kFlatMassThreads / 32];
  const int row = blockIdx.x / a.parts, part = blockIdx.x % a.parts;
  const FlatInfo info = a.s.info[row];
  if (!info.applicable) return;
  if (threadIdx.x < 64) table[threadIdx.x] = kPow2Neg64[threadIdx.x];
  if (threadIdx.x < kFlatMassThreads / 32) windows[threadIdx.x].count = 0;
  __syncthreads();
  const double k64 = 64.0 * (kLog2e / a.t);
  const WeightRow w{info.max, float(k64), double(info.max), k64, table};
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *x = a.logits + size_t(row) * a.stride;
  const int subs = kFlatSubs / a.parts;
#pragma unroll 1
  for (int s = warp; s < subs; s += kFlatMassThreads / 32) {
    const int sub = part * subs + s;
    const int base = sub * kFlatSub;
    double z = 0, sure_mass = 0;
    if (base + kFlatSub <= a.vocab) mass_sub_region<true>(a, info, w, x, row, base, lane, &windows[warp], &z, &sure_mass);
    else if (base < a.vocab) mass_sub_region<false>(a, info, w, x, row, base, lane, &windows[warp], &z, &sure_mass);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      z += __shfl_xor_sync(0xffffffffu, z, o);
      sure_mass += __shfl_xor_sync(0xffffffffu, sure_mass, o);
    }
    if (lane == 0) {
      a.s.subz[size_t(row) * kFlatSubs + sub] = z;
      a.s.subsure[size_t(row) * kFlatSubs + sub] = sure_mass;
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
  const int tid = threadIdx.x;
  const double inv_t = 1.0 / a.t, m64 = double(info.max);
  const float *x = a.logits + size_t(row) * a.stride;
  const bool full = info.w0 >= kFlatBins;  // top_p = 1: every id is kept
  const int listed = a.s.lcount[row * 4];
  // normaliser, mass and count before the window: fixed order (sub-regions across threads, then the block tree)
  double z = 0, mass_before = 0;
  if (tid < kFlatSubs) {
    z = a.s.subz[size_t(row) * kFlatSubs + tid];
    mass_before = a.s.subsure[size_t(row) * kFlatSubs + tid];
    ksum[tid] = mass_before;
  }
  // the reference's chain for the normaliser rounds by at most 2^-53 times the SUM OF ITS PARTIAL SUMS (each addition
  // errs by half an ulp of its own result); that sum is at most 1024 * (normaliser through sub-region j) over the
  // sub-regions j: about half of vocab * z on a row without structure, instead of the worst case vocab * z
  double z_total;
  const double z_through = flat_exclusive(red, z, &z_total) + z;
  const double chain_terms = double(kFlatSub) * flat_sum(red, tid < kFlatSubs ? z_through : 0.0) / z_total * (1.0 + 1e-9);
  z = z_total;
  mass_before = flat_sum(red, mass_before);
  bool ok = listed <= kFlatList && (full || listed >= 1) && (a.s.lcount[row * 4 + 1] & 2) == 0;
  const int n = ok ? listed : 0;
  int pos = -1;
  int status = 0;
  Cut cut{-CUDART_INF_F, -1};
  int kept = a.vocab;
  if (!full) {
    int padded = 64;
    while (padded < n) padded <<= 1;
    for (int i = tid; i < padded; i += kFT) keys[i] = i < n ? a.s.lkeys[size_t(row) * kFlatList + i] : ~0ull;
    __syncthreads();
    {
      // bitonic network, two adjacent keys per thread (positions 2 tid, 2 tid + 1): partners at distance 1 are in the
      // same thread, up to distance 32 in the same warp (shuffles), only the wider ones go through shared memory
      const bool live = 2 * tid < padded;
      unsigned long long k0 = live ? keys[2 * tid] : ~0ull, k1 = live ? keys[2 * tid + 1] : ~0ull;
      const int i0 = 2 * tid;
      for (int k = 2; k <= padded; k <<= 1) {
        const bool up = (i0 & k) == 0;   // (bit 0 of the position plays no part for k >= 2)
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
          if (jj == 1) {
            if ((k0 > k1) == up) { const unsigned long long t = k0; k0 = k1; k1 = t; }
            continue;
          }
          unsigned long long o0, o1;
          if (jj <= 32) {
            o0 = __shfl_xor_sync(0xffffffffu, k0, jj >> 1);
            o1 = __shfl_xor_sync(0xffffffffu, k1, jj >> 1);
          } else {
            __syncthreads();
            if (live) { keys[i0] = k0; keys[i0 + 1] = k1; }
            __syncthreads();
            o0 = live ? keys[i0 ^ jj] : ~0ull;
            o1 = live ? keys[(i0 + 1) ^ jj] : ~0ull;
          }
          const bool keep_min = ((i0 & jj) == 0) == up;
          k0 = keep_min ? (k0 < o0 ? k0 : o0) : (k0 < o0 ? o0 : k0);
          k1 = keep_min ? (k1 < o1 ? k1 : o1) : (k1 < o1 ? o1 : k1);
        }
      }
      __syncthreads();
      if (live) { keys[i0] = k0; keys[i0 + 1] = k1; }
      __syncthreads();
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
    // The reference's test is chain(p_i, i <= k) >= top with p_i = w_i / chain(w, all n ids): its two chains round by at
    // most (k - 1) units (k <= the ids above the window plus the window's) and chain_terms units (see above; at most
    // n - 1); the sums here add a few hundred.
    const double k_bound = fmin(double(a.vocab), double(info.n_before) + double(n));
    const double rel = (k_bound + fmin(double(a.vocab), chain_terms) + 2.0 * kFlatWeightUlps + 512.0) * kU * a.bound_scale;
    const double target_p = a.top_p * z, lo = target_p * (1.0 - rel), hi = target_p * (1.0 + rel);
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
    if (!(ok && mass_before < lo && pos != 0x7fffffff)) ok = false;
    if (ok && (pos >> 1) == tid) {
      const int i = pos & 1;
      const double mass_at = i ? through1 : through0, prev_at = mass_at - e[i];
      cut_amb = ((mass_at < hi) || (prev_at >= lo)) ? 1 : 0;
      cut_y = ys[i]; cut_id = ids[i];
    }
    __syncthreads();
    if (ok) {
      // kept mass per sub-region: the ids before the window plus the window's ids up to the cut
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (2 * tid + i <= pos) atomicAdd(&ksum[ids[i] / kFlatSub], e[i]);
      cut = Cut{cut_y, cut_id};
      kept = min(a.vocab, info.n_before + pos + 1);  // ids with weight in the draw: those above the window and the window's up to the cut
      status = cut_amb ? 2 : 0;  // inside the FP64 bound: decided, flagged like every other path does
    }
    __syncthreads();
  }
  if (!ok) {  // uniform in the CTA: the cluster kernel redoes the row (the nucleus may be wide: no candidate set covers it)
    if (tid == 0) { a.tokens[row] = -1; a.status[row] = kNeedsCluster; atomicAdd(a.s.pending, 1); }
    return;
  }
  // ---- inverse CDF in id order (sampling.cpp:18-21): sub-region that holds u * total, then its ids one by one
  const double k0 = tid < kFlatSubs / 2 ? ksum[2 * tid] : 0.0, k1 = tid < kFlatSubs / 2 ? ksum[2 * tid + 1] : 0.0;
  const double pre0 = flat_prefix2(red, k0, k1), pre1 = pre0 + k1;  // kept mass through sub-region 2*tid (and 2*tid+1)
  if (tid == kFT - 1) cut_mass[1] = pre1;  // total (threads beyond the sub-regions add zeros)
  if (tid == 0) found_at = 0x7fffffff;
  __syncthreads();
  const double total = cut_mass[1];
  const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
  const double target = u * total, slack = 2.0 * (double(kept) + kFlatWeightUlps) * kU * total * a.bound_scale;
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
    __syncthreads();
    if (tid == 0) found_at = -1;
    __syncthreads();
    if (tid < kFlatSubs && ksum[tid] > 0) atomicMax(&found_at, tid);
    __syncthreads();
    sub = found_at;
  }
  if (sub < 0) {  // cannot happen (the maximum has weight 1): leave the row to the other paths
    if (tid == 0) { a.tokens[row] = -1; a.status[row] = kNeedsCluster; atomicAdd(a.s.pending, 1); }
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
    __syncthreads();
    if (tid == 0) found_at = -1;
    __syncthreads();
    if (v[1] > 0) atomicMax(&found_at, 2 * tid + 1); else if (v[0] > 0) atomicMax(&found_at, 2 * tid);
    __syncthreads();
    if (tid == 0) {
      a.tokens[row] = found_at >= 0 ? sub * kFlatSub + found_at : -1;
      a.status[row] = found_at >= 0 ? (status | 1) : kNeedsCluster;
      if (found_at < 0) atomicAdd(a.s.pending, 1);
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
}

// Test hook: the weights of n logits of a row with maximum max_logit, as the FP64 pass forms them.
__global__ void flat_weight_probe_kernel(const float *y, float max_logit, double t, double *out, int n) {
  __shared__ double table[64];
  if (threadIdx.x < 64) table[threadIdx.x] = kPow2Neg64[threadIdx.x];
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double k64 = 64.0 * (kLog2e / t);
  const WeightRow w{max_logit, float(k64), double(max_logit), k64, table};
  out[i] = row_weight(y[i], w);
}

}  // namespace

cudaError_t launch_flat_weight_probe(const float *y, float max_logit, double t, double *out, int n, cudaStream_t stream) {
  flat_weight_probe_kernel<<<(n + 255) / 256, 256, 0, stream>>>(y, max_logit, t, out, n);
  return cudaGetLastError();
}

size_t flat_scratch_bytes(int rows) {
  size_t per_row = 4 * sizeof(int) + kFlatBins * sizeof(unsigned long long) + kFlatMaxParts * sizeof(FlatPartial) +
                   sizeof(FlatInfo) + kFlatSubs * (2 * sizeof(double)) +
                   kFlatList * sizeof(unsigned long long);
  return size_t(rows) * per_row + 256;
}

const int *flat_pending(const void *scratch) { return static_cast<const int *>(scratch); }

cudaError_t launch_flat(FlatArgs a, void *scratch, cudaStream_t stream) {
  // carve (every array is a multiple of 16 bytes per row; the zeroed ones come first, in one block)
  unsigned char *p = static_cast<unsigned char *>(scratch);
  const size_t rows = size_t(a.rows);
  a.s.pending = reinterpret_cast<int *>(p); p += 4 * sizeof(int);
  a.s.lcount = reinterpret_cast<int *>(p); p += rows * 4 * sizeof(int);
  a.s.hist = reinterpret_cast<unsigned long long *>(p); p += rows * kFlatBins * sizeof(unsigned long long);
  a.s.lkeys = reinterpret_cast<unsigned long long *>(p); p += rows * kFlatList * sizeof(unsigned long long);
  a.s.subz = reinterpret_cast<double *>(p); p += rows * kFlatSubs * sizeof(double);
  a.s.subsure = reinterpret_cast<double *>(p); p += rows * kFlatSubs * sizeof(double);
  a.s.info = reinterpret_cast<FlatInfo *>(p); p += rows * sizeof(FlatInfo);
  a.s.partial = reinterpret_cast<FlatPartial *>(p);
  // CTAs per row: one at large batches (the histogram then needs no global atomics and no clearing), more, shorter
  // ones as the batch shrinks, so that the grid still fills the GPU
  int parts = 1;
  while (parts < kFlatMaxParts && a.rows * parts < 1024) parts <<= 1;
  a.parts = parts;
  const bool full = a.top_p >= 1.0;
  const size_t zeroed = 4 * sizeof(int) + rows * 4 * sizeof(int) + (parts > 1 && !full ? rows * kFlatBins * sizeof(unsigned long long) : 0);
  cudaError_t e = cudaMemsetAsync(scratch, 0, zeroed, stream);
  if (e != cudaSuccess) return e;
  phase_restart();
  phase_mark(stream);
  if (!a.head_stats) flat_stats_kernel<<<a.rows * parts, kFT, 0, stream>>>(a);
  phase_mark(stream);
  if (!full) flat_hist_kernel<<<a.rows * parts, kFT, 0, stream>>>(a);
  phase_mark(stream);
  flat_window_kernel<<<a.rows, kFT, 0, stream>>>(a);
  phase_mark(stream);
  // the mass pass: four warps per CTA, one 1024-id sub-region per warp and round.  Five CTAs fit an SM (740 at a time on
  // the GPU), so the rows are cut into as many pieces as give about four waves or more: a grid of 1.4 waves (256 rows x
  // 4 pieces) left a third of the SMs idle through its second wave
  int mass_parts = 4;
  while (mass_parts < 16 && a.rows * mass_parts < 2960) mass_parts <<= 1;
  FlatArgs m = a;
  m.parts = mass_parts;
  flat_mass_kernel<<<a.rows * mass_parts, kFlatMassThreads, 0, stream>>>(m);
  phase_mark(stream);
  flat_resolve_kernel<<<a.rows, kFT, 0, stream>>>(a);
  phase_mark(stream);
  return cudaGetLastError();
}

}  // namespace ds41
