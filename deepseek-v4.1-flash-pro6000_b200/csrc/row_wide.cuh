// Wide-nucleus path of the row kernel: top-p rows whose nucleus may hold thousands of ids (flat distributions, e.g.
// the logits of a randomly initialised head).  The cost that matters is the FP64 exponential, so the row gets exactly
// ONE FP64 pass; what only has to be approximately right is done first in FP32-class arithmetic:
//   W1a  coarse COUNT histogram (256 bins over the row's logit range, 32-bit shared atomics) and the FP32-class total
//        z32; a bin's mass is bracketed by its count times the weights of its two edges, which yields a window of
//        coarse bins that contains the crossing of top_p * z;
//   W1b  FP32-class mass of the ids before the window, and a COUNT histogram of the window 1024 times finer; the same
//        bracketing now yields a BAND of fine bins (a few dozen ids) that provably contains the crossing;
//   W2   the FP64 pass: normaliser z, mass of the ids before the band per warp region (kept for sure), and the band's
//        ids appended to per-warp lists (positions from votes, no atomics);
//   then rank 0 ranks the band's ids exactly, walks them sequentially from the mass before the band as the reference
//   walks its sorted prefix (sampling.cpp:36), and the cut returns to every CTA, which adds its kept band ids to its
//   region sums.  The inverse-CDF draw is draw_token() as for every other row.
// Histogram totals are pulled by rank 0 from the other CTAs' shared memory.  Every step checks itself (crossing
// before / after the band, band larger than the list); on any doubt the whole cluster gets "not applicable" and the
// general search runs instead.
#pragma once
#include "row_core.cuh"

namespace ds41 {

constexpr int kBandPerWarp = 256;
constexpr int kCoarse = 256, kFine = 1024;  // histogram resolutions of the two FP32-class levels

struct WideOutcome {
  int applicable;  // 0: the general path must run (same answer in every CTA)
  Cut cut;
  int kept;
  double z, e_kept;
  int ambiguous;
};

__device__ __forceinline__ float ex2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Brackets the running mass of a count histogram and returns, to lane 0 of the calling warp, the first bin at which
// the upper bracket reaches t_lo (*first_may) and the first bin at which the lower bracket reaches t_hi (*first_sure);
// -1 if never.  Bin b covers distances whose weights lie between 2^-(x0 + b*step) and 2^-(x0 + (b+1)*step).
__device__ __forceinline__ void bracket_scan(const int *counts, int n_bins, float x0, float step, double run_lo,
                                             double run_hi, double t_lo, double t_hi, int lane, int *first_may,
                                             int *first_sure) {
  int may_bin = -1, sure_bin = -1;
  for (int base = 0; base < n_bins; base += 32) {
    const int b = base + lane;
    const double cnt = double(counts[b]);
    double hi = cnt * double(exp2f(-(x0 + float(b) * step))) * 1.00001;
    double lo = cnt * double(exp2f(-(x0 + float(b + 1) * step))) * 0.99999;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double th = __shfl_up_sync(0xffffffffu, hi, o), tl = __shfl_up_sync(0xffffffffu, lo, o);
      if (lane >= o) { hi += th; lo += tl; }
    }
    const unsigned may = __ballot_sync(0xffffffffu, run_hi + hi >= t_lo);
    const unsigned sure = __ballot_sync(0xffffffffu, run_lo + lo >= t_hi);
    if (may && may_bin < 0) may_bin = base + __ffs(may) - 1;
    if (sure && sure_bin < 0) sure_bin = base + __ffs(sure) - 1;
    run_hi += __shfl_sync(0xffffffffu, hi, 31);
    run_lo += __shfl_sync(0xffffffffu, lo, 31);
  }
  *first_may = may_bin;
  *first_sure = sure_bin;
}

// Preconditions: T > 0, top_p < 1, no top-k, the row is valid and has a finite range min_logit < max_logit.
// On success warp_sum[] holds the region sums of the kept ids.
__device__ inline WideOutcome wide_nucleus(RowCtx &c, float max_logit, float min_logit, double t, double top_p,
                                           int allowed) {
  RowSmem *s = c.s;
  WideOutcome out{};
  const float m = max_logit, c32 = float(1.4426950408889634074 / t), mc = m * c32;
  const float range = (m - min_logit) * 1.0001f + 1e-30f;
  const float inv_w = float(kCoarse) / range;
  auto coarse_bin = [&](float y) { return min(kCoarse - 1, int((m - y) * inv_w)); };
  int *bins = s->bin_count;
  // eps: relative error of an FP32-class mass (ex2.approx 2^-22, three FP32 roundings in its argument: (3+|x|)*2^-22)
  const double eps = 6e-5;

  // ---------------------------------------------------------------- W1a
  for (int j = c.tid; j < kCoarse; j += kThreads) bins[j] = 0;
  if (c.tid == 0) s->list_count = 0;
  __syncthreads();
  double sum32 = 0;
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    if (j < c.len) {
      const float y = s->y[j];
      if (y > -CUDART_INF_F) {
        atomicAdd(&bins[coarse_bin(y)], 1);
        sum32 += double(ex2_fast(fmaf(y, c32, -mc)));
      }
    }
  }
  Slot a{};
  a.d[0] = block_sum(c, sum32);
  c.cluster.sync();  // every CTA's histogram is complete; nobody touches its bins again before the exchange below
  if (c.rank == 0)
    for (int j = c.tid; j < kCoarse; j += kThreads) {
      int tot = 0;
      for (int r = 0; r < c.nranks; ++r) tot += *c.cluster.map_shared_rank(&bins[j], r);
      s->u.w.total_count[j] = tot;
    }
  const Slot *all_a = exchange(c, a);  // its barrier also orders rank 0's totals before the scan below
  double z32 = 0;
  for (int r = 0; r < c.nranks; ++r) z32 += all_a[r].d[0];
  Slot wv{};
  if (c.rank == 0) {
    if (c.warp == 0) {
      const double target = top_p * z32;
      int w0, w1;
      bracket_scan(s->u.w.total_count, kCoarse, 0.f, range / float(kCoarse) * c32, 0.0, 0.0, target * (1.0 - eps),
                   target * (1.0 + eps), c.lane, &w0, &w1);
      // a nucleus that certainly fits the candidate list is the small-support path's case
      int through = 0;
      for (int b = c.lane; b <= w1; b += 32) through += s->u.w.total_count[b];
      through = __reduce_add_sync(0xffffffffu, through);
      if (c.lane == 0) {
        s->verdict.i[0] = (w0 >= 0 && w1 >= w0 && through > kListCap / 2) ? 1 : 0;
        s->verdict.i[1] = w0; s->verdict.i[2] = w1;
      }
    }
    __syncthreads();
    wv = s->verdict;
    __syncthreads();
  }
  wv = exchange(c, wv)[0];
  if (!wv.i[0]) return out;  // same verdict in every CTA
  const int w0 = wv.i[1], w1 = wv.i[2];

  // ---------------------------------------------------------------- W1b
  const float lo_d = float(w0) / inv_w, fine_scale = float(kFine) / (float(w1 + 1) / inv_w - lo_d);
  auto fine_bin = [&](float y) { return max(0, min(kFine - 1, int(((m - y) - lo_d) * fine_scale))); };
  for (int j = c.tid; j < kFine; j += kThreads) bins[j] = 0;
  __syncthreads();
  double before32 = 0;
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    if (j < c.len) {
      const float y = s->y[j];
      if (y > -CUDART_INF_F) {
        const int cb = coarse_bin(y);
        if (cb < w0) before32 += double(ex2_fast(fmaf(y, c32, -mc)));
        else if (cb <= w1) atomicAdd(&bins[fine_bin(y)], 1);
      }
    }
  }
  Slot bb{};
  bb.d[0] = block_sum(c, before32);
  c.cluster.sync();
  if (c.rank == 0)
    for (int j = c.tid; j < kFine; j += kThreads) {
      int tot = 0;
      for (int r = 0; r < c.nranks; ++r) tot += *c.cluster.map_shared_rank(&bins[j], r);
      s->u.w.total_count[j] = tot;
    }
  const Slot *all_b = exchange(c, bb);
  double before_window = 0;
  for (int r = 0; r < c.nranks; ++r) before_window += all_b[r].d[0];
  Slot bv{};
  if (c.rank == 0) {
    if (c.warp == 0) {
      // band [f_lo, f_hi]: before f_lo even the upper bracket of the running mass is safely below the target, through
      // f_hi even the lower bracket is safely above it
      const double target = top_p * z32, t_lo = target * (1.0 - eps), t_hi = target * (1.0 + eps);
      int f_lo, f_hi;
      bracket_scan(s->u.w.total_count, kFine, lo_d * c32, c32 / fine_scale, before_window * (1.0 - eps),
                   before_window * (1.0 + eps), t_lo, t_hi, c.lane, &f_lo, &f_hi);
      if (c.lane == 0) {
        const bool ok = before_window * (1.0 + eps) < t_lo && f_lo >= 0 && f_hi >= f_lo;
        s->verdict.i[0] = ok ? 1 : 0; s->verdict.i[1] = f_lo; s->verdict.i[2] = f_hi;
      }
    }
    __syncthreads();
    bv = s->verdict;
    __syncthreads();
  }
  bv = exchange(c, bv)[0];
  if (!bv.i[0]) return out;
  const int f_lo = bv.i[1], f_hi = bv.i[2];
  // position of an id relative to the band: 0 before (kept for sure), 1 inside, 2 after
  auto where = [&](float y) {
    const int cb = coarse_bin(y);
    if (cb < w0) return 0;
    if (cb > w1) return 2;
    const int fb = fine_bin(y);
    return fb < f_lo ? 0 : (fb <= f_hi ? 1 : 2);
  };

  // ---------------------------------------------------------------- W2: the one FP64 pass
  uint16_t *band = reinterpret_cast<uint16_t *>(s->bin_mass) + c.warp * kBandPerWarp;
  const double inv_t = 1.0 / t;  // see the note on `weight` in row_kernel.cuh
  double z_lane = 0, def_lane = 0;
  int def_count = 0, n_band = 0;  // n_band is warp-uniform
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    int pos = 2;
    if (j < c.len) {
      const float y = s->y[j];
      if (y > -CUDART_INF_F) {
        const double e = exp((double(y) - double(m)) * inv_t);
        z_lane += e;
        pos = where(y);
        if (pos == 0) { def_lane += e; ++def_count; }
      }
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, pos == 1);
    if (pos == 1) {
      const int slot = n_band + __popc(ballot & ((1u << c.lane) - 1u));
      if (slot < kBandPerWarp) band[slot] = uint16_t(it + c.lane);
    }
    n_band += __popc(ballot);
  }
  double warp_def = def_lane;  // region sum of the ids kept for sure (lanes stride the region, xor tree across lanes)
#pragma unroll
  for (int o = 16; o; o >>= 1) warp_def += __shfl_xor_sync(0xffffffffu, warp_def, o);
  Slot mine{};
  mine.d[0] = block_sum(c, z_lane);
  mine.d[1] = block_sum(c, def_lane);
  mine.i[0] = block_sum(c, def_count);
  mine.i[1] = block_sum(c, c.lane == 0 ? min(n_band, kBandPerWarp) : 0);
  mine.i[2] = block_or(c, n_band > kBandPerWarp ? 1 : 0);
  const Slot *all = exchange(c, mine);
  double z = 0, mass_before = 0;
  int n_before = 0, n_in_band = 0, overflow = 0;
  for (int r = 0; r < c.nranks; ++r) {
    z += all[r].d[0]; mass_before += all[r].d[1]; n_before += all[r].i[0]; n_in_band += all[r].i[1]; overflow |= all[r].i[2];
  }
  if (overflow || n_in_band > kListCap || n_in_band == 0) return out;
  {
    int *list_count0 = c.cluster.map_shared_rank(&s->list_count, 0);
    float *list_y0 = c.cluster.map_shared_rank(s->u.w.list_y, 0);
    int *list_id0 = c.cluster.map_shared_rank(s->u.w.list_id, 0);
    for (int q = c.lane; q < n_band; q += 32) {
      const int j = c.warp * c.region + band[q];
      const int slot = atomicAdd(list_count0, 1);
      if (slot < kListCap) { list_y0[slot] = s->y[j]; list_id0[slot] = c.begin + j; }
    }
  }
  c.cluster.sync();
  Slot v{};
  if (c.rank == 0) {
    const int n = min(s->list_count, kListCap);
    double *e_sorted = reinterpret_cast<double *>(s->u.w.total_mass);
    for (int i = c.tid; i < n; i += kThreads) {  // exact position in the stable order by counting
      const float yi = s->u.w.list_y[i];
      const int idi = s->u.w.list_id[i];
      int pos = 0;
      for (int k = 0; k < n; ++k) pos += (s->u.w.list_y[k] > yi || (s->u.w.list_y[k] == yi && s->u.w.list_id[k] < idi)) ? 1 : 0;
      s->u.w.sorted_y[pos] = yi; s->u.w.sorted_id[pos] = idi;
      e_sorted[pos] = exp((double(yi) - double(m)) * inv_t);
    }
    __syncthreads();
    if (c.tid == 0) {
      const double rel = 2.0 * (double(allowed) + 256.0) * kU;
      const double target = top_p * z, lo = target * (1.0 - rel), hi = target * (1.0 + rel);
      int ok = 1, amb = 0, pos = -1;
      double mass = mass_before;
      if (mass >= lo) ok = 0;  // the crossing is (or may be) before the band: not this path's case
      for (int r = 0; r < n && ok; ++r) {
        const double prev = mass;
        mass += e_sorted[r];
        if (mass >= target) { pos = r; amb = (mass < hi) || (prev >= lo); break; }
      }
      if (pos < 0) ok = 0;  // not reached inside the band
      s->verdict.i[0] = ok; s->verdict.i[1] = amb;
      if (ok) {
        s->verdict.f[0] = s->u.w.sorted_y[pos]; s->verdict.i[2] = s->u.w.sorted_id[pos];
        s->verdict.i[3] = n_before + pos + 1; s->verdict.d[0] = mass;
      }
      s->list_count = 0;
    }
    __syncthreads();
    v = s->verdict;
    __syncthreads();
  }
  v = exchange(c, v)[0];
  if (!v.i[0]) return out;
  out.cut.y = v.f[0]; out.cut.id = v.i[2]; out.kept = v.i[3]; out.e_kept = v.d[0]; out.z = z; out.ambiguous = v.i[1];
  // ---- region sums of the kept ids: the sure ones plus this warp's band ids that made the cut (list order = id order)
  double extra = 0;
  for (int q = c.lane; q < n_band; q += 32) {
    const int j = c.warp * c.region + band[q];
    const float y = s->y[j];
    if (survives(y, c.begin + j, out.cut)) extra += exp((double(y) - double(m)) * inv_t);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) extra += __shfl_xor_sync(0xffffffffu, extra, o);
  if (c.lane == 0) s->warp_sum[c.warp] = warp_def + extra;
  __syncthreads();
  out.applicable = 1;
  return out;
}

}  // namespace ds41
