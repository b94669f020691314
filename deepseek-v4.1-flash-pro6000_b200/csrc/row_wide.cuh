// Wide-nucleus path of the row kernel: top-p rows whose nucleus may hold thousands of ids (flat distributions, e.g.
// the logits of a randomly initialised head).  What only has to be approximately right is done in FP32-class
// arithmetic with a rigorous error bracket, and the row gets exactly ONE FP64 pass:
//   W1  histogram over the row's logit range (1024 bins, shared-memory atomics): per bin the exact count and an
//       FP32-class mass (ex2.approx of an FP32 argument, float atomic adds).  Each bin's true mass lies within
//       (count + 3 ln2 |x| + 6) * 2^-24 of the measured one (accumulation, argument roundings, ex2.approx), so rank 0
//       can bracket the running mass and the total, and obtains a WINDOW of bins (normally one or two) that provably
//       contains the crossing of top_p * z;
//   W2  the FP64 pass: normaliser z, mass of the ids before the window per warp region (kept for sure), and the
//       window's ids appended to per-warp lists (positions from votes, no atomics);
//   then rank 0 sorts the window's ids exactly (bitonic network on (logit descending, id ascending) keys), takes
//   FP64 prefix sums from the mass before the window as the reference walks its sorted prefix (sampling.cpp:36), and
//   the cut returns to every CTA, which adds its kept window ids to its region sums.  The inverse-CDF draw is
//   draw_token() as for every other row.
// Histogram totals are pulled by rank 0 from the other CTAs' shared memory.  Every step checks itself (crossing
// before / after the window, window larger than the list); on any doubt the whole cluster gets "not applicable" and
// the general search runs instead.
#pragma once
#include "row_core.cuh"

namespace ds41 {

constexpr int kBandPerWarp = 256;
constexpr int kWideBins = 1024;  // = kBins: the histogram arrays of RowSmem are reused
static_assert(kWideBins == kBins && kWideBins == 2 * kThreads, "two bins per thread");

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

// Inclusive prefix sums over 2 * kThreads values, two consecutive ones per thread (v0 at 2*tid, v1 at 2*tid+1), all
// threads of one CTA; returns the prefix through v0 (the one through v1 is that plus v1).
__device__ __forceinline__ double block_prefix2(RowCtx &c, double v0, double v1) {
  RowSmem *s = c.s;
  double scan = v0 + v1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(0xffffffffu, scan, o);
    if (c.lane >= o) scan += up;
  }
  if (c.lane == 31) s->red_d[c.warp] = scan;
  __syncthreads();
  double base = 0;
  for (int w = 0; w < c.warp; ++w) base += s->red_d[w];
  __syncthreads();
  return base + scan - v1;
}
// The same for three sequences at once (a and b doubles, n integers) with one pair of barriers; also returns the OR of
// `flag` over the CTA.
__device__ __forceinline__ void block_prefix2x3(RowCtx &c, const double (&a)[2], const double (&b)[2], const int (&n)[2],
                                                int flag, double *a0, double *b0, int *n0, int *any) {
  RowSmem *s = c.s;
  double sa = a[0] + a[1], sb = b[0] + b[1];
  int sn = n[0] + n[1];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double ua = __shfl_up_sync(0xffffffffu, sa, o), ub = __shfl_up_sync(0xffffffffu, sb, o);
    const int un = __shfl_up_sync(0xffffffffu, sn, o);
    if (c.lane >= o) { sa += ua; sb += ub; sn += un; }
  }
  flag = int(__reduce_or_sync(0xffffffffu, unsigned(flag)));
  if (c.lane == 31) {
    s->red_d[c.warp] = sa; s->red_q[c.warp] = (unsigned long long)__double_as_longlong(sb);
    s->red_i[c.warp] = sn; s->red_j[c.warp] = flag;
  }
  __syncthreads();
  double base_a = 0, base_b = 0;
  int base_n = 0, f = 0;
  for (int w = 0; w < kWarps; ++w) {
    if (w < c.warp) { base_a += s->red_d[w]; base_b += __longlong_as_double((long long)s->red_q[w]); base_n += s->red_i[w]; }
    f |= s->red_j[w];
  }
  __syncthreads();
  *a0 = base_a + sa - a[1]; *b0 = base_b + sb - b[1]; *n0 = base_n + sn - n[1]; *any = f;
}

// Preconditions: T > 0, top_p < 1, no top-k, the row is valid and has a finite range min_logit < max_logit.
// On success warp_sum[] holds the region sums of the kept ids.
__device__ inline WideOutcome wide_nucleus(RowCtx &c, float max_logit, float min_logit, double t, double top_p,
                                           int allowed) {
  RowSmem *s = c.s;
  WideOutcome out{};
  const float m = max_logit, c32 = float(1.4426950408889634074 / t);
  const float range = (m - min_logit) * 1.0001f + 1e-30f;
  const float inv_w = float(kWideBins) / range;
  int *bins = s->bin_count;
  unsigned *qmass = reinterpret_cast<unsigned *>(s->bin_mass);
  // per-bin mass in fixed point, relative to the weight at the bin's near edge: an id of bin b adds
  // round(2^20 * w / 2^-(b*step)), a number in (2^19, 2^20], so integer atomics accumulate it exactly
  const float step = range / float(kWideBins) * c32;  // bin width in units of the exponent of 2

  for (int j = c.tid; j < kWideBins; j += kThreads) { bins[j] = 0; qmass[j] = 0u; }
  if (c.tid == 0) s->list_count = 0;
  __syncthreads();
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    if (j < c.len) {
      const float y = s->y[j];
      if (y > -CUDART_INF_F) {
        const float d = m - y;
        const int b = min(kWideBins - 1, int(d * inv_w));
        atomicAdd(&bins[b], 1);
        atomicAdd(&qmass[b], __float2uint_rn(1048576.f * ex2_fast(fmaf(float(b), step, -(d * c32)))));
      }
    }
  }
  c.cluster.sync();  // every CTA's histogram is complete; nobody touches it again before the outcome exchange below
  // Every CTA totals its own segment of the bins over all CTAs' histograms (remote shared-memory loads), brackets
  // the masses, and takes prefix sums inside the segment; the segment totals then go round the cluster, which gives
  // every CTA the total bracket and its segment's offset, and a second round agrees on the window.
  const int seg = kWideBins / c.nranks;  // cluster sizes are powers of two
  const int b0 = c.rank * seg + 2 * c.tid;
  const bool active = 2 * c.tid < seg;
  int cnt[2] = {0, 0};
  double lo[2] = {0, 0}, hi[2] = {0, 0};
  bool crowded = false;  // a CTA put 4096 or more ids into one bin: its 32-bit mass may have wrapped
  if (active) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int b = b0 + i;
      int pc[kMaxCluster];
      unsigned pm[kMaxCluster];  // independent remote loads, all in flight together
#pragma unroll
      for (int r = 0; r < kMaxCluster; ++r) {
        pc[r] = r < c.nranks ? *c.cluster.map_shared_rank(&bins[b], r) : 0;
        pm[r] = r < c.nranks ? *c.cluster.map_shared_rank(&qmass[b], r) : 0u;
      }
      unsigned long long q = 0;
#pragma unroll
      for (int r = 0; r < kMaxCluster; ++r) { cnt[i] += pc[r]; q += pm[r]; crowded |= pc[r] >= 4096; }
      // Measured mass = q * 2^-20 * 2^-(b*step).  Per id: the FP32 argument carries three roundings relative to
      // |x| <= (b+1)*step plus one of the product b*step (together < 2.8 |x| * 2^-24 in the weight; 5.6 allowed),
      // ex2.approx is within 2^-22, the product by 2^20 within 2^-24, the rounding to an integer within 2^-21 of a
      // value near 2^20; the edge weight below is an FP64 exp2 of the same FP32 product.  The last bin also takes
      // ids whose quotient rounds past the range; the absolute slack on the target covers what they weigh.
      const double x_far = (double(b) + 1.0) * double(step) * 1.0001;
      const double e = (5.6 * x_far + 41.0) * 5.9604644775390625e-8;
      const double mass = double(q) * 9.5367431640625e-7 * exp2(-double(float(b) * step));
      lo[i] = mass * (1.0 - e); hi[i] = mass * (1.0 + e);
    }
  }
  double lo0, hi0;
  int cn0, crowd;
  block_prefix2x3(c, lo, hi, cnt, crowded ? 1 : 0, &lo0, &hi0, &cn0, &crowd);
  if (c.tid == kThreads - 1) { s->outcome.d[0] = lo0 + lo[1]; s->outcome.d[1] = hi0 + hi[1]; s->outcome.i[0] = cn0 + cnt[1]; }
  __syncthreads();
  Slot totals{};
  totals.d[0] = s->outcome.d[0]; totals.d[1] = s->outcome.d[1]; totals.i[1] = s->outcome.i[0]; totals.i[0] = crowd;
  if (c.tid == 0) { s->bcast_i[0] = 0x7fffffff; s->bcast_i[1] = 0x7fffffff; }
  const Slot *all1 = exchange(c, totals);
  double base_lo = 0, base_hi = 0, z_lo = 0, z_hi = 0;
  int any_crowd = 0, base_cn = 0, n_all = 0;
  for (int r = 0; r < c.nranks; ++r) {
    if (r == c.rank) { base_lo = z_lo; base_hi = z_hi; base_cn = n_all; }
    z_lo += all1[r].d[0]; z_hi += all1[r].d[1]; n_all += all1[r].i[1]; any_crowd |= all1[r].i[0];
  }
  const double t_lo = top_p * z_lo * (1.0 - 1e-12), t_hi = top_p * z_hi * (1.0 + 1e-12);
  // w0: first bin through which the running mass MAY reach the target; w1: first through which it SURELY does
  const double H0 = base_hi + hi0, H1 = H0 + hi[1], L0 = base_lo + lo0, L1 = L0 + lo[1];
  const int C0 = base_cn + cn0, C1 = C0 + cnt[1];  // ids through bin b0 and through bin b0 + 1
  if (active) {
    if (H0 >= t_lo) atomicMin(&s->bcast_i[0], b0); else if (H1 >= t_lo) atomicMin(&s->bcast_i[0], b0 + 1);
    if (L0 >= t_hi) atomicMin(&s->bcast_i[1], b0); else if (L1 >= t_hi) atomicMin(&s->bcast_i[1], b0 + 1);
  }
  __syncthreads();
  const int my_w0 = s->bcast_i[0], my_w1 = s->bcast_i[1];
  if (active && (my_w0 == b0 || my_w0 == b0 + 1)) s->outcome.i[2] = my_w0 == b0 ? C0 - cnt[0] : C0;  // ids before
  if (active && (my_w1 == b0 || my_w1 == b0 + 1)) s->outcome.i[3] = my_w1 == b0 ? C0 : C1;            // ids through
  __syncthreads();
  Slot cand{};
  cand.i[0] = my_w0; cand.i[1] = my_w1; cand.i[2] = s->outcome.i[2]; cand.i[3] = s->outcome.i[3];
  __syncthreads();
  const Slot *all2 = exchange(c, cand);
  int w0 = 0x7fffffff, w1 = 0x7fffffff, before_w0 = 0, through = 0;
  for (int r = c.nranks - 1; r >= 0; --r) {  // segments are in bin order: the lowest rank with a candidate holds the first
    if (all2[r].i[0] != 0x7fffffff) { w0 = all2[r].i[0]; before_w0 = all2[r].i[2]; }
    if (all2[r].i[1] != 0x7fffffff) { w1 = all2[r].i[1]; through = all2[r].i[3]; }
  }
  // not this path's case: no window, a nucleus that certainly fits the candidate list (the small-support path's
  // case), a window larger than the list, or a wrapped mass -- the same outcome in every CTA
  if (w0 == 0x7fffffff || w1 == 0x7fffffff || w1 < w0 || through <= kListCap / 2 || through - before_w0 > kListCap || any_crowd)
    return out;

  // ---------------------------------------------------------------- W2: the one FP64 pass
  uint16_t *band = reinterpret_cast<uint16_t *>(s->bin_mass) + c.warp * kBandPerWarp;
  const double inv_t = 1.0 / t;  // see the note on `weight` in row_kernel.cuh
  double z_lane = 0, def_lane = 0;
  int def_count = 0, n_band = 0;  // n_band is warp-uniform
  const float edge0 = float(w0), edge1 = w1 >= kWideBins - 1 ? CUDART_INF_F : float(w1 + 1);
  // (the mass histogram shares its memory with the lists: rank 0 pulled it before the outcome exchange above)
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    bool inside = false;
    if (j < c.len) {
      const float y = s->y[j];
      if (y > -CUDART_INF_F) {
        const double e = exp_nonpos((double(y) - double(m)) * inv_t);
        z_lane += e;
        // bin(y) < w0 and bin(y) <= w1 without forming the bin: int(v) < k is v < k for v >= 0
        const float v = (m - y) * inv_w;
        const bool sure = v < edge0;
        if (sure) { def_lane += e; ++def_count; }
        inside = !sure && v < edge1;
      }
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, inside);
    if (inside) {
      const int slot = n_band + __popc(ballot & ((1u << c.lane) - 1u));
      if (slot < kBandPerWarp) band[slot] = uint16_t(it + c.lane);
    }
    n_band += __popc(ballot);
  }
  // fused block reduction of (z, sure mass, sure count, listed count, overflow)
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    z_lane += __shfl_xor_sync(0xffffffffu, z_lane, o);
    def_lane += __shfl_xor_sync(0xffffffffu, def_lane, o);
  }
  const double warp_def = def_lane;  // region sum of the ids kept for sure
  def_count = __reduce_add_sync(0xffffffffu, def_count);
  if (c.lane == 0) {
    s->red_d[c.warp] = z_lane; s->red_q[c.warp] = (unsigned long long)__double_as_longlong(def_lane);
    s->red_i[c.warp] = def_count; s->red_j[c.warp] = n_band;
  }
  __syncthreads();
  Slot mine{};
  for (int w = 0; w < kWarps; ++w) {
    mine.d[0] += s->red_d[w]; mine.d[1] += __longlong_as_double((long long)s->red_q[w]);
    mine.i[0] += s->red_i[w]; mine.i[1] += min(s->red_j[w], kBandPerWarp); mine.i[2] |= s->red_j[w] > kBandPerWarp ? 1 : 0;
  }
  __syncthreads();
  const Slot *all = exchange(c, mine);
  double z = 0, mass_before = 0;
  int n_before = 0, n_in_band = 0, overflow = 0;
  for (int r = 0; r < c.nranks; ++r) {
    z += all[r].d[0]; mass_before += all[r].d[1]; n_before += all[r].i[0]; n_in_band += all[r].i[1]; overflow |= all[r].i[2];
  }
  if (overflow || n_in_band > kListCap || n_in_band == 0) return out;
  {
    int *list_count0 = c.cluster.map_shared_rank(&s->list_count, 0);
    unsigned long long *keys0 = c.cluster.map_shared_rank(s->u.w.total_mass, 0);
    for (int q = c.lane; q < n_band; q += 32) {
      const int j = c.warp * c.region + band[q];
      const int slot = atomicAdd(list_count0, 1);
      // ascending 64-bit key = (logit descending, id ascending); +0 and -0 compare equal as logits, so both map to +0
      const float y = s->y[j] == 0.f ? 0.f : s->y[j];
      const uint32_t bits = __float_as_uint(y), ordered = bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
      if (slot < kListCap) keys0[slot] = (unsigned long long)(~ordered) << 32 | uint32_t(c.begin + j);
    }
  }
  c.cluster.sync();
  Slot v{};
  if (c.rank == 0) {
    const int n = min(s->list_count, kListCap);
    unsigned long long *keys = s->u.w.total_mass;
    int padded = 64;
    while (padded < n) padded <<= 1;
    for (int i = n + c.tid; i < padded; i += kThreads) keys[i] = ~0ull;
    __syncthreads();
    if (padded <= kThreads) {
      // bitonic network, one key per thread: partners closer than a warp exchange by shuffle, the others through
      // shared memory
      unsigned long long key = c.tid < padded ? keys[c.tid] : ~0ull;
      for (int k = 2; k <= padded; k <<= 1) {
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
          unsigned long long other;
          if (jj < 32) {
            other = __shfl_xor_sync(0xffffffffu, key, jj);
          } else {
            keys[c.tid] = key;
            __syncthreads();
            other = keys[c.tid ^ jj];
            __syncthreads();
          }
          const bool keep_min = ((c.tid & jj) == 0) == ((c.tid & k) == 0);
          key = keep_min ? (key < other ? key : other) : (key < other ? other : key);
        }
      }
      keys[c.tid] = key;
      __syncthreads();
    } else {
      for (int k = 2; k <= padded; k <<= 1) {      // the same network, two keys per thread, every step through memory
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
          for (int i = c.tid; i < padded / 2; i += kThreads) {
            const int lo_i = ((i / jj) * 2 * jj) + (i % jj), hi_i = lo_i + jj;
            const bool up = (lo_i & k) == 0;
            const unsigned long long a = keys[lo_i], b = keys[hi_i];
            if ((a > b) == up) { keys[lo_i] = b; keys[hi_i] = a; }
          }
          __syncthreads();
        }
      }
    }
    // FP64 weights in sorted order and their prefix sums from the mass before the window
    double e[2];
    float ys[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = 2 * c.tid + i;
      const uint32_t ordered = r < n ? ~uint32_t(keys[r] >> 32) : 0x80000000u;
      ys[i] = __uint_as_float(ordered ^ ((ordered >> 31) ? 0x80000000u : 0xffffffffu));
      e[i] = r < n ? exp_nonpos((double(ys[i]) - double(m)) * inv_t) : 0.0;
    }
    const double through0 = mass_before + block_prefix2(c, e[0], e[1]);  // running mass through sorted id 2*tid
    const double rel = 2.0 * (double(allowed) + 256.0) * kU;
    const double target = top_p * z, lo = target * (1.0 - rel), hi = target * (1.0 + rel);
    if (c.tid == 0) s->bcast_i[0] = 0x7fffffff;
    __syncthreads();
    const double through1 = through0 + e[1];
    int mine_pos = -1;
    if (2 * c.tid < n && through0 >= target) mine_pos = 2 * c.tid;
    else if (2 * c.tid + 1 < n && through1 >= target) mine_pos = 2 * c.tid + 1;
    if (mine_pos >= 0) atomicMin(&s->bcast_i[0], mine_pos);
    __syncthreads();
    const int pos = s->bcast_i[0];
    if (c.tid == 0) {
      s->list_count = 0;
      // mass_before >= lo: the crossing is (or may be) before the window; pos unset: not reached inside it
      s->outcome.i[0] = (mass_before < lo && pos != 0x7fffffff) ? 1 : 0;
    }
    if (pos != 0x7fffffff && (pos >> 1) == c.tid) {
      const int i = pos & 1;
      const double mass_at = i ? through1 : through0, prev_at = mass_at - e[i];
      s->outcome.i[1] = ((mass_at < hi) || (prev_at >= lo)) ? 1 : 0;
      s->outcome.f[0] = ys[i]; s->outcome.i[2] = int(uint32_t(keys[pos]));
      s->outcome.i[3] = n_before + pos + 1; s->outcome.d[0] = mass_at;
    }
    __syncthreads();
    v = s->outcome;
    __syncthreads();
  }
  v = exchange(c, v)[0];
  if (!v.i[0]) return out;
  out.cut.y = v.f[0]; out.cut.id = v.i[2]; out.kept = v.i[3]; out.e_kept = v.d[0]; out.z = z; out.ambiguous = v.i[1];
  // ---- region sums of the kept ids: the sure ones plus this warp's window ids that made the cut
  double extra = 0;
  for (int q = c.lane; q < n_band; q += 32) {
    const int j = c.warp * c.region + band[q];
    const float y = s->y[j];
    if (survives(y, c.begin + j, out.cut)) extra += exp_nonpos((double(y) - double(m)) * inv_t);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) extra += __shfl_xor_sync(0xffffffffu, extra, o);
  if (c.lane == 0) s->warp_sum[c.warp] = warp_def + extra;
  __syncthreads();
  out.applicable = 1;
  return out;
}

}  // namespace ds41
