// The per-row kernel: stage -> penalties/mask -> first maximum -> top-k cut -> normaliser (+ top-p cut) -> either
// the inverse-CDF draw (sampler) or a RowStats record (verifier).  One cluster per row; see row_core.cuh.
#pragma once
#include "row_core.cuh"
#include "row_fast.cuh"
#include "row_wide.cuh"

namespace ds41 {

enum RowMode { kModeSample = 0, kModeStats = 1 };

struct RowArgs {
  const float *logits;
  long long logits_stride;
  int vocab;
  double temperature;  // already floored; 0 = greedy
  double top_p;
  int top_k;
  float repetition, presence, frequency;
  const int32_t *history;
  long long history_stride;
  const int32_t *history_len;
  const uint32_t *mask;
  long long mask_stride;
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens;
  int32_t *status;
  RowStats *stats;
  int only_uncovered;  // 1: process only rows the streaming path reported as not covered, leave the others alone
  const int *pending;  // optional, with only_uncovered: number of such rows; 0 = nothing to do, every CTA returns at once
  int rows;            // set by launch_rows: a cluster walks rows cluster, cluster + clusters, ... below this
};

// Region sums of a non-negative per-id value (value(j) for local index j < len, 0 for ids outside the support):
// lanes stride the warp's region in id order, the warp total lands in warp_sum[warp].  Fixed order => same bits
// every run.
template <class Value>
__device__ __forceinline__ void region_sums(RowCtx &c, Value value) {
  double acc = 0;
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    if (j < c.len) acc += value(j);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (c.lane == 0) c.s->warp_sum[c.warp] = acc;
  __syncthreads();
}

// Inverse CDF in id order (reference: draw(), third_party/spark/src/sampling.cpp:18-21): the first id whose running
// sum exceeds u * total, else the last id with a positive value.  warp_sum[] must hold the region sums of `value`.
// Returns the token to every thread of every CTA; *ambiguous is set when the target lies within
// rel_bound*total + abs_bound of a CDF step on either side of the chosen id; *total_out receives the total.
template <class Value>
__device__ int draw_token(RowCtx &c, double u, double rel_bound, double abs_bound, Value value, int *ambiguous,
                          double *total_out) {
  RowSmem *s = c.s;
  if (c.tid == 0) s->bcast_i[2] = 0;
  double block_total = 0;
  for (int w = 0; w < kWarps; ++w) block_total += s->warp_sum[w];
  Slot mine{};
  mine.d[0] = block_total;
  const Slot *all = exchange(c, mine);
  double prefix = 0, total = 0;
  for (int r = 0; r < c.nranks; ++r) {
    if (r == c.rank) prefix = total;
    total += all[r].d[0];
  }
  *total_out = total;
  const double target = u * total;
  const double slack = rel_bound * total + abs_bound;
  // Which warp region of this CTA holds the target, if any (the regions' intervals tile [0, total), so exactly one
  // region of the cluster does); every thread evaluates the same sums, so the answer is uniform in the CTA.
  int owner_warp = -1, amb = 0;
  double region_start = 0;
  {
    double inner = 0;
    for (int w = 0; w < kWarps; ++w) {
      const double start = prefix + inner, end = prefix + (inner + s->warp_sum[w]);
      if (owner_warp < 0 && start <= target && target < end) { owner_warp = w; region_start = start; }
      inner += s->warp_sum[w];
    }
  }
  if (owner_warp >= 0) {
    // The whole CTA walks the owning region: warp v takes chunk v of it (one or two 32-id blocks, values kept in
    // registers), the chunk sums locate the chunk that holds the target, and that chunk's warp walks its values.
    const int blocks = (c.region / kWarps + 31) / 32;  // 32-id blocks per chunk: 1 or 2 (region <= 1024)
    const int first = owner_warp * c.region + c.warp * blocks * 32;
    double v[2] = {0.0, 0.0};
    int last_mine = -1;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int idx = c.warp * blocks * 32 + b * 32 + c.lane, j = first + b * 32 + c.lane;
      const bool in = b < blocks && idx < c.region && j < c.len;
      const double w = value(in ? j : 0);
      v[b] = in ? w : 0.0;
      if (v[b] > 0) last_mine = j;
    }
    double chunk = v[0] + v[1];
#pragma unroll
    for (int o = 16; o; o >>= 1) chunk += __shfl_xor_sync(0xffffffffu, chunk, o);
    last_mine = __reduce_max_sync(0xffffffffu, last_mine);
    if (c.lane == 0) { s->red_d[c.warp] = chunk; s->red_i[c.warp] = last_mine; }
    __syncthreads();
    int owner_chunk = -1, last_positive = -1;
    double carry = region_start;
    {
      double run = region_start;
      for (int w = 0; w < kWarps; ++w) {
        const double through = run + s->red_d[w];
        if (owner_chunk < 0 && s->red_d[w] > 0 && target < through) { owner_chunk = w; carry = run; }
        run = through;
        last_positive = max(last_positive, s->red_i[w]);
      }
    }
    if (last_positive >= 0) last_positive += c.begin;
    int found = -1;
    if (c.warp == (owner_chunk < 0 ? 0 : owner_chunk)) {
      for (int b = 0; b < blocks && found < 0 && owner_chunk >= 0; ++b) {
        const double vb = b ? v[1] : v[0];
        double sc = vb;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const double up = __shfl_up_sync(0xffffffffu, sc, o);
          if (c.lane >= o) sc += up;
        }
        const double cum = carry + sc;
        const unsigned hit = __ballot_sync(0xffffffffu, vb > 0 && target < cum);
        if (hit) {
          const int h = __ffs(hit) - 1;
          found = c.begin + first + b * 32 + h;
          const double cum_h = __shfl_sync(0xffffffffu, cum, h);
          const double v_h = __shfl_sync(0xffffffffu, vb, h);
          const double below = cum_h - v_h;  // CDF before the chosen id
          amb = (cum_h - target < slack) || (below > 0 && target - below < slack);
        } else {
          carry = __shfl_sync(0xffffffffu, cum, 31);
        }
      }
      if (found < 0) { found = last_positive; amb = 1; }  // rounding left the target past the region's last step
      if (c.lane == 0) { s->bcast_i[0] = found; s->bcast_i[1] = amb; s->bcast_i[2] = 1; }
    }
  }
  __syncthreads();
  Slot res{};
  res.i[0] = -1;
  if (s->bcast_i[2] == 1) { res.i[0] = s->bcast_i[0]; res.i[1] = s->bcast_i[1]; }  // at most one CTA has an owner
  __syncthreads();
  const Slot *got = exchange(c, res);
  int token = -1;
  for (int r = 0; r < c.nranks; ++r)
    if (got[r].i[0] >= 0) { token = got[r].i[0]; amb = got[r].i[1]; }
  if (token < 0) {
    // target >= total (only possible by rounding): the reference returns the last id with positive probability
    int last = -1;
    for (int it = 0; it < c.region; it += 32) {
      const int j = c.warp * c.region + it + c.lane;
      if (j < c.len && value(j) > 0) last = max(last, c.begin + j);
    }
    Slot m2{};
    m2.i[0] = block_max(c, last);
    const Slot *g2 = exchange(c, m2);
    for (int r = 0; r < c.nranks; ++r) token = max(token, g2[r].i[0]);
    amb = 1;
  }
  *ambiguous = amb;
  return token;
}

// One row, start to finish, by the whole cluster.  Shared memory needs no particular content on entry.
template <int kMode>
__device__ __forceinline__ void row_body(const RowArgs &a, RowCtx &c, RowSmem *s, const int row) {
  const float *logits = a.logits + size_t(row) * a.logits_stride;

  bool used_tma;
  stage_begin(c, logits, used_tma);
  if (a.mask) {
    const uint32_t *mw = a.mask + size_t(row) * a.mask_stride + (c.begin >> 5);
    for (int w = c.tid; w < (c.len + 31) / 32; w += kThreads) s->mask_words[w] = __ldg(mw + w);
  }
  // ---- history counts (16-bit counters packed in pairs; remote shared-memory atomics route each id to its owner)
  const bool penalised = a.history != nullptr && (a.repetition != 1.f || a.presence != 0.f || a.frequency != 0.f);
  int hist_len = penalised ? (a.history_len ? a.history_len[row] : int(a.history_stride)) : 0;
  const bool bad_history = hist_len < 0 || hist_len > 65535 || (long long)hist_len > a.history_stride;
  if (bad_history) hist_len = 0;
  if (hist_len > 0) {
    for (int j = c.tid; j < kSliceCap / 2; j += kThreads) s->u.count_pairs[j] = 0;
    c.cluster.sync();
    const int32_t *h = a.history + size_t(row) * a.history_stride;
    const int per = (hist_len + c.nranks - 1) / c.nranks;
    const int h0 = min(hist_len, c.rank * per), h1 = min(hist_len, h0 + per);
    for (int base = h0 + c.warp * 32; base < h1; base += kThreads) {
      const int i = base + c.lane;
      const int id = i < h1 ? __ldg(h + i) : -1;
      const bool valid = id >= 0 && id < a.vocab;
      const unsigned peers = __match_any_sync(0xffffffffu, valid ? id : -1);
      if (valid && c.lane == __ffs(peers) - 1) {
        const int owner = id / c.stride_ids, local = id - owner * c.stride_ids;
        atomicAdd(c.cluster.map_shared_rank(&s->u.count_pairs[local >> 1], owner),
                  uint32_t(__popc(peers)) << ((local & 1) * 16));
      }
    }
    c.cluster.sync();
  }
  const bool landed = stage_wait(c, used_tma);

  // ---- effective logits, first maximum, allowed count
  int flags = (landed ? 0 : 8) | (bad_history ? 4 : 0);
  float best = -CUDART_INF_F, lowest = CUDART_INF_F;  // lowest: smallest finite effective logit
  int best_id = 0x7fffffff, allowed = 0;
  for (int it = 0; it < c.region; it += 32) {
    const int j = c.warp * c.region + it + c.lane;
    if (j >= c.len) continue;
    float x = s->y[j];
    if ((__float_as_uint(x) & 0x7f800000u) == 0x7f800000u) flags |= 1;
    if (hist_len > 0) {
      const uint32_t cnt = (s->u.count_pairs[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      if (cnt) {
        const float v = x > 0.f ? __fdiv_rn(x, a.repetition) : __fmul_rn(x, a.repetition);
        x = __fsub_rn(v, __fadd_rn(a.presence, __fmul_rn(a.frequency, float(cnt))));
        if ((__float_as_uint(x) & 0x7f800000u) == 0x7f800000u) flags |= 2;
      }
    }
    const bool ok = !a.mask || ((s->mask_words[j >> 5] >> (j & 31)) & 1u);
    if (!ok) x = -CUDART_INF_F;
    s->y[j] = x;
    if (ok) {
      ++allowed;
      if (x > best) { best = x; best_id = c.begin + j; }
      if (x > -CUDART_INF_F) lowest = fminf(lowest, x);
    }
  }
  __syncthreads();
  {
    Slot mine{};
    // one fused block reduction: (best, best_id) by "larger value, then lower id", lowest, flags, allowed
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
      lowest = fminf(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
    }
    flags = int(__reduce_or_sync(0xffffffffu, unsigned(flags)));
    allowed = __reduce_add_sync(0xffffffffu, allowed);
    if (c.lane == 0) {
      s->red_f[c.warp] = best; s->red_j[c.warp] = best_id; s->red_d[c.warp] = double(lowest);
      s->red_q[c.warp] = (unsigned long long)(unsigned(allowed)) << 32 | unsigned(flags);
    }
    __syncthreads();
    best = s->red_f[0]; best_id = s->red_j[0]; lowest = float(s->red_d[0]);
    flags = int(unsigned(s->red_q[0])); allowed = int(s->red_q[0] >> 32);
#pragma unroll
    for (int w = 1; w < kWarps; ++w) {
      const float ov = s->red_f[w];
      const int oi = s->red_j[w];
      if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
      lowest = fminf(lowest, float(s->red_d[w]));
      flags |= int(unsigned(s->red_q[w]));
      allowed += int(s->red_q[w] >> 32);
    }
    __syncthreads();
    mine.f[0] = best; mine.i[0] = best_id; mine.f[1] = lowest;
    mine.i[1] = flags;
    mine.i[2] = allowed;
    const Slot *all = exchange(c, mine);
    best = all[0].f[0]; best_id = all[0].i[0]; flags = all[0].i[1]; allowed = all[0].i[2];
    for (int r = 1; r < c.nranks; ++r) {
      if (all[r].f[0] > best || (all[r].f[0] == best && all[r].i[0] < best_id)) { best = all[r].f[0]; best_id = all[r].i[0]; }
      flags |= all[r].i[1];
      allowed += all[r].i[2];
    }
    for (int r = 0; r < c.nranks; ++r) lowest = fminf(lowest, all[r].f[1]);
  }
  int status = 0;
  c.timed_out = (flags & 8) ? 1 : 0;
  if (flags & 8) status = -5;
  else if (flags & 1) status = -1;
  else if (flags & 4) status = -7;
  else if (flags & 2) status = -3;
  else if (allowed == 0) status = -2;

  const float max_logit = best;
  const double t = a.temperature;
  // exp((y - max)/T) with the division replaced by a multiplication: the argument moves by at most one ulp, the
  // value by |argument| * 2^-53 relative (< 100 u), which every comparison made on sums of these weights allows for
  const double inv_t = t > 0 ? 1.0 / t : 0.0;
  auto weight = [max_logit, inv_t](float y) { return exp_nonpos((double(y) - double(max_logit)) * inv_t); };
  Cut cut{-CUDART_INF_F, -1};
  // value of local id j for the sums and the draw: exp weight of a survivor of the CURRENT cut, else 0
  auto value = [&cut, &c, s, weight](int j) {
    const float y = s->y[j];
    const double w = weight(y);  // unconditional (0 for an excluded id): independent calls overlap
    return survives(y, c.begin + j, cut) ? w : 0.0;
  };
  int entered = allowed, kept = allowed;
  double z = 0, e_kept = 0;
  int token = -1;

  bool wide_done = false;
  if (status == 0 && t != 0 && a.top_p < 1.0 && (a.top_k <= 0 || a.top_k >= allowed) && allowed > 2 * kListCap &&
      lowest < max_logit) {
    const WideOutcome w = wide_nucleus(c, max_logit, lowest, t, a.top_p, allowed);
    if (w.applicable) {
      wide_done = true;
      cut = w.cut; kept = w.kept; z = w.z; e_kept = w.e_kept;
      if (w.ambiguous) status |= 2;
    }
  }
  if (!wide_done) {
    if (status == 0 && t != 0) {
      const double u = kMode == kModeSample ? philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose) : 0.0;
      const FastOutcome f = fast_small_support(c, max_logit, t, allowed, a.top_k, a.top_p, u, kMode == kModeSample);
      if (f.applicable) {
        // ranks other than 0 are done after the gather; rank 0 finishes alone and touches only its own shared memory
        if (c.rank == 0 && c.tid == 0) {
          if (kMode == kModeSample) {
            a.tokens[row] = f.token;
            if (a.status) a.status[row] = f.status;
          } else {
            RowStats st;
            st.z = f.z; st.e_kept = f.e_kept; st.max_logit = max_logit; st.argmax = best_id; st.cut = f.cut;
            st.kept = f.kept; st.entered = f.entered; st.status = f.status; st.pad = 0;
            a.stats[row] = st;
          }
        }
        return;
      }
    }
  }
  if (wide_done) {
    // cut, sums and region sums are in place
  } else if (status == 0 && t == 0) {
    token = best_id;
    kept = 1; z = 1; e_kept = 1;
    cut.y = max_logit; cut.id = best_id;
  } else if (status == 0) {
    // ---- top-k
    if (a.top_k > 0 && a.top_k < allowed) {
      CutResult r = find_cut<false>(c, max_logit, 16.f / kBins, a.top_k, 0.0, allowed,
                                    [](float y, int) { return y > -CUDART_INF_F; }, weight);
      if (r.error) status = r.error;
      else { cut = r.cut; entered = kept = a.top_k; }
    }
    const Cut base = cut;
    // ---- normaliser and top-p
    if (status == 0 && a.top_p < 1.0) {
      CutResult r = find_cut<true>(c, max_logit, float(48.0 * t) / kBins, 0, a.top_p, entered,
                                   [base](float y, int id) { return survives(y, id, base); }, weight);
      if (r.error) status = r.error;
      else {
        z = r.z; e_kept = r.e_kept; kept = r.kept;
        if (r.cut.id >= 0) cut = r.cut;
        if (r.ambiguous) status |= 2;
      }
      if (status >= 0 && kMode == kModeSample) region_sums(c, value);
    } else if (status == 0) {
      region_sums(c, value);
      double block_total = 0;
      for (int w = 0; w < kWarps; ++w) block_total += s->warp_sum[w];
      Slot mine{};
      mine.d[0] = block_total;
      const Slot *all = exchange(c, mine);
      for (int r = 0; r < c.nranks; ++r) z += all[r].d[0];
      e_kept = z;
    }
  }
  if (status >= 0 && t != 0 && kMode == kModeSample) {
    const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
    int amb = 0;
    double total;
    token = draw_token(c, u, (2.0 * kept + 512.0) * kU, 0.0, value, &amb, &total);
    if (amb) status |= 1;
  }
  if (c.rank == 0 && c.tid == 0) {
    if (kMode == kModeSample) {
      a.tokens[row] = status < 0 ? -1 : token;
      if (a.status) a.status[row] = status;
    } else {
      RowStats st;
      st.z = z; st.e_kept = e_kept; st.max_logit = max_logit; st.argmax = best_id; st.cut = cut;
      st.kept = kept; st.entered = entered; st.status = status; st.pad = 0;
      a.stats[row] = st;
    }
  }
}

// A cluster takes rows cluster, cluster + clusters, ...: one row per cluster when the launch has a cluster per row; a
// small persistent grid when only the rows another path left over (status -8 / -9) are wanted, so that a launch with
// nothing to do costs a few status reads instead of thousands of cluster launches.
template <int kMode>
__global__ void __launch_bounds__(kThreads, 2) row_kernel(RowArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  RowSmem *s = reinterpret_cast<RowSmem *>(smem_raw);
  if (a.only_uncovered && a.pending && *a.pending == 0) return;  // the same in every CTA of the grid
  RowCtx c = make_ctx(s, a.vocab);
  const int clusters = int(gridDim.x) / c.nranks;
  for (int row = int(blockIdx.x) / c.nranks; row < a.rows; row += clusters) {
    if (a.only_uncovered) {  // same answer in every CTA of the cluster
      const int st = kMode == kModeSample ? a.status[row] : a.stats[row].status;
      if (st != -8 && st != -9) continue;  // -9: handed on by the batch path for wide nuclei (flat.cuh)
    }
    row_body<kMode>(a, c, s, row);
    // no CTA may exit, or stage the next row, while a peer can still address its shared memory
    c.cluster.sync();
    if (c.timed_out) {  // a bounded wait expired: this cluster reports its remaining rows and stops
      if (c.rank == 0 && c.tid == 0) {
        for (int r = row + clusters; r < a.rows; r += clusters) {
          if (kMode == kModeSample) {
            if (a.only_uncovered && a.status[r] != -8 && a.status[r] != -9) continue;
            a.tokens[r] = -1;
            if (a.status) a.status[r] = -5;
          } else if (!a.only_uncovered || a.stats[r].status == -8) {
            a.stats[r].status = -5;
          }
        }
      }
      break;
    }
  }
}

}  // namespace ds41
