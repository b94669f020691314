// Fast path of the row kernel for rows whose surviving support is small (top-k, or a top-p nucleus of at most
// kListCap ids, or a small vocabulary): the handful of ids that can survive are gathered into rank 0 of the
// cluster, and ONE thread there runs the reference's arithmetic on them literally -- same operations, same order
// (third_party/spark/src/sampling.cpp:18-21,34-36): sequential normaliser in id order, p/z, sequential prefix of the
// stable descending order until top_p is reached, p/mass, sequential inverse CDF in id order.
//
// What cannot be literal is the normaliser of a top-p row WITHOUT top-k: it runs over the whole vocabulary.  It is
// summed in parallel in mixed precision -- ids within kHeavySpan*T of the maximum in FP64 (their indices compacted per
// warp so that the FP64 work is dense), the light tail in FP32 with an explicit error bound -- and the top-p
// crossing is certified against that bound; everything after the crossing is literal again (the normaliser cancels
// in p/mass up to rounding).
//
// The path needs 4 cluster barriers per row; CTAs other than rank 0 leave after the gather.
#pragma once
#include "row_core.cuh"

namespace ds41 {

constexpr float kHeavySpan = 20.f;  // ids with (max - y)/T below this are summed in FP64
constexpr int kChunk = 256;         // ids per warp between two compaction flushes

struct FastOutcome {
  int applicable;  // 0: not handled, the general path must run (every CTA of the cluster gets the same answer)
  int finished;    // 1: this CTA has nothing left to do (ranks other than 0 after the gather)
  int token, status, kept, entered;
  Cut cut;
  double z, e_kept;
};

// `want_draw`: draw a token with uniform u; otherwise only the statistics are produced.
__device__ inline FastOutcome fast_small_support(RowCtx &c, float max_logit, double t, int allowed, int top_k, double top_p,
                                          double u, bool want_draw) {
  RowSmem *s = c.s;
  FastOutcome out{};
  const bool count_mode = top_k > 0 && top_k < allowed;
  const bool everything = allowed <= kListCap;  // the whole allowed set fits the list: no histogram needed
  if (!everything && !count_mode && !(top_p < 1.0)) return out;
  out.applicable = 1;
  out.entered = count_mode ? top_k : allowed;
  const float inv_t = float(1.0 / t);
  const float span = count_mode ? 16.f : kHeavySpan * float(t);  // histogram range in logit units
  const float inv_w = float(kBins) / span;
  double z_tilde = 0, z_err = 0;  // MASS: parallel normaliser and its absolute error bound
  int pick = kBins;               // ids with bin <= pick are gathered (kBins = everything in range and beyond)

  if (!everything) {
    // ---------------------------------------------------------------- histogram pass
    for (int j = c.tid; j < kBins; j += kThreads) { s->bin_count[j] = 0; s->bin_mass[j] = 0; }
    __syncthreads();
    uint16_t *heavy = reinterpret_cast<uint16_t *>(s->u.w.sorted_y) + c.warp * kChunk;  // 8 KB, free until the tail
    double sum64 = 0;
    float sum32 = 0.f, err32 = 0.f;
    int beyond = 0;
    for (int chunk = 0; chunk < c.region; chunk += kChunk) {
      int n_heavy = 0;
      for (int it = chunk; it < min(chunk + kChunk, c.region); it += 32) {
        const int j = c.warp * c.region + it + c.lane;
        bool is_heavy = false;
        if (j < c.len) {
          const float y = s->y[j];
          if (y > -CUDART_INF_F) {
            const float d = max_logit - y;
            if (d < span) {
              is_heavy = true;
            } else {
              ++beyond;
              if (!count_mode) {
                const float a = d * inv_t;
                const float e = __expf(-a);
                sum32 += e;
                err32 = fmaf(e, 2.f + a, err32);
              }
            }
          }
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, is_heavy);
        if (is_heavy) heavy[n_heavy + __popc(ballot & ((1u << c.lane) - 1u))] = uint16_t(j - c.warp * c.region);
        n_heavy += __popc(ballot);
      }
      __syncwarp();
      for (int q = c.lane; q < n_heavy; q += 32) {
        const int j = c.warp * c.region + heavy[q];
        const float y = s->y[j];
        int b = int((max_logit - y) * inv_w);
        b = b < 0 ? 0 : (b >= kBins ? kBins - 1 : b);
        atomicAdd(&s->bin_count[b], 1);
        if (!count_mode) {
          const double e = exp((double(y) - double(max_logit)) / t);
          sum64 += e;
          atomicAdd(&s->bin_mass[b], (unsigned long long)(e * kFix));
        }
      }
      __syncwarp();
    }
    Slot mine{};
    mine.i[0] = block_sum(c, beyond);
    if (!count_mode) {
      mine.d[0] = block_sum(c, sum64);
      mine.d[1] = block_sum(c, double(sum32));
      mine.d[2] = block_sum(c, double(err32));
    }
    c.cluster.sync();  // every CTA's histogram is complete
    {
      const int share = kBins / c.nranks;
      for (int j = c.tid; j < share; j += kThreads) {
        const int b = c.rank * share + j;
        int tc = 0;
        unsigned long long tm = 0;
        for (int r = 0; r < c.nranks; ++r) {
          tc += *c.cluster.map_shared_rank(&s->bin_count[b], r);
          if (!count_mode) tm += *c.cluster.map_shared_rank(&s->bin_mass[b], r);
        }
        for (int r = 0; r < c.nranks; ++r) {
          *c.cluster.map_shared_rank(&s->u.w.total_count[b], r) = tc;
          if (!count_mode) *c.cluster.map_shared_rank(&s->u.w.total_mass[b], r) = tm;
        }
      }
    }
    const Slot *all = exchange(c, mine);
    double z64 = 0, z32 = 0, e32 = 0;
    int n_beyond = 0;
    for (int r = 0; r < c.nranks; ++r) { z64 += all[r].d[0]; z32 += all[r].d[1]; e32 += all[r].d[2]; n_beyond += all[r].i[0]; }
    z_tilde = z64 + z32;
    // FP64 part: tree-vs-sequential summation and exp ulps; FP32 part: ex2.approx + argument rounding per id
    // ((2+a)*2^-22 relative, accumulated above) and FP32 accumulation of at most 32 terms per lane
    z_err = (double(allowed - n_beyond) + 64.0) * kU * z64 + 1.01 * e32 * 0x1p-22 + z32 * 0x1p-18;
    unsigned long long target_fix = count_mode ? 0ull : (unsigned long long)(top_p * z_tilde * kFix);
    // ---- crossing bin (warp 0)
    if (c.warp == 0) {
      int found = -1, run_c = 0;
      unsigned long long run_m = 0;
      for (int base = 0; base < kBins && found < 0; base += 32) {
        const int vc = s->u.w.total_count[base + c.lane];
        const unsigned long long vm = count_mode ? 0ull : s->u.w.total_mass[base + c.lane];
        int sc = vc;
        unsigned long long sm = vm;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int tc = __shfl_up_sync(0xffffffffu, sc, o);
          const unsigned long long tm = __shfl_up_sync(0xffffffffu, sm, o);
          if (c.lane >= o) { sc += tc; sm += tm; }
        }
        const bool hit = vc > 0 && (count_mode ? (run_c + sc >= top_k) : (run_m + sm >= target_fix));
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (ballot) {
          const int l = __ffs(ballot) - 1;
          found = base + l;
          run_c += __shfl_sync(0xffffffffu, sc, l);  // ids up to and including the crossing bin
        } else {
          run_c += __shfl_sync(0xffffffffu, sc, 31);
          run_m += __shfl_sync(0xffffffffu, sm, 31);
        }
      }
      if (c.lane == 0) { s->bcast_i[0] = found; s->bcast_i[1] = run_c; }
    }
    __syncthreads();
    const int found = s->bcast_i[0], through = s->bcast_i[1];
    __syncthreads();
    if (found < 0 || through > kListCap) { out.applicable = 0; return out; }  // same outcome in every CTA
    pick = found;
  }

  // ------------------------------------------------------------------ gather every id up to the crossing bin
  if (c.tid == 0) s->list_count = 0;
  c.cluster.sync();
  {
    int *list_count0 = c.cluster.map_shared_rank(&s->list_count, 0);
    float *list_y0 = c.cluster.map_shared_rank(s->u.w.list_y, 0);
    int *list_id0 = c.cluster.map_shared_rank(s->u.w.list_id, 0);
    for (int it = 0; it < c.region; it += 32) {
      const int j = c.warp * c.region + it + c.lane;
      if (j >= c.len) continue;
      const float y = s->y[j];
      if (!(y > -CUDART_INF_F)) continue;
      if (!everything) {
        const float d = max_logit - y;
        if (!(d < span)) continue;
        int b = int(d * inv_w);
        b = b < 0 ? 0 : (b >= kBins ? kBins - 1 : b);
        if (b > pick) continue;
      }
      const int slot = atomicAdd(list_count0, 1);
      if (slot < kListCap) { list_y0[slot] = y; list_id0[slot] = c.begin + j; }
    }
  }
  c.cluster.sync();
  if (c.rank != 0) { out.finished = 1; return out; }

  // ------------------------------------------------------------------ rank 0: the reference's arithmetic, literally
  const int n = min(s->list_count, kListCap);
  double *e_sorted = reinterpret_cast<double *>(s->bin_mass);       // [n] exp weights in the stable order
  double *p_sorted = reinterpret_cast<double *>(s->u.w.total_mass); // [n] probabilities in the stable order
  int *pos_by_id = s->u.w.total_count;                              // [n] stable-order position of the q-th id
  for (int i = c.tid; i < n; i += kThreads) {
    const float yi = s->u.w.list_y[i];
    const int idi = s->u.w.list_id[i];
    int before_y = 0, before_id = 0;
    for (int k = 0; k < n; ++k) {
      const float yk = s->u.w.list_y[k];
      const int idk = s->u.w.list_id[k];
      before_y += (yk > yi || (yk == yi && idk < idi)) ? 1 : 0;
      before_id += idk < idi ? 1 : 0;
    }
    s->u.w.sorted_y[before_y] = yi;
    s->u.w.sorted_id[before_y] = idi;
    e_sorted[before_y] = exp((double(yi) - double(max_logit)) / t);
    pos_by_id[before_id] = before_y;
  }
  __syncthreads();
  if (c.tid == 0) {
    const int entered = count_mode ? top_k : n;  // ids that enter the softmax among the gathered ones
    int status = 0;
    double z = z_tilde;
    if (count_mode || everything) {  // normaliser over the survivors only: sequential in id order, as the reference
      z = 0;
      for (int q = 0; q < n; ++q) { const int pos = pos_by_id[q]; if (pos < entered) z += e_sorted[pos]; }
    }
    int kept = entered;
    double mass = 1.0;
    if (!(top_p < 1.0)) {
      for (int i = 0; i < entered; ++i) p_sorted[i] = e_sorted[i] / z;
    } else {
      // do { mass += p[idx[k++]]; } while (k < n && mass < top);   (sampling.cpp:36); p = e/z computed on the way
      mass = 0;
      int k = 0;
      double prev = 0;
      do {
        prev = mass;
        const double p = e_sorted[k] / z;
        p_sorted[k++] = p;
        mass += p;
      } while (k < entered && mass < top_p);
      kept = k;
      if (!(count_mode || everything)) {
        // the normaliser is the parallel one: certify the crossing against its error bound
        const double rel = z_err / z + (double(k) + 8.0) * kU;
        if (mass < top_p) status |= 2;  // not reached inside the gathered ids (only possible within the bound)
        else if (mass < top_p * (1.0 + rel) || prev >= top_p * (1.0 - rel)) status |= 2;
      }
      for (int i = 0; i < kept; ++i) p_sorted[i] /= mass;
    }
    double e_kept = 0;
    for (int i = 0; i < kept; ++i) e_kept += e_sorted[i];
    out.kept = kept; out.z = z; out.e_kept = e_kept; out.entered = count_mode ? top_k : allowed;
    out.cut.y = s->u.w.sorted_y[kept - 1]; out.cut.id = s->u.w.sorted_id[kept - 1];
    if (want_draw) {
      // draw(): z2 = sum p in id order; t = u*z2; first id with t < running sum, else the last positive id
      double z2 = 0;
      for (int q = 0; q < n; ++q) { const int pos = pos_by_id[q]; if (pos < kept) z2 += p_sorted[pos]; }
      const double target = u * z2, slack = (4.0 * kept + 64.0) * kU * z2;
      double run = 0;
      int token = -1, last = -1;
      for (int q = 0; q < n; ++q) {
        const int pos = pos_by_id[q];
        if (pos >= kept) continue;
        const double v = p_sorted[pos], below = run;
        run += v;
        if (v > 0) last = s->u.w.sorted_id[pos];
        if (target < run) {
          token = s->u.w.sorted_id[pos];
          if (run - target < slack || (below > 0 && target - below < slack)) status |= 1;
          break;
        }
      }
      if (token < 0) { token = last; status |= 1; }
      out.token = token;
    }
    out.status = status;
    s->outcome.i[0] = out.token; s->outcome.i[1] = out.status; s->outcome.i[2] = out.kept; s->outcome.i[3] = out.cut.id;
    s->outcome.f[0] = out.cut.y; s->outcome.d[0] = out.z; s->outcome.d[1] = out.e_kept;
  }
  __syncthreads();
  out.token = s->outcome.i[0]; out.status = s->outcome.i[1]; out.kept = s->outcome.i[2]; out.cut.id = s->outcome.i[3];
  out.cut.y = s->outcome.f[0]; out.z = s->outcome.d[0]; out.e_kept = s->outcome.d[1];
  out.entered = count_mode ? top_k : allowed;
  return out;
}

}  // namespace ds41
