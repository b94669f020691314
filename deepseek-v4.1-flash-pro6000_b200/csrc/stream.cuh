// Kernels of the streaming sampler (types and the description are in stream_types.cuh).  Included by stream.cu only.
#pragma once
#include "stream_types.cuh"

namespace ds41 {

constexpr int kWarpNear = 512;     // per-warp capacity of the list of ids near the chunk maximum
constexpr int kFineBins = 256;     // fine count histogram over [0, reach)

struct __align__(128) ChunkSmem {
  float y[kChunkIds];
  int bins[kFineBins];
  uint16_t near_ids[kChunkWarps][kWarpNear];
  float red_f[kChunkWarps];
  int red_i[kChunkWarps], red_j[kChunkWarps];
  double acc_d[4];  // FP64 accumulators filled with shared-memory atomics by warp leaders
  int ladder_count[12];
  unsigned long long mbar;
  int sent_count, overflow;
  int bcast[4];
};

__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per (row, chunk).  Thread t handles the four consecutive ids 4*(t + 256*i) .. +3, i = 0..7 (128-bit shared
// loads).  Passes over shared memory: (A) maximum + finiteness; (B) FP32-class sum of exponentials of every id,
// accumulated in FP64; (C) the ids near the maximum -> per-warp index lists (vote-based, no atomics) + a fine count
// histogram; then the lists only: the ids in the bins BEFORE the one that holds the 64th id are the candidates (a
// prefix of the stable order of fewer than 64 ids, so nothing has to be sorted), their exponentials redone in FP64.
__global__ void __launch_bounds__(kChunkThreads, 4) chunk_kernel(ChunkArgs a) {
  __shared__ ChunkSmem s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x / a.chunks, chunk = blockIdx.x % a.chunks;
  if (a.only_uncovered && a.only_uncovered[row] != kNotCovered) return;  // the same in every thread
  const int begin = min(a.vocab_local, chunk * kChunkIds);
  const int len = min(a.vocab_local, begin + kChunkIds) - begin;
  ChunkRecord *out = a.out + size_t(row) * a.chunks + chunk;
  const double t = a.temperature;
  if (tid < kCand) { out->cand[tid].y = -CUDART_INF_F; out->cand[tid].id = -1; }
  if (len <= 0) {  // padding chunk of an uneven shard
    if (tid == 0) { out->z = 0; out->max_logit = -CUDART_INF_F; out->argmax = 0x7fffffff; out->count = 0; out->status = 0; out->complete = 1; out->z_err = 0.f; }
    return;
  }
  // ---- stage: one thread issues the bulk copy and polls the mbarrier (bounded); everybody else waits at the barrier
  const float *src = a.logits + size_t(row) * a.stride + begin;
  const uint32_t bytes = uint32_t(len) * 4u;
  const bool tma = (bytes & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  if (tid == 0) {
    s.sent_count = 0; s.overflow = 0; s.bcast[2] = 1;
    s.acc_d[0] = s.acc_d[1] = s.acc_d[2] = s.acc_d[3] = 0.0;
    if (tma) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s.mbar)));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&s.mbar)), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(s.y)),
                   "l"(src), "r"(bytes), "r"(smem_u32(&s.mbar))
                   : "memory");
    }
  }
  if (tid < 12) s.ladder_count[tid] = 0;
  s.bins[tid] = 0;  // kFineBins == kChunkThreads
  if (tma) {
    if (tid == 0) {
      uint32_t done = 0;
      for (int spin = 0; spin < (1 << 22) && !done; ++spin)
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(smem_u32(&s.mbar)) : "memory");
      s.bcast[2] = int(done);
    }
  } else {
    for (int j = tid; j < len; j += kChunkThreads) s.y[j] = __ldg(src + j);
  }
  __syncthreads();
  if (!s.bcast[2]) {  // the bounded wait expired: report, do not touch the data
    if (tid == 0) { out->status = -5; out->count = 0; out->complete = 0; out->z = 0; out->max_logit = 0; out->argmax = -1; out->z_err = 0.f; }
    return;
  }
  const int vecs = len >> 2, tail0 = vecs << 2;  // full vectors; ids tail0..len-1 (at most 3) are handled by scalar code
  const float4 *y4 = reinterpret_cast<const float4 *>(s.y);

  // ---- (A) maximum (first index) and finiteness (0*y is NaN exactly when y is NaN or infinite)
  float best = -CUDART_INF_F, poison = 0.f;
  int best_j = 0x7fffffff;
  for (int v = tid; v < vecs; v += kChunkThreads) {
    const float4 q = y4[v];
    poison = fmaf(q.x, 0.f, fmaf(q.y, 0.f, fmaf(q.z, 0.f, fmaf(q.w, 0.f, poison))));
    const float mq = fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w));
    if (mq > best) {  // first index of the vector's maximum
      best = mq;
      best_j = 4 * v + (q.x == mq ? 0 : q.y == mq ? 1 : q.z == mq ? 2 : 3);
    }
  }
  if (tid < len - tail0) {
    const float y = s.y[tail0 + tid];
    poison = fmaf(y, 0.f, poison);
    if (y > best) { best = y; best_j = tail0 + tid; }
  }
  const float own_best = best;  // this thread's maximum: the 256 of them sample the top of the chunk
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oj = __shfl_xor_sync(0xffffffffu, best_j, o);
    if (ov > best || (ov == best && oj < best_j)) { best = ov; best_j = oj; }
  }
  int bad = __any_sync(0xffffffffu, !(poison == 0.f));
  if (lane == 0) { s.red_f[warp] = best; s.red_j[warp] = best_j; s.red_i[warp] = bad; }
  __syncthreads();
  best = s.red_f[0]; best_j = s.red_j[0]; bad = s.red_i[0];
#pragma unroll
  for (int w = 1; w < kChunkWarps; ++w) {
    if (s.red_f[w] > best || (s.red_f[w] == best && s.red_j[w] < best_j)) { best = s.red_f[w]; best_j = s.red_j[w]; }
    bad |= s.red_i[w];
  }
  if (bad || t == 0) {
    if (tid == 0) {
      out->z = 0; out->max_logit = best; out->argmax = bad ? -1 : best_j + begin + a.id_offset; out->count = 0;
      out->status = bad ? -1 : 0; out->complete = 0; out->z_err = 0.f;
    }
    return;
  }
  const float m = best;
  // how far below the maximum do the first 64 ids reach?  The 256 per-thread maxima are a sample of the top of the
  // chunk: the smallest ladder distance that holds 64 of them holds at least 64 ids.
  {
    const float ladder[12] = {0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 16.f, 24.f, 32.f};
    const float d = m - own_best;
#pragma unroll
    for (int k = 0; k < 12; ++k) {
      const unsigned ballot = __ballot_sync(0xffffffffu, d < ladder[k]);
      if (lane == 0 && ballot) atomicAdd(&s.ladder_count[k], __popc(ballot));
    }
  }

  // ---- (B) sum of exp((y-m)/T) over EVERY id in FP32-class arithmetic: x = y*c - m*c (one FMA), ex2.approx; relative
  // error per id <= (3 + |x|) * 2^-22; ids with |x| > 32 weigh less than 2^-32 each, so sum * 35 * 2^-22 + 1e-10 bounds
  // the total.  Every term is added to an FP64 accumulator on its own (a large term must not swallow the low bits of
  // small ones: the candidates are subtracted again below).
  const float c32 = float(1.4426950408889634074 / t), mc = m * c32;
  double sum_all = 0;
  for (int v = tid; v < vecs; v += kChunkThreads) {
    const float4 q = y4[v];
    const float e0 = ex2_approx(fmaf(q.x, c32, -mc)), e1 = ex2_approx(fmaf(q.y, c32, -mc));
    const float e2 = ex2_approx(fmaf(q.z, c32, -mc)), e3 = ex2_approx(fmaf(q.w, c32, -mc));
    sum_all += (double(e0) + double(e1)) + (double(e2) + double(e3));
  }
  if (tid < len - tail0) sum_all += double(ex2_approx(fmaf(s.y[tail0 + tid], c32, -mc)));
  {
    const double wa = warp_sum(sum_all);
    if (lane == 0) atomicAdd(&s.acc_d[0], wa);
  }
  __syncthreads();  // also publishes ladder_count
  float reach = 32.f;
  {
    const float ladder[12] = {0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 16.f, 24.f, 32.f};
    int k = 0;
    while (k < 11 && s.ladder_count[k] < kCand) ++k;
    reach = ladder[k];
  }
  const float bin_scale = float(kFineBins) / reach, near_above = m - reach;

  // ---- (C) vectors holding an id near the maximum -> this warp's list of vector indices (positions from one vote
  // per vector, no atomics); then the fine count histogram over the listed vectors only
  int n_mine = 0;  // warp-uniform
  for (int v0 = warp * 32; v0 < vecs; v0 += kChunkThreads) {
    const int v = v0 + lane;
    float4 q = make_float4(-3.0e38f, -3.0e38f, -3.0e38f, -3.0e38f);
    if (v < vecs) q = y4[v];
    const bool any = fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)) > near_above;
    const unsigned ballot = __ballot_sync(0xffffffffu, any);
    if (any) {
      const int slot = n_mine + __popc(ballot & ((1u << lane) - 1u));
      if (slot < kWarpNear) s.near_ids[warp][slot] = uint16_t(v);
    }
    n_mine += __popc(ballot);
  }
  if (n_mine > kWarpNear && lane == 0) s.overflow = 1;
  const int n_list = min(n_mine, kWarpNear);
  __syncwarp();
  for (int q = lane; q < n_list; q += 32) {
    const float4 w = y4[s.near_ids[warp][q]];
    const float e[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (e[k] > near_above) atomicAdd(&s.bins[min(kFineBins - 1, int((m - e[k]) * bin_scale))], 1);
  }
  if (tid < len - tail0) {  // the (at most 3) tail ids are handled by threads 0..2 directly
    const float y = s.y[tail0 + tid];
    if (y > near_above) atomicAdd(&s.bins[min(kFineBins - 1, int((m - y) * bin_scale))], 1);
  }
  __syncthreads();
  // ---- bin that holds the 64th id: block-wide inclusive scan of the 256 bins (one bin per thread)
  {
    const int v = s.bins[tid];
    int sc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int tv = __shfl_up_sync(0xffffffffu, sc, o);
      if (lane >= o) sc += tv;
    }
    if (lane == 31) s.red_i[warp] = sc;
    if (tid == 0) s.bcast[0] = -1;
    __syncthreads();
    int before = 0;
#pragma unroll
    for (int w = 0; w < kChunkWarps; ++w) before += w < warp ? s.red_i[w] : 0;
    if (v > 0 && before + sc >= kCand && before + sc - v < kCand) s.bcast[0] = tid;
    __syncthreads();
  }
  const int found = s.bcast[0];
  // status -4 (the cluster kernel decides): the first bin alone holds 64 or more ids, or a warp's list overflowed
  const int status = (found == 0 || s.overflow) ? -4 : 0;
  const int pick = found < 0 ? kFineBins : found;  // candidates: near ids in bins < pick (fewer than 64 of them)
  const double inv_t = 1.0 / t;
  double e64 = 0, e32 = 0;
  auto consider = [&](float y, int j) {
    if (y > near_above && min(kFineBins - 1, int((m - y) * bin_scale)) < pick) {
      const int slot = atomicAdd(&s.sent_count, 1);
      if (slot < kCand) { out->cand[slot].y = y; out->cand[slot].id = j + begin + a.id_offset; }
      e64 += exp((double(y) - double(m)) * inv_t);
      e32 += double(ex2_approx(fmaf(y, c32, -mc)));  // bit-identical to the term added in (B)
    }
  };
  if (status == 0) {
    for (int q = lane; q < n_list; q += 32) {
      const int v = s.near_ids[warp][q];
      const float4 w = y4[v];
      consider(w.x, 4 * v); consider(w.y, 4 * v + 1); consider(w.z, 4 * v + 2); consider(w.w, 4 * v + 3);
    }
    if (tid < len - tail0) consider(s.y[tail0 + tid], tail0 + tid);
    const double a64 = warp_sum(e64), a32 = warp_sum(e32);
    if (lane == 0) { atomicAdd(&s.acc_d[2], a64); atomicAdd(&s.acc_d[3], a32); }
  }
  __syncthreads();
  if (tid == 0) {
    // candidates in FP64; the rest = (all - candidates) of the FP32-class sum (FP64 accumulation makes the subtraction
    // clean to ~1e-13 of the total)
    const int n = status == 0 ? min(s.sent_count, kCand) : 0;
    const double z_all = s.acc_d[0], z_list = s.acc_d[2];
    const double z_rest = fmax(0.0, z_all - s.acc_d[3]);
    out->z = z_list + z_rest;
    out->z_err = float((z_rest * 35.0 * 0x1p-22 + 1e-10 + z_all * 1e-12 + z_list * (double(n) + 16.0) * kU) * 1.000001);
    out->max_logit = m; out->argmax = best_j + begin + a.id_offset;
    out->count = n; out->status = status;
    out->complete = (status == 0 && n == len) ? 1 : 0;
  }
}

// ---------------------------------------------------------------------------------------------------------------
constexpr int kCombineThreads = 256;
constexpr int kMaxCandAll = kMaxRecords * kCand;
constexpr int kCombineBins = 512;

struct CombineSmem {
  float cy[kMaxCandAll];   // all candidates as received
  int cid[kMaxCandAll];
  int crec[kMaxCandAll];   // record of each candidate
  float fy[kMaxCandAll];   // filtered candidates (those that can still be kept)
  int fid[kMaxCandAll];
  int frec[kMaxCandAll];   // record of each filtered candidate
  float sy[kMaxCandAll];   // filtered candidates in the stable order
  int sid[kMaxCandAll];
  double se[kMaxCandAll];
  double sp[kMaxCandAll];
  int by_id[kMaxCandAll];
  float bin_mass[kCombineBins];
  int bin_count[kCombineBins];
  int base[kMaxRecords + 1], complete[kMaxRecords], worst[kMaxRecords], ranked[kMaxRecords];
  double hz[kMaxRecords], hw[kMaxRecords];
  float hmax[kMaxRecords], hzerr[kMaxRecords];
  int harg[kMaxRecords], hcount[kMaxRecords], hstatus[kMaxRecords];
  int i_out[6];
  double d_out[3];
  int n_filtered;
};

template <int kMode>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineArgs a) {
  extern __shared__ __align__(16) unsigned char combine_raw[];
  CombineSmem &s = *reinterpret_cast<CombineSmem *>(combine_raw);
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (a.only_uncovered && a.status[row] != kNotCovered) return;  // the same in every thread
  const int nrec = a.groups * a.per_group;
  const double t = a.temperature;
  auto rec = [&](int r) -> const ChunkRecord & {
    return a.records[(size_t(r / a.per_group) * a.rows + row) * a.per_group + r % a.per_group];
  };
  // ---- headers into shared memory (one thread per record), then everything else reads them from there
  if (tid < nrec) {
    const ChunkRecord &h = rec(tid);
    s.hz[tid] = h.z; s.hmax[tid] = h.max_logit; s.harg[tid] = h.argmax; s.hcount[tid] = h.count;
    s.hstatus[tid] = h.status; s.complete[tid] = h.complete; s.hzerr[tid] = h.z_err;
    s.worst[tid] = -1; s.ranked[tid] = 0;
  }
  for (int j = tid; j < kCombineBins; j += kCombineThreads) { s.bin_mass[j] = 0.f; s.bin_count[j] = 0; }
  if (tid == 0) s.n_filtered = 0;
  __syncthreads();
  float m = -CUDART_INF_F;
  int arg = 0x7fffffff, status = 0;
  {
    int error = 0, escalate = 0;
    for (int r = 0; r < nrec; ++r) {  // records are in ascending id order, so the first record wins ties of the maximum
      if (s.hstatus[r] == -4) escalate = 1;  // tie group too large for the chunk list: the cluster kernel decides
      else if (s.hstatus[r] < 0 && error == 0) error = s.hstatus[r];
      if (s.hstatus[r] == 0 && (s.hmax[r] > m || (s.hmax[r] == m && s.harg[r] < arg))) { m = s.hmax[r]; arg = s.harg[r]; }
    }
    status = error ? error : (escalate ? kNotCovered : 0);
  }
  if (status < 0 || t == 0) {
    if (tid == 0) {
      if (kMode == kCombineDraw) { a.tokens[row] = status < 0 ? -1 : arg; if (a.status) a.status[row] = status; }
      else {
        RowStats st{};
        st.z = 1; st.e_kept = 1; st.max_logit = m; st.argmax = arg; st.cut.y = m; st.cut.id = arg; st.kept = 1;
        st.entered = a.vocab; st.status = status;
        a.stats[row] = st;
      }
    }
    return;
  }
  if (tid < nrec) s.hw[tid] = s.hz[tid] > 0 ? exp((double(s.hmax[tid]) - double(m)) / t) : 0.0;
  if (tid == 0) {
    s.base[0] = 0;
    for (int r = 0; r < nrec; ++r) s.base[r + 1] = s.base[r] + s.hcount[r];
  }
  __syncthreads();
  double z = 0, z_err = 0;
  for (int r = 0; r < nrec; ++r) { z += s.hz[r] * s.hw[r]; z_err += double(s.hzerr[r]) * s.hw[r]; }
  z_err += 4.0 * nrec * kU * z;
  const int n = s.base[nrec];
  const bool count_mode = a.top_k > 0 && a.top_k < a.vocab;
  // ---- candidates into shared memory + coarse histogram over d = m - y (1/32 logit bins, d >= 16 in the last bin):
  // counts for top-k, FP32 masses for top-p.  It only selects which candidates can possibly be kept.
  const float inv_t = float(1.0 / t);
  for (int idx = tid; idx < nrec * kCand; idx += kCombineThreads) {
    const int r = idx / kCand, i = idx % kCand;
    if (i < s.hcount[r]) {
      const ChunkRecord &h = rec(r);
      const float y = h.cand[i].y;
      const int q = s.base[r] + i;
      s.cy[q] = y; s.cid[q] = h.cand[i].id; s.crec[q] = r;
      const float d = m - y;
      if (d < 16.f) {  // candidates further down can only matter if no crossing is found at all (then all are ranked)
        const int b = int(d * 32.f);
        atomicAdd(&s.bin_count[b], 1);
        if (!count_mode) atomicAdd(&s.bin_mass[b], __expf(-d * inv_t));
      }
    }
  }
  __syncthreads();
  if (warp == 0) {  // crossing bin; two bins of slack (the FP32 masses are approximate)
    int found = -1;
    int run_c = 0;
    float run_m = 0.f;
    const float target = float(a.top_p * z) * 1.0001f;
    for (int base = 0; base < kCombineBins && found < 0; base += 32) {
      const int vc = s.bin_count[base + lane];
      const float vm = s.bin_mass[base + lane];
      int sc = vc;
      float sm = vm;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int tc = __shfl_up_sync(0xffffffffu, sc, o);
        const float tm = __shfl_up_sync(0xffffffffu, sm, o);
        if (lane >= o) { sc += tc; sm += tm; }
      }
      const bool hit = vc > 0 && (count_mode ? (run_c + sc >= a.top_k) : (a.top_p < 1.0 && run_m + sm >= target));
      const unsigned ballot = __ballot_sync(0xffffffffu, hit);
      if (ballot) found = base + __ffs(ballot) - 1;
      run_c += __shfl_sync(0xffffffffu, sc, 31);
      run_m += __shfl_sync(0xffffffffu, sm, 31);
    }
    if (lane == 0) s.i_out[5] = found < 0 ? kCombineBins : min(kCombineBins - 2, found + 2);
  }
  __syncthreads();
  const int last_bin = s.i_out[5];  // candidates in bins <= last_bin are ranked exactly (all of them if no crossing)
  for (int q = tid; q < n; q += kCombineThreads) {
    const float d = m - s.cy[q];
    const int b = d < 16.f ? int(d * 32.f) : kCombineBins - 1;  // far candidates: ranked only when last_bin == kCombineBins
    if (b <= last_bin) {
      const int slot = atomicAdd(&s.n_filtered, 1);
      s.fy[slot] = s.cy[q]; s.fid[slot] = s.cid[q]; s.frec[slot] = s.crec[q];
      atomicAdd(&s.ranked[s.crec[q]], 1);
    }
  }
  __syncthreads();
  const int nf = s.n_filtered;
  const bool filtered_all = nf == n;
  // ---- exact stable order of the filtered candidates by counting
  for (int i = tid; i < nf; i += kCombineThreads) {
    const float yi = s.fy[i];
    const int idi = s.fid[i];
    int pos = 0;
    for (int k = 0; k < nf; ++k) pos += (s.fy[k] > yi || (s.fy[k] == yi && s.fid[k] < idi)) ? 1 : 0;
    s.sy[pos] = yi; s.sid[pos] = idi;
    const double e = exp((double(yi) - double(m)) / t);
    s.se[pos] = e;
    s.sp[pos] = e / z;  // p = e/z for the top-p walk (count mode recomputes it with its own normaliser)
    atomicMax(&s.worst[s.frec[i]], pos);  // worst position among this record's ranked candidates
  }
  __syncthreads();
  // ---- thread 0: who enters, normaliser, top-p prefix (the reference's loop), coverage
  if (tid == 0) {
    int st = 0, entered = nf, kept = 0;
    bool covered = true;
    double zz = z, mass = 1.0;
    if (count_mode) {
      entered = min(a.top_k, nf);
      if (nf < a.top_k) {  // fewer candidates than k: fine only if every record sent everything
        if (!filtered_all) covered = false;
        for (int r = 0; r < nrec; ++r) covered = covered && s.complete[r];
      }
      // the k survivors in id order -> sequential normaliser as the reference (insertion sort of <= 64 ids)
      int order[kCand];
      const int ne = min(entered, kCand);
      if (entered > kCand) covered = false;
      for (int i = 0; i < ne; ++i) {
        int j = i;
        while (j > 0 && s.sid[order[j - 1]] > s.sid[i]) { order[j] = order[j - 1]; --j; }
        order[j] = i;
      }
      zz = 0;
      for (int i = 0; i < ne; ++i) zz += s.se[order[i]];
      z_err = 0;
    }
    kept = entered;
    if (!(a.top_p < 1.0)) {
      if (count_mode)
        for (int i = 0; i < entered; ++i) s.sp[i] = s.se[i] / zz;
      if (!count_mode) {  // top_p = 1 without top-k keeps every id: only covered if every record is complete
        if (!filtered_all) covered = false;
        for (int r = 0; r < nrec; ++r) covered = covered && s.complete[r];
      }
    } else {
      if (count_mode)
        for (int i = 0; i < entered; ++i) s.sp[i] = s.se[i] / zz;
      mass = 0;
      int k = 0;
      double prev = 0;
      do {
        prev = mass;
        mass += s.sp[k++];
      } while (k < entered && mass < a.top_p);
      kept = k;
      if (!count_mode) {
        const double rel = z_err / zz + (double(k) + 8.0) * kU;
        if (mass < a.top_p) {
          // not reached inside the ranked candidates: everything is kept only if nothing else exists anywhere
          if (!filtered_all) covered = false;
          for (int r = 0; r < nrec; ++r) covered = covered && s.complete[r];
          if (!(mass < a.top_p * (1.0 - rel))) st |= 2;
        } else if (mass < a.top_p * (1.0 + rel) || prev >= a.top_p * (1.0 - rel)) st |= 2;
      }
    }
    // a record that did not send all of its ids must have its WORST candidate outside the surviving prefix (ids it
    // did not send are worse still).  A record with a candidate beyond the ranked bins is fine: that one is outside.
    const int limit = count_mode ? entered : kept;
    for (int r = 0; r < nrec; ++r) {
      if (s.complete[r]) continue;
      if (s.hcount[r] == 0 || (s.ranked[r] == s.hcount[r] && s.worst[r] < limit)) covered = false;
    }
    double e_kept = 0;
    for (int i = 0; i < kept; ++i) e_kept += s.se[i];
    s.i_out[0] = covered ? st : kNotCovered; s.i_out[1] = kept; s.i_out[2] = count_mode ? a.top_k : a.vocab;
    s.d_out[0] = zz; s.d_out[1] = e_kept; s.d_out[2] = mass;
  }
  __syncthreads();
  status = s.i_out[0];
  const int kept = s.i_out[1];
  if (status == kNotCovered) {
    if (tid == 0) {
      if (kMode == kCombineDraw) { a.tokens[row] = -1; if (a.status) a.status[row] = kNotCovered; }
      else { RowStats st{}; st.status = kNotCovered; st.max_logit = m; st.argmax = arg; a.stats[row] = st; }
    }
    return;
  }
  if (kMode == kCombineStats) {
    if (tid == 0) {
      RowStats st;
      st.z = s.d_out[0]; st.e_kept = s.d_out[1]; st.max_logit = m; st.argmax = arg;
      st.cut.y = s.sy[kept - 1]; st.cut.id = s.sid[kept - 1]; st.kept = kept; st.entered = s.i_out[2]; st.status = status; st.pad = 0;
      a.stats[row] = st;
    }
    return;
  }
  // ---- survivors in id order, then the reference's draw
  const double kept_mass = s.d_out[2];
  for (int i = tid; i < kept; i += kCombineThreads) {
    int pos = 0;
    for (int k = 0; k < kept; ++k) pos += s.sid[k] < s.sid[i] ? 1 : 0;
    s.by_id[pos] = i;
    if (a.top_p < 1.0) s.sp[i] /= kept_mass;  // p / mass (sampling.cpp:36), one id per thread
  }
  __syncthreads();
  if (tid == 0) {
    double z2 = 0;
    for (int q = 0; q < kept; ++q) z2 += s.sp[s.by_id[q]];
    const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
    const double target = u * z2, slack = (4.0 * kept + 64.0) * kU * z2;
    double run = 0;
    int token = -1, last = -1, st = status;
    for (int q = 0; q < kept; ++q) {
      const int i = s.by_id[q];
      const double v = s.sp[i], below = run;
      run += v;
      if (v > 0) last = s.sid[i];
      if (target < run) {
        token = s.sid[i];
        if (run - target < slack || (below > 0 && target - below < slack)) st |= 1;
        break;
      }
    }
    if (token < 0) { token = last; st |= 1; }
    a.tokens[row] = token;
    if (a.status) a.status[row] = st;
  }
}

}  // namespace ds41
