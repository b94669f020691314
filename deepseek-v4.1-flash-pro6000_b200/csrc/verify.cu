// Speculative verification from logits (MTP accept / resample), batched over sequences.
//
// Rule reproduced: verify_impl, engine/third_party/spark/src/sampling.cpp:39-53, with p and q rows produced by the
// sampler's probability rule (engine/src/sampling.cpp:142-219), i.e. the sequence
//   probabilities_rows(target) ; probabilities(draft_k) ; reject_sample(...)   (engine/src/speculation.cpp:126-182).
// Two launches:
//   1. row statistics for every target and draft row (row_kernel<kModeStats>): first maximum, normaliser, top-p cut
//      and kept mass, written to caller-provided scratch;
//   2. one cluster per sequence walks the positions: accept test from the two rows' statistics and the two logits at
//      the draft id; on the first rejection the residual max(0,p-q) is drawn by an inverse CDF streamed from the two
//      rows (normally still L2 resident), otherwise the bonus token is drawn from the last target row.
#include <atomic>
#include "ds41_b200.h"
#include "host_error.h"
#include "replay.cuh"
#include "row_kernel.cuh"
#include "stream_types.cuh"
#include <cmath>

namespace ds41 {

template <int kMode>
cudaError_t launch_rows(const RowArgs &a, int rows, cudaStream_t stream);
int cluster_size_for(int vocab);
int chunks_for(int vocab);
cudaError_t launch_chunks(const ChunkArgs &a, int rows, cudaStream_t stream);
cudaError_t launch_combine(const CombineArgs &a, bool stats, cudaStream_t stream);

struct VerifyArgs {
  const float *target, *draft;
  const int32_t *ids;
  const RowStats *pstats, *qstats;
  int drafts, vocab;
  double temperature;
  const uint64_t *seeds, *steps;
  ds41_spark_result *results;
  int32_t *status;
  double bound_scale;   // 1 (tests widen the bounds to exercise the replay)
};

struct Measure {  // one row's probability measure: P(id) = survives ? exp((x-max)/T) / e_kept : 0
  const float *x;
  RowStats st;
  double inv_t, inv_kept;  // 1/T and 1/e_kept: multiplications instead of divisions (a few ulp, inside bound())
  __device__ __forceinline__ double at(int id) const {
    const float y = __ldg(x + id);
    return survives(y, id, st.cut) ? exp_nonpos((double(y) - double(st.max_logit)) * inv_t) * inv_kept : 0.0;
  }
  __device__ __forceinline__ double bound() const { return 2.0 * (double(st.kept) + 256.0) * kU; }
};

__global__ void __launch_bounds__(kThreads, 2) verify_kernel(VerifyArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  RowSmem *s = reinterpret_cast<RowSmem *>(smem_raw);
  RowCtx c = make_ctx(s, a.vocab);
  const int seq = blockIdx.x / c.nranks;
  const int D = a.drafts;
  const bool greedy = a.temperature == 0;
  const uint64_t seed = a.seeds[seq], step = a.steps[seq];
  ds41_spark_result r{};
  int status = 0;
  // any rejected row of this transaction rejects the transaction (the reference computes every p and q row first)
  for (int k = 0; k <= D; ++k) {
    const int st = a.pstats[size_t(seq) * (D + 1) + k].status;
    if (st < 0 && status >= 0) status = st;
    else if (st > 0 && status >= 0) status |= st;
  }
  if (!greedy)
    for (int k = 0; k < D; ++k) {
      const int st = a.qstats[size_t(seq) * D + k].status;
      if (st < 0 && status >= 0) status = st;
      else if (st > 0 && status >= 0) status |= st;
    }
  for (int k = 0; k < D && status >= 0 && !r.rejected; ++k) {
    const int d = a.ids[size_t(seq) * D + k];
    if (d < 0 || d >= a.vocab) { status = -6; break; }  // checked only when the position is reached (sampling.cpp:44)
    const RowStats ps = a.pstats[size_t(seq) * (D + 1) + k];
    Measure P{a.target + (size_t(seq) * (D + 1) + k) * a.vocab, ps, greedy ? 0.0 : 1.0 / a.temperature, 1.0 / ps.e_kept};
    bool accept;
    if (greedy) {
      accept = d == P.st.argmax;
      if (!accept) { r.tokens[r.emitted++] = P.st.argmax; r.rejected = 1; }
    } else {
      const RowStats qs = a.qstats[size_t(seq) * D + k];
      Measure Q{a.draft + (size_t(seq) * D + k) * a.vocab, qs, 1.0 / a.temperature, 1.0 / qs.e_kept};
      const double pd = P.at(d), qd = Q.at(d);
      if (!(qd > 0)) { status = -6; break; }
      const double ratio = fmin(1.0, pd / qd);
      const double u = philox_uniform(seed, step, uint32_t(k), 2);
      accept = u < ratio;
      if (ratio < 1.0 && fabs(u - ratio) <= (P.bound() + Q.bound() + 16 * kU) * a.bound_scale * ratio) status |= 4;
      if (!accept) {
        // residual draw: inverse CDF over max(0, P - Q) in id order
        auto value = [&](int j) { const int id = c.begin + j; return fmax(0.0, P.at(id) - Q.at(id)); };
        region_sums(c, value);
        int amb = 0;
        double total = 0;
        const int support = min(a.vocab, P.st.kept + Q.st.kept);
        const int token = draw_token(c, philox_uniform(seed, step, uint32_t(k), 3),
                                     (2.0 * support + 256.0) * kU * a.bound_scale, (P.bound() + Q.bound()) * a.bound_scale,
                                     value, &amb, &total);
        if (!(total > 0) || token < 0) { status = -2; break; }
        if (amb) status |= 8;
        r.tokens[r.emitted++] = token;
        r.rejected = 1;
      }
    }
    if (accept) { r.tokens[r.emitted++] = d; ++r.accepted_drafts; }
  }
  if (status >= 0 && !r.rejected) {
    const RowStats ps = a.pstats[size_t(seq) * (D + 1) + D];
    Measure P{a.target + (size_t(seq) * (D + 1) + D) * a.vocab, ps, greedy ? 0.0 : 1.0 / a.temperature, 1.0 / ps.e_kept};
    if (greedy) {
      r.tokens[r.emitted++] = P.st.argmax;
    } else {
      auto value = [&](int j) { return P.at(c.begin + j) * P.st.e_kept; };  // unnormalised weights, as the sampler
      region_sums(c, value);
      int amb = 0;
      double total = 0;
      const int token = draw_token(c, philox_uniform(seed, step, uint32_t(D), 0),
                                   (2.0 * P.st.kept + 256.0) * kU * a.bound_scale, 0.0, value, &amb, &total);
      if (amb) status |= 1;
      r.tokens[r.emitted++] = token;
    }
  }
  r.accepted_input_rows = r.accepted_drafts + 1;
  if (status < 0) { r = ds41_spark_result{}; r.emitted = -1; }
  if (c.rank == 0 && c.tid == 0) {
    a.results[seq] = r;
    if (a.status) a.status[seq] = status;
  }
  c.cluster.sync();
}

}  // namespace ds41

namespace ds41 {
namespace {
// [row statistics][chunk records of the streaming path], rounded up to 16 bytes; the replay's rows follow
size_t verify_streaming_bytes(int sequences, int drafts, int vocab) {
  const size_t rows = size_t(sequences) * size_t(2 * drafts + 1);
  return (rows * sizeof(RowStats) + rows * chunks_for(vocab) * sizeof(ChunkRecord) + 15) & ~size_t(15);
}
}  // namespace
}  // namespace ds41

using namespace ds41;

extern "C" size_t ds41_b200_verify_scratch_bytes_for(int sequences, int drafts, int vocab) {
  if (sequences < 1 || drafts < 0 || drafts > 5 || vocab < 1 || vocab > DS41_B200_MAX_VOCAB) return 0;
  return verify_streaming_bytes(sequences, drafts, vocab) + verify_replay_scratch_bytes();
}
extern "C" size_t ds41_b200_verify_scratch_bytes(int sequences, int drafts) {
  return ds41_b200_verify_scratch_bytes_for(sequences, drafts, DS41_B200_MAX_VOCAB);
}

extern "C" int ds41_b200_verify_logits(const ds41_b200_verify_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_verify_args)) return invalid("verify args: struct size / ABI mismatch");
  if (p->sequences < 1 || p->drafts < 0 || p->drafts > 5 || p->vocab < 1 || p->vocab > DS41_B200_MAX_VOCAB)
    return invalid("verify arguments");
  if (!std::isfinite(p->temperature) || p->temperature < 0 || !std::isfinite(p->top_p) || p->top_p <= 0 || p->top_p > 1)
    return invalid("temperature/top_p/logits");
  const bool greedy = p->temperature == 0;
  if (!p->target_logits || !p->seeds || !p->steps || !p->results ||
      (p->drafts && (!p->draft_ids || (!p->draft_logits && !greedy))))
    return invalid("verify arguments");
  const size_t stat_rows = size_t(p->sequences) * size_t(2 * p->drafts + 1);
  if (!p->scratch || p->scratch_bytes < stat_rows * sizeof(RowStats) || (reinterpret_cast<uintptr_t>(p->scratch) & 15u))
    return invalid("verify scratch too small or misaligned");
  RowStats *pstats = static_cast<RowStats *>(p->scratch);
  RowStats *qstats = pstats + size_t(p->sequences) * (p->drafts + 1);
  // with room for the chunk records the row statistics come from the streaming path (cluster kernel only for rows
  // it cannot cover); with statistics-only scratch every row goes through the cluster kernel
  const size_t streaming_need = verify_streaming_bytes(p->sequences, p->drafts, p->vocab);
  const bool streaming = p->scratch_bytes >= streaming_need;
  ChunkRecord *records = reinterpret_cast<ChunkRecord *>(pstats + stat_rows);
  RowArgs a{};
  a.vocab = p->vocab; a.logits_stride = p->vocab;
  a.temperature = p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0;
  a.top_p = p->top_p; a.top_k = 0; a.repetition = 1.f;
  cudaError_t e = cudaSuccess;
  auto row_stats = [&](const float *logits, RowStats *stats, int rows, ChunkRecord *rec) -> cudaError_t {
    a.logits = logits; a.stats = stats; a.only_uncovered = 0;
    if (streaming) {
      const int chunks = chunks_for(p->vocab);
      ChunkArgs c{logits, p->vocab, p->vocab, 0, chunks, a.temperature, rec};
      cudaError_t err = launch_chunks(c, rows, stream);
      if (err != cudaSuccess) return err;
      CombineArgs m{rec, rows, 1, chunks, p->vocab, a.temperature, p->top_p, 0, nullptr, nullptr, 0, 0, nullptr, nullptr, stats};
      err = launch_combine(m, true, stream);
      if (err != cudaSuccess) return err;
      a.only_uncovered = 1;
    }
    return launch_rows<kModeStats>(a, rows, stream);
  };
  e = row_stats(p->target_logits, pstats, p->sequences * (p->drafts + 1), records);
  if (e != cudaSuccess) return int(e);
  if (p->drafts && !greedy) {
    e = row_stats(p->draft_logits, qstats, p->sequences * p->drafts,
                  records + size_t(p->sequences) * (p->drafts + 1) * chunks_for(p->vocab));
    if (e != cudaSuccess) return int(e);
  }
  static thread_local int configured_device = -1;
  int dev = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return int(e);
  if (configured_device != dev) {
    e = cudaFuncSetAttribute(verify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(RowSmem)));
    if (e != cudaSuccess) return int(e);
    configured_device = dev;
  }
  VerifyArgs v{p->target_logits, p->draft_logits, p->draft_ids, pstats, qstats, p->drafts, p->vocab, a.temperature,
               p->seeds, p->steps, p->results, p->status, bound_scale()};
  const int cl = cluster_size_for(p->vocab);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(p->sequences) * cl);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = sizeof(RowSmem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, verify_kernel, v);
  if (e != cudaSuccess) return int(e);
  // transactions with a certification bit set: redone in the reference's order of operations, when the caller gave
  // the status words and room for two probability rows per CTA (the scratch-free entry point has neither)
  if (!greedy && p->status && p->scratch_bytes >= streaming_need + verify_replay_scratch_bytes()) {
    VerifyReplayArgs r{p->target_logits, p->draft_logits, p->draft_ids, p->sequences, p->drafts, p->vocab, a.temperature,
                       p->top_p, p->seeds, p->steps, p->results, p->status,
                       static_cast<unsigned char *>(p->scratch) + streaming_need};
    e = launch_verify_replay(r, stream);
  }
  return int(e);
}

// ---------------------------------------------------------------------------------------------------------------
// Verification without any caller-provided or library-allocated scratch.
//
// Some hosts of this library may not allocate device memory at the point where they verify a speculative step: an
// engine that has handed all of its HBM to weight / KV / expert pools at start-up and runs with a fixed memory plan,
// or a plugin loaded into a process whose allocator it must not touch.  For them the row statistics live in a
// fixed-size array that is part of the library image itself, so the call needs nothing but the inputs and outputs.
//
// The array is device memory reserved on EVERY GPU that loads the library, from load until the process exits
// (kStaticStatRows * sizeof(RowStats) = 48 KiB).  Its name is only a host-side handle: the address the kernels need
// is looked up once per device with cudaGetSymbolAddress, with that device current, on the first call made for the
// device.  That first call therefore does a little set-up work (it may load the module) and should be made before
// any stream capture begins; later calls only enqueue kernels.  No cudaMalloc / cudaFree or allocating library
// routine is ever called on this path.
//
// All calls share the one array.  Every record a call reads is written earlier by that same call (the statistics
// kernels fill all sequences*(2*drafts+1) records before the per-sequence kernel starts), so nothing has to be
// cleared between calls and stale contents of a previous, larger call are never read.  Two calls that overlap on
// the GPU (different streams, or different host threads without ordering) would overwrite each other's records:
// the caller must serialise them, as the reference requires for its own sampler object (spark.h:35-36).
namespace ds41 {
namespace {
constexpr int kStaticStatRows = 1024;  // sequences * (2*drafts + 1) may not exceed this
static __device__ __align__(256) unsigned char g_static_stats[kStaticStatRows * sizeof(RowStats)];
constexpr int kMaxDevices = 64;
std::atomic<void *> g_static_stats_addr[kMaxDevices];   // zero-initialised (static storage)
}  // namespace
}  // namespace ds41

extern "C" int ds41_b200_verify_logits_static_max_rows(void) { return ds41::kStaticStatRows; }

extern "C" int ds41_b200_verify_logits_static(const ds41_b200_verify_args *p, cudaStream_t stream) {
  using namespace ds41;
  if (!p || p->struct_bytes != sizeof(ds41_b200_verify_args)) return invalid("verify args: struct size / ABI mismatch");
  if (p->sequences < 1 || p->drafts < 0 || p->drafts > 5) return invalid("verify arguments");
  const long long rows = (long long)p->sequences * (2 * p->drafts + 1);
  if (rows > kStaticStatRows)
    return invalid("ds41_b200_verify_logits_static: sequences*(2*drafts+1) exceeds the built-in limit of 1024 "
                   "statistics records; use ds41_b200_verify_logits with caller scratch");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return int(e);
  if (dev < 0 || dev >= kMaxDevices) return invalid("device ordinal beyond the static scratch table");
  void *addr = g_static_stats_addr[dev].load(std::memory_order_relaxed);
  if (!addr) {  // first call on this device: resolve the device address of the array (idempotent, so a race between
                // two first calls only repeats the lookup)
    e = cudaGetSymbolAddress(&addr, g_static_stats);
    if (e != cudaSuccess) return int(e);
    if (!addr) return invalid("cudaGetSymbolAddress returned a null address");
    g_static_stats_addr[dev].store(addr, std::memory_order_relaxed);
  }
  ds41_b200_verify_args with_scratch = *p;
  with_scratch.scratch = addr;
  with_scratch.scratch_bytes = sizeof(g_static_stats);
  return ds41_b200_verify_logits(&with_scratch, stream);
}
