// C-ABI entry points of the sampler and of the host-side Philox helpers.  See include/ds41_b200.h.
#include "ds41_b200.h"
#include "row_kernel.cuh"
#include "stream_types.cuh"
#include "flat.cuh"
#include "replay.cuh"
#include "phase_events.h"
#include "host_error.h"
#include <cmath>
#include <cstdlib>

namespace ds41 {

int cluster_size_for(int vocab) {
  int n = 1;
  while (n < kMaxCluster && vocab > n * kSliceCap) n <<= 1;
  // more CTAs per row than strictly needed keep the per-CTA slice short (latency) once the row is large
  if (vocab > 32768) n = kMaxCluster;
  return n;
}

template <int kMode>
cudaError_t launch_rows(const RowArgs &a, int rows, cudaStream_t stream) {
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (configured_device != dev) {
    e = cudaFuncSetAttribute(row_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(RowSmem)));
    if (e != cudaSuccess) return e;
    configured_device = dev;
  }
  const int cl = cluster_size_for(a.vocab);
  RowArgs args = a;
  args.rows = rows;
  // left-over rows only: a persistent grid of two clusters per 8 SMs walks the status words
  const int clusters = a.only_uncovered ? (rows < 74 ? rows : 74) : rows;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(clusters) * cl);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = sizeof(RowSmem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, row_kernel<kMode>, args);
}
template cudaError_t launch_rows<kModeSample>(const RowArgs &, int, cudaStream_t);
template cudaError_t launch_rows<kModeStats>(const RowArgs &, int, cudaStream_t);

int chunks_for(int vocab);
cudaError_t launch_chunks(const ChunkArgs &a, int rows, cudaStream_t stream);
cudaError_t launch_combine(const CombineArgs &a, bool stats, cudaStream_t stream);

}  // namespace ds41

using namespace ds41;

namespace {
// [chunk records][status words when the caller passes none][batch path for wide nuclei]
size_t streaming_bytes(int rows, int vocab) {
  return size_t(rows) * chunks_for(vocab) * sizeof(ChunkRecord) + ((size_t(rows) * 4 + 15) & ~size_t(15));
}
// DS41_FLAT_MIN_ROWS (read once) moves the batch size from which the batch path for wide nuclei is used
int flat_min_rows() {
  static const int value = [] {
    const char *e = getenv("DS41_FLAT_MIN_ROWS");
    const int v = e ? atoi(e) : 0;
    return v >= 1 ? v : kFlatMinRows;
  }();
  return value;
}
bool flat_shape(int rows, int vocab) { return rows >= flat_min_rows() && vocab >= kFlatMinVocab; }
}  // namespace

namespace ds41 {
// DS41_BOUND_SCALE (read once; tests only) multiplies the certification bounds of the batch path and of the
// verification kernel, so that many decisions are flagged as uncertified and take the exact replay
double bound_scale() {
  static const double value = [] {
    const char *e = getenv("DS41_BOUND_SCALE");
    const double v = e ? atof(e) : 0.0;
    return v >= 1.0 ? v : 1.0;
  }();
  return value;
}
PhaseEvents &phase_events() {
  static PhaseEvents p;
  return p;
}
}  // namespace ds41

extern "C" int ds41_b200_profile_phases(int enable) {
  ds41::PhaseEvents &p = ds41::phase_events();
  if (enable && !p.on) {
    for (int i = 0; i < ds41::kPhaseMarks; ++i) {
      const cudaError_t e = cudaEventCreate(&p.events[i]);
      if (e != cudaSuccess) return int(e);
    }
    p.on = true;
  } else if (!enable && p.on) {
    p.on = false;
    for (int i = 0; i < ds41::kPhaseMarks; ++i) cudaEventDestroy(p.events[i]);
  }
  p.next = 0;
  return 0;
}

extern "C" int ds41_b200_profile_read(float *ms, int capacity) {
  ds41::PhaseEvents &p = ds41::phase_events();
  if (!p.on || p.next < 2 || !ms) return 0;
  if (cudaEventSynchronize(p.events[p.next - 1]) != cudaSuccess) return -1;
  int n = 0;
  for (int i = 0; i + 1 < p.next && n < capacity; ++i, ++n)
    if (cudaEventElapsedTime(&ms[n], p.events[i], p.events[i + 1]) != cudaSuccess) return -1;
  return n;
}

extern "C" size_t ds41_b200_sample_scratch_bytes(int rows, int vocab) {
  if (rows < 1 || vocab < 1 || vocab > DS41_B200_MAX_VOCAB) return 0;
  return streaming_bytes(rows, vocab) + (flat_shape(rows, vocab) ? flat_scratch_bytes(rows) : 0) + replay_scratch_bytes();
}

extern "C" uint32_t ds41_spark_rng_word_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw) {
  if (slot > 5 || purpose > 3 || draw / 4 > UINT32_MAX) { set_error("Philox v2 address out of range"); return 0; }
  return philox_word(seed, step, slot, purpose, draw);
}
extern "C" double ds41_spark_uniform_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw) {
  if (slot > 5 || purpose > 3 || draw > 8589934591ULL) { set_error("Philox v2 address out of range"); return NAN; }
  return philox_uniform(seed, step, slot, purpose, draw);
}
extern "C" const char *ds41_spark_error(void) { return last_error(); }

extern "C" int ds41_b200_sample_logits(const ds41_b200_sample_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_sample_args)) return invalid("sample args: struct size / ABI mismatch");
  if (p->rows < 1 || p->vocab < 1 || p->vocab > DS41_B200_MAX_VOCAB) return invalid("sample args: rows/vocab out of range");
  if (!p->logits || (p->logits_stride < p->vocab && p->logits_stride != 0) || !p->seeds || !p->steps || !p->tokens) return invalid("sample args: null buffer or short stride");
  if (!std::isfinite(p->temperature) || p->temperature < 0 || !std::isfinite(p->top_p) || p->top_p <= 0 || p->top_p > 1)
    return invalid("temperature/top_p/logits");
  if (p->top_k < 0 || !(p->repetition > 0) || !std::isfinite(p->repetition) || !std::isfinite(p->presence) || !std::isfinite(p->frequency))
    return invalid("penalty/top_k arguments");
  if (p->slot > 5 || p->purpose > 3) return invalid("Philox v2 address out of range");
  if (p->history && (p->history_stride < 0 || (!p->history_len && p->history_stride > DS41_B200_MAX_HISTORY)))
    return invalid("history longer than DS41_B200_MAX_HISTORY");
  if (p->mask && p->mask_stride < (p->vocab + 31) / 32) return invalid("mask stride shorter than the vocabulary");
  RowArgs a{};
  a.logits = p->logits; a.logits_stride = p->logits_stride; a.vocab = p->vocab;
  a.temperature = p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0;  // engine/src/sampling.cpp:209-210
  a.top_p = p->top_p; a.top_k = p->top_k;
  a.repetition = p->repetition; a.presence = p->presence; a.frequency = p->frequency;
  a.history = p->history; a.history_stride = p->history_stride; a.history_len = p->history_len;
  a.mask = p->mask; a.mask_stride = p->mask_stride;
  a.seeds = p->seeds; a.steps = p->steps; a.slot = p->slot; a.purpose = p->purpose;
  a.tokens = p->tokens; a.status = p->status; a.stats = nullptr;
  const bool penalised = p->history && (p->repetition != 1.f || p->presence != 0.f || p->frequency != 0.f);
  const size_t need = ds41_b200_sample_scratch_bytes(p->rows, p->vocab);
  const bool scratch_ok = p->scratch && p->scratch_bytes >= need && !(reinterpret_cast<uintptr_t>(p->scratch) & 15u) &&
                          !penalised && !p->mask && p->top_k <= kCand;
  // Batches of rows that are only cut by top-p first go through the batch path; it answers the rows it fits and marks
  // the others -8 / -9, and the paths below then only touch those.
  const bool flat = scratch_ok && flat_shape(p->rows, p->vocab) && p->top_k == 0 && p->temperature > 0 &&
                    p->logits_stride != 0 && p->logits_stride % 4 == 0 && !(reinterpret_cast<uintptr_t>(p->logits) & 15u);
  // the streaming path covers small nuclei only: a full-vocabulary draw never fits its candidate sets
  const bool streaming = scratch_ok && (p->top_p < 1.0 || p->top_k > 0 || p->temperature == 0);
  if (!flat && !streaming) return int(launch_rows<kModeSample>(a, p->rows, stream));
  const int chunks = chunks_for(p->vocab);
  ChunkRecord *records = static_cast<ChunkRecord *>(p->scratch);
  int32_t *status = p->status ? p->status : reinterpret_cast<int32_t *>(records + size_t(p->rows) * chunks);
  cudaError_t e;
  if (flat) {
    FlatArgs f{};
    f.logits = p->logits; f.stride = p->logits_stride; f.vocab = p->vocab; f.rows = p->rows;
    f.t = a.temperature; f.top_p = p->top_p; f.seeds = p->seeds; f.steps = p->steps; f.slot = p->slot;
    f.purpose = p->purpose; f.tokens = p->tokens; f.status = status;
    f.head_stats = static_cast<const HeadRowStats *>(p->row_extremes);
    f.bound_scale = bound_scale();
    void *flat_scratch = static_cast<unsigned char *>(p->scratch) + streaming_bytes(p->rows, p->vocab);
    e = launch_flat(f, flat_scratch, stream);
    if (e != cudaSuccess) return int(e);
    // what the batch path could not take (plateaus of equal logits at the cut, ranges beyond its exponent limit) goes to
    // the cluster kernel: a small persistent grid that returns at once when no row was handed on
    a.status = status;
    a.only_uncovered = 1;
    a.pending = flat_pending(flat_scratch);
    e = launch_rows<kModeSample>(a, p->rows, stream);
    if (e != cudaSuccess) return int(e);
    phase_mark(stream);
    // rows whose decision fell inside the rounding bound of the parallel sums: redone in the reference's own order
    ReplayArgs r{p->logits, p->logits_stride, p->vocab, p->rows, a.temperature, p->top_p, p->seeds, p->steps, p->slot,
                 p->purpose, p->tokens, status,
                 static_cast<unsigned char *>(flat_scratch) + flat_scratch_bytes(p->rows),
                 const_cast<int *>(flat_pending(flat_scratch)) + 1};
    e = launch_replay(r, stream);
    phase_mark(stream);
    return int(e);
  }
  if (streaming) {
    // streaming path: chunk records -> combine -> cluster kernel only for the rows the combine could not cover
    ChunkArgs c{p->logits, p->logits_stride, p->vocab, 0, chunks, a.temperature, records, nullptr};
    e = launch_chunks(c, p->rows, stream);
    if (e != cudaSuccess) return int(e);
    CombineArgs m{records, p->rows, 1, chunks, p->vocab, a.temperature, p->top_p, p->top_k, p->seeds, p->steps, p->slot,
                  p->purpose, p->tokens, status, nullptr, 0};
    e = launch_combine(m, false, stream);
    if (e != cudaSuccess) return int(e);
  }
  a.status = status;
  a.only_uncovered = 1;
  return int(launch_rows<kModeSample>(a, p->rows, stream));
}

namespace ds41 {
__global__ void exp_probe_kernel(const double *x, double *out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = exp_nonpos(x[i]);
}
}  // namespace ds41

namespace ds41 {
cudaError_t launch_flat_weight_probe(const float *y, float max_logit, double t, double *out, int n, cudaStream_t stream);
}
extern "C" int ds41_b200_test_batch_weight(const float *y, float max_logit, double temperature, double *out, int n,
                                           cudaStream_t stream) {
  if (!y || !out || n < 1 || !(temperature > 0)) return invalid("weight probe arguments");
  return int(ds41::launch_flat_weight_probe(y, max_logit, temperature, out, n, stream));
}

extern "C" int ds41_b200_test_exp_nonpos(const double *x, double *out, int n, cudaStream_t stream) {
  if (!x || !out || n < 1) return invalid("exp probe arguments");
  ds41::exp_probe_kernel<<<(n + 255) / 256, 256, 0, stream>>>(x, out, n);
  return int(cudaGetLastError());
}

