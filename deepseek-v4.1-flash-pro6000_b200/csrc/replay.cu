// Exact replay of rows whose decision the parallel paths could not certify.
//
// The fast paths sum in parallel and certify every decision against a bound on the difference to the reference's
// sequential FP64 sums; a row whose decision falls inside that bound (status bits 1 / 2), or whose cut search gave up
// (-4), is redone here in the reference's own order of operations, one CTA per row:
//   ds41_spark_probabilities (engine/third_party/spark/src/sampling.cpp:30-38): first maximum b;
//     p[i] = exp((double(x[i]) - x[b]) / t); z = sum of p[i] for i = 0..n-1 IN THAT ORDER; p[i] /= z; for top_p < 1 the
//     ids are ordered by p descending (ties: lower id first, std::stable_sort), mass += p[idx[k++]] while k < n and
//     mass < top_p, the rest is zeroed and every p[i] divided by mass;
//   draw (sampling.cpp:18-21): z = sum of p[i] in id order, t = u * z, c += p[i] until t < c.
// The sums run on one thread, in order, so they round exactly as the reference's do; only exp() itself can differ from
// the host library's in the last place, which moves a sum by a few 2^-53 relative instead of by vocab * 2^-53.  A
// decision that is still closer than 16 * 2^-53 to its threshold keeps its status bit; every other replayed row
// leaves with status 0.  The sums follow the reference's chain of roundings exactly but in parallel (integer prefix sums
// inside each binade of the accumulator, replay_core.cuh), and the order is never put together: the top-p loop consumes
// whole ranges of the key as integer sums and sorts only the few chunks in which it needs the terms one by one.  A
// full-vocabulary row costs a little under a millisecond; the parallel bound flags a few rows in 10^5.
#include "replay_core.cuh"
#include <atomic>

namespace ds41 {
namespace {

constexpr double kStillClose = 16.0 * kU;

__global__ void __launch_bounds__(kRT) replay_sample_kernel(ReplayArgs a) {
  __shared__ ReplaySmem s;
  extern __shared__ __align__(16) unsigned char dynamic[];
  unsigned char *mine = a.scratch + size_t(blockIdx.x) * kReplayBytesPerCta;
  double *p = reinterpret_cast<double *>(mine);
  unsigned long long *key = reinterpret_cast<unsigned long long *>(mine + size_t(kReplayPad) * 8);
  int *idx = reinterpret_cast<int *>(mine + size_t(kReplayPad) * 16);
  // Which rows are this CTA's: the status words are read kRT at a time; in the common case (nothing to redo) the
  // kernel is one coalesced read and a vote.
  for (int first = 0; first < a.rows; first += kRT) {
    const int candidate = first + threadIdx.x;
    const int st0 = candidate < a.rows ? a.status[candidate] : 0;
    const bool flagged = st0 > 0 || st0 == -4;
    if (!__syncthreads_or(flagged)) continue;
    for (int row = first + blockIdx.x; row < min(a.rows, first + kRT); row += gridDim.x) {
      const int st = a.status[row];   // the same in every thread
      if (!(st > 0 || st == -4)) continue;
      const float *x = a.logits + size_t(row) * a.stride;
      const Replayed r = replay_probabilities(s, x, a.vocab, a.t, a.top_p, p, key, idx, dynamic);
      const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
      double draw_margin;
      const int token = replay_draw(s, a.vocab, u, [p](int i) { return p[i]; }, &draw_margin);
      if (threadIdx.x == 0) {
        a.tokens[row] = token;
        a.status[row] = (r.cut_margin < kStillClose ? 2 : 0) | (draw_margin < kStillClose ? 1 : 0);
        if (a.replayed) atomicAdd(a.replayed, 1);
      }
      __syncthreads();
    }
  }
}

}  // namespace

cudaError_t launch_replay(const ReplayArgs &a, cudaStream_t stream) {
  const int ctas = a.rows < kReplayCtas ? a.rows : kReplayCtas;
  static std::atomic<int> opted{0};   // one-time attribute per process (every device shares the function's image)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(opted.load() & (1 << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(replay_sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               int(kReplayDynamicBytes));
    if (e != cudaSuccess) return e;
    opted.fetch_or(1 << (dev & 31));
  }
  replay_sample_kernel<<<ctas, kRT, kReplayDynamicBytes, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ds41

// Test hook: the chain acc += v[i] over n doubles with every rounding of the one-thread loop.  mode 0: the sum; 1: stop
// when !(acc < threshold); 2: stop when threshold < acc.  out = {index or -1, acc, acc before that term}.
namespace ds41 {
namespace {
__global__ void __launch_bounds__(kRT) sequential_probe_kernel(const double *v, int n, int mode, double threshold, double *out) {
  __shared__ ReplaySmem s;
  SeqResult r;
  if (mode == 1) r = exact_sequential(s, n, [v](int i) { return v[i]; }, [threshold](double a) { return !(a < threshold); });
  else if (mode == 2) r = exact_sequential(s, n, [v](int i) { return v[i]; }, [threshold](double a) { return threshold < a; });
  else r = exact_sequential(s, n, [v](int i) { return v[i]; }, [](double) { return false; });
  if (threadIdx.x == 0) { out[0] = double(r.found); out[1] = r.acc; out[2] = r.before; }
}
}  // namespace
}  // namespace ds41

extern "C" int ds41_b200_test_sequential(const double *v, int n, int mode, double threshold, double *out, cudaStream_t stream) {
  ds41::sequential_probe_kernel<<<1, ds41::kRT, 0, stream>>>(v, n, mode, threshold, out);
  return int(cudaGetLastError());
}
