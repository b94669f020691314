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
// leaves with status 0.  Cost: a few milliseconds per row (sort of 131072 keys + four sequential passes); the parallel
// bound flags about one row in 10^5.
#include "replay_core.cuh"

namespace ds41 {
namespace {

constexpr double kStillClose = 16.0 * kU;

__global__ void __launch_bounds__(kRT) replay_sample_kernel(ReplayArgs a) {
  __shared__ ReplaySmem s;
  unsigned char *mine = a.scratch + size_t(blockIdx.x) * kReplayBytesPerCta;
  double *p = reinterpret_cast<double *>(mine);
  unsigned long long *key = reinterpret_cast<unsigned long long *>(mine + size_t(kReplayPad) * 8);
  int *idx = reinterpret_cast<int *>(mine + size_t(kReplayPad) * 16);
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const int st = a.status[row];   // the same in every thread
    if (!(st > 0 || st == -4)) continue;
    const float *x = a.logits + size_t(row) * a.stride;
    const Replayed r = replay_probabilities(s, x, a.vocab, a.t, a.top_p, p, key, idx);
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

}  // namespace

cudaError_t launch_replay(const ReplayArgs &a, cudaStream_t stream) {
  const int ctas = a.rows < kReplayCtas ? a.rows : kReplayCtas;
  replay_sample_kernel<<<ctas, kRT, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ds41
