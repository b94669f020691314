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
#include "replay.cuh"

#include "row_core.cuh"

namespace ds41 {
namespace {

constexpr int kRT = kReplayThreads;
constexpr int kTile = 2048;   // elements sorted / summed out of shared memory at a time

struct ReplaySmem {
  unsigned long long key[kTile];
  int idx[kTile];
  double stage[kTile];
  float red_f[kRT / 32];
  int red_i[kRT / 32];
  double bcast_d[4];
  int bcast_i[4];
};

__device__ __forceinline__ bool key_less(unsigned long long ka, int ia, unsigned long long kb, int ib) {
  return ka < kb || (ka == kb && ia < ib);
}

// Ascending bitonic sort of (key, idx) pairs, kReplayPad of them, in global memory.  Tiles of kTile elements are first
// sorted out of shared memory; after that every merge step runs its wide strides on global memory and its strides below
// kTile again out of shared memory.
__device__ void sort_pairs(ReplaySmem &s, unsigned long long *key, int *idx) {
  const int tid = threadIdx.x;
  auto local_stages = [&](int base, int k, int j_first) {  // strides j_first, j_first / 2 ... 1 of merge step k
    for (int jj = j_first; jj > 0; jj >>= 1) {
      for (int i = tid; i < kTile / 2; i += kRT) {
        const int lo = 2 * jj * (i / jj) + (i % jj), hi = lo + jj;
        const bool up = ((base + lo) & k) == 0;
        const unsigned long long ka = s.key[lo], kb = s.key[hi];
        const int ia = s.idx[lo], ib = s.idx[hi];
        if (key_less(kb, ib, ka, ia) == up) { s.key[lo] = kb; s.key[hi] = ka; s.idx[lo] = ib; s.idx[hi] = ia; }
      }
      __syncthreads();
    }
  };
  for (int base = 0; base < kReplayPad; base += kTile) {
    for (int i = tid; i < kTile; i += kRT) { s.key[i] = key[base + i]; s.idx[i] = idx[base + i]; }
    __syncthreads();
    for (int k = 2; k <= kTile; k <<= 1) local_stages(base, k, k >> 1);
    for (int i = tid; i < kTile; i += kRT) { key[base + i] = s.key[i]; idx[base + i] = s.idx[i]; }
    __syncthreads();
  }
  for (int k = 2 * kTile; k <= kReplayPad; k <<= 1) {
    for (int j = k >> 1; j >= kTile; j >>= 1) {  // partners further apart than a tile
      for (int i = tid; i < kReplayPad / 2; i += kRT) {
        const int lo = 2 * j * (i / j) + (i % j), hi = lo + j;
        const bool up = (lo & k) == 0;
        const unsigned long long ka = key[lo], kb = key[hi];
        const int ia = idx[lo], ib = idx[hi];
        if (key_less(kb, ib, ka, ia) == up) { key[lo] = kb; key[hi] = ka; idx[lo] = ib; idx[hi] = ia; }
      }
      __syncthreads();
    }
    for (int base = 0; base < kReplayPad; base += kTile) {
      for (int i = tid; i < kTile; i += kRT) { s.key[i] = key[base + i]; s.idx[i] = idx[base + i]; }
      __syncthreads();
      local_stages(base, k, kTile >> 1);
      for (int i = tid; i < kTile; i += kRT) { key[base + i] = s.key[i]; idx[base + i] = s.idx[i]; }
      __syncthreads();
    }
  }
}

// sum of v[0..n) in index order, on one thread (tiles staged through shared memory); returned to every thread
__device__ double sequential_sum(ReplaySmem &s, const double *v, int n) {
  double acc = 0;
  for (int base = 0; base < n; base += kTile) {
    const int m = min(kTile, n - base);
    for (int i = threadIdx.x; i < m; i += kRT) s.stage[i] = v[base + i];
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 0; i < m; ++i) acc += s.stage[i];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) s.bcast_d[0] = acc;
  __syncthreads();
  acc = s.bcast_d[0];
  __syncthreads();
  return acc;
}

struct Replayed {
  int first_max;
  double cut_margin;   // relative distance of the top-p crossing from its threshold (inf without a cut)
};

// p[0..n) = the reference's probability row of x; key / idx are work space of kReplayPad entries.
__device__ Replayed replay_probabilities(ReplaySmem &s, const float *x, int n, double t, double top, double *p,
                                         unsigned long long *key, int *idx) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // first maximum
  float best = -CUDART_INF_F;
  int best_id = 0x7fffffff;
  for (int i = tid; i < n; i += kRT) {
    const float v = x[i];
    if (v > best) { best = v; best_id = i; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
  }
  if (lane == 0) { s.red_f[warp] = best; s.red_i[warp] = best_id; }
  __syncthreads();
  for (int w = 0; w < kRT / 32; ++w)
    if (s.red_f[w] > best || (s.red_f[w] == best && s.red_i[w] < best_id)) { best = s.red_f[w]; best_id = s.red_i[w]; }
  __syncthreads();
  Replayed out{best_id, CUDART_INF};
  const double xb = double(best);
  for (int i = tid; i < n; i += kRT) p[i] = exp_nonpos((double(x[i]) - xb) / t);
  __syncthreads();
  const double z = sequential_sum(s, p, n);
  for (int i = tid; i < n; i += kRT) p[i] /= z;
  __syncthreads();
  if (top < 1.0) {
    // order: p descending, id ascending (positive doubles order like their bit patterns)
    for (int i = tid; i < kReplayPad; i += kRT) {
      key[i] = i < n ? ~(unsigned long long)__double_as_longlong(p[i]) : ~0ull;
      idx[i] = i < n ? i : 0x7fffffff;
    }
    __syncthreads();
    sort_pairs(s, key, idx);
    // mass += p[idx[k++]] while k < n and mass < top, on one thread
    double mass = 0, prev = 0;
    int k = 0;
    bool done = false;
    for (int base = 0; base < n && !done; base += kTile) {
      const int m = min(kTile, n - base);
      for (int i = tid; i < m; i += kRT) s.stage[i] = p[idx[base + i]];
      __syncthreads();
      if (tid == 0) {
        int i = 0;
        do { prev = mass; mass += s.stage[i++]; ++k; } while (i < m && k < n && mass < top);
        s.bcast_i[0] = (k >= n || !(mass < top)) ? 1 : 0;
        s.bcast_i[1] = k; s.bcast_d[0] = mass; s.bcast_d[1] = prev;
      }
      __syncthreads();
      done = s.bcast_i[0] != 0;
      __syncthreads();
    }
    k = s.bcast_i[1]; mass = s.bcast_d[0]; prev = s.bcast_d[1];
    __syncthreads();
    // how far the crossing is from flipping: the kept prefix reached top by (mass - top), the one before missed it by (top - prev)
    out.cut_margin = k >= n && mass < top ? (top - mass) / top : fmin(mass - top, top - prev) / top;
    for (int i = k + tid; i < n; i += kRT) p[idx[i]] = 0.0;
    __syncthreads();
    for (int i = tid; i < n; i += kRT) p[i] /= mass;
    __syncthreads();
  }
  return out;
}

// draw(p, n, u) of the reference; *margin = relative distance of u * z from the two CDF steps around the chosen id
__device__ int replay_draw(ReplaySmem &s, const double *p, int n, double u, double *margin) {
  const double z = sequential_sum(s, p, n);
  const double target = u * z;
  double c = 0;
  int last = -1, found = -1;
  double c_at = 0, c_before = 0;
  for (int base = 0; base < n && found < 0; base += kTile) {
    const int m = min(kTile, n - base);
    for (int i = threadIdx.x; i < m; i += kRT) s.stage[i] = p[base + i];
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 0; i < m; ++i) {
        const double before = c;
        c += s.stage[i];
        if (s.stage[i] > 0) last = base + i;
        if (target < c) { found = base + i; c_at = c; c_before = before; break; }
      }
      s.bcast_i[0] = found; s.bcast_i[1] = last; s.bcast_d[0] = c_at; s.bcast_d[1] = c_before;
    }
    __syncthreads();
    found = s.bcast_i[0];
    __syncthreads();
  }
  last = s.bcast_i[1]; c_at = s.bcast_d[0]; c_before = s.bcast_d[1];
  __syncthreads();
  if (found < 0) { *margin = 0.0; return last; }  // rounding left the target past the last step: the reference returns `last`
  *margin = fmin(c_at - target, target - c_before) / z;
  return found;
}

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
    const int token = replay_draw(s, p, a.vocab, u, &draw_margin);
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
