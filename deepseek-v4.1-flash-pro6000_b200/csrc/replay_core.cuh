// Device routines that follow the reference's host arithmetic literally: sums on one thread in index order, the stable
// order of the probabilities, the sequential inverse CDF (engine/third_party/spark/src/sampling.cpp:12-38).  Shared by
// the replay of uncertified rows (replay.cu) and by the operators on probability rows (prob.cu).  One CTA of
// kReplayThreads threads works on one row.
#pragma once
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

// sum of value(0) .. value(n-1) in index order, on one thread (tiles staged through shared memory by all threads);
// returned to every thread
template <class Value>
__device__ double sequential_sum(ReplaySmem &s, int n, Value value) {
  double acc = 0;
  for (int base = 0; base < n; base += kTile) {
    const int m = min(kTile, n - base);
    for (int i = threadIdx.x; i < m; i += kRT) s.stage[i] = value(base + i);
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
  const double z = sequential_sum(s, n, [p](int i) { return p[i]; });
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

// draw(p, n, u) of the reference over the values value(0) .. value(n-1); *margin = relative distance of u * z from the two
// CDF steps around the chosen id; *total = z.  Returns -1 when z is not positive (the reference throws "empty residual
// support").
template <class Value>
__device__ int replay_draw(ReplaySmem &s, int n, double u, Value value, double *margin, double *total = nullptr) {
  const double z = sequential_sum(s, n, value);
  if (total) *total = z;
  if (!(z > 0)) { *margin = 0.0; return -1; }
  const double target = u * z;
  double c = 0;
  int last = -1, found = -1;
  double c_at = 0, c_before = 0;
  for (int base = 0; base < n && found < 0; base += kTile) {
    const int m = min(kTile, n - base);
    for (int i = threadIdx.x; i < m; i += kRT) s.stage[i] = value(base + i);
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

}  // namespace
}  // namespace ds41
