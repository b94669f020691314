// Vocabulary-sharded sampling (large batch on several GPUs): each rank owns a contiguous slice of the vocabulary.
//   1. ds41_b200_shard_candidates: per row, the rank's maximum, its partial normaliser and its first 64 ids of the
//      stable order (logit descending, id ascending) -- row_kernel<kModeShard>, one cluster per row;
//   2. the records of all ranks are all-gathered by the caller (NCCL) into local memory;
//   3. ds41_b200_shard_combine: per row, global first maximum, normaliser z = sum_r z_r * exp((m_r - m)/T), the
//      top-p cut over the union of candidates walked sequentially in the stable order, a COVERAGE check (a rank
//      whose 64th candidate still survives the cut may hold survivors that were not sent: the row is then flagged
//      with DS41_B200_ROW_NOT_COVERED and must be redone from full logits), and the Philox inverse-CDF draw in id order.
// The reference has no multi-GPU path; the contract is "same token ids as the single-GPU rule", which holds for every
// certified row because both paths are certified against the same reference rule (sampling.cpp:18-21,30-38).
#include "ds41_b200.h"
#include "host_error.h"
#include "row_kernel.cuh"
#include <cmath>

namespace ds41 {

template <int kMode>
cudaError_t launch_rows(const RowArgs &a, int rows, cudaStream_t stream);

static_assert(sizeof(ShardRow) == sizeof(ds41_b200_shard_row), "shard record layout");

constexpr int kCombineThreads = 256;
constexpr int kMaxShards = 8;
constexpr int kMaxCand = kMaxShards * kShardCand;

struct CombineArgs {
  const ShardRow *gathered;  // [ranks][rows]
  int rows, ranks, vocab;
  double temperature, top_p;
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens, *status;
};

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineArgs a) {
  __shared__ float cy[kMaxCand];
  __shared__ int cid[kMaxCand], crank[kMaxCand], sid[kMaxCand], srank[kMaxCand], by_id[kMaxCand];
  __shared__ double se[kMaxCand];
  __shared__ int base[kMaxShards + 1], complete[kMaxShards];
  __shared__ int out_status, n_keep;
  const int row = blockIdx.x, tid = threadIdx.x;
  const double t = a.temperature;
  // headers: global first maximum, status, rescaled normaliser (sequential over ranks = a fixed order)
  float m = -CUDART_INF_F;
  int arg = 0x7fffffff, status = 0;
  for (int r = 0; r < a.ranks; ++r) {
    const ShardRow &h = a.gathered[size_t(r) * a.rows + row];
    if (h.status < 0 && status >= 0) status = h.status;
    if (h.status == 0 && (h.max_logit > m || (h.max_logit == m && h.argmax < arg))) { m = h.max_logit; arg = h.argmax; }
  }
  if (status < 0 || t == 0) {
    if (tid == 0) { a.tokens[row] = status < 0 ? -1 : arg; if (a.status) a.status[row] = status; }
    return;
  }
  double z = 0;
  if (tid == 0) base[0] = 0;
  __syncthreads();
  for (int r = 0; r < a.ranks; ++r) {
    const ShardRow &h = a.gathered[size_t(r) * a.rows + row];
    z += h.z * exp((double(h.max_logit) - double(m)) / t);
    if (tid == 0) { base[r + 1] = base[r] + h.count; complete[r] = h.complete; }
  }
  __syncthreads();
  const int n = base[a.ranks];
  for (int r = 0; r < a.ranks; ++r) {
    const ShardRow &h = a.gathered[size_t(r) * a.rows + row];
    for (int i = tid; i < h.count; i += kCombineThreads) {
      cy[base[r] + i] = h.cand[i].y; cid[base[r] + i] = h.cand[i].id; crank[base[r] + i] = r;
    }
  }
  __syncthreads();
  // exact positions in the stable order by counting
  for (int i = tid; i < n; i += kCombineThreads) {
    const float yi = cy[i];
    const int idi = cid[i];
    int pos = 0;
    for (int k = 0; k < n; ++k) pos += (cy[k] > yi || (cy[k] == yi && cid[k] < idi)) ? 1 : 0;
    sid[pos] = idi; srank[pos] = crank[i];
    se[pos] = exp((double(yi) - double(m)) / t);
  }
  __syncthreads();
  if (tid == 0) {
    const double rel = 2.0 * (double(a.vocab) + 64.0 + 8.0 * a.ranks) * kU;
    const double target = a.top_p * z, lo = target * (1.0 - rel), hi = target * (1.0 + rel);
    int st = 0, pos = -1;
    double mass = 0;
    if (a.top_p < 1.0) {
      for (int i = 0; i < n; ++i) {
        const double prev = mass;
        mass += se[i];
        if (mass >= target) { pos = i; if (mass < hi || prev >= lo) st |= 2; break; }
      }
    }
    // coverage: a rank that sent a full list must have its LAST candidate outside the nucleus
    bool covered = pos >= 0;
    if (covered) {
      int worst[kMaxShards];
      for (int r = 0; r < a.ranks; ++r) worst[r] = -1;
      for (int i = 0; i < n; ++i) worst[srank[i]] = i;  // ascending i, so the last write is the largest position
      for (int r = 0; r < a.ranks; ++r) {
        if (!complete[r] && worst[r] <= pos) covered = false;
      }
    } else {
      // no crossing inside the candidates (or top_p == 1): covered only if every rank sent all of its ids
      covered = true;
      for (int r = 0; r < a.ranks; ++r)
        if (!complete[r]) covered = false;
      if (covered) { pos = n - 1; if (a.top_p < 1.0 && !(mass < lo)) st |= 2; }
    }
    if (!covered) st = DS41_B200_ROW_NOT_COVERED;
    out_status = st;
    n_keep = covered ? pos + 1 : 0;
  }
  __syncthreads();
  const int keep = n_keep;
  if (out_status == DS41_B200_ROW_NOT_COVERED) {
    if (tid == 0) { a.tokens[row] = -1; if (a.status) a.status[row] = DS41_B200_ROW_NOT_COVERED; }
    return;
  }
  // survivors in id order
  for (int i = tid; i < keep; i += kCombineThreads) {
    int pos = 0;
    for (int k = 0; k < keep; ++k) pos += sid[k] < sid[i] ? 1 : 0;
    by_id[pos] = i;
  }
  __syncthreads();
  if (tid == 0) {
    double total = 0;
    for (int i = 0; i < keep; ++i) total += se[by_id[i]];
    const double u = philox_uniform(a.seeds[row], a.steps[row], a.slot, a.purpose);
    const double target = u * total, slack = (2.0 * keep + 256.0) * kU * total;
    double run = 0;
    int token = -1, last = -1, st = out_status;
    for (int i = 0; i < keep; ++i) {
      const double v = se[by_id[i]], below = run;
      run += v;
      if (v > 0) last = sid[by_id[i]];
      if (target < run) {
        token = sid[by_id[i]];
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

using namespace ds41;

extern "C" int ds41_b200_shard_candidates(const ds41_b200_shard_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_shard_args)) return invalid("shard args: struct size / ABI mismatch");
  if (p->rows < 1 || p->vocab_local < 1 || p->vocab_local > DS41_B200_MAX_VOCAB || p->vocab_offset < 0 || !p->logits ||
      p->logits_stride < p->vocab_local || !p->out)
    return invalid("shard arguments");
  if (!std::isfinite(p->temperature) || p->temperature < 0) return invalid("temperature/top_p/logits");
  RowArgs a{};
  a.logits = p->logits; a.logits_stride = p->logits_stride; a.vocab = p->vocab_local;
  a.temperature = p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0;
  a.top_p = 1.0; a.repetition = 1.f;
  a.shard_out = reinterpret_cast<ShardRow *>(p->out); a.id_offset = p->vocab_offset;
  return int(launch_rows<kModeShard>(a, p->rows, stream));
}

extern "C" int ds41_b200_shard_combine(const ds41_b200_shard_combine_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_shard_combine_args)) return invalid("combine args: struct size / ABI mismatch");
  if (p->rows < 1 || p->ranks < 1 || p->ranks > kMaxShards || p->vocab < 1 || !p->gathered || !p->seeds || !p->steps || !p->tokens)
    return invalid("combine arguments");
  if (!std::isfinite(p->temperature) || p->temperature < 0 || !std::isfinite(p->top_p) || p->top_p <= 0 || p->top_p > 1)
    return invalid("temperature/top_p/logits");
  if (p->slot > 5 || p->purpose > 3) return invalid("Philox v2 address out of range");
  CombineArgs a{reinterpret_cast<const ShardRow *>(p->gathered), p->rows, p->ranks, p->vocab,
                p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0, p->top_p, p->seeds, p->steps, p->slot,
                p->purpose, p->tokens, p->status};
  combine_kernel<<<p->rows, kCombineThreads, 0, stream>>>(a);
  return int(cudaGetLastError());
}
