// The reference engine's sampler surface on top of libds41_b200.so.
//
// This translation unit implements the functions and classes that the reference declares in
// engine/include/ds41/engine.hpp:181-298 -- Rng, AttemptCounter, probabilities, probabilities_rows, sample, argmax,
// reject_sample, SpeculativeStep, Forward::demand_counters -- in place of engine/src/sampling.cpp and
// engine/src/speculation.cpp.  It is compiled against the reference's own header (which is not part of this
// repository: pass its include directories to the compiler), so an engine built with this file instead of those two
// keeps its call sites unchanged while every computation runs on the GPU:
//   * SpeculativeStep is the decode path: proposals are drawn on the device from the draft logits
//     (ds41_b200_sample_logits, slot = k, purpose Draft), the draft logits stay on the device as the measure q, and the
//     target rows are verified from logits in one fused call (ds41_b200_verify_logits).  No probability row is formed.
//   * probabilities / sample / reject_sample keep the reference's value semantics (FP64 rows in host vectors) for
//     callers that want the rows themselves; they run the library's exact operators on probability rows.
// Errors follow the reference: argument errors are std::invalid_argument, failures of the sampler are
// std::runtime_error, counter exhaustion is std::overflow_error.  The confidence stop rule of the reference's draft loop
// (DS41_SPARK_STOP_*: a host-side scheduling policy) is not part of this file.
#include "ds41/engine.hpp"

#include "ds41_b200.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <cuda_runtime.h>
#include <limits>
#include <mutex>
#include <stdexcept>
#include <string>

namespace ds41e {
namespace {

double now_ms() {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void cuda_check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("ds41_b200 adapter: ") + what + ": " + cudaGetErrorString(e));
}
void lib_check(int rc, const char *what) {
  if (rc) throw std::runtime_error(std::string("ds41_b200 sampler: ") + what + ": " + ds41_spark_error());
}
int checked_width(size_t n) {
  if (!n || n > size_t(DS41_B200_MAX_VOCAB)) throw std::invalid_argument("empty/oversized sampler vocabulary");
  return int(n);
}

// Device memory of one host thread's sampler calls: grown on demand, never shrunk, released with the thread.
class Device {
  void *blocks_[8] = {};
  size_t sizes_[8] = {};

public:
  cudaStream_t stream = nullptr;
  Device() { cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "stream"); }
  ~Device() {
    for (void *p : blocks_)
      if (p) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }
  template <class T> T *block(int which, size_t count) {
    const size_t bytes = std::max<size_t>(256, count * sizeof(T));
    if (sizes_[which] < bytes) {
      if (blocks_[which]) cuda_check(cudaFree(blocks_[which]), "free");
      blocks_[which] = nullptr; sizes_[which] = 0;
      cuda_check(cudaMalloc(&blocks_[which], bytes), "allocation");
      sizes_[which] = bytes;
    }
    return static_cast<T *>(blocks_[which]);
  }
  template <class T> void upload(T *dst, const T *src, size_t count) {
    cuda_check(cudaMemcpyAsync(dst, src, count * sizeof(T), cudaMemcpyHostToDevice, stream), "host to device copy");
  }
  template <class T> void download(T *dst, const T *src, size_t count) {
    cuda_check(cudaMemcpyAsync(dst, src, count * sizeof(T), cudaMemcpyDeviceToHost, stream), "device to host copy");
    cuda_check(cudaStreamSynchronize(stream), "synchronise");
  }
};
Device &device() {
  static thread_local Device d;
  return d;
}
enum Block { kLogits = 0, kDraftLogits, kProbs, kDraftProbs, kScratch, kSmall, kResults };

// Layout of the small per-call words in block kSmall (64-bit aligned).
struct Small {
  uint64_t seeds[8], steps[8];
  int32_t ids[8], tokens[8], status[8];
};

[[noreturn]] void throw_row_status(int status) {
  switch (status) {
    case DS41_B200_ROW_NONFINITE: throw std::runtime_error("ds41_b200 sampler: nonfinite logits or invalid probability");
    case DS41_B200_ROW_NOT_NORMALIZED: throw std::runtime_error("ds41_b200 sampler: probabilities must be normalized");
    case DS41_B200_ROW_EMPTY: throw std::runtime_error("ds41_b200 sampler: empty residual support");
    case DS41_B200_ROW_DRAFT: throw std::runtime_error("ds41_b200 sampler: draft id out of range or impossible under logged q");
    default: throw std::runtime_error("ds41_b200 sampler: row status " + std::to_string(status));
  }
}

// logits rows (host) -> FP64 probability rows (host), through ds41_b200_probabilities
std::vector<Distribution> device_probabilities(const std::vector<const std::vector<float> *> &rows, double temperature,
                                               double top_p) {
  const int vocab = checked_width(rows.at(0)->size());
  for (auto *r : rows)
    if (r->size() != size_t(vocab)) throw std::invalid_argument("target vocabulary mismatch");
  Device &d = device();
  const int n = int(rows.size());
  float *logits = d.block<float>(kLogits, size_t(n) * vocab);
  double *probs = d.block<double>(kProbs, size_t(n) * vocab);
  int32_t *status = d.block<int32_t>(kSmall, sizeof(Small) / 4 + n) + sizeof(Small) / 4;
  for (int r = 0; r < n; ++r) d.upload(logits + size_t(r) * vocab, rows[r]->data(), vocab);
  ds41_b200_prob_args a{};
  a.struct_bytes = sizeof(a); a.rows = n; a.vocab = vocab; a.logits = logits; a.logits_stride = vocab;
  a.temperature = temperature; a.top_p = top_p; a.probabilities = probs; a.status = status;
  a.scratch_bytes = ds41_b200_probabilities_scratch_bytes(n);
  a.scratch = d.block<unsigned char>(kScratch, a.scratch_bytes);
  lib_check(ds41_b200_probabilities(&a, d.stream), "probabilities");
  std::vector<int32_t> st(n);
  d.download(st.data(), status, n);
  for (int s : st)
    if (s) throw_row_status(s);
  std::vector<Distribution> out(n, Distribution(vocab));
  for (int r = 0; r < n; ++r) d.download(out[r].data(), probs + size_t(r) * vocab, vocab);
  return out;
}
}  // namespace

// ---------------------------------------------------------------------------------------------------------------
uint64_t AttemptCounter::take() {
  if (exhausted_) throw std::overflow_error("transaction nonce exhausted");
  const uint64_t out = next_;
  if (next_ == std::numeric_limits<uint64_t>::max()) exhausted_ = true;
  else ++next_;
  return out;
}
uint32_t Rng::word(uint64_t step, uint32_t slot, Purpose purpose, uint64_t draw) const {
  if (draw / 4 > std::numeric_limits<uint32_t>::max() || slot > 5 || uint32_t(purpose) > 3)
    throw std::overflow_error("Philox draw counter");
  return ds41_spark_rng_word_v2(seed, step, slot, uint32_t(purpose), draw);
}
double Rng::uniform(uint64_t step, uint32_t slot, Purpose purpose, uint64_t draw) const {
  if (draw > 8589934591ULL || slot > 5 || uint32_t(purpose) > 3) throw std::overflow_error("Philox draw counter");
  return ds41_spark_uniform_v2(seed, step, slot, uint32_t(purpose), draw);
}

Distribution probabilities(const std::vector<float> &logits, double temperature, double top_p) {
  return std::move(device_probabilities({&logits}, temperature, top_p)[0]);
}
std::vector<Distribution> probabilities_rows(const std::vector<std::vector<float>> &rows, double temperature,
                                             double top_p) {
  if (rows.empty()) return {};
  std::vector<const std::vector<float> *> refs;
  for (auto &r : rows) refs.push_back(&r);
  return device_probabilities(refs, temperature, top_p);
}

int argmax(const std::vector<float> &logits) {
  const int vocab = checked_width(logits.size());
  Device &d = device();
  float *x = d.block<float>(kLogits, vocab);
  Small *small = d.block<Small>(kSmall, 1);
  d.upload(x, logits.data(), vocab);
  cuda_check(cudaMemsetAsync(small, 0, sizeof(Small), d.stream), "memset");
  ds41_b200_sample_args a{};
  a.struct_bytes = sizeof(a); a.rows = 1; a.vocab = vocab; a.logits = x; a.logits_stride = vocab;
  a.temperature = 0; a.top_p = 1; a.repetition = 1;
  a.seeds = small->seeds; a.steps = small->steps; a.tokens = small->tokens; a.status = small->status;
  lib_check(ds41_b200_sample_logits(&a, d.stream), "argmax");
  int32_t out[2];
  d.download(&out[0], small->tokens, 1);
  d.download(&out[1], small->status, 1);
  if (out[1] < 0) throw std::runtime_error("non-finite target logits");
  return out[0];
}

int sample(const Distribution &p, const Rng &rng, uint64_t step, uint32_t slot, Purpose purpose) {
  const int vocab = checked_width(p.size());
  if (slot > 5 || uint32_t(purpose) > 3) throw std::runtime_error("ds41_b200 sampler: sample v2 arguments");
  Device &d = device();
  double *row = d.block<double>(kProbs, vocab);
  Small *small = d.block<Small>(kSmall, 1);
  Small host{};
  host.seeds[0] = rng.seed; host.steps[0] = step;
  d.upload(row, p.data(), vocab);
  d.upload(small, &host, 1);
  lib_check(ds41_b200_sample_probabilities(row, 1, vocab, vocab, small->seeds, small->steps, slot, uint32_t(purpose),
                                           small->tokens, small->status, d.stream), "sample");
  int32_t out[2];
  d.download(&out[0], small->tokens, 1);
  d.download(&out[1], small->status, 1);
  if (out[1] < 0) throw_row_status(out[1]);
  return out[0];
}

Verification reject_sample(const std::vector<int> &proposals, const std::vector<Distribution> &q,
                           const std::vector<Distribution> &p, const Rng &rng, uint64_t step, double temperature) {
  const bool greedy = temperature == 0;
  if (!std::isfinite(temperature) || temperature < 0 || proposals.size() > 5 ||
      ((!greedy || !q.empty()) && q.size() != proposals.size()) || p.size() != proposals.size() + 1)
    throw std::invalid_argument("speculative row count");
  const int vocab = checked_width(p[0].size());
  const int drafts = int(proposals.size());
  Device &d = device();
  double *dp = d.block<double>(kProbs, size_t(drafts + 1) * vocab);
  double *dq = q.empty() ? nullptr : d.block<double>(kDraftProbs, size_t(drafts) * vocab);
  for (int k = 0; k <= drafts; ++k) {
    if (p[k].size() != size_t(vocab)) throw std::invalid_argument("target vocabulary mismatch");
    d.upload(dp + size_t(k) * vocab, p[k].data(), vocab);
  }
  for (int k = 0; k < int(q.size()); ++k) {
    if (q[k].size() != size_t(vocab)) throw std::invalid_argument("draft vocabulary mismatch");
    d.upload(dq + size_t(k) * vocab, q[k].data(), vocab);
  }
  Small *small = d.block<Small>(kSmall, 1);
  Small host{};
  host.seeds[0] = rng.seed; host.steps[0] = step;
  for (int k = 0; k < drafts; ++k) host.ids[k] = proposals[k];
  d.upload(small, &host, 1);
  ds41_spark_result *result = d.block<ds41_spark_result>(kResults, 1);
  lib_check(ds41_b200_verify_probabilities(drafts ? small->ids : nullptr, dq, dp, 1, drafts, vocab, greedy ? 1 : 0,
                                           small->seeds, small->steps, result, small->status, d.stream), "verify");
  ds41_spark_result r;
  int32_t status;
  d.download(&r, result, 1);
  d.download(&status, small->status, 1);
  if (status < 0 || r.emitted < 0) throw_row_status(status);
  Verification out;
  out.emitted.assign(r.tokens, r.tokens + r.emitted);
  out.accepted = size_t(r.accepted_drafts);
  out.accepted_input_rows = size_t(r.accepted_input_rows);
  out.rejected = r.rejected != 0;
  return out;
}

// ---------------------------------------------------------------------------------------------------------------
DemandCounters Forward::demand_counters() const {
  const Json j = counters();
  auto read = [&](const char *name) {
    const double v = j.value(name, 0.0);
    if (!std::isfinite(v) || v < 0) throw std::runtime_error("invalid target tier counter");
    return v;
  };
  return {read("expert_host_hits"), read("expert_nvme_misses")};
}

namespace {
double counter_delta(double before, double after) {
  if (!std::isfinite(before) || !std::isfinite(after) || before < 0 || after < 0)
    throw std::runtime_error("invalid target tier counter");
  if (after < before) throw std::runtime_error("target tier counter moved backwards");
  return after - before;
}

// One speculative transaction on the device: target rows [width, vocab] and draft rows [width - 1, vocab] as logits.
Verification verify_on_device(const std::vector<std::vector<float>> &target_rows, int drafts, const int32_t *proposals,
                              const Sampling &sampling, uint64_t step) {
  const int vocab = checked_width(target_rows.at(0).size());
  Device &d = device();
  float *target = d.block<float>(kLogits, size_t(drafts + 1) * vocab);
  float *draft = d.block<float>(kDraftLogits, size_t(std::max(drafts, 1)) * vocab);  // filled by the draft loop
  for (int k = 0; k <= drafts; ++k) d.upload(target + size_t(k) * vocab, target_rows[k].data(), vocab);
  Small *small = d.block<Small>(kSmall, 1);
  Small host{};
  host.seeds[0] = sampling.seed; host.steps[0] = step;
  for (int k = 0; k < drafts; ++k) host.ids[k] = proposals[k];
  d.upload(small, &host, 1);
  ds41_spark_result *result = d.block<ds41_spark_result>(kResults, 1);
  ds41_b200_verify_args a{};
  a.struct_bytes = sizeof(a); a.sequences = 1; a.drafts = drafts; a.vocab = vocab;
  a.target_logits = target; a.draft_logits = drafts && sampling.temperature != 0 ? draft : nullptr;
  a.draft_ids = drafts ? small->ids : nullptr;
  a.temperature = sampling.temperature; a.top_p = sampling.top_p;
  a.seeds = small->seeds; a.steps = small->steps; a.results = result; a.status = small->status;
  a.scratch_bytes = ds41_b200_verify_scratch_bytes_for(1, drafts, vocab);
  a.scratch = d.block<unsigned char>(kScratch, a.scratch_bytes);
  lib_check(ds41_b200_verify_logits(&a, d.stream), "verify");
  ds41_spark_result r;
  int32_t status;
  d.download(&r, result, 1);
  d.download(&status, small->status, 1);
  if (status < 0 || r.emitted < 0) throw_row_status(status);
  Verification out;
  out.emitted.assign(r.tokens, r.tokens + r.emitted);
  out.accepted = size_t(r.accepted_drafts);
  out.accepted_input_rows = size_t(r.accepted_input_rows);
  out.rejected = r.rejected != 0;
  return out;
}

// Proposal k from the draft logits: uploaded into draft row k (where they stay as q for the verifier) and sampled on
// the device at the address (seed, step, slot = k, Draft); greedy takes the first maximum.
int propose_on_device(const std::vector<float> &logits, int k, const Sampling &sampling, uint64_t step) {
  const int vocab = checked_width(logits.size());
  Device &d = device();
  float *draft = d.block<float>(kDraftLogits, size_t(5) * vocab);
  float *row = draft + size_t(k) * vocab;
  d.upload(row, logits.data(), vocab);
  Small *small = d.block<Small>(kSmall, 1);
  Small host{};
  host.seeds[0] = sampling.seed; host.steps[0] = step;
  d.upload(small, &host, 1);
  ds41_b200_sample_args a{};
  a.struct_bytes = sizeof(a); a.rows = 1; a.vocab = vocab; a.logits = row; a.logits_stride = vocab;
  a.temperature = sampling.temperature; a.top_p = sampling.top_p; a.repetition = 1;
  a.seeds = small->seeds; a.steps = small->steps; a.slot = uint32_t(k); a.purpose = uint32_t(Purpose::Draft);
  a.tokens = small->tokens; a.status = small->status;
  lib_check(ds41_b200_sample_logits(&a, d.stream), "draft sample");
  int32_t out[2];
  d.download(&out[0], small->tokens, 1);
  d.download(&out[1], small->status, 1);
  if (out[1] < 0) throw_row_status(out[1]);
  return out[0];
}
}  // namespace

SpeculativeStep::SpeculativeStep(Forward &target, DraftProvider *draft, int anchor, int64_t committed,
                                 const Sampling &sampling, uint64_t position, uint64_t step, int maximum)
    : target_(target), draft_(draft), begin_(committed) {
  started_ms_ = now_ms();
  observed_.nonce = step;
  if (committed < 0 || position != uint64_t(committed) + 1 || maximum < 1 || maximum > 6 || anchor < 0 ||
      anchor >= target.vocab())
    throw std::invalid_argument("speculative step position/width/anchor");
  std::vector<int32_t> proposals;
  try {
    // the width is fixed before any proposal is drawn (spark.h:122-128)
    draft_attempt_ = draft != nullptr;
    int width = 1;
    if (draft) width = draft->prepare(DraftContext{anchor, maximum, committed, step, sampling.temperature, sampling.top_p});
    if (width < 1 || width > maximum) throw std::runtime_error("draft policy returned invalid width");
    observed_.width = width;
    inputs_.push_back(anchor);
    if (width > 1) {
      double t0 = now_ms();
      draft->begin(anchor);
      observed_.draft_ms += now_ms() - t0;
      width = draft->finalize_width(width);
      if (width < 1 || width > maximum) throw std::runtime_error("final draft width outside negotiated capacity");
      t0 = now_ms();
      for (int k = 0; k + 1 < width; ++k) {
        const std::vector<float> logits = draft->logits(k, inputs_.back());
        if (logits.size() != size_t(target.vocab())) throw std::runtime_error("draft vocabulary mismatch");
        const int token = propose_on_device(logits, k, sampling, step);
        proposals.push_back(token);
        inputs_.push_back(token);
      }
      observed_.width = int(inputs_.size());
      observed_.draft_ms += now_ms() - t0;
    }
    // target-only demand deltas around the verify call
    const DemandCounters before = target.demand_counters();
    const double t0 = now_ms();
    rows_ = target.verify(inputs_);
    pending_ = true;
    observed_.verify_ms = std::max(now_ms() - t0, std::numeric_limits<double>::min());
    const DemandCounters after = target.demand_counters();
    observed_.nvme_misses = counter_delta(before.nvme_misses, after.nvme_misses);
    observed_.host_misses = observed_.nvme_misses + counter_delta(before.host_hits, after.host_hits);
    if (rows_.size() != inputs_.size()) throw std::runtime_error("target verify returned wrong row count");
    for (const auto &row : rows_)
      if (row.size() != size_t(target.vocab())) throw std::runtime_error("target vocabulary mismatch");
    result_ = verify_on_device(rows_, int(proposals.size()), proposals.data(), sampling, step);
    observed_.accepted_drafts = result_.accepted;
    observed_.tested_drafts = result_.accepted + size_t(result_.rejected);
  } catch (...) {
    // nothing of a failed attempt may stay pending: zero rows are committed, the drafter returns to the frontier, the
    // nonce is retired
    if (pending_) {
      try { target_.commit(0); pending_ = false; } catch (...) {}
    }
    if (draft_) {
      try { draft_->rollback(begin_); } catch (...) {}
    }
    abort_draft();
    throw;
  }
}

SpeculativeStep::~SpeculativeStep() {
  if (pending_) {  // abandoned: the target and the drafter stay at the committed frontier
    try {
      target_.commit(0);
      if (draft_) draft_->rollback(begin_);
    } catch (...) {}
  }
  abort_draft();
}

void SpeculativeStep::abort_draft() noexcept {
  if (!draft_attempt_) return;
  draft_attempt_ = false;
  try { draft_->abort(observed_.nonce); } catch (...) {}
}

size_t SpeculativeStep::finish(size_t delivered, bool terminal, bool cancelled) {
  const bool whole = delivered == result_.emitted.size();
  if (!pending_ || delivered > result_.emitted.size() || (!terminal && !whole) || (cancelled && !terminal))
    throw std::invalid_argument("speculative delivered prefix/transaction");
  // the anchor row and the accepted inputs that were actually delivered; never the correction / bonus token
  const size_t rows = 1 + std::min(delivered, result_.accepted);
  try {
    target_.commit(rows);
    pending_ = false;
    if (draft_) {
      draft_->rollback(begin_ + int64_t(rows));
      observed_.accepted_drafts = std::min(delivered, result_.accepted);
      observed_.tested_drafts = observed_.accepted_drafts + ((whole && result_.rejected) ? 1 : 0);
      observed_.other_ms = std::max(0.0, now_ms() - started_ms_ - observed_.draft_ms - observed_.verify_ms);
      if (cancelled) {
        abort_draft();
      } else {
        draft_->complete(observed_, terminal);
        draft_attempt_ = false;
      }
    }
  } catch (...) {
    abort_draft();
    throw;
  }
  return rows;
}

}  // namespace ds41e
