// Exact replay of rows the parallel paths could not certify (kernel and description in replay.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ds41 {

constexpr int kReplayThreads = 1024;
constexpr int kReplayPad = 131072;   // sort length: the largest vocabulary, a power of two
constexpr int kReplayCtas = 4;       // rows replayed side by side
// per CTA: probabilities (double), sort keys (64-bit), sorted ids (32-bit)
constexpr size_t kReplayBytesPerCta = size_t(kReplayPad) * (8 + 8 + 4);

struct ReplayArgs {
  const float *logits;
  long long stride;
  int vocab, rows;
  double t, top_p;             // t > 0 (greedy rows are never uncertified)
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens, *status;
  unsigned char *scratch;      // kReplayCtas * kReplayBytesPerCta bytes, 16-byte aligned
  int *replayed;               // optional counter of replayed rows
};

// Verification: transactions whose status carries a certification bit are redone from the logits in the reference's
// order of operations (probability rows by the rule above, then verify_impl, sampling.cpp:39-53).
struct VerifyReplayArgs {
  const float *target, *draft;   // [sequences, drafts + 1, vocab], [sequences, drafts, vocab]
  const int32_t *ids;            // [sequences, drafts]
  int sequences, drafts, vocab;
  double t, top_p;               // t > 0
  const uint64_t *seeds, *steps;
  void *results;                 // ds41_spark_result [sequences]
  int32_t *status;               // [sequences]: read to find the transactions, rewritten for those redone
  unsigned char *scratch;        // verify_replay_scratch_bytes(), 16-byte aligned
};
constexpr int kVerifyReplayCtas = 2;
// per CTA: a target and a draft probability row (double), sort keys (64-bit), ids (32-bit)
inline size_t verify_replay_scratch_bytes() { return size_t(kVerifyReplayCtas) * size_t(kReplayPad) * (8 + 8 + 8 + 4); }
cudaError_t launch_verify_replay(const VerifyReplayArgs &a, cudaStream_t stream);
double bound_scale();   // test hook (DS41_BOUND_SCALE): factor on the certification bounds

inline size_t replay_scratch_bytes() { return size_t(kReplayCtas) * kReplayBytesPerCta; }
// Walks the status words; rows with a certification bit set (or -4) are redone in the reference's order of operations.
cudaError_t launch_replay(const ReplayArgs &a, cudaStream_t stream);

}  // namespace ds41
