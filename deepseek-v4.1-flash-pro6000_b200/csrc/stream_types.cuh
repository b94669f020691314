// Streaming sampler: one pass over the logits by independent CTAs (no cluster), then a small per-row combine.
//
//   chunk_kernel   : one CTA per (row, 8192-id chunk).  The chunk is staged in shared memory by one bulk copy, then:
//                    chunk maximum (first index), partial normaliser relative to that maximum (ids within
//                    kHeavySpan*T of it in FP64, the rest in FP32 with an error bound), and the chunk's first 64 ids of
//                    the stable order (logit descending, id ascending), in no particular order.  Output: one ChunkRecord.
//   combine_kernel : one CTA per row over all of the row's records (from one GPU, or all-gathered from several):
//                    global first maximum, normaliser, exact stable order of the candidates, then the reference's
//                    arithmetic run literally on them (same steps as row_fast.cuh) and a COVERAGE check: a chunk
//                    that sent 64 ids but not all of its ids must have its last candidate outside the kept set,
//                    otherwise ids that were not sent might survive and the row is reported NOT_COVERED (the caller
//                    then runs the cluster kernel, which handles any support size, on that row).
// The same two kernels serve the single-GPU sampler, the verifier's row statistics and the vocabulary-sharded path
// (a shard is just a set of chunks).
#pragma once
#include "row_core.cuh"
#include "row_fast.cuh"

namespace ds41 {

constexpr int kChunkIds = 8192;
constexpr int kChunkThreads = 256;
constexpr int kChunkWarps = kChunkThreads / 32;
constexpr int kChunkRegion = kChunkIds / kChunkWarps;  // 1024 ids per warp
constexpr int kChunkBins = 512;                        // count histogram over d in [0,16), 1/32 logit per bin
constexpr int kChunkList = 256;
constexpr int kCand = 64;
constexpr int kMaxRecords = 17;                        // ceil(131072 / 8192) + 1 for uneven shards
constexpr int kNotCovered = -8;

struct ChunkRecord {  // layout = ds41_b200_shard_row
  double z;           // sum over the chunk's ids of exp((y - max_logit)/T)
  float max_logit;    // chunk maximum
  int argmax;         // its global id (first maximum)
  int count;          // candidates present
  int status;         // 0, or a negative row error
  int complete;       // 1: cand[] holds every id of the chunk
  float z_err;        // absolute error bound of z (same scale as z)
  struct { float y; int id; } cand[kCand];  // a prefix of the stable order (as a set; unordered)
};
static_assert(sizeof(ChunkRecord) == 544, "record layout");

struct ChunkArgs {
  const float *logits;
  long long stride;
  int vocab_local, id_offset, chunks;  // chunks per row (>= ceil(vocab_local/kChunkIds); extra chunks are empty)
  double temperature;
  ChunkRecord *out;  // [rows][chunks]
  const int32_t *only_uncovered;  // if set: only rows whose status word there is -8 are processed
};

enum CombineMode { kCombineDraw = 0, kCombineStats = 1 };

struct CombineArgs {
  const ChunkRecord *records;  // [groups][rows][per_group]: groups = ranks (all-gathered) or 1
  int rows, groups, per_group, vocab;
  double temperature, top_p;
  int top_k;
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens, *status;
  RowStats *stats;
  int only_uncovered;  // only rows whose status word is -8 are processed (the others already have their answer)
};


}  // namespace ds41
