// Types of the sampler's batch path (kernels and launcher in flat.cu): top-p rows without penalties, mask or top-k,
// decided by four grid-wide kernels over the whole batch.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ds41 {

constexpr int kFlatThreads = 512;
constexpr int kFlatMassThreads = 128;
constexpr int kFlatSub = 1024;      // ids per sub-region: the granularity of the inverse-CDF search
constexpr int kFlatSubs = 128;      // sub-regions per row (covers the largest vocabulary, 131072)
constexpr int kFlatBins = 2048;     // histogram bins over the row's logit range
constexpr int kFlatFrac = 128;      // positions inside a bin that the histogram records (first moment of the ids' places)
constexpr int kFlatQMax = kFlatBins * kFlatFrac - 1;
constexpr int kFlatList = 1024;     // ids of the window that can be sorted exactly
constexpr int kFlatMaxParts = 32;   // CTAs per row of the streaming passes: 1, 2, 4 ... 32 (fewer rows: more, shorter CTAs)
constexpr int kFlatMinRows = 1;
constexpr int kFlatMinVocab = 16384;
constexpr double kFlatMaxExponent = 600.0;  // rows whose range * log2(e)/T exceeds this go to the other paths
// internal status word: this path could not certify the row and its nucleus may be wide; only the cluster kernel may
// take it (the streaming path's candidate sets never cover such a row).  Never returned to the caller.
constexpr int kNeedsCluster = -9;

struct FlatPartial { float max, min; int argmax, flags; };
// Row statistics as the FP8 head's epilogue leaves them (ds41_b200_head_fp8_stats): zero-initialised, then raised with
// atomic maxima.  max_key = (order-preserving bits of the largest logit) << 32 | (0xffffffff - its first id);
// min_key = ~(order-preserving bits of the smallest logit); flags bit 0: a non-finite logit was seen.
struct HeadRowStats { unsigned long long max_key; unsigned int min_key; unsigned int flags; };
struct FlatInfo {
  float max, min;
  int argmax, applicable;
  int w0, w1;             // window of bins that holds the top-p crossing (w0 = kFlatBins: no cut, every id is kept)
  int n_before, n_window; // ids in the bins before the window / inside it (exact: the histogram counts are)
  // the mass pass sorts the ids by two thresholds on the logit itself (a quarter of a bin outside the window's edges):
  // y > y_sure: before the window; y < y_tail: beyond it; the rest goes to the list
  float y_sure, y_tail;
  int pad[2];
};
struct FlatScratch {
  int *pending;                // [4]: rows handed on to the cluster kernel (status -8 / -9); rows replayed   (zeroed every call)
  int *lcount;                 // [rows][4]: window list length, histogram field overflow flag   (zeroed every call)
  unsigned long long *hist;    // [rows][kFlatBins]: count << 32 | sum of the ids' positions inside the bin
  FlatPartial *partial;        // [rows][kFlatMaxParts]
  FlatInfo *info;              // [rows]
  double *subz, *subsure;      // [rows][kFlatSubs]: FP64 mass of every id / of the ids before the window
  unsigned long long *lkeys;   // [rows][kFlatList]
};
struct FlatArgs {
  const float *logits;         // rows 16-byte aligned: base and stride
  long long stride;
  int vocab, rows;
  int parts;                   // CTAs per row in the statistics / histogram / mass passes (set by launch_flat)
  double t, top_p;             // t > 0
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens, *status;    // status is required here
  const HeadRowStats *head_stats;  // optional [rows]: maximum / minimum / finiteness already known (skips the first pass)
  double bound_scale;              // 1; larger values widen the certification bounds (a test hook: more rows get flagged)
  FlatScratch s;
};

size_t flat_scratch_bytes(int rows);
// The word (inside `scratch`) that counts the rows launch_flat handed on; valid once its kernels have run.
const int *flat_pending(const void *scratch);
// Rows this path decides get their token and status (0 or certification bits); the others get token -1 and status
// -8 / -9 (to be redone by another path) or -1 (non-finite logits, final).
cudaError_t launch_flat(FlatArgs a, void *scratch, cudaStream_t stream);

}  // namespace ds41
