// Types of the sampler's batch path for wide nuclei (kernels and launcher in flat.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ds41 {

constexpr int kFlatMaxChunks = 8;   // CTAs per row in the streaming passes: 4 (large batches) or 8 (fewer rows, shorter CTAs)
constexpr int kFlatThreads = 512;
constexpr int kFlatSub = 1024;      // ids per sub-region: the granularity of the inverse-CDF search
constexpr int kFlatSubs = 128;      // sub-regions per row (covers the largest vocabulary, 131072)
constexpr int kFlatBins = 1024;
constexpr int kFlatList = 1024;     // ids of the window that can be sorted exactly
constexpr int kFlatMinNucleus = 512;  // nuclei that certainly hold fewer ids are the other paths' case
constexpr int kFlatMinRows = 128;   // measured on flat rows: 64 rows 133 us against 110 for a cluster per row, 128 rows 170 against 217
constexpr int kFlatMinVocab = 16384;
// internal status word: the row has a wide nucleus but this path could not certify it; only the cluster kernel may
// take it (the streaming path's candidate sets never cover such a row).  Never returned to the caller.
constexpr int kNeedsCluster = -9;

struct FlatPartial { float max, min; int argmax, flags; };
struct FlatInfo {
  float max, min;
  int argmax, applicable, w0, w1;
  double tail;  // mass of the ids beyond the window as the histogram pass has it
};
struct FlatScratch {
  FlatPartial *partial;        // [rows][kFlatMaxChunks]
  unsigned long long *hmass;   // [rows][kFlatBins], fixed point relative to the bin's near edge
  FlatInfo *info;              // [rows]
  double *subz, *subsure;      // [rows][kFlatSubs]: FP64 mass of the ids up to the window's far edge / before the window
  int *subcnt;                 // [rows][kFlatSubs]
  int *lcount;                 // [rows][4]: window list length, "a 32-bit mass may have wrapped" flag
  unsigned long long *lkeys;   // [rows][kFlatList]
};
struct FlatArgs {
  const float *logits;         // rows 16-byte aligned: base and stride
  long long stride;
  int vocab, rows;
  int chunks;                  // 4 or 8 (set by launch_flat)
  double t, top_p;             // t > 0, top_p < 1
  const uint64_t *seeds, *steps;
  uint32_t slot, purpose;
  int32_t *tokens, *status;    // status is required here
  FlatScratch s;
};

size_t flat_scratch_bytes(int rows);
// Rows this path decides get their token and status (0 or certification bits); the others get token -1 and status
// -8 (to be redone by another path) or -1 (non-finite logits, final).
cudaError_t launch_flat(FlatArgs a, void *scratch, cudaStream_t stream);

}  // namespace ds41
