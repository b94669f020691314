// Thread-local message for argument errors, read back through ds41_spark_error()
// (same contract as the reference: third_party/spark/src/sampling.cpp:9-10).
#pragma once
#include <cuda_runtime_api.h>
namespace ds41 {
void set_error(const char *message);
const char *last_error();
inline int invalid(const char *message) {
  set_error(message);
  return int(cudaErrorInvalidValue);
}
}  // namespace ds41
