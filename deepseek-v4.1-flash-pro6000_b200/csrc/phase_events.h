// Measurement hook: CUDA events recorded between the kernels of one sampler call (the batch path), so that a bench can
// time each kernel on the launching stream without a profiler.  Process-wide and not thread-safe: switch it on, make
// one call, read, switch it off.  Off (the default) it costs one predictable branch per mark.
#pragma once
#include <cuda_runtime.h>

namespace ds41 {

constexpr int kPhaseMarks = 8;   // start, then after: statistics, histogram, window, masses, resolve, cluster kernel, replay

struct PhaseEvents {
  cudaEvent_t events[kPhaseMarks];
  bool on = false;
  int next = 0;
};
PhaseEvents &phase_events();

inline void phase_restart() { phase_events().next = 0; }
inline void phase_mark(cudaStream_t stream) {
  PhaseEvents &p = phase_events();
  if (p.on && p.next < kPhaseMarks) cudaEventRecord(p.events[p.next++], stream);
}

}  // namespace ds41
