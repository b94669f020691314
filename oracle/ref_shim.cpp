// TEST INFRASTRUCTURE ONLY.  C-ABI shim over the reference's own C++ sampler adapter so that ctypes can call it.
// Compiled together with the reference's engine/src/sampling.cpp and third_party/spark/src/sampling.cpp (from
// the reference tree, in place) into oracle/_ref/libds41_ref.so.  Nothing here restates the algorithm: each
// function forwards to the reference function of the same name in namespace ds41e (engine.hpp:181-227).
#include "ds41/engine.hpp"
#include "ds41/spark.h"
#include <cstring>
#include <string>
namespace {
thread_local std::string last_error;
template <class F> int guarded(F f) {
  try { f(); return 0; } catch (const std::exception &e) { last_error = e.what(); return -1; }
}
}
extern "C" {
const char *ref_error(void) { return last_error.c_str(); }
int ref_probabilities(const float *x, double *p, int n, double t, double top) {
  return guarded([&] {
    auto d = ds41e::probabilities(std::vector<float>(x, x + n), t, top);
    std::memcpy(p, d.data(), sizeof(double) * n);
  });
}
int ref_probabilities_rows(const float *x, double *p, int rows, int n, double t, double top) {
  return guarded([&] {
    std::vector<std::vector<float>> in(rows);
    for (int r = 0; r < rows; ++r) in[r].assign(x + size_t(r) * n, x + size_t(r + 1) * n);
    auto d = ds41e::probabilities_rows(in, t, top);
    for (int r = 0; r < rows; ++r) std::memcpy(p + size_t(r) * n, d[r].data(), sizeof(double) * n);
  });
}
int ref_sample(const double *p, int n, uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, int32_t *out) {
  return guarded([&] {
    *out = ds41e::sample(ds41e::Distribution(p, p + n), ds41e::Rng{seed}, step, slot, ds41e::Purpose(purpose));
  });
}
int ref_argmax(const float *x, int n, int32_t *out) {
  return guarded([&] { *out = ds41e::argmax(std::vector<float>(x, x + n)); });
}
// proposals[count], q[count,n] (may be null when temperature==0), p[count+1,n]
int ref_reject_sample(const int32_t *proposals, const double *q, const double *p, int count, int n, uint64_t seed,
                      uint64_t step, double temperature, int32_t *emitted, int *n_emitted, int *accepted,
                      int *accepted_rows, int *rejected) {
  return guarded([&] {
    std::vector<int> ids(proposals, proposals + count);
    std::vector<ds41e::Distribution> qq, pp;
    if (q) for (int k = 0; k < count; ++k) qq.emplace_back(q + size_t(k) * n, q + size_t(k + 1) * n);
    for (int k = 0; k <= count; ++k) pp.emplace_back(p + size_t(k) * n, p + size_t(k + 1) * n);
    auto v = ds41e::reject_sample(ids, qq, pp, ds41e::Rng{seed}, step, temperature);
    *n_emitted = int(v.emitted.size());
    for (size_t i = 0; i < v.emitted.size(); ++i) emitted[i] = v.emitted[i];
    *accepted = int(v.accepted); *accepted_rows = int(v.accepted_input_rows); *rejected = v.rejected ? 1 : 0;
  });
}
uint64_t ref_attempt_counter_take2(uint64_t first, int *threw) {
  // two takes starting at `first`; reports whether a third take throws (core.cpp:32-34)
  ds41e::AttemptCounter c(first);
  uint64_t a = c.take(); (void)a; uint64_t b = c.take();
  *threw = 0; try { c.take(); } catch (const std::overflow_error &) { *threw = 1; }
  return b;
}
}
