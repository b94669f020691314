// TEST INFRASTRUCTURE ONLY -- CPU oracle for the decode-tail path (LM head -> sampler -> MTP verify).
//
// This file restates, in independent code, the reference's host sampling rule so that the CUDA path can be
// checked against it.  It is never linked into, imported by or called from the product library: only the
// test-suite, the smoke check and the bench's CPU-baseline leg may load it.
//
// Every function names the reference source it follows (paths are relative to the reference project):
//   Philox v2 addressing ....... engine/third_party/spark/include/ds41/spark_rng.h:23-36
//   softmax / top-p rule ....... engine/third_party/spark/src/sampling.cpp:30-38
//   temperature floor .......... engine/src/sampling.cpp:205-219 (and :144)
//   validate + inverse CDF ..... engine/third_party/spark/src/sampling.cpp:12-21, :59
//   speculative verify ......... engine/third_party/spark/src/sampling.cpp:39-56
//   first-maximum argmax ....... engine/src/sampling.cpp:133-139
//   FP8 e4m3 element decode .... components/dense/src/dense.cu:77-80
//   activation quantisation .... components/dense/src/dense.cu:8-16 (group widened from 32 to 128)
//
// Parts with NO counterpart in the reference ("parity unpinned", the rule is defined here and mirrored by the
// CUDA path): top-k, repetition / presence / frequency penalties, the allowed-token bitmask, batching, and the
// FP8 LM head with one fp32 weight scale per 128x128 block.
//
// Pinning: tests/test_oracle_golden.py checks this file against the reference's own known answers
// (engine/tests/core.cpp:22-42,50-60) and, when the reference library has been compiled into oracle/_ref,
// bit for bit against the reference functions on random inputs.
//
// Build: make -C oracle   (g++ -O2 -ffp-contract=off: no fused multiply-add may be introduced, because the
// extension rule below is defined with individually rounded FP32 operations).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;

struct Fail {
  std::string what;
};
[[noreturn]] void fail(const char *m) { throw Fail{m}; }

// ---------------------------------------------------------------- Philox4x32-10, v2 address
// spark_rng.h:23-31.  key = seed halves; counter = (step_lo, step_hi, draw/4, tag | purpose<<3 | slot).
uint32_t philox_word(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw) {
  uint32_t ctr[4] = {uint32_t(step), uint32_t(step >> 32), uint32_t(draw >> 2), 0x53500000u | (purpose << 3) | slot};
  uint32_t key[2] = {uint32_t(seed), uint32_t(seed >> 32)};
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = uint64_t(0xD2511F53u) * ctr[0];
    const uint64_t p1 = uint64_t(0xCD9E8D57u) * ctr[2];
    const uint32_t n0 = uint32_t(p1 >> 32) ^ ctr[1] ^ key[0];
    const uint32_t n1 = uint32_t(p1);
    const uint32_t n2 = uint32_t(p0 >> 32) ^ ctr[3] ^ key[1];
    const uint32_t n3 = uint32_t(p0);
    ctr[0] = n0; ctr[1] = n1; ctr[2] = n2; ctr[3] = n3;
    key[0] += 0x9E3779B9u;
    key[1] += 0xBB67AE85u;
  }
  return ctr[draw & 3];
}
// spark_rng.h:32-36.  53 bits: 27 from word 2d, 26 from word 2d+1.
double philox_uniform(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw = 0) {
  const uint64_t hi = philox_word(seed, step, slot, purpose, 2 * draw) >> 5;
  const uint64_t lo = philox_word(seed, step, slot, purpose, 2 * draw + 1) >> 6;
  return double((hi << 26) | lo) * 0x1p-53;
}

// ---------------------------------------------------------------- A7 tail: top-p on a normalised row
// sampling.cpp:35-36.  Stable descending order (ties keep the lower id first); do-while keeps the crossing id.
void nucleus(double *p, int n, double top) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return p[a] > p[b]; });
  double mass = 0;
  int kept = 0;
  do {
    mass += p[order[kept++]];
  } while (kept < n && mass < top);
  for (int j = kept; j < n; ++j) p[order[j]] = 0;
  for (int i = 0; i < n; ++i) p[i] /= mass;
}

// sampling.cpp:30-38 (ds41_spark_probabilities).  No temperature floor here: that is the adapter's job.
void probabilities_core(const float *x, double *p, int n, double t, double top) {
  if (!x || !p || n < 1 || !std::isfinite(t) || t < 0 || !std::isfinite(top) || top <= 0 || top > 1)
    fail("temperature/top_p/logits");
  int b = 0;
  for (int i = 0; i < n; ++i) {
    if (!std::isfinite(x[i])) fail("nonfinite logits");
    if (x[i] > x[b]) b = i;
  }
  std::fill(p, p + n, 0.0);
  if (t == 0) {
    p[b] = 1;
    return;
  }
  double z = 0;
  for (int i = 0; i < n; ++i) {
    p[i] = std::exp((double(x[i]) - x[b]) / t);
    z += p[i];
  }
  for (int i = 0; i < n; ++i) p[i] /= z;
  if (top < 1) nucleus(p, n, top);
}

// engine/src/sampling.cpp:205-219: the adapter raises a positive temperature to at least 1e-5.
double floored(double t) { return t > 0 ? std::max(t, 1e-5) : t; }

// sampling.cpp:12-17
double validate(const double *p, int n) {
  if (!p || n < 1) fail("null/empty probability row");
  double z = 0;
  for (int i = 0; i < n; ++i) {
    if (!std::isfinite(p[i]) || p[i] < 0) fail("invalid probability");
    z += p[i];
  }
  if (std::abs(z - 1) > 1e-8) fail("probabilities must be normalized");
  return z;
}
// sampling.cpp:18-21: inverse CDF in id order, first id whose running sum exceeds u*z, else last positive id.
int inverse_cdf(const double *p, int n, double u) {
  double z = 0;
  for (int i = 0; i < n; ++i) z += p[i];
  if (!(z > 0)) fail("empty residual support");
  const double target = u * z;
  double run = 0;
  int last = -1;
  for (int i = 0; i < n; ++i) {
    run += p[i];
    if (p[i] > 0) last = i;
    if (target < run) return i;
  }
  return last;
}
int first_max(const double *p, int n) { return int(std::max_element(p, p + n) - p); }

struct Result {  // layout of ds41_spark_result (spark.h:106-108)
  int32_t tokens[6];
  int emitted, accepted_drafts, accepted_input_rows, rejected;
};

// sampling.cpp:39-53 (verify_impl, v2 addressing).
void verify_core(const int32_t *d, const double *q, const double *p, int count, int n, int greedy, uint64_t seed,
                 uint64_t step, Result *out) {
  if (!out || count < 0 || count > 5 || n < 1 || !p || (count && (!d || (!q && !greedy)))) fail("verify arguments");
  Result r{};
  for (int k = 0; k <= count; ++k) validate(p + size_t(k) * n, n);
  for (int k = 0; k < count; ++k) {
    if (d[k] < 0 || d[k] >= n) fail("draft id");
    const double *pk = p + size_t(k) * n;
    const double *qk = q ? q + size_t(k) * n : nullptr;
    bool accept;
    if (greedy) {
      accept = d[k] == first_max(pk, n);
    } else {
      validate(qk, n);
      if (qk[d[k]] <= 0) fail("draft impossible under logged q");
      accept = philox_uniform(seed, step, k, 2) < std::min(1.0, pk[d[k]] / qk[d[k]]);
    }
    if (accept) {
      r.tokens[r.emitted++] = d[k];
      ++r.accepted_drafts;
      continue;
    }
    if (greedy) {
      r.tokens[r.emitted++] = first_max(pk, n);
    } else {
      std::vector<double> residual(n);
      for (int i = 0; i < n; ++i) residual[i] = std::max(0.0, pk[i] - qk[i]);
      r.tokens[r.emitted++] = inverse_cdf(residual.data(), n, philox_uniform(seed, step, k, 3));
    }
    r.rejected = 1;
    break;
  }
  if (!r.rejected) {
    const double *last = p + size_t(count) * n;
    r.tokens[r.emitted++] = greedy ? first_max(last, n) : inverse_cdf(last, n, philox_uniform(seed, step, count, 0));
  }
  r.accepted_input_rows = r.accepted_drafts + 1;
  *out = r;
}

// ---------------------------------------------------------------- extension rule (no reference counterpart)
// Penalties, allowed-token bitmask and top-k in front of the reference's softmax / top-p / draw.
//   1. every raw logit must be finite (same check as sampling.cpp:32, made before anything else);
//   2. counts[id] = occurrences of id in the history (ids outside [0,n) are padding and ignored);
//   3. for ids with count>0, in FP32 with each operation rounded to nearest separately:
//        y = x>0 ? x/repetition : x*repetition;   y = y - (presence + frequency*float(count));
//      the result must still be finite;
//   4. an id is allowed iff the mask is absent or its bit (word id/32, bit id%32) is set; an empty allowed set
//      is an error (the reference's draw throws on empty support, sampling.cpp:19);
//   5. top_k>0 keeps the top_k allowed ids in the order (y descending, id ascending);
//   6. b = first maximum among survivors; t==0 -> one-hot at b; else p[i]=exp((double(y[i])-double(y[b]))/t)
//      for survivors and 0 otherwise, z summed in id order, p/=z, then the reference's top-p and draw unchanged.
struct Extension {
  const int32_t *history = nullptr;
  int history_len = 0;
  float repetition = 1.f, presence = 0.f, frequency = 0.f;
  const uint32_t *mask = nullptr;
  int top_k = 0;
};

void extended_probabilities(const float *x, double *p, int n, double t, double top, const Extension &e,
                            std::vector<float> *effective = nullptr) {
  if (!x || !p || n < 1 || !std::isfinite(t) || t < 0 || !std::isfinite(top) || top <= 0 || top > 1)
    fail("temperature/top_p/logits");
  if (!(e.repetition > 0) || !std::isfinite(e.repetition) || !std::isfinite(e.presence) ||
      !std::isfinite(e.frequency) || e.top_k < 0 || e.history_len < 0)
    fail("penalty/top_k arguments");
  for (int i = 0; i < n; ++i)
    if (!std::isfinite(x[i])) fail("nonfinite logits");
  std::vector<float> y(x, x + n);
  const bool penalised = e.history && e.history_len > 0 &&
                         (e.repetition != 1.f || e.presence != 0.f || e.frequency != 0.f);
  if (penalised) {
    std::vector<int32_t> count(n, 0);
    for (int j = 0; j < e.history_len; ++j) {
      const int32_t id = e.history[j];
      if (id >= 0 && id < n) ++count[id];
    }
    for (int i = 0; i < n; ++i) {
      if (!count[i]) continue;
      volatile float v = y[i] > 0 ? y[i] / e.repetition : y[i] * e.repetition;
      volatile float scaled = e.frequency * float(count[i]);
      volatile float pen = e.presence + scaled;
      volatile float w = v - pen;
      if (!std::isfinite(w)) fail("nonfinite penalised logit");
      y[i] = w;
    }
  }
  std::vector<char> keep(n, 1);
  if (e.mask)
    for (int i = 0; i < n; ++i) keep[i] = (e.mask[i >> 5] >> (i & 31)) & 1u;
  int allowed = 0;
  for (int i = 0; i < n; ++i) allowed += keep[i];
  if (!allowed) fail("empty allowed set");
  if (e.top_k > 0 && e.top_k < allowed) {
    std::vector<int> order;
    order.reserve(allowed);
    for (int i = 0; i < n; ++i)
      if (keep[i]) order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return y[a] > y[b]; });
    for (size_t j = size_t(e.top_k); j < order.size(); ++j) keep[order[j]] = 0;
  }
  int b = -1;
  for (int i = 0; i < n; ++i)
    if (keep[i] && (b < 0 || y[i] > y[b])) b = i;
  std::fill(p, p + n, 0.0);
  if (effective) {
    *effective = y;
    for (int i = 0; i < n; ++i)
      if (!keep[i]) (*effective)[i] = -INFINITY;
  }
  if (t == 0) {
    p[b] = 1;
    return;
  }
  double z = 0;
  for (int i = 0; i < n; ++i) {
    if (!keep[i]) continue;
    p[i] = std::exp((double(y[i]) - y[b]) / t);
    z += p[i];
  }
  for (int i = 0; i < n; ++i) p[i] /= z;
  if (top < 1) nucleus(p, n, top);
}

// ---------------------------------------------------------------- FP8 head (no reference counterpart)
// e4m3 (finite-only variant): 1 sign, 4 exponent (bias 7), 3 mantissa; 0x7f/0xff are NaN.
float e4m3_decode(uint8_t b) {
  const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) return NAN;
  if (e == 0) v = std::ldexp(float(m), -9);
  else v = std::ldexp(float(8 + m), e - 10);
  return s ? -v : v;
}
// Round to nearest even onto the e4m3 grid, saturating to +-448.
uint8_t e4m3_encode(float v) {
  if (std::isnan(v)) return 0x7f;
  const uint8_t sign = std::signbit(v) ? 0x80 : 0;
  float a = std::fabs(v);
  if (a >= 448.f) return sign | 0x7e;
  if (a < 0x1p-6f) {  // subnormal grid, spacing 2^-9
    const float q = std::nearbyint(a * 512.f);  // default rounding mode: nearest even
    return sign | uint8_t(q);                   // q==8 encodes the first normal, which is correct
  }
  int ex;
  const float fr = std::frexp(a, &ex);           // a = fr * 2^ex, fr in [0.5,1)
  float mant = std::nearbyint(fr * 16.f);        // 8..16
  int e = ex - 1 + 7;
  if (mant == 16.f) { mant = 8.f; ++e; }
  if (e > 15 || (e == 15 && mant > 14.f)) return sign | 0x7e;
  return sign | uint8_t((e << 3) | (int(mant) - 8));
}
float bf16_to_float(uint16_t h) {
  uint32_t u = uint32_t(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
// dense.cu:8-16 with group 128: scale = 2^ceil(log2(max(amax,1e-4)/448)); values divided by it and clamped.
float act_scale(float amax) {
  volatile float scaled = std::max(amax, 1e-4f) * (1.f / 448.f);
  uint32_t bits;
  float s = scaled;
  std::memcpy(&bits, &s, 4);
  const uint32_t exponent = (bits >> 23) + ((bits & 0x7fffffu) != 0);
  bits = exponent << 23;
  std::memcpy(&s, &bits, 4);
  return s;
}

void parallel_rows(int rows, int threads, const std::function<void(int)> &body) {
  if (threads <= 1 || rows <= 1) {
    for (int r = 0; r < rows; ++r) body(r);
    return;
  }
  std::atomic<int> next{0};
  std::vector<std::thread> pool;
  std::atomic<bool> failed{false};
  std::string message;
  std::mutex guard;
  for (int t = 0; t < std::min(threads, rows); ++t)
    pool.emplace_back([&] {
      for (;;) {
        const int r = next.fetch_add(1);
        if (r >= rows || failed.load()) return;
        try {
          body(r);
        } catch (const Fail &f) {
          std::lock_guard<std::mutex> lock(guard);
          if (!failed.exchange(true)) message = f.what;
        }
      }
    });
  for (auto &t : pool) t.join();
  if (failed) throw Fail{message};
}
}  // namespace

#define ORACLE_TRY try {
#define ORACLE_END                 \
  return 0;                        \
  }                                \
  catch (const Fail &f) {          \
    g_error = f.what;              \
    return -1;                     \
  }                                \
  catch (const std::exception &x) {\
    g_error = x.what();            \
    return -1;                     \
  }

extern "C" {

const char *oracle_error(void) { return g_error.c_str(); }

uint32_t oracle_rng_word_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw) {
  if (slot > 5 || purpose > 3 || draw / 4 > UINT32_MAX) {
    g_error = "Philox v2 address out of range";
    return 0;
  }
  return philox_word(seed, step, slot, purpose, draw);
}
double oracle_uniform_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw) {
  if (slot > 5 || purpose > 3 || draw > 8589934591ULL) {
    g_error = "Philox v2 address out of range";
    return NAN;
  }
  return philox_uniform(seed, step, slot, purpose, draw);
}

// Library rule (no temperature floor), as ds41_spark_probabilities.
int oracle_probabilities(const float *x, double *p, int n, double t, double top) {
  ORACLE_TRY probabilities_core(x, p, n, t, top);
  ORACLE_END
}
// Engine-adapter rule (temperature floor applied), as ds41e::probabilities.
int oracle_engine_probabilities(const float *x, double *p, int n, double t, double top) {
  ORACLE_TRY probabilities_core(x, p, n, floored(t), top);
  ORACLE_END
}
int oracle_sample_v2(const double *p, int n, uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose,
                     int32_t *out) {
  ORACLE_TRY if (!out || slot > 5 || purpose > 3) fail("sample v2 arguments");
  validate(p, n);
  *out = inverse_cdf(p, n, philox_uniform(seed, step, slot, purpose, 0));
  ORACLE_END
}
int oracle_verify_v2(const int32_t *d, const double *q, const double *p, int count, int n, int greedy, uint64_t seed,
                     uint64_t step, void *out) {
  ORACLE_TRY verify_core(d, q, p, count, n, greedy, seed, step, static_cast<Result *>(out));
  ORACLE_END
}
int oracle_argmax(const float *x, int n, int32_t *out) {
  ORACLE_TRY if (!x || n < 1 || !out) fail("argmax arguments");
  int b = 0;
  for (int i = 0; i < n; ++i) {
    if (!std::isfinite(x[i])) fail("non-finite target logits");
    if (x[i] > x[b]) b = i;
  }
  *out = b;
  ORACLE_END
}

// BF16 head in the reference kernels' own arithmetic order (components/fuse-head/src/head_half_tree.cu:7-21 and
// head_half_tune.cu:7-22): sixteen FP32 chains per output, chain l = fused multiply-adds over k = l, l+16, ... in
// ascending order; then four tree levels over the chain index (distance 8, 4, 2, 1; a chain without a partner at that
// distance adds itself, as the width-16 shuffle does, which never reaches chain 0); then + 0.f.
int oracle_head_bf16(const float *x, const uint16_t *w_bits, float *y, int M, int N, int K) {
  ORACLE_TRY if (!x || !w_bits || !y || M < 1 || N < 1 || K < 1) fail("bf16 head arguments");
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < M; ++m) {
      float c[16];
      for (int l = 0; l < 16; ++l) {
        float acc = 0.f;
        for (int k = l; k < K; k += 16) {
          uint32_t bits = uint32_t(w_bits[size_t(n) * K + k]) << 16;
          float weight;
          std::memcpy(&weight, &bits, 4);
          acc = std::fmaf(weight, x[size_t(m) * K + k], acc);
        }
        c[l] = acc;
      }
      for (int d = 8; d; d >>= 1) {
        float next[16];
        for (int i = 0; i < 16; ++i) next[i] = c[i] + (i + d < 16 ? c[i + d] : c[i]);
        std::memcpy(c, next, sizeof c);
      }
      y[size_t(m) * N + n] = c[0] + 0.f;
    }
  ORACLE_END
}

static float bf16_value(uint16_t bits) {
  uint32_t wide = uint32_t(bits) << 16;
  float v;
  std::memcpy(&v, &wide, 4);
  return v;
}
static uint16_t bf16_round(float v) {  // round to nearest even, as __float2bfloat16_rn (finite inputs)
  uint32_t bits;
  std::memcpy(&bits, &v, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return uint16_t((bits >> 16) | 0x40);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return uint16_t(bits >> 16);
}

// The drafter's BF16 head in the reference kernel's own arithmetic order (components/dense/src/compact.cu:10-24):
// 32 lanes per output; lane l takes k = 8 l + 256 i; element j of its eight goes to accumulator j % 4 by fused
// multiply-add; (a0 + a1) + (a2 + a3); then five shuffle-down levels (distance 16, 8, 4, 2, 1: lane i adds lane i + d,
// lanes without a partner add their own value, which never reaches lane 0).
int oracle_head_compact(const float *x, const uint16_t *w_bits, float *y, int M, int N, int K) {
  ORACLE_TRY if (!x || !w_bits || !y || M < 1 || M > 8 || N < 1 || K < 256 || K % 256) fail("compact head arguments");
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < M; ++m) {
      float lane_sum[32];
      for (int l = 0; l < 32; ++l) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = l * 8; k < K; k += 256)
          for (int j = 0; j < 8; ++j)
            acc[j & 3] = std::fmaf(bf16_value(w_bits[size_t(n) * K + k + j]), x[size_t(m) * K + k + j], acc[j & 3]);
        lane_sum[l] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      }
      for (int d = 16; d; d >>= 1) {
        float next[32];
        for (int i = 0; i < 32; ++i) next[i] = lane_sum[i] + (i + d < 32 ? lane_sum[i + d] : lane_sum[i]);
        std::memcpy(lane_sum, next, sizeof lane_sum);
      }
      y[size_t(m) * N + n] = lane_sum[0];
    }
  ORACLE_END
}

// Draft logits of one position: U + W_markov . emb (engine/third_party/spark/src/forward.cu:46,135-139), the dot product
// in the compact head's order for K = 256, then one rounded addition.
int oracle_markov_logits(const float *u, const uint16_t *w_bits, const uint16_t *emb_bits, float *out, int vocab) {
  ORACLE_TRY if (!u || !w_bits || !emb_bits || !out || vocab < 1) fail("Markov logits arguments");
  float e[256];
  for (int k = 0; k < 256; ++k) e[k] = bf16_value(emb_bits[k]);
  std::vector<float> bias(vocab);
  int rc = oracle_head_compact(e, w_bits, bias.data(), 1, vocab, 256);
  if (rc) return rc;
  for (int n = 0; n < vocab; ++n) out[n] = u[n] + bias[n];
  ORACLE_END
}

// HC-pre mix -> RMSNorm -> BF16 -> FP32 (engine/src/hotpath/batch.inc:487-492; components/dense/src/ops.cu:10-27,45-48,
// 102,110-112) with the reference's reduction geometry.  The device takes rsqrtf() of mean + eps; this restatement takes
// 1 / sqrt in FP32, which can differ from it in the last place, so a comparison with the device allows the BF16 result
// to move by one unit in a few entries (the bit-exact comparison is against the reference kernels themselves).
int oracle_final_norm(const uint16_t *h_bits, const float *pre, const uint16_t *w_bits, float *out, int M, int K, float eps) {
  ORACLE_TRY if (!h_bits || !pre || !w_bits || !out || M < 1 || M > 8 || K < 128 || K % 4) fail("final norm arguments");
  int height = 1;
  while (height * 2 <= M && height * 2 <= 16) height *= 2;
  int n = 1;
  while (n * 2 <= K / 4 && n * 2 <= 512) n *= 2;
  const int width = n < 512 / height ? n : 512 / height;
  const int threads = K / width >= height * 16 ? width * height : width;
  std::vector<uint16_t> x(K);
  std::vector<float> sh(threads), sum(threads);
  for (int row = 0; row < M; ++row) {
    for (int k = 0; k < K; ++k) {
      float s = 0.f;
      for (int j = 0; j < 4; ++j) s = s + pre[row * 4 + j] * bf16_value(h_bits[(size_t(row) * 4 + j) * K + k]);
      x[k] = bf16_round(s);
    }
    for (int t = 0; t < threads; ++t) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int i = t * 4; i < K; i += threads * 4)
        for (int j = 0; j < 4; ++j)
          if (i + j < K) {
            const float z = bf16_value(x[i + j]);
            v[j] = v[j] + z * z;
          }
      sum[t] = ((v[0] + v[1]) + v[2]) + v[3];
      sh[t] = sum[t];
    }
    for (int d = width / 2; d >= 32; d >>= 1) {          // halving inside each segment of `width` threads
      std::vector<float> next = sh;
      for (int t = 0; t < threads; ++t)
        if (t % width < d) { sum[t] = sum[t] + sh[t + d]; next[t] = sum[t]; }
      sh = next;
    }
    for (int d = 16; d; d >>= 1) {                        // shuffle-down inside every warp
      std::vector<float> next = sum;
      for (int t = 0; t < threads; ++t) {
        const int lane = t & 31;
        next[t] = sum[t] + (lane + d < 32 && t + d < threads ? sum[t + d] : sum[t]);
      }
      sum = next;
    }
    for (int t = 0; t < threads; ++t)
      if (t % width == 0) sh[t] = sum[t];
    for (int d = (threads / width) / 2; d; d >>= 1) {     // halving over the segments
      std::vector<float> next = sh;
      for (int t = 0; t < threads; ++t)
        if (t % width == 0 && t / width < d) { sum[t] = sum[t] + sh[t + d * width]; next[t] = sum[t]; }
      sh = next;
    }
    const float rstd = 1.f / std::sqrt(sh[0] * (1.f / K) + eps);
    for (int k = 0; k < K; ++k) out[size_t(row) * K + k] = bf16_value(bf16_round((bf16_value(x[k]) * rstd) * bf16_value(w_bits[k])));
  }
  ORACLE_END
}

// Score reporting of one row (engine/src/server.cpp:178-183 log_normalizer: max, then the sequential FP64 sum of
// exp(double(v) - max), result max + log(sum); :730-737 top_order: the first n ids in the order value descending, id
// ascending; :450-461 logprob = double(l[t]) - normalizer).
int oracle_score_row(const float *x, int n, int top, double *logsumexp, int32_t *top1, int32_t *top_ids,
                     double *top_logprob) {
  ORACLE_TRY if (!x || n < 1 || top < 0 || top > n || !logsumexp) fail("score arguments");
  int b = 0;
  for (int i = 0; i < n; ++i) {
    if (!std::isfinite(x[i])) fail("non-finite target logits");
    if (x[i] > x[b]) b = i;
  }
  const double mx = x[b];
  double sum = 0;
  for (int i = 0; i < n; ++i) sum += std::exp(double(x[i]) - mx);
  *logsumexp = mx + std::log(sum);
  if (top1) *top1 = b;
  std::vector<int> ids(n);
  for (int i = 0; i < n; ++i) ids[i] = i;
  std::partial_sort(ids.begin(), ids.begin() + top, ids.end(),
                    [&](int a, int c) { return x[a] == x[c] ? a < c : x[a] > x[c]; });
  for (int k = 0; k < top; ++k) {
    top_ids[k] = ids[k];
    top_logprob[k] = double(x[ids[k]]) - *logsumexp;
  }
  ORACLE_END
}

// Extended single row: effective (nullable) receives the penalised logits with excluded ids at -inf.
int oracle_extended_probabilities(const float *x, double *p, int n, double t, double top, int top_k,
                                  const int32_t *history, int history_len, float repetition, float presence,
                                  float frequency, const uint32_t *mask, float *effective) {
  ORACLE_TRY Extension e;
  e.history = history; e.history_len = history_len;
  e.repetition = repetition; e.presence = presence; e.frequency = frequency;
  e.mask = mask; e.top_k = top_k;
  std::vector<float> eff;
  extended_probabilities(x, p, n, floored(t), top, e, effective ? &eff : nullptr);
  if (effective) std::memcpy(effective, eff.data(), sizeof(float) * n);
  ORACLE_END
}

// Batched logits -> token, one row per (seed, step, slot): the engine path probabilities() + sample()
// (engine/src/sampling.cpp:205-226) applied per row, with the extension rule in front when requested.
// t==0 returns the first maximum (server.cpp:623-625 uses argmax for greedy requests).
// history: [rows, history_stride] with history_len[r] valid entries (history_len may be null -> history_stride).
// mask: [rows, mask_stride] words or null.  status[r] = 0 ok, -1 row rejected (message via oracle_error()).
int oracle_sample_rows(const float *logits, int rows, int n, int64_t stride, double t, double top, int top_k,
                       const int32_t *history, int64_t history_stride, const int32_t *history_len, float repetition,
                       float presence, float frequency, const uint32_t *mask, int64_t mask_stride,
                       const uint64_t *seeds, const uint64_t *steps, uint32_t slot, uint32_t purpose,
                       int32_t *tokens, int32_t *status, int threads) {
  ORACLE_TRY if (!logits || rows < 1 || n < 1 || !seeds || !steps || !tokens || slot > 5 || purpose > 3)
      fail("sample_rows arguments");
  const bool extended = top_k > 0 || mask || (history && (repetition != 1.f || presence != 0.f || frequency != 0.f));
  parallel_rows(rows, threads, [&](int r) {
    std::vector<double> p(n);
    try {
      const float *x = logits + size_t(r) * stride;
      if (extended) {
        Extension e;
        e.history = history ? history + size_t(r) * history_stride : nullptr;
        e.history_len = history ? (history_len ? history_len[r] : int(history_stride)) : 0;
        e.repetition = repetition; e.presence = presence; e.frequency = frequency;
        e.mask = mask ? mask + size_t(r) * mask_stride : nullptr;
        e.top_k = top_k;
        extended_probabilities(x, p.data(), n, floored(t), top, e);
      } else {
        probabilities_core(x, p.data(), n, floored(t), top);
      }
      if (t == 0) {
        tokens[r] = first_max(p.data(), n);
      } else {
        validate(p.data(), n);
        tokens[r] = inverse_cdf(p.data(), n, philox_uniform(seeds[r], steps[r], slot, purpose, 0));
      }
      if (status) status[r] = 0;
    } catch (const Fail &f) {
      g_error = f.what;
      tokens[r] = -1;
      if (status) status[r] = -1; else throw;
    }
  });
  ORACLE_END
}

// Batched speculative verification from logits: for each sequence, p rows = probabilities(target logits),
// q rows = probabilities(draft logits), both through the adapter rule, then the reference's verify.
// target: [seqs*(drafts+1), n], draft: [seqs*drafts, n], ids: [seqs*drafts]; results: Result[seqs].
int oracle_verify_rows(const float *target, const float *draft, const int32_t *ids, int seqs, int drafts, int n,
                       double t, double top, const uint64_t *seeds, const uint64_t *steps, void *results,
                       int32_t *status, int threads) {
  ORACLE_TRY if (!target || seqs < 1 || drafts < 0 || drafts > 5 || n < 1 || !seeds || !steps || !results ||
                 (drafts && (!ids || (!draft && t != 0))))
      fail("verify_rows arguments");
  Result *out = static_cast<Result *>(results);
  parallel_rows(seqs, threads, [&](int s) {
    try {
      std::vector<double> p(size_t(drafts + 1) * n), q(size_t(drafts) * n);
      for (int k = 0; k <= drafts; ++k)
        probabilities_core(target + (size_t(s) * (drafts + 1) + k) * n, p.data() + size_t(k) * n, n, floored(t), top);
      if (t != 0)
        for (int k = 0; k < drafts; ++k)
          probabilities_core(draft + (size_t(s) * drafts + k) * n, q.data() + size_t(k) * n, n, floored(t), top);
      verify_core(ids ? ids + size_t(s) * drafts : nullptr, t != 0 && drafts ? q.data() : nullptr, p.data(), drafts, n,
                  t == 0, seeds[s], steps[s], out + s);
      if (status) status[s] = 0;
    } catch (const Fail &f) {
      g_error = f.what;
      Result bad{};
      bad.emitted = -1;
      out[s] = bad;
      if (status) status[s] = -1; else throw;
    }
  });
  ORACLE_END
}

// ---- FP8 head
void oracle_e4m3_table(float *out256) {
  for (int i = 0; i < 256; ++i) out256[i] = e4m3_decode(uint8_t(i));
}
uint8_t oracle_e4m3_encode(float v) { return e4m3_encode(v); }

// Activation quantisation: x bf16 bits [M,K] -> a e4m3 [M,K], scale fp32 [M,K/128].
int oracle_quantize_activations(const uint16_t *x, uint8_t *a, float *scale, int M, int K) {
  ORACLE_TRY if (!x || !a || !scale || M < 1 || K < 128 || K % 128) fail("quantize arguments");
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < K / 128; ++g) {
      float amax = 0;
      for (int k = 0; k < 128; ++k) amax = std::max(amax, std::fabs(bf16_to_float(x[size_t(m) * K + g * 128 + k])));
      const float s = act_scale(amax);
      scale[size_t(m) * (K / 128) + g] = s;
      for (int k = 0; k < 128; ++k) {
        const float v = bf16_to_float(x[size_t(m) * K + g * 128 + k]) / s;  // exact: s is a power of two
        a[size_t(m) * K + g * 128 + k] = e4m3_encode(std::min(448.f, std::max(-448.f, v)));
      }
    }
  ORACLE_END
}

// Weight quantisation used by the synthetic generator: w fp32 [N,K] -> e4m3 + fp32 scale per 128x128 block,
// scale = amax/448 (block amax 0 -> scale 1).  Scales laid out [ceil(N/128), K/128].
int oracle_quantize_weights(const float *w, uint8_t *out, float *scale, int N, int K) {
  ORACLE_TRY if (!w || !out || !scale || N < 1 || K < 128 || K % 128) fail("quantize arguments");
  const int nb = (N + 127) / 128, kb = K / 128;
  for (int bi = 0; bi < nb; ++bi)
    for (int bj = 0; bj < kb; ++bj) {
      float amax = 0;
      for (int r = bi * 128; r < std::min(N, bi * 128 + 128); ++r)
        for (int c = bj * 128; c < bj * 128 + 128; ++c) amax = std::max(amax, std::fabs(w[size_t(r) * K + c]));
      const float s = amax > 0 ? amax / 448.f : 1.f;
      scale[size_t(bi) * kb + bj] = s;
      for (int r = bi * 128; r < std::min(N, bi * 128 + 128); ++r)
        for (int c = bj * 128; c < bj * 128 + 128; ++c) out[size_t(r) * K + c] = e4m3_encode(w[size_t(r) * K + c] / s);
    }
  ORACLE_END
}

// Head reference: logits[m,n] = sum over 128-wide K blocks of sx[m,kb]*sw[n/128,kb]*dot(a[m,kb],w[n,kb]),
// each block dot product exact in FP64 and the block sum carried in FP64; rounded once to FP32 at the end.
int oracle_head_fp8(const uint8_t *a, const float *a_scale, const uint8_t *w, const float *w_scale, float *logits,
                    int M, int N, int K, int threads) {
  ORACLE_TRY if (!a || !a_scale || !w || !w_scale || !logits || M < 1 || N < 1 || K < 128 || K % 128)
      fail("head arguments");
  float table[256];
  oracle_e4m3_table(table);
  const int kb = K / 128;
  std::vector<float> af(size_t(M) * K);
  for (size_t i = 0; i < af.size(); ++i) af[i] = table[a[i]];
  parallel_rows(N, threads, [&](int n) {
    std::vector<float> wf(K);
    for (int k = 0; k < K; ++k) wf[k] = table[w[size_t(n) * K + k]];
    for (int m = 0; m < M; ++m) {
      double total = 0;
      for (int g = 0; g < kb; ++g) {
        double dot = 0;
        for (int k = g * 128; k < g * 128 + 128; ++k) dot += double(af[size_t(m) * K + k]) * double(wf[k]);
        total += double(a_scale[size_t(m) * kb + g]) * double(w_scale[size_t(n / 128) * kb + g]) * dot;
      }
      logits[size_t(m) * N + n] = float(total);
    }
  });
  ORACLE_END
}

// ---- synthetic inputs shared by the oracle and the CUDA path (counter-based, platform independent)
// Standard normal from two Philox uniforms by Box-Muller in FP64.  stream selects the tensor, index the element.
static inline double unit_normal(uint64_t seed, uint64_t stream, uint64_t index) {
  // purposes/slots are not used here: the generator has its own domain (slot 5, purpose 3, high draw numbers
  // would collide with nothing the sampler draws because the key below is different from any request seed used
  // in the tests: key = seed ^ stream-mix).
  const uint64_t key = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
  const uint64_t hi = philox_word(key, index, 0, 0, 0) >> 5, lo = philox_word(key, index, 0, 0, 1) >> 6;
  const uint64_t hi2 = philox_word(key, index, 0, 0, 2) >> 5, lo2 = philox_word(key, index, 0, 0, 3) >> 6;
  const double u1 = (double((hi << 26) | lo) + 0.5) * 0x1p-53, u2 = double((hi2 << 26) | lo2) * 0x1p-53;
  return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
}
static inline uint64_t raw64(uint64_t seed, uint64_t stream, uint64_t index) {
  const uint64_t key = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
  return (uint64_t(philox_word(key, index, 1, 0, 0)) << 32) | philox_word(key, index, 1, 0, 1);
}

// Zipf+Gaussian logits row: x[id] = f32(sigma*N(0,1) - s*ln(rank(id))), rank = 1 + position of id in a seeded
// Fisher-Yates permutation.  One row per call; row index enters the stream so rows are independent.
int oracle_gen_logits(uint64_t seed, uint64_t row, int n, double sigma, double zipf_s, float *out) {
  ORACLE_TRY if (!out || n < 1) fail("gen arguments");
  std::vector<int> perm(n);
  std::iota(perm.begin(), perm.end(), 0);
  for (int i = n - 1; i > 0; --i) {
    const uint64_t j = raw64(seed, 2 * row + 1, uint64_t(i)) % uint64_t(i + 1);
    std::swap(perm[i], perm[int(j)]);
  }
  for (int pos = 0; pos < n; ++pos) {
    const int id = perm[pos];
    out[id] = float(sigma * unit_normal(seed, 2 * row, uint64_t(id)) - zipf_s * std::log(double(pos + 1)));
  }
  ORACLE_END
}
// out[i] = f32(base[i] + sigma*N(0,1)) -- draft logits from target logits.
int oracle_gen_perturbed(uint64_t seed, uint64_t row, int n, double sigma, const float *base, float *out) {
  ORACLE_TRY if (!out || !base || n < 1) fail("gen arguments");
  for (int i = 0; i < n; ++i) out[i] = float(double(base[i]) + sigma * unit_normal(seed, 0x40000000ull + row, uint64_t(i)));
  ORACLE_END
}
// out[i] = sigma*N(0,1) as fp32 (caller converts to bf16 / quantises).
int oracle_gen_normal(uint64_t seed, uint64_t stream, int64_t count, double sigma, float *out) {
  ORACLE_TRY if (!out || count < 1) fail("gen arguments");
  for (int64_t i = 0; i < count; ++i) out[i] = float(sigma * unit_normal(seed, 0x80000000ull + stream, uint64_t(i)));
  ORACLE_END
}
// Token history from a Zipf(s) law over a seeded permutation of ids (inverse CDF over a precomputed table).
int oracle_gen_history(uint64_t seed, uint64_t row, int n, int len, double zipf_s, int32_t *out) {
  ORACLE_TRY if (!out || n < 1 || len < 1) fail("gen arguments");
  std::vector<double> cdf(n);
  double z = 0;
  for (int r = 0; r < n; ++r) { z += std::pow(double(r + 1), -zipf_s); cdf[r] = z; }
  std::vector<int> perm(n);
  std::iota(perm.begin(), perm.end(), 0);
  for (int i = n - 1; i > 0; --i) {
    const uint64_t j = raw64(seed, 0xC0000000ull + 2 * row + 1, uint64_t(i)) % uint64_t(i + 1);
    std::swap(perm[i], perm[int(j)]);
  }
  for (int j = 0; j < len; ++j) {
    const double u = double(raw64(seed, 0xC0000000ull + 2 * row, uint64_t(j)) >> 11) * 0x1p-53 * z;
    const int rank = int(std::lower_bound(cdf.begin(), cdf.end(), u, [](double c, double v) { return c <= v; }) - cdf.begin());
    out[j] = perm[std::min(rank, n - 1)];
  }
  ORACLE_END
}
// Allowed-token bitmask with roughly `fraction` of ids set in contiguous runs of 8..263 ids.
int oracle_gen_mask(uint64_t seed, uint64_t row, int n, double fraction, uint32_t *out) {
  ORACLE_TRY if (!out || n < 1 || !(fraction > 0) || fraction > 1) fail("gen arguments");
  const int words = (n + 31) / 32;
  std::fill(out, out + words, 0u);
  const int64_t want = std::max<int64_t>(1, int64_t(fraction * n));
  int64_t have = 0;
  for (uint64_t j = 0; have < want && j < 1000000; ++j) {
    const uint64_t r = raw64(seed, 0xE0000000ull + row, j);
    const int start = int((r >> 16) % uint64_t(n)), len = 8 + int(r & 255);
    for (int i = start; i < std::min(n, start + len); ++i)
      if (!((out[i >> 5] >> (i & 31)) & 1u)) { out[i >> 5] |= 1u << (i & 31); ++have; }
  }
  ORACLE_END
}

}  // extern "C"
