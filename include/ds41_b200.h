/* ds41_b200.h -- C ABI of the B200 (sm_100a) decode-tail library: LM head -> sampler -> MTP verify.
 *
 * Conventions are the reference plugins' own (components/fuse-head/include/ds41/fuse_head.h:8,
 * components/dense/include/ds41/dense.h:8-10, engine/third_party/spark/include/ds41/spark.h:35-36,116-120):
 *   - every tensor argument is DEVICE memory owned by the caller and alive until the stream reaches the call;
 *   - calls only enqueue work on the given stream: no allocation, no synchronisation, no hidden state;
 *   - the return value is a cudaError_t as int (0 = enqueued); argument errors return cudaErrorInvalidValue and
 *     leave a message for ds41_spark_error();
 *   - DATA errors (non-finite logits, empty allowed set, impossible draft ...) are reported in band, per row,
 *     in the caller's status / result buffers, exactly as the reference GPU sampler signals `emitted = -1`
 *     (third_party/spark/src/sampling.cu:29-32).
 * There is no CPU implementation behind any entry point; a machine without a CUDA device gets a CUDA error.
 */
#ifndef DS41_B200_H
#define DS41_B200_H
#include <stddef.h>
#include <stdint.h>
#include <cuda_runtime_api.h>
#ifdef __cplusplus
extern "C" {
#endif

#define DS41_B200_ABI 2
#define DS41_B200_MAX_VOCAB 131072 /* 8 cluster CTAs x 16384 staged logits */
#define DS41_B200_MAX_HISTORY 65535 /* 16-bit shared-memory counters */

/* ---- per-row status words written by the sampler / verifier ------------------------------------------------
 * 0            decision certified: it provably equals the reference FP64 rule for these inputs, assuming only
 *              that both exp() implementations are within 1 ulp.
 * >0 bit set   decision taken but NOT certified (the quantity compared lay inside the rounding-error bound of
 *              the parallel summation): 1 inverse-CDF draw, 2 top-p cut, 4 accept test, 8 residual draw.
 * <0           row rejected, token = -1 / emitted = -1:  */
#define DS41_B200_ROW_NONFINITE (-1)      /* a logit is NaN/Inf   (sampling.cpp:32 "nonfinite logits") */
#define DS41_B200_ROW_EMPTY (-2)          /* bitmask allows no id (sampling.cpp:19 "empty residual support") */
#define DS41_B200_ROW_PENALTY_OVERFLOW (-3)
#define DS41_B200_ROW_TIES (-4)           /* the cut search gave up: more than 1024 ids, not all equal, inside one bin of its finest level */
#define DS41_B200_ROW_TIMEOUT (-5)        /* a bounded device-side wait expired */
#define DS41_B200_ROW_DRAFT (-6)          /* draft id out of range or impossible under q (sampling.cpp:44,47) */
#define DS41_B200_ROW_NOT_COVERED (-8)    /* sharded combine: the candidates of some rank may not contain the whole nucleus; redo the row from full logits */
#define DS41_B200_ROW_NOT_NORMALIZED (-10) /* a probability row does not sum to 1 within 1e-8 (sampling.cpp:15) */
#define DS41_B200_ROW_HISTORY (-7)        /* history_len[r] negative, above DS41_B200_MAX_HISTORY or above history_stride */

/* Same layout as ds41_spark_result (spark.h:106-108). */
typedef struct ds41_spark_result {
  int32_t tokens[6];
  int emitted, accepted_drafts, accepted_input_rows, rejected;
} ds41_spark_result;

/* ---- host-side helpers (pure integer/FP64 arithmetic, no device) --------------------------------------------
 * Replace ds41_spark_rng_word_v2 / ds41_spark_uniform_v2 / ds41_spark_error (spark.h:39,129-130; implementation
 * third_party/spark/src/sampling.cpp:9-10,57-58).  Invalid addresses return 0 / NaN and set the message. */
uint32_t ds41_spark_rng_word_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw);
double ds41_spark_uniform_v2(uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose, uint64_t draw);
const char *ds41_spark_error(void);

/* ---- LM head -------------------------------------------------------------------------------------------
 * FP8 head: logits[m,n] = sum over 128-wide K blocks kb of a_scale[m,kb] * w_scale[n/128,kb] *
 * dot(a[m,kb], w[n,kb]) with e4m3 operands and fp32 output.  There is no FP8 head in the reference; the entry
 * points keep the call shape of ds41_fuse_head_decode (components/fuse-head/include/ds41/fuse_head.h:9-10:
 * activations, weights, fp32 logits [M,N], M, N, K, stream) and the two-step quantise / multiply split of
 * ds41_dense_quant + ds41_dense_fp8 (components/dense/include/ds41/dense.h:10-13; dense.cu:8-16,25-91).
 *   w_e4m3  [N,K] row-major, K % 128 == 0;  w_scale [ceil(N/128), K/128] fp32
 *   a_e4m3  [M,K];  a_scale [M, K/128] fp32 (powers of two, as ds41_dense_quant produces them, group 128)
 *   error_flag: optional device int raised to 1 if a bounded device-side wait expired (logits then invalid). */
int ds41_b200_quantize_activations(const void *x_bf16, void *a_e4m3, float *a_scale, int M, int K,
                                   cudaStream_t stream);
int ds41_b200_head_fp8(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                       float *logits, int64_t logits_stride, int M, int N, int K, int *error_flag,
                       cudaStream_t stream);
/* The same head, which also leaves per-row records (first maximum and its id, minimum, finiteness) of the logits it
 * produced in row_extremes [M] (DS41_B200_ROW_EXTREMES_BYTES each, 16-byte aligned, cleared by the call): pass them to
 * ds41_b200_sample_logits as args->row_extremes and the sampler's batch path skips its own first pass over the logits.
 * No counterpart in the reference (its sampler runs on the host). */
#define DS41_B200_ROW_EXTREMES_BYTES 16
int ds41_b200_head_fp8_stats(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                             float *logits, int64_t logits_stride, int M, int N, int K, void *row_extremes,
                             int *error_flag, cudaStream_t stream);
/* Quantise + multiply in one call: x_bf16 [M,K] -> logits fp32 [M,N] (stride N).  workspace: caller-owned device
 * memory of ds41_fuse_head_fp8_workspace_bytes(M,K) bytes, 256-byte aligned. */
size_t ds41_fuse_head_fp8_workspace_bytes(int M, int K);
int ds41_fuse_head_fp8(const void *x_bf16, const void *w_e4m3, const float *w_scale, float *logits, int M, int N,
                       int K, void *workspace, size_t workspace_bytes, int *error_flag, cudaStream_t stream);

/* BF16 head: the reference engine's head plugin symbol, same signature and argument check
 * (components/fuse-head/include/ds41/fuse_head.h:9-10; src/head_decode.cpp:4-10: 1 <= M <= 6, N == 129280, K == 5120),
 * x fp32 [M,K], weights bf16 [N,K] row-major, out fp32 [M,N].  The FP32 arithmetic order of the reference kernels
 * (head_half_tree.cu:7-21: sixteen fused-multiply-add chains over k = l + 16 j, a four-level tree, +0.f) is kept, so
 * the results equal the reference plugin's bit for bit.  ds41_b200_head_bf16 is the same operator for any N and any K
 * that is a multiple of 256 with M*K*4 bytes of activations + 68 KB within 227 KB of shared memory (K <= 6656 at
 * M = 6); weights 16-byte aligned. */
int ds41_fuse_head_decode(const float *x, const void *weights_bf16, float *out, int M, int N, int K,
                          cudaStream_t stream);
int ds41_b200_head_bf16(const float *x, const void *weights_bf16, float *out, int M, int N, int K,
                        cudaStream_t stream);

/* FP32 head: y[m, n] = sum_k w[n, k] * x[m, k] with FP32 weights [N, K] (K contiguous), x [M, K], y [M, N], M <= 8, K a
 * multiple of 128, M * K * 4 <= 224 KB.  Stands in for the reference's default target head, ds41_dense_cublas(f32 = 1)
 * on FP32-promoted weights (components/dense/src/ops.cu:120-128; engine/src/forward.cu:1306-1318).  cuBLAS does not
 * specify its order of summation, so there is nothing to match bit for bit: the order here is fixed (stated in
 * csrc/head_f32.cu) and the result is within the FP32 bound of the exact product. */
int ds41_b200_head_f32(const float *x, const float *w, float *y, int M, int N, int K, cudaStream_t stream);

/* Drafter head: the reference's own symbol and argument check (components/dense/include/ds41/dense.h;
 * src/compact.cu:10-24,44-50: 1 <= M <= 8, K a multiple of 256), x fp32 [M,K], weights bf16 [N,K], y fp32 [M,N].  The
 * reference kernel's FP32 order is kept (four fused-multiply-add chains per lane over 8-wide loads,
 * (a0+a1)+(a2+a3), 32-lane shuffle-down tree), so the results equal the reference's bit for bit.  Additional limits of
 * this implementation: M*K*4 bytes within 224 KB of shared memory, x and weights 16-byte aligned. */
int ds41_dense_head_compact(const float *x, const void *w_bf16, float *y, int M, int N, int K, cudaStream_t stream);
/* Draft logits of one position: logits[n] = draft_row[n] + bias[n], bias = markov_weight [vocab,256] (bf16) times the
 * previous token's Markov embedding [256] (bf16, promoted to fp32): the reference's markov() + add_bias
 * (engine/third_party/spark/src/forward.cu:46,135-139) in one kernel.  The reference forms the bias with a library GEMV
 * whose summation order is not specified; here it is the compact head's order for K = 256, followed by the reference's
 * single rounded addition. */
int ds41_b200_markov_logits(const float *draft_row, const void *markov_weight_bf16, const void *embedding_bf16,
                            float *logits, int vocab, cudaStream_t stream);
/* What the reference runs in front of the target head (engine/src/hotpath/batch.inc:487-492): HC-pre mix of the four
 * streams h [M,4,K] (bf16) with pre [M,4] -> RMSNorm with norm_weight [K] (bf16), eps -> bf16 -> fp32 x [M,K], as one
 * kernel with the arithmetic and the M-dependent reduction geometry of ds41_dense_hc_pre, ds41_dense_rms and
 * ds41_dense_promote (components/dense/src/ops.cu:10-27,45-48,102,110-112): bit-identical to running those three.
 * 1 <= M <= 8, K a multiple of 4 in 128..16384. */
int ds41_b200_final_norm(const void *h_bf16, const float *pre, const void *norm_weight_bf16, float *x_f32, int M, int K,
                         float eps, cudaStream_t stream);

/* ---- sampler: logits -> token ids -----------------------------------------------------------------------
 * Replaces, fused and batched on the device, the engine's per-token host sequence
 *   probabilities(logits, T, top_p)  (engine/src/sampling.cpp:205-219 -> spark sampling.cpp:30-38)
 *   sample(p, rng, step, slot, purpose) (engine/src/sampling.cpp:220-226 -> spark sampling.cpp:18-21,59)
 *   argmax(logits) for temperature 0   (engine/src/sampling.cpp:133-139; server.cpp:623-625)
 * Row r draws with the Philox address (seeds[r], steps[r], slot, purpose) (spark_rng.h:23-36).
 * The temperature floor max(T,1e-5) of the adapter is applied here (engine/src/sampling.cpp:209-210).
 * top_k, the three penalties and the bitmask have no counterpart in the reference.  Their rule: count[id] =
 * occurrences of id in the row's history; for count > 0, in FP32 with every operation rounded separately,
 * y = x > 0 ? x / repetition : x * repetition, then y -= (presence + frequency * float(count)) (a non-finite result
 * rejects the row); ids whose mask bit is 0 are excluded (no id left rejects the row); top_k keeps the first k
 * remaining ids in the order (y descending, id ascending); the reference rule then runs on the survivors.  The CPU
 * oracle of the tests implements the same rule. */
typedef struct ds41_b200_sample_args {
  uint32_t struct_bytes;      /* sizeof(ds41_b200_sample_args): ABI check */
  int32_t rows, vocab;        /* 1 <= vocab <= DS41_B200_MAX_VOCAB */
  const float *logits;        /* [rows, logits_stride] fp32 */
  int64_t logits_stride;      /* elements between rows: >= vocab, or 0 to give every row the same logits */
  double temperature;         /* >= 0, finite; 0 = greedy */
  double top_p;               /* (0,1] */
  int32_t top_k;              /* 0 = off */
  float repetition, presence, frequency; /* 1,0,0 = off */
  const int32_t *history;     /* [rows, history_stride] token ids or NULL; ids outside [0,vocab) are padding */
  int64_t history_stride;
  const int32_t *history_len; /* [rows] valid entries per row, or NULL = history_stride for every row */
  const uint32_t *mask;       /* [rows, mask_stride] allowed-token bits (id/32, id%32) or NULL */
  int64_t mask_stride;
  const uint64_t *seeds;      /* [rows] Philox key per row */
  const uint64_t *steps;      /* [rows] attempt counter per row */
  uint32_t slot, purpose;     /* slot 0..5, purpose 0..3 (spark.h:96) */
  int32_t *tokens;            /* [rows] out */
  int32_t *status;            /* [rows] out, see above; may be NULL */
  void *scratch;              /* optional device scratch of ds41_b200_sample_scratch_bytes(rows, vocab) bytes, 16-byte
                                 aligned.  With it, rows without penalties / bitmask and with top_k <= 64 are tried,
                                 per row, by two batch-parallel paths before the cluster kernel: without top_k (rows
                                 16-byte aligned, vocab >= 16384) the batch path (grid-wide kernels: histogram,
                                 window, FP64 masses, resolve), then the streaming path for small nuclei (chunk
                                 records + a per-row combine).  Rows neither can take, and calls without scratch,
                                 use the cluster kernel.  Same results on every path.  With scratch, rows whose
                                 decision fell inside the rounding bound of the parallel sums (status bits 1 / 2) are
                                 redone in the same call in the reference's order of operations and leave with
                                 status 0 (the scratch holds the replay's rows too: about 10 MB). */
  size_t scratch_bytes;
  const void *row_extremes;   /* optional: the [rows] records ds41_b200_head_fp8_stats wrote for these logits (16 bytes
                                 each); the batch path then skips its own maximum / minimum pass.  NULL otherwise. */
} ds41_b200_sample_args;
size_t ds41_b200_sample_scratch_bytes(int rows, int vocab);
int ds41_b200_sample_logits(const ds41_b200_sample_args *args, cudaStream_t stream);

/* ---- MTP speculative verification from logits ---------------------------------------------------------------
 * Replaces probabilities_rows() + reject_sample() (engine/src/speculation.cpp:179-182;
 * engine/src/sampling.cpp:142-204,227-275 -> ds41_spark_verify_v2, spark sampling.cpp:39-56) for `sequences`
 * independent transactions of `drafts` (0..5) proposals each.  p rows come from the target logits, q rows from
 * the draft logits, both through the same temperature/top-p rule, so q is the measure the proposal was drawn
 * from (spark.h:101-105).  Sequence s uses the address (seeds[s], steps[s], slot = position, purpose =
 * ACCEPT / RESIDUAL / TARGET) exactly as the reference.  temperature 0 selects the greedy rule (draft_logits
 * may then be NULL).  `scratch` is caller-owned device memory of ds41_b200_verify_scratch_bytes() bytes (16-byte
 * aligned): 48 bytes of statistics per logits row, the streaming path's chunk records, and 7.3 MB for the replay of
 * transactions whose decisions fell inside the rounding bound (status bits 1 / 2 / 4 / 8: redone in the same call in
 * the reference's order, they leave with status 0).  With less the call still works: without the replay's share the
 * bits stay in the status words; with the statistics alone every row goes through the cluster kernel. */
typedef struct ds41_b200_verify_args {
  uint32_t struct_bytes;
  int32_t sequences, drafts, vocab;
  const float *target_logits;  /* [sequences*(drafts+1), vocab] */
  const float *draft_logits;   /* [sequences*drafts, vocab] */
  const int32_t *draft_ids;    /* [sequences*drafts] */
  double temperature, top_p;
  const uint64_t *seeds, *steps; /* [sequences] */
  ds41_spark_result *results;  /* [sequences] out */
  int32_t *status;             /* [sequences] out, may be NULL */
  void *scratch;
  size_t scratch_bytes;
} ds41_b200_verify_args;
size_t ds41_b200_verify_scratch_bytes(int sequences, int drafts);
size_t ds41_b200_verify_scratch_bytes_for(int sequences, int drafts, int vocab);
int ds41_b200_verify_logits(const ds41_b200_verify_args *args, cudaStream_t stream);

/* Same verification for callers that cannot provide or allocate scratch memory (an engine running on a fixed
 * device-memory plan, a plugin that must not touch its host's allocator).  This entry point has no counterpart in
 * the reference.  args->scratch and args->scratch_bytes are ignored: the per-row statistics live in a 48 KiB device
 * array built into the library, so sequences*(2*drafts+1) may not exceed
 * ds41_b200_verify_logits_static_max_rows() (1024); larger requests return cudaErrorInvalidValue with a message.
 * Small calls (up to five full-vocabulary rows, e.g. one sequence with two drafts) take the chunk + combine path and
 * keep their 544-byte chunk records in the same array, behind the statistics.
 * The first call on each device looks up the array's address (make it before any stream capture); no call
 * allocates.  All calls share the array, so calls that could overlap on the GPU must be serialised by the caller. */
int ds41_b200_verify_logits_static_max_rows(void);
int ds41_b200_verify_logits_static(const ds41_b200_verify_args *args, cudaStream_t stream);

/* ---- operators on probability rows: the reference sampler's C ABI on the device ------------------------------------------
 * For callers that keep the reference's own interface (logits -> probability row -> sample / verify:
 * engine/include/ds41/engine.hpp:211-227) instead of the fused calls above.  Every sum runs on one thread in index
 * order, as the reference's host loops do, so for the same probability rows the tokens and accept / reject records are
 * the reference's bit for bit; ds41_b200_probabilities follows ds41_spark_probabilities operation by operation and can
 * differ from the host's rows only in the last place of exp().  One CTA per row or transaction, milliseconds per
 * full-vocabulary row: compatibility and reporting paths, not the decode-rate path.
 *   ds41_b200_probabilities         <- ds41_spark_probabilities (spark.h:115; sampling.cpp:30-38), temperature floor of
 *                                      the engine adapter (engine/src/sampling.cpp:209-210); non-finite rows: status -1
 *   ds41_b200_sample_probabilities  <- ds41_spark_sample_v2     (spark.h:131; sampling.cpp:12-21,59), row r at the
 *                                      address (seeds[r], steps[r], slot, purpose); rows that are not a probability
 *                                      measure get token -1 and status -1 / -10 / -2
 *   ds41_b200_verify_probabilities  <- ds41_spark_verify_v2     (spark.h:132; sampling.cpp:39-56), `sequences`
 *                                      transactions; q [sequences, drafts, vocab], p [sequences, drafts+1, vocab]
 *   ds41_spark_sample_gpu_v2 / ds41_spark_verify_gpu_v2: the reference's device sampler ABI itself (spark.h:133-134;
 *   third_party/spark/src/sampling.cu:24-39,71-72): FP32 measures normalised in FP64, one row / one transaction, result
 *   in caller-owned device memory, data errors in band (token -1 / emitted -1). */
typedef struct ds41_b200_prob_args {
  uint32_t struct_bytes;
  int32_t rows, vocab;
  const float *logits;       /* [rows, logits_stride] */
  int64_t logits_stride;
  double temperature, top_p;
  double *probabilities;     /* [rows, vocab] out */
  int32_t *status;           /* [rows] out */
  void *scratch;             /* ds41_b200_probabilities_scratch_bytes(rows) bytes, 16-byte aligned */
  size_t scratch_bytes;
} ds41_b200_prob_args;
size_t ds41_b200_probabilities_scratch_bytes(int rows);
int ds41_b200_probabilities(const ds41_b200_prob_args *args, cudaStream_t stream);
int ds41_b200_sample_probabilities(const double *p, int rows, int vocab, int64_t stride, const uint64_t *seeds,
                                   const uint64_t *steps, uint32_t slot, uint32_t purpose, int32_t *tokens,
                                   int32_t *status, cudaStream_t stream);
int ds41_b200_verify_probabilities(const int32_t *draft_ids, const double *q, const double *p, int sequences,
                                   int drafts, int vocab, int greedy, const uint64_t *seeds, const uint64_t *steps,
                                   ds41_spark_result *results, int32_t *status, cudaStream_t stream);
int ds41_spark_sample_gpu_v2(const float *p, int vocab, uint64_t seed, uint64_t step, uint32_t slot, uint32_t purpose,
                             int32_t *token, void *stream);
int ds41_spark_verify_gpu_v2(const int32_t *draft_ids, const float *q, const float *p, int drafts, int vocab,
                             int greedy, uint64_t seed, uint64_t step, ds41_spark_result *result, void *stream);

/* ---- vocabulary-sharded sampling (several GPUs, one rank per GPU) -----------------------------------------------
 * No counterpart in the reference (single GPU, no collectives: scripts/run.py:228).  Rank r owns the logits of the
 * contiguous id range [vocab_offset, vocab_offset + vocab_local) (e.g. its slice of the head's weight rows).
 *   1. every rank: ds41_b200_shard_candidates -> `chunks` records of 544 bytes per row (one per 8192 ids; pass the
 *      same `chunks` >= ds41_b200_shard_chunks(largest vocab_local) on every rank so that the records line up);
 *   2. caller: all-gather of the records into `gathered` [ranks][rows][chunks] (ncclAllGather on the same stream);
 *   3. every rank: ds41_b200_shard_combine -> the same token ids on every rank (ranks * chunks <= 17).
 * A row whose surviving ids may extend beyond some chunk's 64 candidates gets status DS41_B200_ROW_NOT_COVERED and
 * token -1; the caller must then sample that row from its full logits (ds41_b200_sample_logits).  top_p = 1 without
 * top_k is therefore only covered for tiny vocabularies; top_k must be <= 64. */
#define DS41_B200_SHARD_CANDIDATES 64
typedef struct ds41_b200_shard_row {
  double z;
  float max_logit;
  int32_t argmax, count, status;
  int32_t complete; /* 1: cand[] holds every id of the chunk */
  float z_err;
  struct { float y; int32_t id; } cand[DS41_B200_SHARD_CANDIDATES];
} ds41_b200_shard_row;
typedef struct ds41_b200_shard_args {
  uint32_t struct_bytes;
  int32_t rows, vocab_local, vocab_offset;
  int32_t chunks;           /* records per row; 0 = ds41_b200_shard_chunks(vocab_local) */
  const float *logits;      /* [rows, logits_stride], this rank's id range */
  int64_t logits_stride;
  double temperature;
  ds41_b200_shard_row *out; /* [rows][chunks] */
} ds41_b200_shard_args;
int ds41_b200_shard_chunks(int vocab_local);
int ds41_b200_shard_candidates(const ds41_b200_shard_args *args, cudaStream_t stream);
typedef struct ds41_b200_shard_combine_args {
  uint32_t struct_bytes;
  int32_t rows, ranks, chunks, vocab;    /* vocab = full vocabulary */
  const ds41_b200_shard_row *gathered;   /* [ranks][rows][chunks] */
  double temperature, top_p;
  int32_t top_k;                         /* 0 = off, else <= 64 */
  const uint64_t *seeds, *steps;         /* [rows] */
  uint32_t slot, purpose;
  int32_t *tokens, *status;              /* [rows] out */
} ds41_b200_shard_combine_args;
int ds41_b200_shard_combine(const ds41_b200_shard_combine_args *args, cudaStream_t stream);

/* ---- vocabulary-sharded head with the row exchange fused into its epilogue ----------------------------------------
 * No counterpart in the reference (single GPU).  The batch rows are split over `owners` ranks, rows_per_owner each
 * (the last owner may hold fewer); owner_logits[r] is rank r's full-vocabulary buffer [rows_per_owner, logits_stride],
 * mapped into this process (ds41_b200_peer_open) or local for r = this rank.  The kernel computes this rank's slice
 * [vocab_offset, vocab_offset + N) of every row's logits and stores row m into owner m / rows_per_owner at local row
 * m % rows_per_owner with plain peer stores, so the exchange (vocabulary-sharded -> row-sharded) overlaps the GEMM.
 * The caller orders the owners' readers after every rank's kernel (a stream-ordered collective such as a one-word
 * all-reduce) and the next step's writers after the readers (the token all-gather does that).
 * owner_logits is a HOST array of `owners` device pointers, copied at the call. */
int ds41_b200_head_fp8_scatter(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                               float *const *owner_logits, int owners, int rows_per_owner, int64_t logits_stride,
                               int vocab_offset, int M, int N, int K, int *error_flag, cudaStream_t stream);
/* The same with per-row records for the sampler (see ds41_b200_head_fp8_stats): every owner's buffer holds, behind its
 * logits at byte offset stats_offset_bytes (>= rows_per_owner * logits_stride * 4, a multiple of 16), rows_per_owner
 * 16-byte records.  All ranks merge their slice's first maximum (with its global id), minimum and finiteness flag into
 * the record of the row's owner with system-scope atomic maxima.  The OWNER zeroes its records after it has read them
 * and before the collective that orders the next step's writers after this step's readers. */
int ds41_b200_head_fp8_scatter_stats(const void *a_e4m3, const float *a_scale, const void *w_e4m3, const float *w_scale,
                                     float *const *owner_logits, int owners, int rows_per_owner, int64_t logits_stride,
                                     int vocab_offset, int M, int N, int K, int64_t stats_offset_bytes, int *error_flag,
                                     cudaStream_t stream);
/* Peer-visible device buffers (CUDA IPC; one process per GPU).  alloc: cudaMalloc + a 64-byte handle to hand to the
 * other ranks; open: map another rank's buffer (enables peer access to its device on first use); close / free undo
 * them.  Not stream ordered: set up once, outside the decode loop. */
#define DS41_B200_PEER_HANDLE_BYTES 64
int ds41_b200_peer_alloc(size_t bytes, void **ptr, void *handle);
int ds41_b200_peer_open(const void *handle, void **ptr);
int ds41_b200_peer_close(void *ptr);
int ds41_b200_peer_free(void *ptr);

/* ---- score reporting: log-normaliser and top-N log-probabilities of device logits ------------------------------------
 * Replaces the host passes of the reference's score / logprobs events: log_normalizer (engine/src/server.cpp:178-183),
 * top_order (:730-737: the first n ids in the order logit descending, id ascending) and `double(l[t]) - normalizer`
 * (:450-461, :603-612).  top ids and top1 are exact; logsumexp and the log-probabilities agree with the reference's
 * sequential FP64 sum to a few units in the last place (relative 1e-13 is the tested tolerance).  Rows with a
 * non-finite logit get status DS41_B200_ROW_NONFINITE, NaN values and ids -1.  The logits_sha256 fingerprint of the
 * same event comes from ds41_b200_logits_sha256 below. */
#define DS41_B200_SCORE_MAX_TOP 32
typedef struct ds41_b200_score_args {
  uint32_t struct_bytes;
  int32_t rows, vocab;
  const float *logits;    /* [rows, logits_stride] fp32 */
  int64_t logits_stride;
  int32_t top_n;          /* 0..DS41_B200_SCORE_MAX_TOP */
  double *logsumexp;      /* [rows] out */
  int32_t *top1;          /* [rows] out: first maximum; may be NULL */
  int32_t *top_ids;       /* [rows, top_n] out */
  double *top_logprob;    /* [rows, top_n] out */
  int32_t *status;        /* [rows] out */
} ds41_b200_score_args;
int ds41_b200_score_logits(const ds41_b200_score_args *args, cudaStream_t stream);
/* digests[r, 0..32) = SHA-256 of row r's fp32 logits in little-endian byte order: the logits_sha256 field of the
 * reference's score event (engine/src/server.cpp:184-197), computed where the row lies, so that 32 bytes per row leave
 * the device instead of the row.  One thread per row (a hash is a chain): milliseconds per full-vocabulary row. */
int ds41_b200_logits_sha256(const float *logits, int rows, int vocab, int64_t logits_stride, uint8_t *digests,
                            cudaStream_t stream);

/* Measurement hook (not thread-safe, off by default): with it on, the next ds41_b200_sample_logits call that takes the
 * batch path records CUDA events on its stream between its kernels; ds41_b200_profile_read waits for the last one and
 * returns the milliseconds of each interval, in launch order: statistics, histogram, window, masses, resolve, cluster
 * kernel, replay (DS41_B200_PROFILE_PHASES of them; fewer when the call ended early; -1 on a CUDA error). */
#define DS41_B200_PROFILE_PHASES 7
int ds41_b200_profile_phases(int enable);
int ds41_b200_profile_read(float *ms, int capacity);

/* ---- test hook ---------------------------------------------------------------------------------------------------
 * out[i] = the samplers' own exp(x[i]) for x <= 0 (device pointers), so that its error can be measured against a
 * reference exponential.  No counterpart in the reference. */
int ds41_b200_test_exp_nonpos(const double *x, double *out, int n, cudaStream_t stream);
/* out[i] = the weight exp((y[i] - max_logit) / temperature) as the sampler's batch path computes it in its FP64 pass
 * (y[i] <= max_logit, (max_logit - y[i]) * log2(e) / temperature <= 600; device pointers), for the test of its error
 * bound against a reference exponential. */
int ds41_b200_test_batch_weight(const float *y, float max_logit, double temperature, double *out, int n,
                                cudaStream_t stream);
/* out = {index or -1, acc, acc before that term} of the chain acc += v[i] over n doubles with every rounding of the
 * one-thread loop (the replay's parallel form of the reference's sums).  mode 0: the sum; 1: stop when !(acc <
 * threshold); 2: stop when threshold < acc. */
int ds41_b200_test_sequential(const double *v, int n, int mode, double threshold, double *out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
