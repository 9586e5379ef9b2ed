/*
 * CPU oracle for the Gemma decode hot path.  TEST INFRASTRUCTURE ONLY: it is the
 * checker the CUDA path is compared against and the timed CPU baseline; the
 * product library never links, loads or calls it.
 *
 * Every function restates, in plain C, the scalar CPU algorithm of the reference
 * engine; each declaration cites the reference file:line it follows.  Parity of
 * this restatement is pinned by the reference's own known-answer vectors and by
 * fixtures produced with the reference's CPU code (see tests/golden).
 */
#ifndef GF_ORACLE_H
#define GF_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF tensor type ids, as in include/local_gguf_engine/tensor/dtype.hpp:9-15. */
enum { GFO_F32 = 0, GFO_F16 = 1, GFO_Q8_0 = 8, GFO_Q4_K = 12, GFO_Q6_K = 14 };

/* src/tensor/f16.cpp:7 (decode) and :39 (encode; rounds half UP, not to even). */
float gfo_f16_to_f32(uint16_t bits);
uint16_t gfo_f32_to_f16_half_up(float value);
/* IEEE round-to-nearest-even binary16, the rounding the KV cache store uses
 * (metal_kernels.mm:2441-2517 `half()`; torch `.to(float16)` in the Python oracle). */
uint16_t gfo_f32_to_f16_rne(float value);

/* Block geometry: elements and bytes per block for a quantised dtype (0 if unknown). */
uint32_t gfo_block_elements(int dtype);
uint32_t gfo_block_bytes(int dtype);

/* src/tensor/quantization.cpp:457 (Q8_0), :517 (Q4_K), :590 (Q6_K): decode
 * `block_count` consecutive native blocks to f32, element order preserved. */
void gfo_dequantize(int dtype, const uint8_t* blocks, uint64_t block_count, float* out);

/* src/tensor/backends/cpu_backend.cpp:301-323: out[m,n] = sum_k x[m,k]*deq(w)[n,k],
 * f32, k strictly ascending.  `weight` is the native GGUF payload: output column n
 * owns K/block consecutive blocks (cpu_backend.cpp:49-53). */
void gfo_matmul_quantized(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                          uint64_t k, uint64_t n, float* out);
/* Same loop restricted to columns [n_begin, n_end): lets callers split columns across threads. */
void gfo_matmul_quantized_columns(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                                  uint64_t k, uint64_t n, uint64_t n_begin, uint64_t n_end, float* out);
/* Double-precision decoded dot and sum of |x*w|, the independent bound used by
 * tests/tensor/gemma3_metal_tests.cpp:1257-1285. */
void gfo_matmul_quantized_f64(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                              uint64_t k, uint64_t n, double* out, double* abs_out);

/* src/tensor/ops/normalization.cpp:70-101. */
void gfo_rms_norm(const float* x, const float* gamma, uint32_t rows, uint32_t hidden, float eps,
                  float* out);
/* src/tensor/ops/elementwise.cpp:79-94 times `up` (metal_kernels.mm:1827-1843). */
void gfo_gelu_tanh_multiply(const float* gate, const float* up, uint64_t count, float* out);
/* src/tensor/ops/elementwise.cpp:96-111. */
void gfo_softcap(const float* x, uint64_t count, float softcap, float* out);
/* src/tensor/ops/softmax.cpp:42-72 (double exp-sum). */
void gfo_softmax(const float* x, uint32_t rows, uint32_t columns, float* out);
/* src/tensor/ops/rope.cpp:109-117 + :246-283 (NEOX split-half), with the per-row
 * positions and linear frequency scale of metal_kernels.mm:2160-2167,2406-2439:
 * angle = position * scale / base^(2i/d), evaluated in double. */
void gfo_rope_neox(const float* x, const uint32_t* positions, uint32_t rows, uint32_t heads,
                   uint32_t head_dim, float base, float scale, float* out);

/* Grouped-query attention of one query row over `count` cached rows
 * (src/tensor/ops/attention.cpp:482-548 scores, softmax.cpp:42, :550-612 values).
 * K/V rows are f32 [count, kv_heads*head_dim] in logical order. softcap 0 = none. */
void gfo_attention_row(const float* q, const float* keys, const float* values, uint32_t count,
                       uint32_t heads, uint32_t kv_heads, uint32_t head_dim, float scale,
                       float softcap, float* out);

/* Candidate selection contract of metal_kernels.mm:3444-3589 and sampling.cpp:25-30:
 * optional softcap c*tanh(l/c), best `retain` pairs by (logit desc, token asc), then the
 * logits of `history_count` history tokens appended.  Returns pairs written. */
typedef struct { uint32_t token; float logit; } gfo_token_logit;
uint32_t gfo_select_candidates(const float* logits, uint32_t vocab, float softcap, uint32_t retain,
                               const uint32_t* history, uint32_t history_count,
                               gfo_token_logit* out);

/* ---- sampling / lossless acceptance (src/engine/sampling.cpp) ---- */
typedef struct {
    float temperature; uint32_t top_k; float top_p; float min_p; float repetition_penalty;
} gfo_sampler_options;
typedef struct { uint32_t token; double probability; double weight; } gfo_prob;
typedef struct { gfo_prob values[256]; uint32_t count; double total_weight; } gfo_distribution;

/* sampling.cpp:394-499.  Returns 0, or a negative code on the reference's throw sites. */
int gfo_prepare_distribution(const gfo_token_logit* candidates, uint32_t count,
                             const gfo_sampler_options* options, uint32_t request_top_k,
                             const uint32_t* history, uint32_t history_count,
                             gfo_distribution* out);
/* sampling.cpp:561-630 (gathered draft law): q_mass[i] is the 2^32-scaled draft mass of
 * target.values[i].token; proposal_mass the mass of the proposed token. */
int gfo_prepare_speculative(uint32_t proposal, uint64_t proposal_mass, const uint64_t* q_mass,
                            const gfo_distribution* target, double* acceptance,
                            gfo_distribution* residual);
/* sampling.cpp:632-656 + :247-257. */
int gfo_sample_speculative(uint32_t proposal, double acceptance, const gfo_distribution* residual,
                           double accept_draw, double residual_draw, uint32_t* token,
                           int* accepted);
/* sampling.cpp:247-257. */
uint32_t gfo_select_prepared(const gfo_distribution* d, double draw);

/* std::mt19937_64 and libstdc++'s uniform_real_distribution<double> as used at
 * sampling.cpp:841-842,913-918, and the proposal stream of :45-60. */
typedef struct { uint64_t mt[312]; uint32_t index; } gfo_mt19937_64;
void gfo_mt_seed(gfo_mt19937_64* rng, uint64_t seed);
void gfo_mt_seed_seq(gfo_mt19937_64* rng, const uint32_t* words, uint32_t count);
uint64_t gfo_mt_next(gfo_mt19937_64* rng);
double gfo_uniform_double(gfo_mt19937_64* rng, double a, double b);
void gfo_make_proposal_rng(const gfo_mt19937_64* target_rng, gfo_mt19937_64* out);
uint32_t gfo_next_proposal_word(gfo_mt19937_64* rng);

/* ---- load-time weight transforms (src/tensor/quantization.cpp:634-673,752-800) ---- */
int gfo_quantize_f16_q8_0(const uint16_t* f16, uint64_t block_count, uint8_t* out /* 34 B per block */);
int gfo_requantize_q6k_q4k(const uint8_t* q6, uint64_t block_count, uint8_t* out /* 144 B per block */);

/* ---- drafter proposal law (src/engine/gemma3_draft.mm:191-203,237-294) ----
 * Compact path: logits already include temperature and repetition processing
 * (gd_process).  Builds the support (every token whose score >= the top_k-th best),
 * filters with the ascending-tail top-p rule and min-p, then the integer CDF in token-id
 * order with total exactly 2^32.  Returns support size (0 = overflow >256 / invalid). */
uint32_t gfo_draft_law_compact(const float* scores, uint32_t vocab, uint32_t top_k, float top_p,
                               float min_p, uint32_t* ids, uint64_t* cdf /* count+1 */);
uint32_t gfo_draft_law_full(const float* scores, uint32_t vocab, float temperature, uint32_t top_k,
                            float top_p, float min_p, uint64_t* cdf);
void gfo_draft_process_logits(const float* logits, uint32_t vocab, float temperature,
                              float repetition_penalty, const uint32_t* history,
                              uint32_t history_count, float* scores);

/* ---- whole-model forward (Gemma 2 / Gemma 3 block schedule) ----
 * Equations of scripts/gemma3_target_reference.py:216-254, gemma3_reference_golden.py:166-209
 * and tests/support/gemma2_reference_test_support.cpp:93-205, as a token-at-a-time loop. */
typedef struct {
    int dtype;            /* GFO_* */
    const void* data;     /* native GGUF payload */
    uint64_t k, n;        /* input width, output columns */
} gfo_tensor;

typedef struct {
    gfo_tensor attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down;
    const float *attn_norm, *post_attention_norm, *ffn_norm, *post_ffw_norm, *q_norm, *k_norm;
} gfo_layer;

typedef struct {
    uint32_t hidden, ffn, heads, kv_heads, head_dim, layers, vocab;
    uint32_t sliding_window;
    uint32_t sliding_pattern;   /* 6: local iff (layer+1)%6!=0 (Gemma 3); 2: local iff layer%2==0 (Gemma 2) */
    float rope_base_global, rope_scale_global, rope_base_local, rope_scale_local;
    float rms_eps, attn_softcap, final_softcap;
    int uses_qk_norm;
    int kv_f16;                 /* 1: K/V rounded to binary16 (RNE) when cached */
    float attention_scale;      /* 1/sqrt(head_dim) */
} gfo_model_config;

typedef struct gfo_model gfo_model;
gfo_model* gfo_model_create(const gfo_model_config* config, const gfo_tensor* token_embd,
                            const float* output_norm, const gfo_tensor* output_head /* NULL = tied */,
                            const gfo_layer* layers, uint32_t context);
void gfo_model_destroy(gfo_model* model);
void gfo_model_reset(gfo_model* model);
uint32_t gfo_model_position(const gfo_model* model);
/* Appends one token at the current position.  logits may be NULL (KV only);
 * final_hidden may be NULL. */
void gfo_model_append(gfo_model* model, uint32_t token, float* logits, float* final_hidden);
void gfo_model_truncate(gfo_model* model, uint32_t position);
void gfo_model_set_kv(gfo_model* model, uint32_t layer, uint32_t first, uint32_t count, const float* keys, const float* values);
void gfo_model_seek(gfo_model* model, uint32_t position);
/* Logical cache row (after rounding), [kv_heads*head_dim] floats. */
const float* gfo_model_key(const gfo_model* model, uint32_t layer, uint32_t position);
const float* gfo_model_value(const gfo_model* model, uint32_t layer, uint32_t position);
/* Threads used for the column-parallel GEMV inside gfo_model_append (default 1). */
void gfo_set_threads(int threads);

#ifdef __cplusplus
}
#endif
#endif
