/*
 * guffin_b200 -- C ABI of the B200 (sm_100a) backend for the Gemma decode hot path.
 *
 * This is the boundary a host engine binds instead of the reference's Metal command encoder
 * (src/tensor/backends/metal/metal_command_context.hpp:54-369) and its Metal drafter
 * (include/local_gguf_engine/engine/gemma3_draft.hpp:30-105).  Plain pointers and sizes only.
 *
 * Conventions
 *  - Every function returns GF_OK (0) or a negative status; gf_last_error() gives the text.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Kernels never
 *    allocate; callers own every buffer.  Pointers named *_dev are device pointers.
 *  - A context (stream + its buffers) is used from one thread at a time
 *    (target_verifier.hpp:363-365 states the same contract).
 *  - Weight matrices are logically [K, N]: output column n owns K/block consecutive GGUF
 *    blocks (src/tensor/backends/cpu_backend.cpp:49-53).
 */
#ifndef GUFFIN_B200_H
#define GUFFIN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GF_API __attribute__((visibility("default")))

enum {
    GF_OK = 0,
    GF_ERR_INVALID = -1,      /* std::invalid_argument in the reference (shape / extent) */
    GF_ERR_STATE = -2,        /* std::logic_error (state machine) */
    GF_ERR_CUDA = -3,         /* BackendError{metal_execution_failed} */
    GF_ERR_UNAVAILABLE = -4,  /* BackendError{unavailable_metal_device} */
    GF_ERR_NUMERIC = -5,      /* std::overflow_error: non-finite F16 K/V, poisoned plan */
    GF_ERR_TIMEOUT = -6       /* a bounded device-side wait gave up */
};

/* GGUF tensor type ids (include/local_gguf_engine/tensor/dtype.hpp:9-15). */
enum { GF_F32 = 0, GF_F16 = 1, GF_Q8_0 = 8, GF_Q4_K = 12, GF_Q6_K = 14 };

GF_API const char* gf_last_error(void);
GF_API const char* gf_version(void);

/* ---- device, memory, streams: replaces metal_backend.hpp:17-51 / metal_buffer.hpp:48-84 ---- */
GF_API int gf_device_count(int* count);             /* tensor_backend_is_available (tensor/backend.hpp:10) */
GF_API int gf_set_device(int device);
GF_API int gf_memory_info(size_t* free_bytes, size_t* total_bytes);   /* metal_backend.hpp memory_info */
GF_API int gf_malloc(void** out_dev, size_t bytes);                   /* allocate_backend_buffer */
GF_API int gf_free(void* ptr_dev);
GF_API int gf_host_alloc(void** out_host, size_t bytes);              /* pinned staging */
GF_API int gf_host_free(void* ptr_host);
GF_API int gf_memset(void* dst_dev, int value, size_t bytes, void* stream);
GF_API int gf_upload(void* dst_dev, const void* src_host, size_t bytes, void* stream);    /* copy_tensor_to_backend */
GF_API int gf_download(void* dst_host, const void* src_dev, size_t bytes, void* stream);  /* copy_tensor_from_backend */
GF_API int gf_copy(void* dst_dev, const void* src_dev, size_t bytes, void* stream);
GF_API int gf_stream_create(void** out_stream);
GF_API int gf_stream_destroy(void* stream);
GF_API int gf_stream_synchronize(void* stream);     /* MetalCommandContext::wait_until_completed */
/* Device timestamps on a stream: the gpu_duration_ns of MetalCommandStats
 * (metal_command_context.hpp:19-45) comes from a pair of these. */
GF_API int gf_event_create(void** out_event);
GF_API int gf_event_destroy(void* event);
GF_API int gf_event_record(void* event, void* stream);
GF_API int gf_event_synchronize(void* event);
GF_API int gf_event_elapsed_ms(void* start_event, void* end_event, float* out_ms);

/* ---- weight preparation: replaces repack_kquant_weight_columns8 / restore_native_kquant_weight
 * (src/tensor/kquant_packing.cpp:154,250).  The streaming layout keeps every bit of the native
 * blocks: 8 output columns x one K unit (256 elements; 128 for Q8_0) per contiguous 16-byte
 * aligned group, missing columns zero-filled.  K must be a multiple of the unit. ---- */
GF_API size_t gf_packed_weight_bytes(int dtype, uint64_t k, uint64_t n);
GF_API int gf_pack_weight(int dtype, const void* native_dev, uint64_t k, uint64_t n,
                          void* packed_dev, void* stream);
GF_API int gf_unpack_weight(int dtype, const void* packed_dev, uint64_t k, uint64_t n,
                            void* native_dev, void* stream);

/* ---- dequantisation: Q8_0/Q4_K/Q6_K BlockView::dequantized_value
 * (src/tensor/quantization.cpp:457,517,590), bit-exact, native block order. ---- */
GF_API int gf_dequantize(int dtype, const void* native_dev, uint64_t block_count, float* out_dev,
                         void* stream);

/* ---- load-time weight transforms of the Gemma 2 plan (src/engine/gemma2_metal_plan.cpp:301-316,
 * 495-512), on the device, bit-identical per block to the reference's functions built without
 * floating-point contraction:
 *   gf_quantize_f16_q8_0     quantize_f16_gguf_weight_q8_0_into (src/tensor/quantization.cpp:634-673):
 *                            32 consecutive binary16 values -> one 34-byte Q8_0 block;
 *   gf_requantize_q6_k_q4_k  requantize_q6_k_gguf_weight_q4_k_into, canonical layout (:752-800):
 *                            one 210-byte Q6_K block -> one 144-byte Q4_K block.
 * Blocks keep their order.  *status_dev (optional) gets bit 1 when a source value is not finite
 * (the reference throws std::invalid_argument). ---- */
GF_API int gf_quantize_f16_q8_0(const void* f16_dev, uint64_t block_count, void* q8_0_dev,
                                uint32_t* status_dev, void* stream);
GF_API int gf_requantize_q6_k_q4_k(const void* q6_k_dev, uint64_t block_count, void* q4_k_dev,
                                   uint32_t* status_dev, void* stream);

/* ---- quantised GEMV / small-M GEMM: MetalCommandContext::encode_verifier_matmul
 * (metal_command_context.hpp:94-101; kernels metal_kernels.mm:551-986) and the CPU reference
 * matmul_f32_quantized_gguf_weight (cpu_backend.cpp:301-323).
 * y[m, n] = sum_k x[m, k] * deq(W)[n, k], rows m <= GF_MAX_ROWS, f32 accumulate.  Each row's
 * result is bit-identical whether computed alone or beside other rows, for every row count from
 * 1 to 8 (gemma3_metal_tests.cpp:1223-1256 tests M = 1, 2, 3): up to four rows are one instance of
 * the kernel, five to eight run as two halves of the four-row instance inside one launch, planned
 * from the shape alone, so the same products are added in the same order whatever the count.
 * `workspace_dev` holds split-K partial sums (gf_matmul_workspace_bytes); it may be NULL when
 * that size is 0. ---- */
#define GF_MAX_ROWS 8
GF_API size_t gf_matmul_workspace_bytes(int dtype, uint32_t rows, uint64_t k, uint64_t n);
GF_API int gf_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev,
                     uint32_t rows, uint64_t k, uint64_t n, void* workspace_dev, void* stream);
/* Reads and clears the device error word the streaming kernels set when a bounded wait gives
 * up (GF_ERR_TIMEOUT); synchronises `stream`.  The analogue of reading the command buffer's
 * status after wait_until_completed (metal_command_context.mm:2316-2344). */
GF_API int gf_matmul_check(void* stream);
/* No counterpart in the reference.  gf_matmul for callers that cannot allocate device memory when
 * they need a projection (a latency-critical loop that must avoid cudaMalloc's device-wide stall,
 * a process whose HBM is already fully handed out to its own pools, a plugin that only receives
 * its input and output buffers): the split-K scratch is a fixed array of
 * gf_matmul_static_capacity() bytes (8 MiB) inside the library, held by every GPU that loads it.
 * The caller passes only the weights, x and y.  Shapes whose scratch would not fit are rejected
 * with GF_ERR_INVALID and a message naming both sizes.  No allocation is made, here or in
 * anything this calls.  The first call on a device looks the array's device address up (with that
 * device current); make that first call before starting any stream capture.  All calls on a
 * device share the one array: the call zeroes the counters it needs, but two calls whose kernels
 * can overlap on the GPU (different streams without ordering) race on it.
 * Failures on the device: a bounded wait that gives up sets an error word that also lives in the
 * library's static storage (gf_matmul_check does not see it).  gf_matmul_static_check(stream)
 * synchronises the stream, reads that word without allocating, returns GF_ERR_TIMEOUT and clears
 * it when it is set (y of the failed call is incomplete), GF_OK otherwise.  The word is never
 * cleared by gf_matmul_static itself, so an unread failure survives later calls. */
GF_API size_t gf_matmul_static_capacity(void);
GF_API int gf_matmul_static(int dtype, const void* packed_dev, const float* x_dev, float* y_dev,
                            uint32_t rows, uint64_t k, uint64_t n, void* stream);
GF_API int gf_matmul_static_check(void* stream);
/* The same product for up to 256 rows at once as a dense contraction on the tensor cores: bf16
 * activations, weights dequantised to bf16 in shared memory, f32 accumulation (tcgen05 / TMEM).  The
 * prompt-ingestion shape of encode_verifier_matmul with allow_prefill_matrix
 * (metal_command_context.hpp:94-101; MSL gemma3_matmul_f32_kquant_matrix_impl, metal_kernels.mm:1031-1199;
 * the reference's Gemma 2 path uses half operands the same way, gemma2_runtime.cpp:893-1170).
 * y_dev holds 128 rows of n floats, 256 when rows > 128 (rows beyond `rows` are written as zeros: every dequantised
 * weight tile feeds one 128-row product per half of the rows in use); n must be a multiple of 128,
 * k of 256 (128 for Q8_0); workspace_dev holds gf_prefill_workspace_bytes(k) bytes (the activations in the
 * tensor core's operand order).  Synchronises the stream and returns GF_ERR_TIMEOUT if a bounded wait
 * gave up.  Differs from gf_matmul by the bf16 rounding of both operands (about 4e-3 relative L2). */
GF_API size_t gf_prefill_workspace_bytes(uint64_t k);
GF_API int gf_prefill_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev,
                             uint32_t rows, uint64_t k, uint64_t n, void* workspace_dev, void* stream);
/* Attention of a prompt chunk (up to 256 rows) over the ring and the chunk's private rows of a binary16
 * cache with 256-wide heads, both contractions on the tensor cores with f16 operands (queries rounded to
 * f16 after scaling): the reference's flash prefill attention, encode_f16_prefill_attention
 * (metal_command_context.hpp; MSL metal_kernels.mm:2596-2798).  Same arguments as gf_attention without
 * the workspace; out_dev is [rows][heads * 256] f32.  Agrees with gf_attention to about 1e-3. */
GF_API int gf_prefill_attention(const float* q_dev, const void* ring_k_dev, const void* ring_v_dev,
                                const void* private_k_dev, const void* private_v_dev, float* out_dev,
                                const uint32_t* base_position_dev, uint32_t rows, uint32_t heads,
                                uint32_t kv_heads, uint32_t head_dim, uint32_t ring_rows, uint32_t window,
                                float scale, float softcap, void* stream);
/* Same product from HOST buffers through an internal context: uploads x, runs, downloads y.
 * `packed_dev` stays device-resident (weights are uploaded once at load time). */
GF_API int gf_matmul_host(int dtype, const void* packed_dev, const float* x_host, float* y_host,
                          uint32_t rows, uint64_t k, uint64_t n);

/* ---- block-schedule operators.  Per-pass scalars (the committed position) are read from
 * device memory, so one captured CUDA graph serves every token. ---- */

/* MetalCommandContext::encode_embedding (metal_command_context.hpp:75-82; kernels
 * metal_kernels.mm:235-255,452-474): gathers rows of the packed [K, vocab] matrix, dequantises
 * with the reference's rounding and multiplies by `scale` (sqrt(hidden)).  A token id >= vocab
 * sets status bit 1 and yields NaN for that row.  dtype GF_F16: `packed_dev` is a binary16 table
 * [vocab][k] exactly as the file stores it (the retained Gemma 2 9B embedding). */
GF_API int gf_embedding(int dtype, const void* packed_dev, uint32_t k, uint32_t vocab,
                        const uint32_t* tokens_dev, uint32_t rows, float scale, float* out_dev,
                        uint32_t* status_dev, void* stream);
/* encode_rms_norm / encode_rms_norm_add (metal_command_context.hpp:131-147; CPU reference
 * ops/normalization.cpp:70): out = x * rsqrt(mean(x^2) + eps) * gamma [+ residual]. */
GF_API int gf_rms_norm(const float* x_dev, const float* gamma_dev, float* out_dev, uint32_t rows,
                       uint32_t hidden, float eps, void* stream);
GF_API int gf_rms_norm_add(const float* x_dev, const float* gamma_dev, const float* residual_dev,
                           float* out_dev, uint32_t rows, uint32_t hidden, float eps, void* stream);
/* encode_head_rms_norm + encode_verifier_rope + encode_verifier_kv_store fused
 * (metal_command_context.hpp:121-130,215-241): per-head RMSNorm of Q and K (skipped when the
 * norm pointers are NULL), NEOX rotation at position base+row with
 * angle = position * freq_scale / freq_base^(2i/d), Q written as f32, K and V written to the
 * pass's private rows as F16 (round to nearest even) or F32.  Non-finite F16 sets status bit 8. */
GF_API int gf_qk_norm_rope_store(const float* raw_q_dev, const float* raw_k_dev, const float* raw_v_dev,
                                 const float* q_norm_dev, const float* k_norm_dev, float* q_out_dev,
                                 void* private_k_dev, void* private_v_dev,
                                 const uint32_t* base_position_dev, uint32_t* status_dev, uint32_t rows,
                                 uint32_t heads, uint32_t kv_heads, uint32_t head_dim, float eps,
                                 float freq_base, float freq_scale, int kv_f16, void* stream);
/* encode_verifier_rope and encode_verifier_kv_store as the reference calls them, with one position per row
 * (metal_command_context.hpp:239-263; kernels metal_kernels.mm:1915-1930,2406-2517): row r sits at
 * row_positions_dev[r].  heads = 0 skips the queries, kv_heads = 0 the cache rows; rotary_dim = 0 stores without
 * rotating (values keep their bits before the narrowing), rotary_dim = head_dim rotates whole heads; other
 * values are GF_ERR_INVALID.  status_dev may be NULL when nobody reads the non-finite bit. */
GF_API int gf_rope_store_rows(const float* raw_q_dev, const float* raw_k_dev, const float* raw_v_dev,
                              const float* q_norm_dev, const float* k_norm_dev, float* q_out_dev,
                              void* private_k_dev, void* private_v_dev, const uint32_t* row_positions_dev,
                              uint32_t* status_dev, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                              uint32_t head_dim, uint32_t rotary_dim, float eps, float freq_base,
                              float freq_scale, int kv_f16, void* stream);
/* encode_verifier_attention (metal_command_context.hpp:245-268; kernels
 * metal_kernels.mm:3070-3382): grouped-query attention of rows 0..rows-1 at positions base+row
 * over the committed ring rows inside each row's window followed by the private rows of its
 * chain ancestors, itself included.  window = 0 means a global layer.  head_dim must be 256;
 * every device pointer must be 16-byte aligned. */
GF_API size_t gf_attention_workspace_bytes(uint32_t rows, uint32_t heads);
GF_API int gf_attention(const float* q_dev, const void* ring_k_dev, const void* ring_v_dev,
                        const void* private_k_dev, const void* private_v_dev, float* out_dev,
                        void* workspace_dev, const uint32_t* base_position_dev, uint32_t rows,
                        uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t ring_rows,
                        uint32_t window, float scale, float softcap, int kv_f16, void* stream);
/* encode_gelu_tanh_multiply (metal_command_context.hpp:289-295; ops/elementwise.cpp:79). */
GF_API int gf_gelu_tanh_multiply(const float* gate_dev, const float* up_dev, float* out_dev,
                                 uint64_t count, void* stream);
/* encode_add (metal_command_context.hpp:301-306; ops/elementwise.cpp): out = left + right, elementwise. */
GF_API int gf_add(const float* left_dev, const float* right_dev, float* out_dev, uint64_t count, void* stream);
/* encode_verifier_kv_scatter (metal_command_context.hpp:269-279): publishes private rows
 * 0..rows-1 to ring slots (base + row) & (ring_rows - 1). */
GF_API int gf_kv_scatter(const void* private_k_dev, const void* private_v_dev, void* ring_k_dev,
                         void* ring_v_dev, const uint32_t* base_position_dev, uint32_t rows,
                         uint32_t row_width, uint32_t ring_rows, int kv_f16, void* stream);

/* ---- candidate selection: encode_target_token_candidates / read_target_token_candidates
 * (metal_command_context.hpp:316-323,351-355; kernels metal_kernels.mm:3444-3884).
 * Per row: optional final softcap c*tanh(l/c), the best `retain` = top_k + unique-history pairs
 * by (logit descending, token ascending), then the history tokens' logits.
 * Request row (device): { u32 retain; u32 history_count; u32 history[64] }.
 * Result row  (device): { u32 status; u32 count; { u32 token; f32 logit }[384] }. ---- */
/* Request rows written on the device (gd_requests, src/engine/gemma3_draft.mm:396-400, filling
 * VerifierDeviceSelectionRow, target_verifier.hpp:114-121): base_dev holds { u32 top_k; u32 window_limit;
 * u32 count; u32 tokens[64] } -- the sampler's repetition window, oldest first; row i of requests_dev
 * becomes the request of the context "window, root, chain_dev[1..i]" (the window slides, then its distinct
 * tokens in order of first appearance), so a verification pass whose drafted tokens exist only in device
 * memory needs no host round trip for its requests. */
GF_API size_t gf_selection_base_bytes(void);
GF_API int gf_selection_requests(const void* base_dev, uint32_t root, const uint32_t* chain_dev, uint32_t rows,
                                 void* requests_dev, void* stream);
GF_API size_t gf_selection_request_bytes(void);
GF_API size_t gf_candidate_result_bytes(void);
GF_API size_t gf_token_candidates_workspace_bytes(uint32_t rows, uint32_t vocab);
GF_API int gf_token_candidates(const float* logits_dev, uint32_t rows, uint32_t vocab, float softcap,
                               const void* requests_dev, void* workspace_dev, void* results_dev,
                               void* stream);

/* ---- resident model plan: replaces Gemma2MetalModelPlan + its verifier arena
 * (include/local_gguf_engine/engine/gemma2_metal_plan.hpp:229-319, target_verifier.hpp:228-257)
 * and the block schedule encode_gemma_target_blocks (src/engine/gemma_target_runtime.cpp:13-221).
 * The same plan type serves the 12B target, the Gemma 2 target and the 270M drafter. ---- */
typedef struct gf_model gf_model;

typedef struct gf_model_config {         /* the GemmaModelConfig fields the path uses (engine/model.hpp:52-86) */
    uint32_t hidden, ffn, heads, kv_heads, head_dim, layers, vocab;
    uint32_t sliding_window;
    uint32_t sliding_pattern;            /* 6: local iff (layer+1)%6 != 0; 2: local iff layer%2 == 0; 0: all global */
    float rope_base_global, rope_scale_global, rope_base_local, rope_scale_local;
    float rms_eps, attn_softcap, final_softcap;
    int32_t uses_qk_norm;
    int32_t kv_f16;                      /* 1: K/V cached as binary16 (round to nearest even), 0: f32 */
    float attention_scale;
    uint32_t context;                    /* positions the caches are sized for */
    uint32_t row_capacity;               /* rows per pass, 1..GF_MAX_ROWS (2 = H1 verification) */
} gf_model_config;

enum { GF_MAT_TOKEN_EMBD = 0, GF_MAT_OUTPUT = 1, GF_MAT_ATTN_Q = 2, GF_MAT_ATTN_K = 3, GF_MAT_ATTN_V = 4,
       GF_MAT_ATTN_OUTPUT = 5, GF_MAT_FFN_GATE = 6, GF_MAT_FFN_UP = 7, GF_MAT_FFN_DOWN = 8 };
enum { GF_VEC_OUTPUT_NORM = 0, GF_VEC_ATTN_NORM = 1, GF_VEC_POST_ATTENTION_NORM = 2, GF_VEC_FFN_NORM = 3,
       GF_VEC_POST_FFW_NORM = 4, GF_VEC_ATTN_Q_NORM = 5, GF_VEC_ATTN_K_NORM = 6 };
enum { GF_FORWARD_LOGITS = 1, GF_FORWARD_DEVICE_TOKENS = 2 };

GF_API int gf_model_create(const gf_model_config* config, gf_model** out_model);
GF_API int gf_model_destroy(gf_model* model);
/* Uploads one native GGUF tensor and repacks it on the device (WeightMaterializer,
 * gemma2_metal_plan.cpp:266-336).  GF_MAT_OUTPUT is optional: without it the head is tied to
 * the token embedding (resolve_gemma_output_head_policy, gemma2_metal_plan.cpp:799-828). */
GF_API int gf_model_set_matrix(gf_model* model, int kind, uint32_t layer, int dtype,
                               const void* native_host, uint64_t k, uint64_t n);
GF_API int gf_model_set_vector(gf_model* model, int kind, uint32_t layer, const float* values_host,
                               uint32_t count);
/* gf_model_set_matrix also takes binary16 tables (dtype GF_F16, [K, vocab]) for the token embedding and the
 * output head, the form of the retained Gemma 2 9B file: the embedding is gathered from the binary16 rows
 * as they are, the head -- given, or tied to such an embedding -- is quantised to Q8_0 on the device
 * (WeightMaterializer::q8_head, gemma2_metal_plan.cpp:310-316; policy :799-828).
 * gf_model_set_matrix_requantized binds a Q6_K matrix as Q4_K (WeightMaterializer::requantized_down,
 * gemma2_metal_plan.cpp:301-308: the 9B file's Q6_K ffn_down). */
GF_API int gf_model_set_matrix_requantized(gf_model* model, int kind, uint32_t layer, const void* native_q6_k_host,
                                           uint64_t k, uint64_t n);
/* ---- optional tensor parallelism for one stream's latency.  No counterpart in the reference (one device).  A
 * shard is an ordinary plan built on 1 / G of the query and KV heads, of the FFN width and of the head's
 * vocabulary: Q/K/V, gate and up are split by output column, O and down by input row, so a shard's O and down
 * projections leave PARTIAL sums of the full hidden vector.  The plan calls `hook(user, buffer_dev, count,
 * stream)` behind each of them (2 x layers times per pass); the host sums the buffers of all shards in place,
 * in stream order -- an NCCL all-reduce over NVLink in the multi-process bench, any fixed-order sum elsewhere.
 * The hook is recorded into the plan's CUDA graphs when what it enqueues can be captured (NCCL can).
 * gf_model_set_token_table_vocab lets the token embedding cover the full vocabulary while the head (config.vocab
 * columns, bound as GF_MAT_OUTPUT) is this shard's slice; call it before binding the table.  Candidate ids of a
 * shard are local to its slice. ---- */
typedef int (*gf_reduce_fn)(void* user, float* buffer_dev, uint64_t count, void* stream);
GF_API int gf_model_set_reduce_hook(gf_model* model, gf_reduce_fn hook, void* user);
GF_API int gf_model_set_token_table_vocab(gf_model* model, uint32_t vocab);
/* The same sum without a hook and without a launch of its own: the exchange rides on the projection launches.
 * Each shard owns an arena in its GPU's memory.  The O / down launch mirrors every value it writes into its slot
 * of every peer's arena as an 8-byte (value, stamp) pair -- plain stores over NVLink; the stamp names the pass and
 * the projection -- and the launch that consumes the projection (the next fused Q/K/V, gate/up or head launch)
 * reads its input as the sum of all parts in shard order, so every shard holds the same bits, polling the peers'
 * pairs until they carry the stamp it expects.  The polls are bounded: when they run out the plan's error word is
 * set, the pass goes on with what has arrived and gf_model_status reports GF_ERR_TIMEOUT (the plan is poisoned
 * until gf_model_reset).  Shards are one per
 * GPU and run the same passes in the same order; two shards must never share a GPU (their launches would wait
 * on one another inside one device).
 *   gf_model_shard_prepare      allocates this shard's arena; `ipc_handle_out` (64 bytes, may be null) receives
 *                               the handle another PROCESS maps it with
 *   gf_model_shard_arena        the arena's device pointer (and _bytes its size), for shards that live in one process
 *   gf_model_shard_connect      `arenas[size]`: every shard's arena as addressable in this process (own ignored)
 *   gf_model_shard_connect_ipc  `handles`: size x 64 bytes, every shard's exported handle (own ignored)
 *   gf_model_shard_set_wait_limit  polls (a fraction of a microsecond each) before a wait for a peer's value gives up
 * Connect every shard, and let the host see that all have (a barrier), before the first pass. */
GF_API int gf_model_shard_prepare(gf_model* model, uint32_t rank, uint32_t size, void* ipc_handle_out);
GF_API void* gf_model_shard_arena(gf_model* model);
GF_API size_t gf_model_shard_arena_bytes(gf_model* model);
GF_API int gf_model_shard_connect(gf_model* model, void* const* arenas);
GF_API int gf_model_shard_connect_ipc(gf_model* model, const void* handles);
GF_API int gf_model_shard_set_wait_limit(gf_model* model, uint32_t polls);
/* With global selection a connected shard's gf_model_select / gf_model_read_candidates speak token ids of the whole
 * vocabulary: a request's history tokens go to the shard that owns them, every shard selects in its slice, the
 * candidate rows of all shards are gathered over peer memory and merged on the host -- the same rows on every
 * shard, so one gf_h1 engine per shard (each with its own replica of the drafter, the same options and seeds) runs
 * the speculative cycle in step with the others.  Requests written on the device are not offered in this mode,
 * i.e. engines on shards need a repetition penalty of 1. */
GF_API int gf_model_shard_global_selection(gf_model* model, int enable);
/* Binds every tensor of a GGUF v2/v3 file that the block schedule knows (llama.cpp tensor names,
 * F32 vectors, Q8_0 / Q4_K / Q6_K matrices and binary16 embedding / head tables) through the two calls above: the path's share of
 * read_file_backed_gguf_model (model_format/gguf_reader.hpp:85) and of the WeightMaterializer.
 * The geometry still comes from gf_model_config; *out_bound_tensors (optional) counts the
 * tensors taken.  Call gf_model_finalize afterwards. */
GF_API int gf_model_load_gguf(gf_model* model, const char* path, uint32_t* out_bound_tensors);
/* Checks every tensor is bound and allocates KV rings, private rows and scratch
 * (allocate_kv_cache, gemma2_metal_plan.cpp:514-537). */
GF_API int gf_model_finalize(gf_model* model);
GF_API int gf_model_reset(gf_model* model);
GF_API int gf_model_position(const gf_model* model, uint32_t* out_position);
/* One pass over `rows` chained tokens at positions position..position+rows-1
 * (run_gemma3_resident_decode / run_gemma_target_width_two_verifier,
 * gemma_target_runtime.cpp:390,457): K/V go to private rows, nothing is published.
 * flags: GF_FORWARD_LOGITS computes the final norm and the output head for every row;
 * GF_FORWARD_DEVICE_TOKENS takes the ids already stored in gf_model_tokens_dev().
 * Asynchronous on the model's stream. */
GF_API int gf_model_forward(gf_model* model, const uint32_t* tokens_host, uint32_t rows, uint32_t flags);
/* Publishes private rows 0..rows-1 into the rings and advances the position
 * (publish_contiguous_rows, gemma_target_runtime.cpp:273; provisional commit,
 * target_verifier_runtime.cpp:535).  Rows left unpublished are the rollback. */
GF_API int gf_model_publish(gf_model* model, uint32_t rows);
/* Chunked prompt ingestion through the row path (run_gemma3_resident_prefill semantics,
 * gemma_target_runtime.cpp:420); logits are produced for the last token only. */
GF_API int gf_model_prefill(gf_model* model, const uint32_t* tokens_host, uint32_t count);
GF_API int gf_model_truncate(gf_model* model, uint32_t position);
/* gf_model_prefill ingests prompts of 65 tokens or more in chunks of up to 256 rows, every projection of
 * a chunk as one bf16 tensor-core GEMM (run_gemma3_resident_prefill's 128-row chunks,
 * gemma_target_runtime.cpp:420-455; the last layer of a chunk stops after its K/V rows, :59-61,125), and
 * the last prompt token as an ordinary one-row pass.  K/V rows and logits then differ from the exact row
 * path by the bf16 rounding of activations and weights (about 1e-2 relative L2 on logits).
 * gf_model_use_tensor_prefill(model, 0) keeps every prompt on the exact row path.
 * gf_model_prefill_logits_row: the row of the logits buffer that holds the last prompt token's logits. */
GF_API int gf_model_use_tensor_prefill(gf_model* model, int enable);
GF_API uint32_t gf_model_prefill_logits_row(const gf_model* model);
/* Candidate selection over the last pass's logits; requests_host holds `rows` request rows
 * (gf_selection_request_bytes each).  gf_model_read_candidates synchronises and copies
 * `rows` result rows (gf_candidate_result_bytes each) (read_target_token_candidates). */
GF_API int gf_model_select(gf_model* model, const void* requests_host, uint32_t rows);
GF_API int gf_model_read_candidates(gf_model* model, void* results_host, uint32_t rows);
GF_API int gf_model_read_logits(gf_model* model, uint32_t row, float* logits_host);
/* Committed K and V rows of one layer, positions [first_position, first_position + count), widened
 * to f32: `count` x kv_heads*head_dim values each.  Synchronises.  The rows must still be inside
 * the layer's ring (copy_tensor_from_backend on the plan's cache buffers, backend_buffer.hpp:47-68;
 * the reference's runtime tests read the caches the same way, gemma3_target_runtime_tests.cpp:255-308). */
GF_API int gf_model_read_kv(gf_model* model, uint32_t layer, uint32_t first_position, uint32_t count,
                            float* k_host, float* v_host);
GF_API int gf_model_synchronize(gf_model* model);
/* Synchronises and returns the validation word (bit 1 bad token id, bit 2 bad request,
 * bit 8 non-finite F16 K/V, bit 16 a position beyond the bound context; read_verifier_status)
 * and GF_ERR_TIMEOUT / GF_ERR_NUMERIC / GF_ERR_STATE. */
GF_API int gf_model_status(gf_model* model, uint32_t* out_status);
GF_API void* gf_model_stream(gf_model* model);
GF_API uint32_t* gf_model_tokens_dev(gf_model* model);
GF_API float* gf_model_logits_dev(gf_model* model);
GF_API size_t gf_model_weight_bytes(const gf_model* model, int native);
/* K and V bytes one pass has to read at the current position: the committed rows inside every
 * layer's window, once (the rows of a pass share the cache); 0 for rows = 0. */
GF_API size_t gf_model_kv_bytes_per_pass(const gf_model* model, uint32_t rows);
GF_API uint32_t gf_model_kernel_launches(const gf_model* model);
GF_API int gf_model_use_graph(gf_model* model, int enable);
/* How passes of one or two rows (decode, drafting, verification) are scheduled.  mode 0 (default): one
 * kernel per operator with programmatic dependent launch, replayed as a CUDA graph.  mode 1: one
 * persistent "decode pass" kernel, one CTA per SM, walks the whole block schedule of
 * encode_gemma_target_blocks (gemma_target_runtime.cpp:13-221) with grid-wide barriers between its
 * operators and keeps streaming the next matrix's weights while it waits; attention runs inside it for
 * a binary16 cache and as launches of its own between kernel segments otherwise.  mode 2: as 1 with
 * attention always as launches of its own.  All modes compute bit-identical results; mode 0 measured
 * fastest on B200 (a grid barrier costs more than a dependent-launch boundary).  Wider passes (prompt
 * ingestion) never use the pass kernel. */
GF_API int gf_model_use_pass_kernel(gf_model* model, int mode);
/* Enqueues exactly the weight-streaming GEMVs of one `rows`-row pass (every projection of every
 * layer and the output head, in schedule order) and nothing else: the measurement the
 * reference's quick benchmark calls "effective weight GB/s"
 * (include/local_gguf_engine/benchmarks/quick_benchmark.hpp:24-30).  Scratch activations are
 * reused as inputs; results are not meaningful. */
GF_API int gf_model_weight_sweep(gf_model* model, uint32_t rows, uint32_t* out_launches, uint64_t* out_weight_bytes);

/* ---- independent conversation streams on one GPU.  No counterpart as a type in the reference, which decodes
 * one conversation per process; each row of a step computes the reference's decode graph
 * (run_gemma2_metal_resident_decode_step, src/engine/gemma2_runtime.cpp:250-418; block schedule
 * gemma_target_runtime.cpp:13-221) for its own conversation.  `count` KV caches shaped like the plan's own share
 * the plan's weights; a decode step takes one token per stream and runs the streams in groups of up to
 * row_capacity rows, so the weights are streamed once per group instead of once per stream, while every row is
 * rotated at its stream's position, attends its stream's rings and is published into them.  A stream's results
 * do not depend on which streams share its pass.  Streams are the unit that is spread over the GPUs of a node:
 * one process and one replica of the weights per GPU, no collective.
 * gf_streams_prefill ingests a prompt into one stream through gf_model_prefill's paths (its last token's logits
 * become that stream's row); gf_streams_decode leaves logits for every stream, gf_streams_select /
 * gf_streams_read_candidates run candidate selection over all rows (`count` request / result rows). ---- */
typedef struct gf_streams gf_streams;
GF_API int gf_streams_create(gf_model* model, uint32_t count, gf_streams** out_streams);
GF_API int gf_streams_destroy(gf_streams* streams);
GF_API uint32_t gf_streams_count(const gf_streams* streams);
GF_API int gf_streams_prefill(gf_streams* streams, uint32_t stream, const uint32_t* tokens_host, uint32_t count);
GF_API int gf_streams_decode(gf_streams* streams, const uint32_t* tokens_host /* one id per stream */);
/* How a step computes its projections.  0 (default): the exact row passes described above.  1: ONE pass over
 * all streams of the set (at most 256) whose projections are the prompt path's bf16 tensor-core GEMMs
 * (gf_prefill_matmul): the weights are read and dequantised once per step however many streams there are,
 * and results differ from mode 0 by the bf16 rounding of activations and weights (about 1e-2 relative L2 on
 * logits), the trade the reference makes for its Gemma 2 prompt path (gemma2_runtime.cpp:893-1170). */
GF_API int gf_streams_set_mode(gf_streams* streams, int mode);
GF_API int gf_streams_select(gf_streams* streams, const void* requests_host);
GF_API int gf_streams_read_candidates(gf_streams* streams, void* results_host);
GF_API int gf_streams_read_logits(gf_streams* streams, uint32_t stream, float* logits_host);
GF_API int gf_streams_position(const gf_streams* streams, uint32_t stream, uint32_t* out_position);
/* K and V bytes one decode step reads at the streams' current positions. */
GF_API size_t gf_streams_kv_bytes_per_step(const gf_streams* streams);

/* ---- drafter proposal law: the device sampler of Gemma3DraftPlan::propose and the receipts
 * Gemma3DraftPlan::gather reads (src/engine/gemma3_draft.mm:995-1167,1528-1581; kernels :191-294).
 * Compact law (temperature > 0 and 1 <= top_k <= 64, or a greedy drafter): support = every token whose
 * processed score reaches the top_k-th best, filtered by the ascending-tail top-p rule and min-p,
 * integer CDF of total 2^32 in token-id order; the drafted token is the bin holding `word`.
 * Receipt (device): { u32 status; u32 count; u32 token; u32 word; u32 ids[256]; u64 cdf[257] }.
 * status 20 = the support holds more than 256 tokens: no token was drafted, and the caller builds the
 * full-vocabulary law from the same scores with gf_draft_resolve_overflow (same workspace, same word).
 * Full-vocabulary law (gd_full_merge .. gd_select, gemma3_draft.mm:295-395): taken at once when top_k
 * is 0 or above 64, and by gf_draft_resolve_overflow.  Its receipt has count = 0xffffffff and only the
 * four leading words; the CDF (vocab + 1 bounds, total 2^32) stays inside the workspace and
 * gf_draft_gather_full returns the [begin, end) bounds of up to 257 tokens (2 * count words;
 * synchronises the stream): the non-compact branch of Gemma3DraftPlan::gather (:1528-1581). ---- */
GF_API size_t gf_draft_receipt_bytes(void);
GF_API size_t gf_draft_sample_workspace_bytes(uint32_t vocab);
GF_API int gf_draft_sample(const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k,
                           float top_p, float min_p, float repetition_penalty,
                           const uint32_t* history_host, uint32_t history_count, uint32_t word,
                           void* workspace_dev, void* receipt_dev, uint32_t* out_token_dev, void* stream);
GF_API int gf_draft_resolve_overflow(uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                                     uint32_t word, void* workspace_dev, void* receipt_dev,
                                     uint32_t* out_token_dev, void* stream);
GF_API int gf_draft_gather_full(void* workspace_dev, uint32_t vocab, const uint32_t* tokens_host, uint32_t count,
                                uint64_t* intervals_host, void* stream);

/* ---- host sampler and lossless acceptance: TokenSampler / TokenSamplerFork
 * (include/local_gguf_engine/engine/sampling.hpp:184-395, src/engine/sampling.cpp).  Double
 * precision on the host, two mt19937_64 streams; decisions are bit-identical to the reference
 * for identical candidates, draft masses and seed. ---- */
typedef struct gf_sampler gf_sampler;
typedef struct gf_sampler_options {      /* TokenSamplerOptions (sampling.hpp:184-196) */
    float temperature;
    uint32_t top_k;
    float top_p, min_p, repetition_penalty;
    uint32_t repetition_window;
    uint64_t seed;
} gf_sampler_options;
typedef struct gf_token_logit { uint32_t token; float logit; } gf_token_logit;   /* TokenLogit (sampling.hpp:25-28) */
typedef struct gf_gathered_draft {       /* GatheredDraftTokenDistribution (sampling.hpp:150-156) */
    uint32_t proposal;
    uint32_t count;
    uint64_t proposal_mass, proposal_cdf_begin;
    uint64_t target_mass[256];           /* draft mass of the i-th token of the prepared target support */
} gf_gathered_draft;
GF_API int gf_sampler_create(const gf_sampler_options* options, gf_sampler** out_sampler);
GF_API int gf_sampler_destroy(gf_sampler* sampler);
GF_API int gf_sampler_observe(gf_sampler* sampler, const uint32_t* tokens, uint32_t count);    /* observe_tokens */
GF_API int gf_sampler_preview_proposal_word(const gf_sampler* sampler, uint32_t* out_word);   /* preview_proposal_words(1) */
/* The next `count` (<= 23, the reference's largest horizon) words of the proposal stream without consuming them:
 * word i is the one the i-th acceptance test of a cycle will check (preview_proposal_words, sampling.cpp:62-80,936). */
GF_API int gf_sampler_preview_proposal_words(const gf_sampler* sampler, uint32_t count, uint32_t* out_words);
/* prepare_distribution (sampling.cpp:394-499) for the row whose context is the observed history
 * plus `suffix`: writes the support tokens and their sampling weights. */
GF_API int gf_sampler_prepare(const gf_sampler* sampler, const gf_token_logit* candidates, uint32_t count,
                              const uint32_t* suffix, uint32_t suffix_count, uint32_t* out_tokens,
                              double* out_weights, uint32_t* out_count, double* out_total_weight);
GF_API int gf_sampler_sample(gf_sampler* sampler, const gf_token_logit* candidates, uint32_t count,
                             const uint32_t* suffix, uint32_t suffix_count, uint32_t* out_token);   /* TokenSampler::sample */
/* TokenSamplerFork::sample_speculative with a gathered draft law (sampling.cpp:896-934). */
GF_API int gf_sampler_sample_speculative(gf_sampler* sampler, const gf_gathered_draft* draft,
                                         const gf_token_logit* candidates, uint32_t count,
                                         const uint32_t* suffix, uint32_t suffix_count, uint32_t* out_token,
                                         int* out_accepted, uint32_t* out_target_draws);

/* ---- the speculative cycle: draft -> verify -> accept / rollback.  Replaces StandaloneChatPlan::run
 * (src/engine/standalone_chat.cpp:508-615), ChainChatVerifier::run for one tile of `horizon` drafts and
 * horizon + 1 rows (src/engine/chain_chat.mm:245-543; the unconditional schedule of :64-93) and the
 * speculative branch of the generation loop (src/engine/gemma2_runtime.cpp:1630-1699).  horizon = 1 is
 * the H1 cycle; horizons up to GF_MAX_ROWS - 1 draft a chain of tokens, verify them in one pass of the
 * target and keep the accepted prefix (the drafter rolls back behind it).  One host synchronisation per
 * cycle: with a repetition penalty the selection requests, which name the drafted tokens, are written on
 * the device. ---- */
typedef struct gf_h1 gf_h1;
typedef struct gf_h1_options {
    gf_sampler_options sampler;          /* target sampler; the drafter reuses it (standalone_chat.cpp:11-32) */
    int32_t speculative;                 /* 0: ordinary decode with the target only */
    int32_t forced_schedule;             /* 1: accept/reject control flow follows a seeded Bernoulli schedule
                                            while the real acceptance law still runs and is recorded */
    float forced_accept_probability;
    uint64_t schedule_seed;
    int32_t record_cycles;               /* keep the inputs of every acceptance test for exactness checks */
    uint32_t horizon;                    /* drafts per cycle, 1..GF_MAX_ROWS-1 (0 = 1); the target plan needs
                                            horizon + 1 rows per pass, the drafter max(2, horizon) */
    int32_t conditional;                 /* 1: verify a cycle's drafts as a cascade of passes, each run only when every
                                            draft before it was accepted (chain_chat.mm:63-88; partitions of
                                            make_registered_conditional_chain_schedule, speculative_controller.cpp:590-623:
                                            3 = 2 + 1, 4 = 2 + 2, 7 = 4 + 3, pairs otherwise).  Same tokens as the single
                                            pass, fewer rows after an early rejection, one more pass and host wait per tile */
} gf_h1_options;
typedef struct gf_h1_stats {
    uint64_t cycles, accepted, rejected, ordinary_steps, fallback_cycles, emitted_tokens;
    uint64_t law_agreements;             /* cycles whose real decision equals the forced one (forced mode) */
    uint64_t sampler_launches;           /* kernels of the drafter's device sampler (three per proposal); the plans count
                                            their own in gf_model_kernel_launches */
    uint64_t drafted_tokens, accepted_tokens;   /* over all cycles; accepted / rejected count whole cycles */
    uint64_t full_law_proposals;         /* proposals drawn from the full-vocabulary law; fallback_cycles counts the
                                            verification passes repeated after a compact law overflowed */
    uint64_t verify_passes;              /* target passes run by speculative cycles (one per cycle; one per tile reached
                                            under a conditional schedule) */
} gf_h1_stats;
typedef struct gf_h1_cycle_record {      /* inputs and result of one real acceptance test (`root` = the row's input token) */
    uint32_t root, proposal, word, candidate_count;
    gf_token_logit candidates[384];
    gf_gathered_draft draft;
    uint32_t token;
    int32_t accepted;
    uint32_t target_draws;
    int32_t status;
    uint32_t depth, horizon;             /* this test's place in its cycle's chain (0 = the root's row) and the cycle's drafts */
} gf_h1_cycle_record;
/* The verification passes of a cycle with `horizon` drafts: tile t tests out_drafts[t] drafts in a pass of
 * out_rows[t] rows (at most four tiles; ChainVerifierSchedule, speculative_controller.hpp). */
GF_API int gf_h1_verification_schedule(uint32_t horizon, int conditional, uint32_t* out_drafts, uint32_t* out_rows,
                                       uint32_t* out_tiles);
GF_API int gf_h1_create(gf_model* target, gf_model* draft /* may be NULL when speculative == 0 */,
                        const gf_h1_options* options, gf_h1** out_engine);
GF_API int gf_h1_destroy(gf_h1* engine);
/* Ingests the prompt into both models and samples the first token from the target. */
GF_API int gf_h1_prefill(gf_h1* engine, const uint32_t* tokens_host, uint32_t count);
/* Generates until `max_tokens` tokens have been emitted (the first emitted token is the one
 * sampled by prefill).  Returns the tokens and the number written. */
GF_API int gf_h1_generate(gf_h1* engine, uint32_t max_tokens, uint32_t* out_tokens, uint32_t* out_count);
/* Same, but stops after `steps` cycles (or ordinary steps) as well. */
GF_API int gf_h1_generate_steps(gf_h1* engine, uint32_t steps, uint32_t max_tokens, uint32_t* out_tokens,
                                uint32_t* out_count);
GF_API int gf_h1_stats_read(const gf_h1* engine, gf_h1_stats* out_stats);
/* Restarts the forced accept/reject schedule (options.forced_schedule) from `seed`, so that two
 * measured loops see the same sequence of scheduled outcomes.  Benchmark control only. */
GF_API int gf_h1_reseed_schedule(gf_h1* engine, uint64_t seed);
GF_API int gf_h1_cycle_record_read(const gf_h1* engine, uint32_t index, gf_h1_cycle_record* out_record);
GF_API uint32_t gf_h1_cycle_record_count(const gf_h1* engine);

#ifdef __cplusplus
}
#endif
#endif
