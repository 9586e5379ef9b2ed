// Resident Gemma model plan: packed weights, KV rings + private rows, scratch, and the block
// schedule.  One class serves the 12B target, the Gemma 2 target and the 270M drafter; they
// differ only in configuration (weight types, KV precision, RoPE, softcaps, QK norm).
#pragma once

#include "common.cuh"
#include "ops.cuh"
#include "pass.cuh"
#include "prefill.cuh"

#include <memory>
#include <string>
#include <vector>

namespace gf {

struct PackedMatrix {
    int dtype = 0;
    uint64_t k = 0, n = 0;
    uint8_t* data = nullptr;     // streaming layout, device
    size_t bytes = 0;
    size_t native_bytes = 0;
};

struct LayerWeights {
    PackedMatrix q, k, v, o, gate, up, down;
    float *attn_norm = nullptr, *post_attention_norm = nullptr, *ffn_norm = nullptr, *post_ffw_norm = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr;
};

struct LayerCache {
    void *ring_k = nullptr, *ring_v = nullptr;        // [ring_rows][kv_width]
    void *private_k = nullptr, *private_v = nullptr;  // [row_capacity][kv_width]
    uint32_t ring_rows = 0;                           // power of two (gemma2_metal_plan.cpp:356-366)
    uint32_t window = 0;                              // 0 = global layer
    float rope_base = 0.0f, rope_scale = 1.0f;
    const double* rope_divisors = nullptr;            // [head_dim / 2] rope_base^(2i / head_dim)
    const float2* rope_rotation = nullptr;            // [context + GF_MAX_ROWS][head_dim / 2] (cos, sin) per position
};

enum ForwardFlags : uint32_t {
    kForwardLogits = 1u,        // final norm + output head for every row
    kForwardDeviceTokens = 2u,  // token ids are already in the device token buffer
};

// KV caches of independent conversation streams that share one plan's weights (streams.cu).
constexpr uint32_t kMaxStreams = 256;
struct StreamSet {
    uint32_t count = 0;
    std::vector<std::vector<void*>> ring_k, ring_v;       // [stream][layer], shaped like the plan's own rings
    std::vector<uint32_t> positions_host;
    uint32_t* positions_dev = nullptr;                     // [count]
    StreamRings* rings_dev = nullptr;                      // [layer][count]
    StreamPublishLayer* publish_layers_dev = nullptr;      // [layer]: the plan's private rows
    StreamPublishLayer* wide_publish_layers_dev = nullptr; // [layer]: the private rows of the 128-row arena (tensor-core steps)
    float* logits = nullptr;                               // [max(count, 128)][vocab]
    int mode = 0;                                          // 0: exact row passes in groups; 1: one tensor-core pass over all streams
    cudaGraphExec_t wide_graph = nullptr;
    uint32_t wide_launches = 0;
    void *candidates_ws = nullptr, *requests_dev = nullptr, *results_dev = nullptr, *requests_pinned = nullptr;
    std::vector<void*> allocations;
    // One recorded CUDA graph per group of streams (a group's pointers are fixed): [group] -> executable, rows.
    std::vector<cudaGraphExec_t> group_graphs;
    std::vector<uint32_t> group_launches;
    ~StreamSet();
};

class Model {
public:
    explicit Model(const gf_model_config& config);
    ~Model();
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    int set_matrix(int kind, uint32_t layer, int dtype, const void* native_host, uint64_t k, uint64_t n, bool requantize = false);
    int set_vector(int kind, uint32_t layer, const float* host, uint32_t count);
    int finalize();

    int reset();
    int forward(const uint32_t* tokens_host, uint32_t rows, uint32_t flags);
    int publish(uint32_t rows);
    int select(const void* requests_host, uint32_t rows);
    int read_candidates(void* results_host, uint32_t rows);
    int read_logits(uint32_t row, float* host);
    int read_kv(uint32_t layer, uint32_t first_position, uint32_t count, float* k_host, float* v_host);
    int synchronize();
    int status_word(uint32_t* out);
    int prefill(const uint32_t* tokens_host, uint32_t count);
    int truncate(uint32_t position);
    int weight_sweep(uint32_t rows, uint32_t* out_launches, uint64_t* out_bytes);

    const gf_model_config& config() const { return config_; }
    uint32_t position() const { return position_; }
    cudaStream_t stream() const { return stream_; }
    float* logits_dev() const { return logits_; }
    uint32_t* tokens_dev() const { return tokens_dev_; }
    uint32_t* base_position_dev() const { return state_dev_; }
    void* requests_dev() const { return requests_dev_; }
    void* results_dev() const { return results_dev_; }
    size_t weight_bytes() const { return weight_bytes_; }
    size_t native_weight_bytes() const { return native_weight_bytes_; }
    size_t kv_bytes_per_pass(uint32_t rows) const;
    uint32_t kernel_launches() const { return launches_; }
    void set_use_graph(bool on) { use_graph_ = on; }
    // Prompts longer than kTensorPrefillMinRows go through the 128-row tensor-core path (bf16 operands)
    // unless this is switched off; shorter ones, and every prompt then, through the exact row path.
    void set_tensor_prefill(bool on) { tensor_prefill_ = on; }
    // Row of the logits buffer that holds the last prompt token's logits after prefill().
    uint32_t prefill_logits_row() const { return prefill_logits_row_; }
    // 0: kernel-per-matrix schedule only.  1: passes of one or two rows run as the decode pass kernel
    // (attention inside it where it has an instance, as launches of its own between segments otherwise).
    // 2: as 1, but attention always as launches of its own.
    void set_pass_mode(int mode) { if (mode != pass_mode_) invalidate_passes(); pass_mode_ = mode; }

    // Independent streams over this plan's weights (streams.cu).
    int streams_create(uint32_t count, StreamSet** out);
    int streams_prefill(StreamSet& set, uint32_t stream, const uint32_t* tokens_host, uint32_t count);
    int streams_decode(StreamSet& set, const uint32_t* tokens_host);
    int streams_set_mode(StreamSet& set, int mode);
    int streams_select(StreamSet& set, const void* requests_host);
    int streams_read_candidates(StreamSet& set, void* results_host);
    int streams_read_logits(StreamSet& set, uint32_t stream, float* host);
    size_t streams_kv_bytes(const StreamSet& set) const;

    // Tensor-parallel shards: the token table may cover more ids than the (sharded) head, and partial sums
    // behind the O and down projections go through the host's reduction hook.
    int set_token_table_vocab(uint32_t vocab) {
        if (token_embd_.data) return fail(GF_ERR_STATE, "set the token table's vocabulary before binding it");
        if (vocab < config_.vocab) return fail(GF_ERR_INVALID, "the token table cannot be narrower than the head");
        token_table_vocab_ = vocab;
        return GF_OK;
    }
    void drop_graphs() {
        for (auto& per_rows : graphs_)
            for (cudaGraphExec_t& exec : per_rows)
                if (exec) { cudaGraphExecDestroy(exec); exec = nullptr; }
        invalidate_passes();
    }
    int set_reduce_hook(gf_reduce_fn hook, void* user) {
        reduce_hook_ = hook; reduce_user_ = user;
        drop_graphs();
        return GF_OK;
    }
    uint32_t token_vocab() const { return token_table_vocab_ ? token_table_vocab_ : config_.vocab; }
    bool sharded() const { return reduce_hook_ != nullptr || shard_.connected; }
    // The exchange fused into the projection launches (no host hook, no separate reduction launch): every
    // shard owns an arena its peers write into over NVLink.  shard_prepare allocates it (and exports it for
    // other processes), shard_connect takes every shard's arena as mapped in this process, shard_connect_ipc
    // maps the exported ones first.
    int shard_prepare(uint32_t rank, uint32_t size, void* ipc_handle_out);
    void* shard_arena() const { return shard_.arena; }
    size_t shard_arena_bytes() const { return shard_.bytes; }
    int shard_connect(void* const* arenas);
    int shard_connect_ipc(const void* handles);
    void shard_set_wait_limit(uint32_t polls) { shard_.wait_limit = polls; drop_graphs(); }
    // With global selection a connected shard's select / read_candidates speak ids of the whole vocabulary: the
    // request's history tokens go to the shard that owns them, every shard selects in its slice, the candidate rows
    // of all shards are gathered over peer memory and merged on the host (the same merge on every shard, so the
    // shards' samplers stay in step).  Requests written on the device are not offered in this mode.
    int shard_global_selection(bool enable);

    // Enqueues the selection for rows whose requests already sit in requests_dev().
    int select_device(uint32_t rows);
    // Uploads one token id into the device token buffer slot `row` (asynchronous).
    int set_device_token(uint32_t row, uint32_t token);

private:
    // A recorded pass: the phase table on the device and the launches that walk it.  A segment is one
    // pass-kernel launch over phases [first, first + count); `attention` >= 0 names the attention launch
    // that follows it (an index into `attention_launches`).
    struct PassSegment { uint32_t first, count, first_stream, last_stream; int attention; };
    struct RecordedPass {
        bool ready = false, usable = false;
        PassPhase* table_dev = nullptr;
        uint32_t smem_bytes = 0, phases = 0;
        uint64_t weight_bytes = 0;               // of a recorded weight sweep
        std::vector<PassSegment> segments;
        std::vector<AttentionParams> attention_launches;
    };

    int reduce_partial(float* buffer, size_t count);
    int read_candidates_global(void* results_host, uint32_t rows);
    bool selecting_global_ = false;
    // This shard's side of the fused exchange.  Arena: [2 halves][size shards][row_capacity x hidden] stamped
    // (value, stamp) pairs the peers write, then this GPU's pass counter.  The O projections use half 0, the down
    // projections half 1, so consecutive exchanges never share a half; this shard's own part stays in `projected_`.
    struct ShardExchange {
        uint32_t rank = 0, size = 0;
        bool connected = false;
        uint8_t* arena = nullptr;
        uint8_t* mapped[8] = {};          // every shard's arena as addressed from this process (own at [rank])
        bool opened[8] = {};              // mapped from an exported handle: closed with the plan
        size_t part_values = 0, tick_offset = 0, rows_offset = 0, rows_values = 0, bytes = 0;
        bool global_selection = false;
        uint32_t gathers = 0;             // gathers so far: their stamp, and the parity of the slot they use
        uint32_t* gathered_dev = nullptr; // [size][rows_values]
        uint32_t* gathered_host = nullptr;
        std::vector<uint8_t> global_requests;      // the requests of the selection in flight, as the caller gave them
        uint2* rows_slot(uint8_t* base, uint32_t parity, uint32_t shard) const {
            return reinterpret_cast<uint2*>(base + rows_offset) + ((size_t)parity * size + shard) * rows_values;
        }
        uint32_t wait_limit = 1u << 22;   // polls of a fraction of a microsecond: about a second
        uint2* part(uint8_t* base, uint32_t half, uint32_t shard) const {
            return reinterpret_cast<uint2*>(base) + ((size_t)half * size + shard) * part_values;
        }
        uint32_t* tick() const { return reinterpret_cast<uint32_t*>(arena + tick_offset); }
    } shard_;
    void shard_scatter(struct GemvLaunch& launch, uint32_t half, uint32_t site);
    void shard_gather(struct GemvLaunch& launch, uint32_t half, uint32_t site);
    uint32_t token_table_vocab_ = 0;
    gf_reduce_fn reduce_hook_ = nullptr;
    void* reduce_user_ = nullptr;
    int bind_q8_head_from_f16(const void* f16_dev, uint64_t k, uint64_t n);
    int bind_rings(const std::vector<void*>& ring_k, const std::vector<void*>& ring_v, uint32_t position);
    int encode_stream_group(StreamSet& set, uint32_t first, uint32_t rows);
    int encode_stream_batch(StreamSet& set);
    int encode_blocks(uint32_t rows, uint32_t flags);
    int run_gemv(struct GemvLaunch& launch, uint32_t rows);
    int emit_embedding(uint32_t rows, float scale);
    int emit_attention(const AttentionParams& params);
    int run_graph_or_encode(uint32_t rows, uint32_t flags);
    int record_pass(uint32_t rows, uint32_t flags, bool sweep, RecordedPass& out);
    int finish_recording(uint32_t rows, RecordedPass& out);
    int run_recorded(const RecordedPass& pass, uint32_t rows);
    int encode_sweep(uint32_t rows, uint32_t* out_launches, uint64_t* out_bytes);
    bool layer_is_local(uint32_t layer) const;
    int ensure_prefill_arena();
    int prefill_chunk(const uint32_t* tokens_host, uint32_t rows);

    // Buffers of the 128-row prompt path, allocated when a long prompt first arrives.
    struct PrefillArena {
        bool ready = false;
        uint32_t chunk_rows = 0;
        void *a_hidden = nullptr, *a_q = nullptr, *a_ffn = nullptr;            // tile-major bf16 operands
        float *residual = nullptr, *residual2 = nullptr, *raw_q = nullptr, *raw_k = nullptr, *raw_v = nullptr;
        float *query = nullptr, *attention_out = nullptr, *projected = nullptr, *gate = nullptr, *up = nullptr;
        std::vector<void*> private_k, private_v;                               // per layer [128][kv width]
        KvPublishLayer* publish_layers = nullptr;
        void* attention_ws = nullptr;
        uint32_t* tokens = nullptr;
    } prefill_;
    bool tensor_prefill_ = true;
    uint32_t prefill_logits_row_ = 0;

    // Weight upload at load time: native blocks travel through two pinned host chunks into one of two device
    // staging buffers on a copy stream, while the repack of the previous tensor runs on the plan's stream
    // (the reference overlaps source I/O of the next block with packing of the current one,
    // gemma2_metal_plan.cpp:427-461).  Released by finalize().
    struct WeightStager {
        static constexpr size_t kChunkBytes = 32u << 20;
        cudaStream_t copy_stream = nullptr;
        uint8_t* pinned[2] = {nullptr, nullptr};
        cudaEvent_t chunk_done[2] = {nullptr, nullptr};       // the chunk's device copy has read the pinned buffer
        uint8_t* staging[2] = {nullptr, nullptr};
        size_t staging_bytes[2] = {0, 0};
        cudaEvent_t uploaded[2] = {nullptr, nullptr};         // the tensor is complete in staging[i]
        cudaEvent_t packed[2] = {nullptr, nullptr};           // the repack has finished reading staging[i]
        uint32_t next = 0, chunk = 0;
        bool ready = false;
    } stager_;
    int stage_upload(const void* native_host, size_t bytes, uint8_t** out_staging, uint32_t* out_slot);
    void release_stager();

    gf_model_config config_;
    bool finalized_ = false, use_graph_ = true, poisoned_ = false;
    cudaStream_t stream_ = nullptr;
    PackedMatrix token_embd_, head_;
    bool has_head_ = false;
    float* output_norm_ = nullptr;
    std::vector<LayerWeights> layers_;
    std::vector<LayerCache> caches_;
    std::vector<void*> allocations_;
    size_t weight_bytes_ = 0, native_weight_bytes_ = 0;

    // scratch (rows x width), names after target_verifier.hpp:228-257
    float *residual_ = nullptr, *normalized_ = nullptr, *raw_q_ = nullptr, *raw_k_ = nullptr, *raw_v_ = nullptr;
    float *query_ = nullptr, *attention_out_ = nullptr, *projected_ = nullptr, *post_attention_ = nullptr;
    float *gate_ = nullptr, *up_ = nullptr, *gated_ = nullptr, *logits_ = nullptr;
    void *attention_ws_ = nullptr, *matmul_ws_ = nullptr, *candidates_ws_ = nullptr;
    size_t matmul_ws_bytes_ = 0;
    uint32_t* matmul_counters_ = nullptr;
    size_t matmul_counters_bytes_ = 0;
    KvPublishLayer* publish_layers_ = nullptr;
    uint32_t* head_counters_ = nullptr;
    void *requests_dev_ = nullptr, *results_dev_ = nullptr;
    uint32_t *tokens_dev_ = nullptr, *state_dev_ = nullptr, *status_dev_ = nullptr;
    int* error_flag_ = nullptr;
    uint32_t* tokens_pinned_ = nullptr;
    void* requests_pinned_ = nullptr;
    uint32_t position_ = 0;
    uint32_t launches_ = 0;
    cudaGraphExec_t graphs_[GF_MAX_ROWS + 1][2] = {};
    uint32_t graph_launches_[GF_MAX_ROWS + 1][2] = {};      // kernel nodes of each recorded graph
    // Decode pass kernel: recorded tables per (rows, logits), one for the weight sweep per rows.
    int pass_mode_ = 0, recorded_mode_ = -1;
    RecordedPass passes_[kPassMaxRows + 1][2], sweeps_[kPassMaxRows + 1];
    uint32_t* pass_arrived_ = nullptr;
    uint32_t pass_arrivals_ = 0;                             // value of *pass_arrived_ once every launch so far has finished
    uint32_t pass_poll_limit_ = kPassDefaultPollLimit;
    // While a pass is being recorded, the emitters append phases here instead of launching.
    std::vector<PassPhase>* recording_ = nullptr;
    std::vector<int> recording_breaks_;                      // per recorded phase: attention launch that precedes it, or -1
    RecordedPass* recording_pass_ = nullptr;
    bool recording_failed_ = false;
    int pending_break_ = -1;
    void invalidate_passes();
    cudaEvent_t tokens_copied_ = nullptr, requests_copied_ = nullptr;
};

}  // namespace gf

// The opaque handle of the C ABI.
struct gf_model {
    gf::Model impl;
    explicit gf_model(const gf_model_config& c) : impl(c) {}
};
