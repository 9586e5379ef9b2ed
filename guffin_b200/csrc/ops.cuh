// Small fused operators of the Gemma block schedule (everything that is not a weight GEMV).
// All per-pass scalars (committed position, token ids) are read from device memory so that a
// captured CUDA graph can be replayed for every token without re-recording.
#pragma once

#include "common.cuh"

namespace gf {

constexpr int kMaxAttentionPartitions = 32;   // verifier_max_partitions in the reference
constexpr int kAttentionTokensPerPartition = 32;
constexpr int kAttentionWarps = 8;
constexpr int kAttentionBlocksPerSm = 1;      // registers keep one 8-warp block per SM; 4-warp blocks at 2 or 3 per SM measured no faster

// Status bits shared with the reference's validation word
// (metal_kernels.mm:2332,2357,2370,2484; metal_command_context.hpp:17).
enum : uint32_t { kStatusBadToken = 1u, kStatusBadRequest = 2u, kStatusBadHistory = 4u, kStatusKvNonFinite = 8u, kStatusBadPosition = 16u };

struct RopeStoreParams {
    const float* raw_q;        // [rows][heads*hd]
    const float* raw_k;        // [rows][kv_heads*hd]
    const float* raw_v;        // [rows][kv_heads*hd]
    const float* q_norm;       // [hd] or null (no QK norm)
    const float* k_norm;
    float* q_out;              // [rows][heads*hd]
    void* private_k;           // [row_capacity][kv_heads*hd], f16 or f32
    void* private_v;
    const uint32_t* base_position;   // device scalar: position of row 0
    uint32_t* status;
    const double* divisors;    // [hd / 2] freq_base^(2i / hd), or null to compute them in the kernel
    uint32_t rows, heads, kv_heads, head_dim;
    float eps, freq_base, freq_scale;
    int kv_f16;
    const uint32_t* row_positions = nullptr;   // optional [rows]: row r sits at row_positions[r] instead of base + r (rows of different streams)
    uint32_t rotate = 1;                       // 0: norm and store only (the reference's rope_dimension_count = 0)
};

struct AttentionParams {
    const float* q;            // [rows][heads*hd]
    const void* ring_k;        // [ring_rows][kv_heads*hd]
    const void* ring_v;
    const void* private_k;     // [row_capacity][kv_heads*hd]
    const void* private_v;
    float* out;                // [rows][heads*hd]
    float* partial_out;        // [rows][heads][kMaxAttentionPartitions][hd]
    float* partial_ml;         // [rows][heads][kMaxAttentionPartitions][2]
    uint32_t* counters;        // [row groups][kv_heads] partition arrivals, zero between launches
    const uint32_t* base_position;
    uint32_t rows, heads, kv_heads, head_dim;
    uint32_t ring_mask;        // ring_rows - 1
    uint32_t window;           // 0 = global layer
    uint32_t target_parts;     // partitions the launch has room for per (kv head, row group); set by launch_attention
    float scale, softcap;
    int kv_f16;
    // 0: the block that arrives last merges the partitions into `out`.  1: every block parks its
    // partial result and the consumer merges (the GEMV prologue kPrologueMerge); partition slots
    // the launch did not fill are marked empty, `out` and `counters` are not touched.
    uint32_t defer_merge = 0;
};

// Attention workspace: partial outputs, partial (max, sum) pairs, then the arrival counters.
inline size_t attention_workspace_bytes(uint32_t rows, uint32_t heads) {
    return (size_t)rows * heads * kMaxAttentionPartitions * (256u + 2u) * sizeof(float) + (size_t)rows * heads * sizeof(uint32_t);
}
inline uint32_t* attention_counters(void* workspace, uint32_t rows, uint32_t heads) {
    return reinterpret_cast<uint32_t*>(static_cast<float*>(workspace) + (size_t)rows * heads * kMaxAttentionPartitions * (256u + 2u));
}

struct KvPublishLayer {          // one per layer, device resident
    uint8_t *ring_k, *ring_v;
    const uint8_t *private_k, *private_v;
    uint32_t ring_mask, row_bytes;
};
int launch_kv_publish(const KvPublishLayer* layers_dev, uint32_t layer_count, uint32_t* base_position, uint32_t rows,
                      cudaStream_t stream);

int launch_embedding(int dtype, const void* packed, uint32_t k, uint32_t vocab, const uint32_t* tokens,
                     uint32_t rows, float scale, float* out, uint32_t* status, cudaStream_t stream, bool pdl);
int launch_rms_norm(const float* x, const float* gamma, const float* residual, float* out, uint32_t rows,
                    uint32_t hidden, float eps, cudaStream_t stream, bool pdl);
int launch_rope_store(const RopeStoreParams& p, cudaStream_t stream, bool pdl);
int launch_attention(const AttentionParams& p, cudaStream_t stream, bool pdl);

// Rows that belong to different conversation streams: row s of the launch is one query row of stream s, at
// that stream's own position, over that stream's own rings; its private row is row s of private_k / private_v.
// `p` is laid out for p.rows = streams rows (q, out, private rows, workspace); ring pointers come from the table.
struct StreamRings { const void* ring_k; const void* ring_v; };
int launch_stream_attention(const AttentionParams& p, const StreamRings* rings_dev, const uint32_t* positions_dev, cudaStream_t stream);
// Private row r of every layer into ring slot positions[r] & mask of stream r's rings (rings_dev is
// [layer][stride] with the launch's streams starting at column 0), then positions[r] += 1.
struct StreamPublishLayer { const uint8_t *private_k, *private_v; uint32_t ring_mask, row_bytes; };
int launch_stream_publish(const StreamPublishLayer* layers_dev, uint32_t layer_count, const StreamRings* rings_dev, uint32_t stride,
                          uint32_t* positions_dev, uint32_t rows, cudaStream_t stream);
int launch_geglu(const float* gate, const float* up, float* out, uint64_t count, cudaStream_t stream, bool pdl);
int launch_kv_scatter(const void* private_k, const void* private_v, void* ring_k, void* ring_v,
                      const uint32_t* base_position, uint32_t rows, uint32_t row_width, uint32_t ring_mask,
                      int kv_f16, cudaStream_t stream, bool pdl);

// Tensor-parallel shards: the pass counter of the exchange stamps, and the wait for a projection nobody reads.
struct ShardDrain {
    const uint2* parts[7];        // the peers' stamped parts in this GPU's arena
    const uint32_t* tick;
    uint32_t count, site, values, wait_limit;
    int* error_flag;
};
// The exchange of a whole prompt chunk's partial sums (the tensor-core prompt path of a shard): x holds `splits`
// partial results laid [split][slab]; the kernel adds them in split order, mirrors the sums into the peers'
// arenas as stamped pairs, polls (bounded) the peers' pairs of the same values and leaves the total of all
// shards, added in shard order, in split 0.
struct ShardBulk {
    float* x;
    uint32_t splits, slab, values;      // floats between splits; rows x width, a multiple of 4
    uint2* out[7];                      // this shard's slot in each peer's arena
    const uint2* parts[8];              // the peers' slots in this GPU's arena, by shard (own entry unused)
    uint32_t shards, self, peers;
    const uint32_t* tick;
    uint32_t site, wait_limit;
    int* error_flag;
};
int launch_shard_bulk_exchange(const ShardBulk& bulk, cudaStream_t stream);
// Every shard's copy of a few rows of 32-bit words (the candidate rows of a pass), gathered on every shard:
// gathered[shard][word].  Stamped pairs as above; `stamp` is a count the host keeps (the same on every shard).
struct ShardGather {
    const uint32_t* local;
    uint32_t* gathered;
    uint32_t words;
    uint2* out[7];
    const uint2* parts[8];
    uint32_t shards, self, peers, stamp, wait_limit;
    int* error_flag;
};
int launch_shard_gather(const ShardGather& gather, cudaStream_t stream);
int launch_shard_tick(uint32_t* tick, cudaStream_t stream);
int launch_shard_drain(const ShardDrain& drain, cudaStream_t stream, bool pdl);

// Launch helper: optional programmatic stream serialisation (PDL).
template <typename Kernel, typename... Args>
int launch_kernel(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = pdl ? 1 : 0;
    GF_CUDA(cudaLaunchKernelEx(&config, kernel, args...));
    return GF_OK;
}

}  // namespace gf
