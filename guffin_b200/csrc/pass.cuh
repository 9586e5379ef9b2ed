// The decode pass kernel: one persistent launch (one CTA per SM) that walks a device-resident
// table of phases -- embedding, weight-streaming products with their fused prologues, attention --
// with a grid-wide barrier between phases instead of a kernel boundary.  It replaces the
// kernel-per-matrix schedule of encode_gemma_target_blocks (src/engine/gemma_target_runtime.cpp:13-221)
// for passes of one or two rows.
//
// Why: weights never depend on activations, so every warp's bulk-copy ring keeps filling with the
// NEXT matrix's pair rows while the CTA waits for the current phase's activations; no CTA is torn
// down and set up again between matrices; and a pass is one launch instead of 240.
//
// Every wait is bounded: the barrier poll gives up after `poll_limit` reads (or as soon as another
// CTA has set the error word), the CTA then waits -- bounded again -- for its own copies in flight
// and returns; the host reads the error word as GF_ERR_TIMEOUT.
#pragma once

#include "gemv.cuh"
#include "ops.cuh"

namespace gf {

// First word of a table entry.  kPhaseStream (gemv.cuh) = 1.
enum : uint32_t { kPhaseEmbedding = 2u, kPhaseAttention = 3u };

struct EmbeddingPhase {
    const uint8_t* packed;
    const uint32_t* tokens;
    float* out;
    uint32_t* status;
    int32_t dtype;
    uint32_t k, vocab, rows;
    float scale;
};

struct alignas(16) PassPhase {
    uint32_t kind;
    uint32_t attention_group, attention_rows;     // query heads per KV head and rows per block of an attention phase
    uint32_t reserved;
    WeightStreamParams stream;                    // at byte 16 (phase_stream_params)
    AttentionParams attention;
    EmbeddingPhase embedding;
};

constexpr uint32_t kPassDefaultPollLimit = 1u << 21;     // barrier polls before a CTA gives up (well under a second apart)

struct PassLaunch {
    const PassPhase* table_dev = nullptr;   // device copy of the table
    uint32_t first = 0, count = 0;          // phases [first, first + count) run in this launch
    uint32_t first_stream = ~0u, last_stream = ~0u;   // first and last streaming phase among them, counted from `first` (~0: none)
    uint32_t rows = 1;                      // 1 or 2: the kernel instance
    uint32_t smem_bytes = 0;                // pass_smem_bytes of the table
    uint32_t* arrived_dev = nullptr;        // barrier counter: only ever grows, by (count - 1) * SM count per launch
    uint32_t base = 0;                      // its value when this launch starts (the host keeps count; modulo 2^32)
    int* error_flag = nullptr;
    uint32_t poll_limit = kPassDefaultPollLimit;
    uint32_t skip_arrival = ~0u;            // phase after which CTA 0 leaves out its arrival (~0: never; a testing build's fault seam)
};

// Rows a pass kernel instance exists for.
constexpr uint32_t kPassMaxRows = 2;

// Dynamic shared memory a table needs: the ring, then the largest staging area of any phase.
// Returns 0 when a phase does not fit (the caller then keeps the kernel-per-matrix schedule).
uint32_t pass_smem_bytes(const PassPhase* table_host, uint32_t count, uint32_t rows);
// The attention phase's launch geometry for a plan: partitions per (KV head, row group) and whether the
// pass kernel has an instance for it (binary16 cache, at most four query vectors per block).
bool pass_attention_supported(const AttentionParams& p, uint32_t rows, uint32_t& group, uint32_t& rows_per_block, uint32_t& target_parts);
int launch_pass(const PassLaunch& launch, cudaStream_t stream);

}  // namespace gf
