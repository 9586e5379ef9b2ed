// Prompt ingestion as a dense contraction on the fifth-generation tensor cores (tcgen05 + TMEM).
//
// A chunk of up to 256 prompt rows goes through each projection as ONE GEMM
//     C[256, N] = A[256, K] (bf16 activations) x deq(W)[N, K]^T (bf16, dequantised in shared memory)
// issued as two M = 128 products per dequantised weight tile (one accumulator per half of the rows), so the
// quantised weights are read and dequantised once per 256 rows instead of once per row pair
// (run_gemma3_resident_prefill, src/engine/gemma_target_runtime.cpp:420-455; the reference's matrix
// kernel is gemma3_matmul_f32_kquant_matrix_impl, metal_kernels.mm:1031-1199).
//
// Operands in shared memory use the tensor core's K-major layout without swizzle: a "core matrix" is
// 8 rows x 16 bytes (8 bf16 along K) stored as 128 contiguous bytes; inside a block of 64 K elements
// the core matrices of one 8-row group lie 128 bytes apart along K and the row groups 1024 bytes apart.
// The activations are kept in global memory already in that order ("tile-major": one 16-KB block per
// 64 K elements holding all 128 rows), so a CTA fetches a block with one bulk copy.
#pragma once

#include "common.cuh"

namespace gf {

constexpr uint32_t kPrefillHalf = 128;          // M of the tensor-core instruction
constexpr uint32_t kPrefillRows = 256;          // rows of one chunk: two accumulators share every dequantised weight tile
constexpr uint32_t kPrefillTile = 128;          // output columns per CTA
constexpr uint32_t kPrefillBlockK = 64;         // K elements per shared-memory stage
constexpr uint32_t kPrefillThreads = 576;          // sixteen dequantising warps, the warp that issues the products and the warp that requests the copies
constexpr uint32_t kPrefillBlockBytes = kPrefillRows * kPrefillBlockK * 2u;      // one tile-major activation block

// Byte offset of element (row, k) in a tile-major bf16 activation buffer.
__host__ __device__ inline size_t tile_major_offset(uint32_t row, uint32_t k) {
    return (size_t)(k / kPrefillBlockK) * kPrefillBlockBytes + (row / 8u) * 1024u + ((k % kPrefillBlockK) / 8u) * 128u
           + (row % 8u) * 16u + (k % 8u) * 2u;
}
inline size_t tile_major_bytes(uint64_t k) { return (size_t)((k + kPrefillBlockK - 1u) / kPrefillBlockK) * kPrefillBlockBytes; }

// Rows a chunk of `rows` occupies in operands and results: whole halves.
__host__ __device__ inline uint32_t prefill_padded_rows(uint32_t rows) { return (rows + kPrefillHalf - 1u) / kPrefillHalf * kPrefillHalf; }

struct PrefillMatrix {
    const uint8_t* weight;      // streaming layout (the same bytes the decode kernels read)
    float* out;                 // [padded rows][n] f32
    uint32_t n, dtype, first_tile;
};

struct PrefillGemmParams {
    PrefillMatrix m[3];
    uint32_t matrices, tiles;   // tiles over all matrices (n / kPrefillTile each)
    uint32_t k, units, unit_elems;
    const uint8_t* a;           // tile-major bf16 activations, `k` wide
    int* error_flag;
    uint32_t halves;            // 1 or 2: halves of the chunk that hold rows
};

struct PrefillGemmLaunch {
    struct Matrix { int dtype; const void* packed; float* out; uint64_t n; } matrices[3];
    uint32_t count = 1;
    uint64_t k = 0;
    const void* a = nullptr;
    uint32_t splits = 1;       // K is cut into this many parts; part s writes its rows at out + s * kPrefillRows * n
    uint32_t rows = kPrefillRows;      // rows of the chunk (results are written for whole halves)
};
constexpr uint32_t kPrefillMaxSplits = 4;
int launch_prefill_gemm(const PrefillGemmLaunch& launch, int* error_flag, cudaStream_t stream);
// K splits that finish a launch of n output columns (over all its matrices) in the fewest waves of CTAs.
uint32_t prefill_gemm_splits(uint64_t n, uint64_t k, int dtype);

// Elementwise steps between the GEMMs, each writing the next GEMM's tile-major bf16 operand.
// mode 0: a = rmsnorm(x; gamma1)
// mode 1: r = residual + rmsnorm(x; gamma0) -> residual_out;  a = rmsnorm(r; gamma1)     (gamma1 null: only residual_out)
// x is the sum, in split order, of `splits` partial results laid [split][kPrefillRows][k].
int launch_prefill_norm(const float* x, uint32_t splits, const float* residual, const float* gamma0, const float* gamma1,
                        float* residual_out, void* a_out, uint32_t rows, uint32_t k, float eps, int mode, cudaStream_t stream);
// a = gelu_tanh(gate) * up, gate and up each the sum of `splits` partial results
int launch_prefill_geglu(const float* gate, const float* up, uint32_t splits, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream);
// x[i][0][row][:] = sum over splits of x[i][split][row][:], for `count` <= 3 matrices of n[i] columns
int launch_prefill_reduce(float* const* x, const uint64_t* n, uint32_t count, uint32_t splits, uint32_t rows, cudaStream_t stream);
// Attention of a chunk's rows over ring + private rows of a binary16 cache with 256-wide heads (f32 output
// [rows][heads * 256]); other shapes go through the row kernels (launch_attention).
bool prefill_attention_supported(const struct AttentionParams& p);
int launch_prefill_attention(const struct AttentionParams& p, cudaStream_t stream);
// a = x (f32 rows of width k)
int launch_prefill_pack(const float* x, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream);

}  // namespace gf
