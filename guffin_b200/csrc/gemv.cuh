// Weight-streaming dequant-GEMV core for Q4_K / Q6_K / Q8_0, rows M <= 4.
//
// Work decomposition: an item is (column tile of 8 outputs, K chunk).  A CTA is bound to one
// K chunk and stages that slice of the activation rows in shared memory once; each of its
// warps then streams whole items through a private ring of shared-memory stages filled by
// one-shot TMA bulk copies (cp.async.bulk + mbarrier), so no block-level synchronisation
// happens while weights stream.  A lane owns eight K positions of every unit row and loops
// over the tile's eight columns with the activations held in registers; a unit row's group
// scales are decoded once by the warp (one lane per column x group pair) and exchanged
// through a small shared table.  Row r's arithmetic does not depend on how many rows are
// computed beside it, and partial sums of different K chunks are added in chunk order, so
// results are reproducible and row-count invariant.
#pragma once

#include "common.cuh"

namespace gf {

constexpr int kGemvWarps = 16;       // warps per CTA (one CTA per SM)
constexpr int kGemvStages = 3;       // ring depth per warp
constexpr int kGemvMaxChunkUnits = 16;

__host__ __device__ constexpr int gemv_stage_units(int dtype) { return dtype == GF_Q6_K ? 2 : 3; }
__host__ __device__ constexpr int gemv_table_floats(int dtype) {
    return dtype == GF_Q4_K ? 64 : dtype == GF_Q6_K ? 128 : 32;   // per unit row, per warp
}

struct GemvParams {
    const uint8_t* weight;     // streaming layout
    const float* x;            // [rows][k]
    float* out;                // chunks == 1: y [rows][n]; else partial [chunks][rows][n]
    uint32_t k, n;
    uint32_t units;            // K units per column
    uint32_t tiles;            // ceil(n / 8)
    uint32_t chunks;           // K chunks (gridDim.x is a multiple of this)
    uint32_t chunk_units;      // units per chunk (last chunk may be shorter)
    int* error_flag;           // set to 1 when a bounded wait gives up
};

struct GemvSmemLayout {
    uint32_t xs_bytes, sx_bytes, ring_bytes, table_bytes, total;
};

__host__ __device__ inline GemvSmemLayout gemv_smem_layout(int dtype, int rows, uint32_t chunk_units) {
    GemvSmemLayout s;
    const uint32_t slice = chunk_units * unit_elements(dtype);
    s.xs_bytes = (uint32_t)rows * slice * 4u;
    s.sx_bytes = dtype == GF_Q4_K ? (uint32_t)rows * (slice / 32u) * 4u : 0u;
    s.ring_bytes = (uint32_t)kGemvWarps * kGemvStages * gemv_stage_units(dtype) * unit_row_bytes(dtype);
    s.table_bytes = (uint32_t)kGemvWarps * 2u * gemv_table_floats(dtype) * 4u;
    s.total = s.xs_bytes + s.sx_bytes + s.ring_bytes + s.table_bytes + kGemvWarps * kGemvStages * 8u + 16u;
    return s;
}

#ifdef __CUDACC__

__device__ __forceinline__ float magic_to_float(uint32_t bits, float bias) {
    return __fsub_rn(__uint_as_float(bits), bias);
}

// ---- one unit row (8 columns x one K unit) of each format.  `row` points at the unit row in
// shared memory, `xs` at the activation slice of this unit (row stride `xstride` floats),
// `table` at this warp's scale table for the current parity.

template <int ROWS>
__device__ __forceinline__ void unit_row_q4k(const uint8_t* row, const float* xs, const float* sx,
                                             uint32_t xstride, uint32_t sxstride, float* table,
                                             uint32_t lane, float (&acc)[ROWS][8], float (&macc)[ROWS]) {
    // Phase A: lane (col, pair) decodes the two 6-bit scales and mins of groups 2*pair, 2*pair+1.
    {
        const uint32_t col = lane & 7u, pair = lane >> 3;
        const uint4 hdr = *reinterpret_cast<const uint4*>(row + 1024u + col * 16u);
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const uint32_t sh = (pair & 1u) * 16u;
        const uint32_t a = (hdr.y >> sh) & 0xffffu, b = (hdr.z >> sh) & 0xffffu, c = (hdr.w >> sh) & 0xffffu;
        const bool upper = pair >= 2u;
        const uint32_t sc = upper ? ((c & 0x0f0fu) | ((a >> 2) & 0x3030u)) : (a & 0x3f3fu);
        const uint32_t mn = upper ? (((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u)) : (b & 0x3f3fu);
        float2 ds;
        ds.x = __fmul_rn(d, (float)(sc & 0xffu));
        ds.y = __fmul_rn(d, (float)(sc >> 8));
        *reinterpret_cast<float2*>(table + (col * 4u + pair) * 2u) = ds;
        const float m0 = __fmul_rn(dmin, (float)(mn & 0xffu)), m1 = __fmul_rn(dmin, (float)(mn >> 8));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float2 s = *reinterpret_cast<const float2*>(sx + r * sxstride + pair * 2u);
            macc[r] = fmaf(m0, s.x, fmaf(m1, s.y, macc[r]));
        }
    }
    __syncwarp();
    // Phase B: lane (chunk c, word i) owns nibbles of elements 64c+4i+j (low) and 64c+32+4i+j (high).
    const uint32_t c = lane >> 3, i = lane & 7u;
    float xl[ROWS][4], xh[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const float4 lo = *reinterpret_cast<const float4*>(xs + r * xstride + c * 64u + i * 4u);
        const float4 hi = *reinterpret_cast<const float4*>(xs + r * xstride + c * 64u + 32u + i * 4u);
        xl[r][0] = lo.x; xl[r][1] = lo.y; xl[r][2] = lo.z; xl[r][3] = lo.w;
        xh[r][0] = hi.x; xh[r][1] = hi.y; xh[r][2] = hi.z; xh[r][3] = hi.w;
    }
    const uint32_t* qs = reinterpret_cast<const uint32_t*>(row);
    constexpr uint32_t kMagic = 0x4B000000u;   // 2^23: the nibble lands in the low mantissa bits
    constexpr float kBias = 8388608.0f;
#pragma unroll
    for (int col = 0; col < 8; ++col) {
        const uint32_t w = qs[col * 32 + lane];
        const uint32_t w2 = w >> 16;
        const float2 ds = *reinterpret_cast<const float2*>(table + (col * 4u + c) * 2u);
        // Activations were pre-scaled by 2^-bitpos of their nibble, so q * 2^bitpos * x' = q * x exactly.
        const float l0 = magic_to_float((w & 0x0000000fu) | kMagic, kBias);
        const float l1 = magic_to_float((w & 0x00000f00u) | kMagic, kBias);
        const float l2 = magic_to_float((w2 & 0x0000000fu) | kMagic, kBias);
        const float l3 = magic_to_float((w2 & 0x00000f00u) | kMagic, kBias);
        const float h0 = magic_to_float((w & 0x000000f0u) | kMagic, kBias);
        const float h1 = magic_to_float((w & 0x0000f000u) | kMagic, kBias);
        const float h2 = magic_to_float((w2 & 0x000000f0u) | kMagic, kBias);
        const float h3 = magic_to_float((w2 & 0x0000f000u) | kMagic, kBias);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float lo = fmaf(xl[r][3], l3, fmaf(xl[r][2], l2, fmaf(xl[r][1], l1, xl[r][0] * l0)));
            const float hi = fmaf(xh[r][3], h3, fmaf(xh[r][2], h2, fmaf(xh[r][1], h1, xh[r][0] * h0)));
            acc[r][col] = fmaf(ds.x, lo, fmaf(ds.y, hi, acc[r][col]));
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void unit_row_q6k(const uint8_t* row, const float* xs, uint32_t xstride,
                                             float* table, uint32_t lane, float (&acc)[ROWS][8]) {
    {   // Phase A: lane (col, part) turns int8 sub-scales 4*part..4*part+3 into d*scale.
        const uint32_t col = lane & 7u, part = lane >> 3;
        const uint32_t s4 = *reinterpret_cast<const uint32_t*>(row + 1536u + col * 16u + part * 4u);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + 1664u + col * 2u)));
        const uint32_t h = part >> 1, ab = part & 1u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float s = (float)(int)(signed char)((s4 >> (8 * j)) & 0xffu);
            table[col * 16u + (h * 4u + j) * 2u + ab] = __fmul_rn(d, s);
        }
    }
    __syncwarp();
    // Phase B: lane (half h, plane p, word i): elements h*128+32p+4i+j (low nibble, high bits 2p)
    // and h*128+32(p+2)+4i+j (high nibble, high bits 2p+4); each set lies in one 16-wide group.
    const uint32_t h = lane >> 4, p = (lane >> 3) & 1u, i = lane & 7u;
    float xa[ROWS][4], xb[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const float4 a = *reinterpret_cast<const float4*>(xs + r * xstride + h * 128u + p * 32u + i * 4u);
        const float4 b = *reinterpret_cast<const float4*>(xs + r * xstride + h * 128u + p * 32u + 64u + i * 4u);
        xa[r][0] = a.x; xa[r][1] = a.y; xa[r][2] = a.z; xa[r][3] = a.w;
        xb[r][0] = b.x; xb[r][1] = b.y; xb[r][2] = b.z; xb[r][3] = b.w;
    }
    const uint32_t* ql = reinterpret_cast<const uint32_t*>(row);
    const uint32_t* qh = reinterpret_cast<const uint32_t*>(row + 1024u);
    constexpr uint32_t kMagic = 0x4B000000u;
    constexpr float kBias = 8388608.0f + 32.0f;      // removes the magic exponent and the -32 offset
    const uint32_t shift = p * 2u;
#pragma unroll
    for (int col = 0; col < 8; ++col) {
        const uint32_t wl = ql[col * 32 + h * 16u + p * 8u + i];
        const uint32_t wh = qh[col * 16 + h * 8u + i] >> shift;
        const uint32_t va = (wl & 0x0f0f0f0fu) | ((wh << 4) & 0x30303030u);
        const uint32_t vb = ((wl >> 4) & 0x0f0f0f0fu) | (wh & 0x30303030u);
        const float2 ds = *reinterpret_cast<const float2*>(table + col * 16u + ((h * 2u + p) * 2u + (i >> 2)) * 2u);
        float qa[4], qb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            qa[j] = magic_to_float(__byte_perm(va, kMagic, 0x7540 + j), kBias);
            qb[j] = magic_to_float(__byte_perm(vb, kMagic, 0x7540 + j), kBias);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float da = fmaf(xa[r][3], qa[3], fmaf(xa[r][2], qa[2], fmaf(xa[r][1], qa[1], xa[r][0] * qa[0])));
            const float db = fmaf(xb[r][3], qb[3], fmaf(xb[r][2], qb[2], fmaf(xb[r][1], qb[1], xb[r][0] * qb[0])));
            acc[r][col] = fmaf(ds.x, da, fmaf(ds.y, db, acc[r][col]));
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void unit_row_q80(const uint8_t* row, const float* xs, uint32_t xstride,
                                             float* table, uint32_t lane, float (&acc)[ROWS][8]) {
    {   // Phase A: lane (col, block) widens the block's f16 scale.
        const uint32_t col = lane & 7u, block = lane >> 3;
        table[col * 4u + block] = __half2float(__ushort_as_half(
            *reinterpret_cast<const unsigned short*>(row + 1024u + col * 8u + block * 2u)));
    }
    __syncwarp();
    const uint32_t block = lane >> 3;
    float xv[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(xs + r * xstride + lane * 4u);
        xv[r][0] = v.x; xv[r][1] = v.y; xv[r][2] = v.z; xv[r][3] = v.w;
    }
    const uint32_t* q = reinterpret_cast<const uint32_t*>(row);
    constexpr uint32_t kMagic = 0x4B000000u;
    constexpr float kBias = 8388608.0f + 128.0f;     // int8 + 128 was made unsigned by flipping bit 7
#pragma unroll
    for (int col = 0; col < 8; ++col) {
        const uint32_t w = q[col * 32 + lane] ^ 0x80808080u;
        const float d = table[col * 4u + block];
        float qv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) qv[j] = magic_to_float(__byte_perm(w, kMagic, 0x7540 + j), kBias);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float dot = fmaf(xv[r][3], qv[3], fmaf(xv[r][2], qv[2], fmaf(xv[r][1], qv[1], xv[r][0] * qv[0])));
            acc[r][col] = fmaf(d, dot, acc[r][col]);
        }
    }
}

// Stages this CTA's K slice of the activation rows: xs (Q4_K: scaled by 2^-bitpos of the
// element's nibble) and, for Q4_K, the per-32 sums the min term needs.
template <int DTYPE, int ROWS>
__device__ __forceinline__ void stage_activations(const float* __restrict__ x, uint32_t k, uint32_t first,
                                                  uint32_t count, uint32_t slice, float* xs, float* sx) {
    for (uint32_t e = threadIdx.x; e < (uint32_t)ROWS * slice; e += blockDim.x) {
        const uint32_t r = e / slice, o = e % slice;
        float v = o < count ? x[(size_t)r * k + first + o] : 0.0f;
        if (DTYPE == GF_Q4_K) {
            const float sum = warp_sum(v);   // slice is a multiple of 32 and e is warp-aligned
            if ((threadIdx.x & 31u) == 0u) sx[r * (slice / 32u) + o / 32u] = sum;
            const uint32_t bitpos = 8u * (o & 1u) + ((o & 32u) ? 4u : 0u);
            v *= __uint_as_float((127u - bitpos) << 23);
        }
        xs[e] = v;
    }
}

template <int DTYPE, int ROWS>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) gemv_kernel(GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kUnitRow = DTYPE == GF_Q8_0 ? 1088u : DTYPE == GF_Q4_K ? 1152u : 1680u;
    constexpr uint32_t kUnitElems = DTYPE == GF_Q8_0 ? 128u : 256u;
    constexpr uint32_t kStageUnits = gemv_stage_units(DTYPE);
    constexpr uint32_t kStageBytes = kStageUnits * kUnitRow;
    constexpr uint32_t kTable = gemv_table_floats(DTYPE);

    const GemvSmemLayout lay = gemv_smem_layout(DTYPE, ROWS, p.chunk_units);
    float* xs = reinterpret_cast<float*>(smem);
    float* sx = reinterpret_cast<float*>(smem + lay.xs_bytes);
    uint8_t* ring_base = smem + lay.xs_bytes + lay.sx_bytes;
    float* table_base = reinterpret_cast<float*>(ring_base + lay.ring_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(table_base) + lay.table_bytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint8_t* ring = ring_base + warp * (kGemvStages * kStageBytes);
    float* table = table_base + warp * (2u * kTable);
    uint64_t* bar = bars + warp * kGemvStages;

    // This CTA's K chunk and this warp's sequence of column tiles.
    const uint32_t chunk = blockIdx.x % p.chunks;
    const uint32_t group_ctas = gridDim.x / p.chunks;
    const uint32_t first_unit = chunk * p.chunk_units;
    const uint32_t chunk_count = min(p.chunk_units, p.units - first_unit);
    const uint32_t stride = group_ctas * kGemvWarps;
    const uint32_t first_tile = (blockIdx.x / p.chunks) * kGemvWarps + warp;
    const uint32_t my_tiles = first_tile < p.tiles ? (p.tiles - first_tile + stride - 1u) / stride : 0u;
    const uint32_t stages_per_item = (chunk_count + kStageUnits - 1u) / kStageUnits;
    const uint32_t jobs = my_tiles * stages_per_item;

    if (lane == 0) {
        for (int s = 0; s < kGemvStages; ++s) mbar_init(&bar[s], 1);
        fence_barrier_init();
    }
    __syncwarp();

    auto issue = [&](uint32_t job) {   // lane 0 only
        const uint32_t item = job / stages_per_item, s = job % stages_per_item;
        const uint32_t tile = first_tile + item * stride;
        const uint32_t u0 = s * kStageUnits;
        const uint32_t cnt = min(kStageUnits, chunk_count - u0);
        const uint8_t* src = p.weight + ((size_t)tile * p.units + first_unit + u0) * kUnitRow;
        const uint32_t slot = job % kGemvStages;
        mbar_expect_tx(&bar[slot], cnt * kUnitRow);
        bulk_load(ring + slot * kStageBytes, src, cnt * kUnitRow, &bar[slot]);
    };
    // Weights do not depend on the previous kernel: start streaming before waiting for it.
    if (lane == 0)
        for (uint32_t j = 0; j < (uint32_t)kGemvStages && j < jobs; ++j) issue(j);

    pdl_wait();
    const uint32_t slice = p.chunk_units * kUnitElems;
    stage_activations<DTYPE, ROWS>(p.x, p.k, first_unit * kUnitElems, chunk_count * kUnitElems, slice, xs, sx);
    __syncthreads();
    pdl_launch_dependents();

    float acc[ROWS][8];
    float macc[ROWS];
    bool failed = false;
    for (uint32_t item = 0; item < my_tiles && !failed; ++item) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            macc[r] = 0.0f;
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[r][c] = 0.0f;
        }
        for (uint32_t s = 0; s < stages_per_item; ++s) {
            const uint32_t job = item * stages_per_item + s;
            const uint32_t slot = job % kGemvStages;
            if (!mbar_wait(&bar[slot], (job / kGemvStages) & 1u)) { failed = true; break; }
            const uint32_t u0 = s * kStageUnits;
            const uint32_t cnt = min(kStageUnits, chunk_count - u0);
            const uint8_t* stage = ring + slot * kStageBytes;
            for (uint32_t u = 0; u < cnt; ++u) {
                const uint32_t lu = u0 + u;      // unit index inside the chunk
                float* tbl = table + (lu & 1u) * kTable;
                if constexpr (DTYPE == GF_Q4_K)
                    unit_row_q4k<ROWS>(stage + u * kUnitRow, xs + lu * 256u, sx + lu * 8u, slice, slice / 32u,
                                       tbl, lane, acc, macc);
                else if constexpr (DTYPE == GF_Q6_K)
                    unit_row_q6k<ROWS>(stage + u * kUnitRow, xs + lu * 256u, slice, tbl, lane, acc);
                else
                    unit_row_q80<ROWS>(stage + u * kUnitRow, xs + lu * 128u, slice, tbl, lane, acc);
            }
            __syncwarp();   // every lane has finished reading this slot
            if (lane == 0 && job + kGemvStages < jobs) issue(job + kGemvStages);
        }
        if (failed) break;
        // Reduce the eight column sums across the warp and write this item's outputs.
        const uint32_t tile = first_tile + item * stride;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float total = reduce_columns8(acc[r], lane);
            if constexpr (DTYPE == GF_Q4_K) {
                float m = macc[r];                         // lanes with equal (lane & 7) share a column
                m += __shfl_xor_sync(0xffffffffu, m, 8);
                m += __shfl_xor_sync(0xffffffffu, m, 16);
                total -= __shfl_sync(0xffffffffu, m, column_of_lane(lane));
            }
            const uint32_t column = tile * 8u + column_of_lane(lane);
            if ((lane & 3u) == 0u && column < p.n)
                p.out[((size_t)chunk * ROWS + r) * p.n + column] = total;
        }
    }
    if (failed && lane == 0) atomicExch(p.error_flag, 1);
}

// Adds split-K partials in chunk order: y[r][n] = sum_c partial[c][r][n].
static __global__ void __launch_bounds__(256) gemv_reduce_kernel(const float* __restrict__ partial, float* __restrict__ y,
                                                          uint32_t chunks, uint32_t elements) {
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < elements) {
        float sum = partial[i];
        for (uint32_t c = 1; c < chunks; ++c) sum += partial[(size_t)c * elements + i];
        y[i] = sum;
    }
    pdl_launch_dependents();
}

#endif  // __CUDACC__

// Host-side plan: how a (dtype, rows, K, N) product is decomposed.
struct GemvPlan {
    uint32_t units, tiles, chunks, chunk_units, grid, smem;
};
int gemv_plan(int dtype, uint32_t rows, uint64_t k, uint64_t n, GemvPlan& plan);
int gemv_launch(int dtype, const void* packed, const float* x, float* y, uint32_t rows, uint64_t k, uint64_t n,
                void* workspace, int* error_flag, cudaStream_t stream, bool programmatic);

}  // namespace gf
