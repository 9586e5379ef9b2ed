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

constexpr int kGemvWarps = 8;        // warps per CTA; two CTAs share an SM so that the next
                                     // kernel's CTAs can prefetch weights while this one drains
constexpr int kGemvStages = 3;       // ring depth per warp
constexpr uint32_t kGemvStageBytes = 3456u;          // 3 Q4_K / 2 Q6_K / 3 Q8_0 unit rows
constexpr uint32_t kGemvTableFloats = 128u;          // per unit row, per warp (Q6_K needs 8 x 16)
constexpr uint32_t kGemvSmemBudget = 113u * 1024u;   // two CTAs per SM
constexpr int kGemvMaxMatrices = 3;

__host__ __device__ constexpr uint32_t gemv_stage_units(int dtype) { return dtype == GF_Q6_K ? 2u : 3u; }

// How the activation rows are produced from global memory before the weights are applied.
enum GemvPrologue : uint32_t {
    kProloguePlain = 0,      // xs = in
    kPrologueNorm = 1,       // xs = rmsnorm(in; gamma1)
    kPrologueAddNorm = 2,    // r = residual + rmsnorm(in; gamma0) -> residual_out;  xs = rmsnorm(r; gamma1)
    kPrologueGeglu = 3,      // xs = gelu_tanh(in) * residual
};

struct GemvMatrix {
    const uint8_t* weight;   // streaming layout
    float* out;              // [rows][n]
    uint32_t n, tiles, dtype, first_tile;
};

struct GemvParams {
    GemvMatrix m[kGemvMaxMatrices];
    uint32_t matrices, total_tiles;
    uint32_t k, units, unit_elems;
    uint32_t chunks, chunk_units;
    uint32_t needs_scaled, needs_plain;   // which activation variants the matrices read
    uint32_t prologue;
    const float *in, *residual, *gamma0, *gamma1;
    float* residual_out;
    float eps;
    float* partial;            // [chunks][rows][total_tiles * 8] when chunks > 1
    uint32_t* counters;        // [total_tiles] arrival counts, zero between launches
    int* error_flag;           // set to 1 when a bounded wait gives up
};

struct GemvSmemLayout {
    uint32_t xs_bytes, sx_bytes, ring_bytes, table_bytes, total;
};

__host__ __device__ inline GemvSmemLayout gemv_smem_layout(uint32_t rows, uint32_t chunk_units, uint32_t unit_elems,
                                                           uint32_t variants, bool needs_sums) {
    GemvSmemLayout s;
    const uint32_t slice = chunk_units * unit_elems;
    s.xs_bytes = rows * slice * 4u * variants;
    s.sx_bytes = needs_sums ? rows * (slice / 32u) * 4u : 0u;
    s.ring_bytes = (uint32_t)kGemvWarps * kGemvStages * kGemvStageBytes;
    s.table_bytes = (uint32_t)kGemvWarps * 2u * kGemvTableFloats * 4u;
    s.total = s.xs_bytes + s.sx_bytes + s.ring_bytes + s.table_bytes + kGemvWarps * kGemvStages * 8u + 64u;
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

// ---- activation prologue ----

__device__ __forceinline__ float gelu_tanh_exact(float v) {
    const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
}

// Sum over the block of one value per thread; every thread gets the total (fixed order).
__device__ __forceinline__ float gemv_block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kGemvWarps; ++w) total += scratch[w];
    __syncthreads();
    return total;
}

// Produces this CTA's K slice of the activation rows in shared memory: the plain values, the
// copy pre-scaled by 2^-bitpos of each element's nibble (what the Q4_K lanes multiply with),
// and the per-32 sums the Q4_K min term needs.  The RMS norms of prologues 1 and 2 need the
// whole row, so every CTA recomputes them from global memory (a few tens of KB out of L2).
template <int ROWS>
__device__ __forceinline__ void stage_activations(const GemvParams& p, uint32_t first, uint32_t count, uint32_t slice,
                                                  float* xs_plain, float* xs_scaled, float* sx, float* scratch) {
    float inv0[ROWS], inv1[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { inv0[r] = 1.0f; inv1[r] = 1.0f; }
    if (p.prologue == kPrologueNorm || p.prologue == kPrologueAddNorm) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float* in = p.in + (size_t)r * p.k;
            float sum = 0.0f;
            for (uint32_t c = threadIdx.x; c < p.k; c += blockDim.x) sum = fmaf(in[c], in[c], sum);
            const float total = gemv_block_sum(sum, scratch);
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)p.k), p.eps)));
            if (p.prologue == kPrologueNorm) { inv1[r] = inv; continue; }
            inv0[r] = inv;
            // r = residual + norm(in) * gamma0; its mean square feeds the second norm.
            const float* res = p.residual + (size_t)r * p.k;
            float sum2 = 0.0f;
            for (uint32_t c = threadIdx.x; c < p.k; c += blockDim.x) {
                const float v = __fadd_rn(res[c], __fmul_rn(__fmul_rn(in[c], inv), p.gamma0[c]));
                sum2 = fmaf(v, v, sum2);
                if (blockIdx.x == 0) p.residual_out[(size_t)r * p.k + c] = v;
            }
            const float total2 = gemv_block_sum(sum2, scratch);
            inv1[r] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total2, (float)p.k), p.eps)));
        }
    }
    for (uint32_t e = threadIdx.x; e < (uint32_t)ROWS * slice; e += blockDim.x) {
        const uint32_t r = e / slice, o = e % slice;
        float v = 0.0f;
        if (o < count) {
            const size_t g = (size_t)r * p.k + first + o;
            const uint32_t c = first + o;
            float i0 = 1.0f, i1 = 1.0f;
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) if (rr == (int)r) { i0 = inv0[rr]; i1 = inv1[rr]; }
            if (p.prologue == kProloguePlain) v = p.in[g];
            else if (p.prologue == kPrologueNorm) v = __fmul_rn(__fmul_rn(p.in[g], i1), p.gamma1[c]);
            else if (p.prologue == kPrologueAddNorm) {
                const float t = __fadd_rn(p.residual[g], __fmul_rn(__fmul_rn(p.in[g], i0), p.gamma0[c]));
                v = __fmul_rn(__fmul_rn(t, i1), p.gamma1[c]);
            } else v = __fmul_rn(gelu_tanh_exact(p.in[g]), p.residual[g]);
        }
        if (p.needs_plain) xs_plain[e] = v;
        if (p.needs_scaled) {
            const float sum = warp_sum(v);   // slice is a multiple of 32 and e is warp-aligned
            if ((threadIdx.x & 31u) == 0u) sx[r * (slice / 32u) + o / 32u] = sum;
            const uint32_t bitpos = 8u * (o & 1u) + ((o & 32u) ? 4u : 0u);
            xs_scaled[e] = v * __uint_as_float((127u - bitpos) << 23);
        }
    }
}

template <int ROWS>
__global__ void __launch_bounds__(kGemvWarps * 32, 2) gemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[kGemvWarps];
    const uint32_t variants = p.needs_plain + p.needs_scaled;
    const GemvSmemLayout lay = gemv_smem_layout(ROWS, p.chunk_units, p.unit_elems, variants, p.needs_scaled != 0u);
    const uint32_t slice = p.chunk_units * p.unit_elems;
    float* xs_plain = reinterpret_cast<float*>(smem);
    float* xs_scaled = xs_plain + (p.needs_plain ? (size_t)ROWS * slice : 0u);
    float* sx = reinterpret_cast<float*>(smem + lay.xs_bytes);
    uint8_t* ring_base = smem + lay.xs_bytes + lay.sx_bytes;
    float* table_base = reinterpret_cast<float*>(ring_base + lay.ring_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(table_base) + lay.table_bytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint8_t* ring = ring_base + warp * (kGemvStages * kGemvStageBytes);
    float* table = table_base + warp * (2u * kGemvTableFloats);
    uint64_t* bar = bars + warp * kGemvStages;

    // This CTA's K chunk and this warp's sequence of column tiles (over all matrices).
    const uint32_t chunk = blockIdx.x % p.chunks;
    const uint32_t group_ctas = gridDim.x / p.chunks;
    const uint32_t first_unit = chunk * p.chunk_units;
    const uint32_t chunk_count = min(p.chunk_units, p.units - first_unit);
    const uint32_t stride = group_ctas * kGemvWarps;
    const uint32_t first_tile = (blockIdx.x / p.chunks) * kGemvWarps + warp;
    const uint32_t my_tiles = first_tile < p.total_tiles ? (p.total_tiles - first_tile + stride - 1u) / stride : 0u;

    auto matrix_of = [&](uint32_t tile) -> uint32_t {
        uint32_t m = 0;
        if (p.matrices > 1u && tile >= p.m[1].first_tile) m = 1;
        if (p.matrices > 2u && tile >= p.m[2].first_tile) m = 2;
        return m;
    };
    auto stages_of = [&](uint32_t dtype) { const uint32_t su = gemv_stage_units((int)dtype); return (chunk_count + su - 1u) / su; };

    if (lane == 0) {
        for (int s = 0; s < kGemvStages; ++s) mbar_init(&bar[s], 1);
        fence_barrier_init();
    }
    __syncwarp();

    // Producer cursor (lane 0): the next stage to request, walking items then stages.
    uint32_t prod_item = 0, prod_stage = 0, prod_slot = 0;
    auto issue_next = [&]() -> bool {   // lane 0 only
        if (prod_item >= my_tiles) return false;
        const uint32_t tile = first_tile + prod_item * stride;
        const GemvMatrix& mat = p.m[matrix_of(tile)];
        const uint32_t su = gemv_stage_units((int)mat.dtype), row_bytes = unit_row_bytes((int)mat.dtype);
        const uint32_t u0 = prod_stage * su;
        const uint32_t cnt = min(su, chunk_count - u0);
        const uint8_t* src = mat.weight + ((size_t)(tile - mat.first_tile) * p.units + first_unit + u0) * row_bytes;
        mbar_expect_tx(&bar[prod_slot], cnt * row_bytes);
        bulk_load(ring + prod_slot * kGemvStageBytes, src, cnt * row_bytes, &bar[prod_slot]);
        prod_slot = prod_slot + 1u == (uint32_t)kGemvStages ? 0u : prod_slot + 1u;
        if (++prod_stage == stages_of(mat.dtype)) { prod_stage = 0; ++prod_item; }
        return true;
    };
    // Weights do not depend on the previous kernel: start streaming before waiting for it.
    if (lane == 0)
        for (int j = 0; j < kGemvStages; ++j) issue_next();

    pdl_wait();
    stage_activations<ROWS>(p, first_unit * p.unit_elems, chunk_count * p.unit_elems, slice, xs_plain, xs_scaled, sx, scratch);
    __syncthreads();
    pdl_launch_dependents();

    float acc[ROWS][8];
    float macc[ROWS];
    bool failed = false;
    uint32_t slot = 0, phase = 0;
    for (uint32_t item = 0; item < my_tiles && !failed; ++item) {
        const uint32_t tile = first_tile + item * stride;
        const GemvMatrix& mat = p.m[matrix_of(tile)];
        const uint32_t dtype = mat.dtype, su = gemv_stage_units((int)dtype), row_bytes = unit_row_bytes((int)dtype);
        const uint32_t stages = (chunk_count + su - 1u) / su;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            macc[r] = 0.0f;
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[r][c] = 0.0f;
        }
        for (uint32_t s = 0; s < stages; ++s) {
            if (!mbar_wait(&bar[slot], phase)) { failed = true; break; }
            const uint32_t u0 = s * su;
            const uint32_t cnt = min(su, chunk_count - u0);
            const uint8_t* stage = ring + slot * kGemvStageBytes;
            for (uint32_t u = 0; u < cnt; ++u) {
                const uint32_t lu = u0 + u;      // unit index inside the chunk
                float* tbl = table + (lu & 1u) * kGemvTableFloats;
                if (dtype == GF_Q4_K)
                    unit_row_q4k<ROWS>(stage + u * row_bytes, xs_scaled + lu * 256u, sx + lu * 8u, slice, slice / 32u,
                                       tbl, lane, acc, macc);
                else if (dtype == GF_Q6_K)
                    unit_row_q6k<ROWS>(stage + u * row_bytes, xs_plain + lu * 256u, slice, tbl, lane, acc);
                else
                    unit_row_q80<ROWS>(stage + u * row_bytes, xs_plain + lu * 128u, slice, tbl, lane, acc);
            }
            __syncwarp();   // every lane has finished reading this slot
            if (lane == 0) issue_next();
            if (++slot == (uint32_t)kGemvStages) { slot = 0; phase ^= 1u; }
        }
        if (failed) break;
        // Reduce the eight column sums across the warp.
        float totals[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float total = reduce_columns8(acc[r], lane);
            if (dtype == GF_Q4_K) {
                float m = macc[r];                         // lanes with equal (lane & 7) share a column
                m += __shfl_xor_sync(0xffffffffu, m, 8);
                m += __shfl_xor_sync(0xffffffffu, m, 16);
                total -= __shfl_sync(0xffffffffu, m, column_of_lane(lane));
            }
            totals[r] = total;
        }
        const uint32_t local_tile = tile - mat.first_tile;
        const uint32_t column = local_tile * 8u + column_of_lane(lane);
        if (p.chunks == 1u) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if ((lane & 3u) == 0u && column < mat.n) mat.out[(size_t)r * mat.n + column] = totals[r];
            continue;
        }
        // Split K: park this chunk's partial sums; the warp that arrives last for the tile adds
        // all chunks in chunk order (so the result does not depend on arrival order).
        const size_t width = (size_t)p.total_tiles * 8u;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if ((lane & 3u) == 0u) p.partial[((size_t)chunk * ROWS + r) * width + (size_t)tile * 8u + column_of_lane(lane)] = totals[r];
        __threadfence();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atomicAdd(&p.counters[tile], 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == p.chunks - 1u) {
            __threadfence();
            const uint32_t col = lane & 7u, r = lane >> 3;
            if (r < (uint32_t)ROWS) {
                float sum = 0.0f;
                for (uint32_t c = 0; c < p.chunks; ++c)
                    sum += __ldcg(&p.partial[((size_t)c * ROWS + r) * width + (size_t)tile * 8u + col]);
                const uint32_t out_column = local_tile * 8u + col;
                if (out_column < mat.n) mat.out[(size_t)r * mat.n + out_column] = sum;
            }
            if (lane == 0) p.counters[tile] = 0u;
        }
    }
    if (failed) {
        // Give outstanding copies a bounded chance to land before the shared memory is released.
        for (int s = 0; s < kGemvStages; ++s) mbar_wait(&bar[s], 0);
        if (lane == 0) atomicExch(p.error_flag, 1);
    }
}

#endif  // __CUDACC__

// Host-side description of one fused launch.
struct GemvMatrixDesc { int dtype; const void* packed; float* out; uint64_t n; };
struct GemvLaunch {
    GemvMatrixDesc matrices[kGemvMaxMatrices];
    uint32_t count = 1;
    uint64_t k = 0;
    uint32_t rows = 1;
    uint32_t prologue = kProloguePlain;
    const float *in = nullptr, *residual = nullptr, *gamma0 = nullptr, *gamma1 = nullptr;
    float* residual_out = nullptr;
    float eps = 1e-6f;
};
struct GemvPlan { uint32_t units, unit_elems, total_tiles, chunks, chunk_units, grid, smem, needs_scaled, needs_plain; };

int gemv_plan(const GemvLaunch& launch, GemvPlan& plan);
// Split-K scratch of one launch: `partial` bytes of sums, and one arrival counter per column tile.
// Counters must be zero before a launch and are left zero by it; they must not share memory
// with any launch's partial sums.
size_t gemv_partial_bytes(const GemvLaunch& launch);
size_t gemv_counter_bytes(const GemvLaunch& launch);
int gemv_launch(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                cudaStream_t stream, bool programmatic);

}  // namespace gf
