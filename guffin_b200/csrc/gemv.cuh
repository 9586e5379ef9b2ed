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

// ---- packed f32x2 arithmetic (sm_100): one instruction issues two independent f32 operations,
// halving the issue slots of the conversion and multiply-add stream.  Each half rounds exactly
// like the scalar instruction.
typedef unsigned long long f32x2;
// The "magic" exponent word 0x4B000000 (2^23) held in a register the compiler cannot fold: a
// logic instruction encodes only one immediate, so (w & mask) | magic is a single LOP3 only when
// the magic operand comes from a register.
__device__ __forceinline__ uint32_t magic_register() {
    uint32_t r;
    asm("mov.u32 %0, 0x4B000000;" : "=r"(r));
    return r;
}
__device__ __forceinline__ f32x2 pack2(uint32_t lo, uint32_t hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pack2f(float lo, float hi) { return pack2(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ float2 unpack2(f32x2 v) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Two codes of one word become a pair of exact floats in one go: (w & mask) | magic for each half
// (a single three-input logic instruction each, the magic word coming from a register), then
// one packed add of -bias.  MASK_LO / MASK_HI select the code of the even / odd element.
template <uint32_t MASK_LO, uint32_t MASK_HI>
__device__ __forceinline__ f32x2 masked_pair(uint32_t w, uint32_t magic, f32x2 neg_bias) {
    f32x2 r;
    asm("{\n\t.reg .b32 lo, hi;\n\t.reg .b64 p;\n\t"
        "lop3.b32 lo, %1, %2, %4, 0xEA;\n\t"
        "lop3.b32 hi, %1, %3, %4, 0xEA;\n\t"
        "mov.b64 p, {lo, hi};\n\t"
        "add.rn.f32x2 %0, p, %5;\n\t}"
        : "=l"(r) : "r"(w), "n"(MASK_LO), "n"(MASK_HI), "r"(magic), "l"(neg_bias));
    return r;
}
// Bytes SEL and SEL+1 of `v` (each < 256) become a pair of exact floats minus the bias.
template <uint32_t SEL>
__device__ __forceinline__ f32x2 byte_pair(uint32_t v, uint32_t magic, f32x2 neg_bias) {
    f32x2 r;
    asm("{\n\t.reg .b32 lo, hi;\n\t.reg .b64 p;\n\t"
        "prmt.b32 lo, %1, %2, %3;\n\t"
        "prmt.b32 hi, %1, %2, %4;\n\t"
        "mov.b64 p, {lo, hi};\n\t"
        "add.rn.f32x2 %0, p, %5;\n\t}"
        : "=l"(r) : "r"(v), "r"(magic), "n"(0x7540u + SEL), "n"(0x7541u + SEL), "l"(neg_bias));
    return r;
}

// Sums four per-lane column values over the 16 lanes of a half warp; afterwards the lanes
// with (lane & 3) == 0 hold the total of column half_column_of_lane(lane).
__device__ __forceinline__ float reduce_columns4(float (&v)[4], uint32_t lane) {
    const bool b8 = lane & 8u, b4 = lane & 4u;
    float u[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float keep = b8 ? v[i + 2] : v[i];
        const float send = b8 ? v[i] : v[i + 2];
        u[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float keep = b4 ? u[1] : u[0];
    const float send = b4 ? u[0] : u[1];
    float w = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    w += __shfl_xor_sync(0xffffffffu, w, 2);
    w += __shfl_xor_sync(0xffffffffu, w, 1);
    return w;
}
__device__ __forceinline__ uint32_t half_column_of_lane(uint32_t lane) {
    return (lane >> 4) * 4u + ((lane & 8u) ? 2u : 0u) + ((lane & 4u) ? 1u : 0u);
}

// ---- one unit row (8 columns x one K unit) of each format.  `row` points at the unit row in
// shared memory, `xs` at the activation slice of this unit (row stride `xstride` floats),
// `table` at this warp's scale table for the current parity.  Each half warp owns four of the
// eight columns; a lane owns sixteen K positions and keeps their activations in registers as
// f32x2 pairs.  acc[r][cc] is a pair of partial sums of row r, column half*4+cc.

template <int ROWS>
__device__ __forceinline__ void unit_row_q4k(const uint8_t* row, const float* xs, const float* sx,
                                             uint32_t xstride, uint32_t sxstride, float* table,
                                             uint32_t lane, f32x2 (&acc)[ROWS][4], float (&macc)[ROWS]) {
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
        const float ds0 = __fmul_rn(d, (float)(sc & 0xffu)), ds1 = __fmul_rn(d, (float)(sc >> 8));
        // Each scale is stored twice so that Phase B reads it as a ready-made f32x2 pair.
        *reinterpret_cast<float4*>(table + (col * 4u + pair) * 4u) = make_float4(ds0, ds0, ds1, ds1);
        const float m0 = __fmul_rn(dmin, (float)(mn & 0xffu)), m1 = __fmul_rn(dmin, (float)(mn >> 8));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float2 s = *reinterpret_cast<const float2*>(sx + r * sxstride + pair * 2u);
            macc[r] = fmaf(m0, s.x, fmaf(m1, s.y, macc[r]));
        }
    }
    __syncwarp();
    // Phase B: lane (half, chunk c, piece i) owns the nibbles of elements 64c+8i+j (low) and
    // 64c+32+8i+j (high), j < 8, of the half's four columns.
    const uint32_t half = lane >> 4, t = lane & 15u, c = t >> 2, i = t & 3u;
    f32x2 xl[ROWS][4], xh[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const ulonglong2* lo = reinterpret_cast<const ulonglong2*>(xs + r * xstride + c * 64u + i * 8u);
        const ulonglong2* hi = reinterpret_cast<const ulonglong2*>(xs + r * xstride + c * 64u + 32u + i * 8u);
        const ulonglong2 l0 = lo[0], l1 = lo[1], h0 = hi[0], h1 = hi[1];
        xl[r][0] = l0.x; xl[r][1] = l0.y; xl[r][2] = l1.x; xl[r][3] = l1.y;
        xh[r][0] = h0.x; xh[r][1] = h0.y; xh[r][2] = h1.x; xh[r][3] = h1.y;
    }
    const uint2* qs = reinterpret_cast<const uint2*>(row);
    const uint32_t magic = magic_register();
    const f32x2 neg_bias = pack2f(-8388608.0f, -8388608.0f);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
        const uint32_t col = half * 4u + cc;
        const uint2 w = qs[col * 16u + t];
        const ulonglong2 ds = *reinterpret_cast<const ulonglong2*>(table + (col * 4u + c) * 4u);
        const uint32_t w0 = w.x, w0h = w.x >> 16, w1 = w.y, w1h = w.y >> 16;
        // Pair = (even element, odd element): bits 0-3 / 8-11 of a half word hold the low nibbles,
        // bits 4-7 / 12-15 the high nibbles.  Activations were pre-scaled by 2^-bitpos of their
        // nibble, so q * 2^bitpos * x' = q * x exactly.
        const f32x2 qa0 = masked_pair<0x0000000fu, 0x00000f00u>(w0, magic, neg_bias), qb0 = masked_pair<0x000000f0u, 0x0000f000u>(w0, magic, neg_bias);
        const f32x2 qa1 = masked_pair<0x0000000fu, 0x00000f00u>(w0h, magic, neg_bias), qb1 = masked_pair<0x000000f0u, 0x0000f000u>(w0h, magic, neg_bias);
        const f32x2 qa2 = masked_pair<0x0000000fu, 0x00000f00u>(w1, magic, neg_bias), qb2 = masked_pair<0x000000f0u, 0x0000f000u>(w1, magic, neg_bias);
        const f32x2 qa3 = masked_pair<0x0000000fu, 0x00000f00u>(w1h, magic, neg_bias), qb3 = masked_pair<0x000000f0u, 0x0000f000u>(w1h, magic, neg_bias);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const f32x2 lo = fma2(xl[r][3], qa3, fma2(xl[r][2], qa2, fma2(xl[r][1], qa1, mul2(xl[r][0], qa0))));
            const f32x2 hi = fma2(xh[r][3], qb3, fma2(xh[r][2], qb2, fma2(xh[r][1], qb1, mul2(xh[r][0], qb0))));
            acc[r][cc] = fma2(ds.x, lo, fma2(ds.y, hi, acc[r][cc]));
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void unit_row_q6k(const uint8_t* row, const float* xs, uint32_t xstride,
                                             float* table, uint32_t lane, f32x2 (&acc)[ROWS][4]) {
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
    // Phase B: lane (half, t = (h, p, i)): elements h*128+32p+8i+j (low nibble, high bits 2p) and
    // h*128+32(p+2)+8i+j (high nibble, high bits 2p+4), j < 8; each set lies in one 16-wide group.
    const uint32_t half = lane >> 4, t = lane & 15u, h = t >> 3, p = (t >> 2) & 1u, i = t & 3u;
    f32x2 xa[ROWS][4], xb[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const ulonglong2* a = reinterpret_cast<const ulonglong2*>(xs + r * xstride + h * 128u + p * 32u + i * 8u);
        const ulonglong2* b = reinterpret_cast<const ulonglong2*>(xs + r * xstride + h * 128u + p * 32u + 64u + i * 8u);
        const ulonglong2 a0 = a[0], a1 = a[1], b0 = b[0], b1 = b[1];
        xa[r][0] = a0.x; xa[r][1] = a0.y; xa[r][2] = a1.x; xa[r][3] = a1.y;
        xb[r][0] = b0.x; xb[r][1] = b0.y; xb[r][2] = b1.x; xb[r][3] = b1.y;
    }
    const uint2* ql = reinterpret_cast<const uint2*>(row);
    const uint2* qh = reinterpret_cast<const uint2*>(row + 1024u);
    const uint32_t kMagic = magic_register();
    const f32x2 neg_bias = pack2f(-(8388608.0f + 32.0f), -(8388608.0f + 32.0f));   // magic exponent and the -32 offset
    const uint32_t shift = p * 2u;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
        const uint32_t col = half * 4u + cc;
        const uint2 wl = ql[col * 16u + t];
        const uint2 whr = qh[col * 8u + h * 4u + i];
        const float2 ds = *reinterpret_cast<const float2*>(table + col * 16u + ((h * 2u + p) * 2u + (i >> 1)) * 2u);
        const uint32_t wh0 = whr.x >> shift, wh1 = whr.y >> shift;
        const uint32_t va0 = (wl.x & 0x0f0f0f0fu) | ((wh0 << 4) & 0x30303030u);
        const uint32_t vb0 = ((wl.x >> 4) & 0x0f0f0f0fu) | (wh0 & 0x30303030u);
        const uint32_t va1 = (wl.y & 0x0f0f0f0fu) | ((wh1 << 4) & 0x30303030u);
        const uint32_t vb1 = ((wl.y >> 4) & 0x0f0f0f0fu) | (wh1 & 0x30303030u);
        const f32x2 qa0 = byte_pair<0>(va0, kMagic, neg_bias), qa1 = byte_pair<2>(va0, kMagic, neg_bias);
        const f32x2 qa2 = byte_pair<0>(va1, kMagic, neg_bias), qa3 = byte_pair<2>(va1, kMagic, neg_bias);
        const f32x2 qb0 = byte_pair<0>(vb0, kMagic, neg_bias), qb1 = byte_pair<2>(vb0, kMagic, neg_bias);
        const f32x2 qb2 = byte_pair<0>(vb1, kMagic, neg_bias), qb3 = byte_pair<2>(vb1, kMagic, neg_bias);
        const f32x2 dsa = pack2f(ds.x, ds.x), dsb = pack2f(ds.y, ds.y);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const f32x2 da = fma2(xa[r][3], qa3, fma2(xa[r][2], qa2, fma2(xa[r][1], qa1, mul2(xa[r][0], qa0))));
            const f32x2 db = fma2(xb[r][3], qb3, fma2(xb[r][2], qb2, fma2(xb[r][1], qb1, mul2(xb[r][0], qb0))));
            acc[r][cc] = fma2(dsa, da, fma2(dsb, db, acc[r][cc]));
        }
    }
}

template <int ROWS>
__device__ __forceinline__ void unit_row_q80(const uint8_t* row, const float* xs, uint32_t xstride,
                                             float* table, uint32_t lane, f32x2 (&acc)[ROWS][4]) {
    {   // Phase A: lane (col, block) widens the block's f16 scale.
        const uint32_t col = lane & 7u, block = lane >> 3;
        table[col * 4u + block] = __half2float(__ushort_as_half(
            *reinterpret_cast<const unsigned short*>(row + 1024u + col * 8u + block * 2u)));
    }
    __syncwarp();
    // Phase B: lane (half, t) owns elements 8t..8t+7 (block t/4) of the half's four columns.
    const uint32_t half = lane >> 4, t = lane & 15u, block = t >> 2;
    f32x2 xv[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const ulonglong2* v = reinterpret_cast<const ulonglong2*>(xs + r * xstride + t * 8u);
        const ulonglong2 v0 = v[0], v1 = v[1];
        xv[r][0] = v0.x; xv[r][1] = v0.y; xv[r][2] = v1.x; xv[r][3] = v1.y;
    }
    const uint2* q = reinterpret_cast<const uint2*>(row);
    const uint32_t kMagic = magic_register();
    const f32x2 neg_bias = pack2f(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f));   // int8 + 128 made unsigned by flipping bit 7
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
        const uint32_t col = half * 4u + cc;
        const uint2 raw = q[col * 16u + t];
        const uint32_t w0 = raw.x ^ 0x80808080u, w1 = raw.y ^ 0x80808080u;
        const float d = table[col * 4u + block];
        const f32x2 q0 = byte_pair<0>(w0, kMagic, neg_bias), q1 = byte_pair<2>(w0, kMagic, neg_bias);
        const f32x2 q2 = byte_pair<0>(w1, kMagic, neg_bias), q3 = byte_pair<2>(w1, kMagic, neg_bias);
        const f32x2 dd = pack2f(d, d);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const f32x2 dot = fma2(xv[r][3], q3, fma2(xv[r][2], q2, fma2(xv[r][1], q1, mul2(xv[r][0], q0))));
            acc[r][cc] = fma2(dd, dot, acc[r][cc]);
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

    f32x2 acc[ROWS][4];
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
            for (int c = 0; c < 4; ++c) acc[r][c] = 0ull;
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
        // Reduce each half warp's four column sums; lanes with (lane & 3) == 0 hold the eight totals.
        const uint32_t my_column = half_column_of_lane(lane);
        float totals[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float sums[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) { const float2 v = unpack2(acc[r][c]); sums[c] = v.x + v.y; }
            float total = reduce_columns4(sums, lane);
            if (dtype == GF_Q4_K) {
                float m = macc[r];                         // lanes with equal (lane & 7) share a column
                m += __shfl_xor_sync(0xffffffffu, m, 8);
                m += __shfl_xor_sync(0xffffffffu, m, 16);
                total -= __shfl_sync(0xffffffffu, m, my_column);
            }
            totals[r] = total;
        }
        const uint32_t local_tile = tile - mat.first_tile;
        const uint32_t column = local_tile * 8u + my_column;
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
            if ((lane & 3u) == 0u) p.partial[((size_t)chunk * ROWS + r) * width + (size_t)tile * 8u + my_column] = totals[r];
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
