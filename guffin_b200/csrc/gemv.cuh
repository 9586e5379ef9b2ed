// Weight-streaming dequant-GEMV core for Q4_K / Q6_K / Q8_0, rows M <= 4.
//
// Work decomposition: an item is (column pair of 16 outputs, K chunk).  A CTA is bound to one
// K chunk and stages that slice of the activation rows in shared memory once; each of its
// warps then streams whole items through a private ring of shared-memory slots filled by
// one-shot TMA bulk copies (cp.async.bulk + mbarrier), so no block-level synchronisation
// happens while weights stream.
//
// Arithmetic: the quantised codes are integers below 256, so they are exact in bf16; a logic
// instruction per two codes turns the packed nibbles into bf16 pairs in the register layout of
// the A operand of mma.m16n8k16 (16 output columns x 16 K positions).  The B operand holds the
// activations: every f32 activation is split exactly into three bf16 terms (8 + 8 + 8 mantissa
// bits), which occupy three of the eight B columns, so one tensor-core instruction multiplies
// 256 weights with the full-precision activations of up to two rows and accumulates in f32.
// That removes the per-element conversion and multiply-add instructions that bound a
// CUDA-core dequant-GEMV on issue slots rather than on HBM bandwidth.  Group scales are applied
// to the accumulator of each scale group (two packed f32 multiply-adds per instruction group);
// the constant offsets of the code encodings and the Q4_K minima reduce to one dot product per
// column with the per-group activation sums, taken while the scales are decoded.
//
// Row r's arithmetic does not depend on how many rows are computed beside it (its three B
// columns are independent of the others), and partial sums of different K chunks are added in
// chunk order, so results are reproducible and row-count invariant.
#pragma once

#include "common.cuh"

namespace gf {

constexpr int kGemvWarps = 16;       // warps per CTA; one CTA per SM
constexpr int kGemvSlots = 3;        // ring depth per warp, one pair row per slot
constexpr uint32_t kGemvSmemLimit = 226u * 1024u;    // dynamic part; the static arrays take the rest of the 227 KB
constexpr int kGemvMaxMatrices = 3;

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
    uint32_t n, pairs, dtype, first_pair;
};

struct GemvParams {
    GemvMatrix m[kGemvMaxMatrices];
    uint32_t matrices, total_pairs;
    uint32_t k, units, unit_elems;
    uint32_t chunks, chunk_units;
    uint32_t slot_bytes, table_bytes;     // ring slot size; scale table bytes per warp
    uint32_t prologue;
    const float *in, *residual, *gamma0, *gamma1;
    float* residual_out;
    float eps;
    float* partial;            // [chunks][rows][total_pairs * 16] when chunks > 1
    uint32_t* counters;        // [total_pairs] arrival counts, zero between launches
    int* error_flag;           // set to 1 when a bounded wait gives up
};

// Columns of the B operand kept per 16-element group: three bf16 terms per row, padded to a
// power of two (one row) or to whole n-tiles of eight.
__host__ __device__ constexpr uint32_t gemv_fragment_columns(uint32_t rows) {
    return rows == 1u ? 4u : ((3u * rows + 7u) / 8u) * 8u;
}
__host__ __device__ constexpr uint32_t gemv_table_bytes(int dtype) {   // per warp: 16 columns x groups x (a, a)
    return dtype == GF_Q6_K ? 2048u : dtype == GF_Q4_K ? 1024u : 512u;
}

struct GemvSmemLayout {
    uint32_t frag_bytes, sums_bytes, ring_bytes, table_bytes, total;
};

__host__ __device__ inline GemvSmemLayout gemv_smem_layout(uint32_t rows, uint32_t chunk_units, uint32_t unit_elems,
                                                           uint32_t slot_bytes, uint32_t table_bytes) {
    GemvSmemLayout s;
    const uint32_t slice = chunk_units * unit_elems;
    s.frag_bytes = slice * gemv_fragment_columns(rows) * 2u;
    s.sums_bytes = rows * (slice / 16u) * 4u;
    s.ring_bytes = (uint32_t)kGemvWarps * kGemvSlots * slot_bytes;
    s.table_bytes = (uint32_t)kGemvWarps * table_bytes;
    s.total = s.frag_bytes + s.sums_bytes + s.ring_bytes + s.table_bytes + kGemvWarps * kGemvSlots * 8u + 64u;
    return s;
}

#ifdef __CUDACC__

// ---- packed f32x2 arithmetic (sm_100): one instruction issues two independent f32 operations.
// Each half rounds exactly like the scalar instruction.
typedef unsigned long long f32x2;
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

// A constant the compiler cannot fold into an immediate: a logic instruction encodes only one
// immediate, so (w & mask) | magic is a single instruction only when the magic word is a register.
__device__ __forceinline__ uint32_t opaque_constant(uint32_t value) {
    uint32_t r;
    asm("mov.u32 %0, %1;" : "=r"(r) : "r"(value));
    return r;
}
// (v & MASK) | orend: one three-input logic instruction.
template <uint32_t MASK>
__device__ __forceinline__ uint32_t and_or(uint32_t v, uint32_t orend) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(v), "n"(MASK), "r"(orend));
    return r;
}
// Bytes SEL and SEL+1 of `v` (each < 256) become a pair of exact floats minus the bias
// (magic = 0x4B000000, the exponent word of 2^23).
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

// D = A (16 x 16, bf16) * B (16 x 8, bf16) + C, f32 accumulation.  Lane (g, t): A registers are
// (row g, k 2t..2t+1), (row g+8, same k), (row g, k 2t+8..2t+9), (row g+8, same k); B registers
// are (k 2t..2t+1, column g), (k 2t+8..2t+9, column g); C/D are (row g, columns 2t..2t+1),
// (row g+8, columns 2t..2t+1).
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// Nibble codes as bf16 pairs.  A code n sits in mantissa bits 3..6 of the bf16 word 0x4180
// (16.0, whose mantissa step at those bits is 1), so the word reads 16 + n; the constant 16 per
// element is removed through the activation sums.  Bytes (0, 2) of a 32-bit word give the pair
// of elements (0, 2) and bytes (1, 3) the pair (1, 3), matching the activation fragments.
constexpr uint32_t kNibbleMask = 0x00780078u;
constexpr uint32_t kNibbleMagic = 0x41804180u;
constexpr float kNibbleOffset = 16.0f;
// a[0..3] for the low (HIGH = 0) or high (HIGH = 1) nibbles of word wa (column g) and wb (column g+8).
template <int HIGH>
__device__ __forceinline__ void nibble_fragment(uint32_t wa, uint32_t wb, uint32_t magic, uint32_t (&a)[4]) {
    if (HIGH) {
        a[0] = and_or<kNibbleMask>(wa >> 1, magic); a[1] = and_or<kNibbleMask>(wb >> 1, magic);
        a[2] = and_or<kNibbleMask>(wa >> 9, magic); a[3] = and_or<kNibbleMask>(wb >> 9, magic);
    } else {
        a[0] = and_or<kNibbleMask>(wa << 3, magic); a[1] = and_or<kNibbleMask>(wb << 3, magic);
        a[2] = and_or<kNibbleMask>(wa >> 5, magic); a[3] = and_or<kNibbleMask>(wb >> 5, magic);
    }
}

// ---- one pair row (16 columns x one K unit) of each format.  `row` points at the pair row in
// shared memory, `frag` at this lane's activation fragments of the unit's first 32-element
// group, `sums` at the unit's first per-16 activation sum of row 0, `table` at this warp's
// scale table.  accA / accB are (columns 2t, 2t+1 of the B operand) for output column g / g + 8;
// macc[r] collects this lane's share of the correction dot product of column (lane & 15).
// FRAG_STRIDE = bytes between consecutive 32-element groups of fragments.

template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q4k(const uint8_t* row, const uint8_t* frag, const float* sums,
                                             uint32_t sums_stride, uint8_t* table, uint32_t lane,
                                             f32x2 (&accA)[NT], f32x2 (&accB)[NT], float (&macc)[ROWS]) {
    // Phase A: lane (column, half) decodes the 6-bit scales and minima of groups 4*half .. 4*half+3.
    {
        const uint32_t col = lane & 15u, hf = lane >> 4;
        const uint4 hdr = *reinterpret_cast<const uint4*>(row + 2048u + col * 16u);
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const uint32_t sc4 = hf ? ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u)) : (hdr.y & 0x3f3f3f3fu);
        const uint32_t mn4 = hf ? (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u)) : (hdr.z & 0x3f3f3f3fu);
        const uint32_t magic = opaque_constant(0x4B000000u);
        const f32x2 neg_bias = pack2f(-8388608.0f, -8388608.0f);
        const f32x2 dd = pack2f(d, d), mm = pack2f(dmin, dmin);
        const float2 a01 = unpack2(mul2(dd, byte_pair<0>(sc4, magic, neg_bias)));
        const float2 a23 = unpack2(mul2(dd, byte_pair<2>(sc4, magic, neg_bias)));
        const float2 m01 = unpack2(mul2(mm, byte_pair<0>(mn4, magic, neg_bias)));
        const float2 m23 = unpack2(mul2(mm, byte_pair<2>(mn4, magic, neg_bias)));
        float4* dst = reinterpret_cast<float4*>(table + (col * 8u + hf * 4u) * 8u);
        dst[0] = make_float4(a01.x, a01.x, a01.y, a01.y);
        dst[1] = make_float4(a23.x, a23.x, a23.y, a23.y);
        // Every code carries +16 and every element the group minimum: both multiply the group's
        // activation sum.
        const float b0 = fmaf(kNibbleOffset, a01.x, m01.x), b1 = fmaf(kNibbleOffset, a01.y, m01.y);
        const float b2 = fmaf(kNibbleOffset, a23.x, m23.x), b3 = fmaf(kNibbleOffset, a23.y, m23.y);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4* s = reinterpret_cast<const float4*>(sums + r * sums_stride + hf * 8u);
            const float4 s0 = s[0], s1 = s[1];
            macc[r] = fmaf(b0, s0.x + s0.y, macc[r]);
            macc[r] = fmaf(b1, s0.z + s0.w, macc[r]);
            macc[r] = fmaf(b2, s1.x + s1.y, macc[r]);
            macc[r] = fmaf(b3, s1.z + s1.w, macc[r]);
        }
    }
    __syncwarp();
    // Phase B: chunk c = elements 64c .. 64c+63; its low nibbles are group 2c, its high nibbles 2c+1.
    const uint32_t g = lane >> 2;
    const uint32_t magic = opaque_constant(kNibbleMagic);
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + c * 512 + lane * 16u);
        const ulonglong2 sA = *reinterpret_cast<const ulonglong2*>(table + (g * 8u + 2u * c) * 8u);
        const ulonglong2 sB = *reinterpret_cast<const ulonglong2*>(table + ((g + 8u) * 8u + 2u * c) * 8u);
        uint32_t lo0[4], lo1[4], hi0[4], hi1[4];
        nibble_fragment<0>(w.x, w.z, magic, lo0);
        nibble_fragment<0>(w.y, w.w, magic, lo1);
        nibble_fragment<1>(w.x, w.z, magic, hi0);
        nibble_fragment<1>(w.y, w.w, magic, hi1);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 bl = *reinterpret_cast<const uint4*>(frag + (2 * c) * FRAG_STRIDE + nt * 512);
            const uint4 bh = *reinterpret_cast<const uint4*>(frag + (2 * c + 1) * FRAG_STRIDE + nt * 512);
            float cl[4], ch[4];
            mma_bf16(cl, lo0, bl.x, bl.y, zero);
            mma_bf16(ch, hi0, bh.x, bh.y, zero);
            mma_bf16(cl, lo1, bl.z, bl.w, cl);
            mma_bf16(ch, hi1, bh.z, bh.w, ch);
            accA[nt] = fma2(sA.x, pack2f(cl[0], cl[1]), accA[nt]);
            accB[nt] = fma2(sB.x, pack2f(cl[2], cl[3]), accB[nt]);
            accA[nt] = fma2(sA.y, pack2f(ch[0], ch[1]), accA[nt]);
            accB[nt] = fma2(sB.y, pack2f(ch[2], ch[3]), accB[nt]);
        }
    }
}

// Q6_K codes: low nibble from ql, two high bits from qh, placed in bits 0..5 of the bf16 word
// 0x4300 (128.0, mantissa step 1), so the word reads 128 + code = 160 + q.
constexpr float kQ6Offset = 160.0f;
__device__ __forceinline__ uint32_t q6_pair(uint32_t ql_shifted, uint32_t qh_shifted, uint32_t magic) {
    return and_or<0x000f000fu>(ql_shifted, and_or<0x00300030u>(qh_shifted, magic));
}

template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q6k(const uint8_t* row, const uint8_t* frag, const float* sums,
                                             uint32_t sums_stride, uint8_t* table, uint32_t lane,
                                             f32x2 (&accA)[NT], f32x2 (&accB)[NT], float (&macc)[ROWS]) {
    {   // Phase A: lane (column, half) turns int8 sub-scales 8*half .. 8*half+7 into d*scale.
        const uint32_t col = lane & 15u, hf = lane >> 4;
        const uint2 s8 = *reinterpret_cast<const uint2*>(row + 3072u + col * 16u + hf * 8u);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + 3328u + col * 2u)));
        const uint32_t magic = opaque_constant(0x4B000000u);
        const f32x2 neg_bias = pack2f(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f));   // int8 made unsigned by flipping bit 7
        const f32x2 dd = pack2f(d, d);
        const uint32_t u0 = s8.x ^ 0x80808080u, u1 = s8.y ^ 0x80808080u;
        float a[8];
        { const float2 v = unpack2(mul2(dd, byte_pair<0>(u0, magic, neg_bias))); a[0] = v.x; a[1] = v.y; }
        { const float2 v = unpack2(mul2(dd, byte_pair<2>(u0, magic, neg_bias))); a[2] = v.x; a[3] = v.y; }
        { const float2 v = unpack2(mul2(dd, byte_pair<0>(u1, magic, neg_bias))); a[4] = v.x; a[5] = v.y; }
        { const float2 v = unpack2(mul2(dd, byte_pair<2>(u1, magic, neg_bias))); a[6] = v.x; a[7] = v.y; }
        float4* dst = reinterpret_cast<float4*>(table + (col * 16u + hf * 8u) * 8u);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_float4(a[2 * j], a[2 * j], a[2 * j + 1], a[2 * j + 1]);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4* s = reinterpret_cast<const float4*>(sums + r * sums_stride + hf * 8u);
            const float4 s0 = s[0], s1 = s[1];
            macc[r] = fmaf(a[0], s0.x, macc[r]); macc[r] = fmaf(a[1], s0.y, macc[r]);
            macc[r] = fmaf(a[2], s0.z, macc[r]); macc[r] = fmaf(a[3], s0.w, macc[r]);
            macc[r] = fmaf(a[4], s1.x, macc[r]); macc[r] = fmaf(a[5], s1.y, macc[r]);
            macc[r] = fmaf(a[6], s1.z, macc[r]); macc[r] = fmaf(a[7], s1.w, macc[r]);
        }
    }
    __syncwarp();
    // Phase B: half h = elements 128h .. 128h+127 = four quarters q of 32; 16-element group
    // (q, s) is scale group 8h + 2q + s.  ql byte l of the half serves quarters 0 (low nibble)
    // and 2 (high nibble), byte 32 + l quarters 1 and 3; qh byte l holds two bits per quarter.
    const uint32_t g = lane >> 2;
    const uint32_t magic = opaque_constant(0x43004300u);
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 qa = *reinterpret_cast<const uint4*>(row + h * 1536 + lane * 16u);
        const uint4 qb = *reinterpret_cast<const uint4*>(row + h * 1536 + 512 + lane * 16u);
        const uint4 qh = *reinterpret_cast<const uint4*>(row + h * 1536 + 1024 + lane * 16u);
        uint4 bf[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q)
                bf[nt][q] = *reinterpret_cast<const uint4*>(frag + (4 * h + q) * FRAG_STRIDE + nt * 512);
        ulonglong2 sA[4], sB[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            sA[q] = *reinterpret_cast<const ulonglong2*>(table + (g * 16u + 8u * h + 2u * q) * 8u);
            sB[q] = *reinterpret_cast<const ulonglong2*>(table + ((g + 8u) * 16u + 8u * h + 2u * q) * 8u);
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const uint32_t ae = s ? qa.z : qa.x, ao = s ? qa.w : qa.y;
            const uint32_t be = s ? qb.z : qb.x, bo = s ? qb.w : qb.y;
            const uint32_t ha = s ? qh.y : qh.x, hb = s ? qh.w : qh.z;
            uint32_t a[4][4];
            a[0][0] = q6_pair(ae, ha << 4, magic);       a[0][1] = q6_pair(be, hb << 4, magic);
            a[0][2] = q6_pair(ae >> 8, ha >> 4, magic);  a[0][3] = q6_pair(be >> 8, hb >> 4, magic);
            a[1][0] = q6_pair(ao, ha << 2, magic);       a[1][1] = q6_pair(bo, hb << 2, magic);
            a[1][2] = q6_pair(ao >> 8, ha >> 6, magic);  a[1][3] = q6_pair(bo >> 8, hb >> 6, magic);
            a[2][0] = q6_pair(ae >> 4, ha, magic);       a[2][1] = q6_pair(be >> 4, hb, magic);
            a[2][2] = q6_pair(ae >> 12, ha >> 8, magic); a[2][3] = q6_pair(be >> 12, hb >> 8, magic);
            a[3][0] = q6_pair(ao >> 4, ha >> 2, magic);  a[3][1] = q6_pair(bo >> 4, hb >> 2, magic);
            a[3][2] = q6_pair(ao >> 12, ha >> 10, magic); a[3][3] = q6_pair(bo >> 12, hb >> 10, magic);
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float c[4];
                    mma_bf16(c, a[q], s ? bf[nt][q].z : bf[nt][q].x, s ? bf[nt][q].w : bf[nt][q].y, zero);
                    accA[nt] = fma2(s ? sA[q].y : sA[q].x, pack2f(c[0], c[1]), accA[nt]);
                    accB[nt] = fma2(s ? sB[q].y : sB[q].x, pack2f(c[2], c[3]), accB[nt]);
                }
        }
    }
}

// Q8_0: the byte with bit 7 flipped is v = q + 128 = 16 * hi + lo; both nibbles use the 16 + n
// encoding, so (low product) + 16 * (high product) = sum (272 + v) x = sum (400 + q) x.
constexpr float kQ80Offset = 400.0f;

template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q80(const uint8_t* row, const uint8_t* frag, const float* sums,
                                             uint32_t sums_stride, uint8_t* table, uint32_t lane,
                                             f32x2 (&accA)[NT], f32x2 (&accB)[NT], float (&macc)[ROWS]) {
    {   // Phase A: lane (column, half) widens the f16 scales of blocks 2*half, 2*half+1.
        const uint32_t col = lane & 15u, hf = lane >> 4;
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(row + 2048u + col * 8u + hf * 4u);
        const float d0 = __half2float(__ushort_as_half((unsigned short)(raw & 0xffffu)));
        const float d1 = __half2float(__ushort_as_half((unsigned short)(raw >> 16)));
        *reinterpret_cast<float4*>(table + (col * 4u + hf * 2u) * 8u) = make_float4(d0, d0, d1, d1);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4 s = *reinterpret_cast<const float4*>(sums + r * sums_stride + hf * 4u);
            macc[r] = fmaf(d0, s.x + s.y, macc[r]);
            macc[r] = fmaf(d1, s.z + s.w, macc[r]);
        }
    }
    __syncwarp();
    const uint32_t g = lane >> 2;
    const uint32_t magic = opaque_constant(kNibbleMagic);
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const f32x2 sixteen = pack2f(16.0f, 16.0f);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        uint4 w = *reinterpret_cast<const uint4*>(row + b * 512 + lane * 16u);
        w.x ^= 0x80808080u; w.y ^= 0x80808080u; w.z ^= 0x80808080u; w.w ^= 0x80808080u;
        const f32x2 dA = *reinterpret_cast<const f32x2*>(table + (g * 4u + b) * 8u);
        const f32x2 dB = *reinterpret_cast<const f32x2*>(table + ((g + 8u) * 4u + b) * 8u);
        uint32_t lo0[4], lo1[4], hi0[4], hi1[4];
        nibble_fragment<0>(w.x, w.z, magic, lo0);
        nibble_fragment<0>(w.y, w.w, magic, lo1);
        nibble_fragment<1>(w.x, w.z, magic, hi0);
        nibble_fragment<1>(w.y, w.w, magic, hi1);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 bq = *reinterpret_cast<const uint4*>(frag + b * FRAG_STRIDE + nt * 512);
            float cl[4], ch[4];
            mma_bf16(cl, lo0, bq.x, bq.y, zero);
            mma_bf16(ch, hi0, bq.x, bq.y, zero);
            mma_bf16(cl, lo1, bq.z, bq.w, cl);
            mma_bf16(ch, hi1, bq.z, bq.w, ch);
            accA[nt] = fma2(dA, fma2(sixteen, pack2f(ch[0], ch[1]), pack2f(cl[0], cl[1])), accA[nt]);
            accB[nt] = fma2(dB, fma2(sixteen, pack2f(ch[2], ch[3]), pack2f(cl[2], cl[3])), accB[nt]);
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

// Exact split of two floats into three bf16 terms each: out[i] = (term i of a) | (term i of b) << 16.
__device__ __forceinline__ void split_bf16x3(float a, float b, uint32_t (&out)[3]) {
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        uint32_t bits;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(bits) : "f"(b), "f"(a));   // first source -> upper half
        out[i] = bits;
        a = __fsub_rn(a, __uint_as_float(bits << 16));
        b = __fsub_rn(b, __uint_as_float(bits & 0xffff0000u));
    }
}

// Produces this CTA's K slice of the activation rows in shared memory as B-operand fragments:
// for 32-element group G2, B column n and lane position t the 16 bytes at
// ((G2 * NCP + n) * 4 + t) * 16 hold {(x0, x2), (x1, x3)} of elements 4t .. 4t+3 of the first
// 16 elements and the same of the second 16, as bf16 pairs of term n % 3 of row n / 3.  Also the
// f32 sum of every 16 consecutive elements.  The RMS norms of prologues 1 and 2 need the whole
// row, so every CTA recomputes them from global memory (a few tens of KB out of L2).
template <int ROWS>
__device__ __forceinline__ void stage_activations(const GemvParams& p, uint32_t first, uint32_t count, uint32_t slice,
                                                  uint8_t* frags, float* sums, float* scratch) {
    constexpr uint32_t NCP = gemv_fragment_columns(ROWS);
    float inv0[ROWS], inv1[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { inv0[r] = 1.0f; inv1[r] = 1.0f; }
    if (p.prologue == kPrologueNorm || p.prologue == kPrologueAddNorm) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4* in = reinterpret_cast<const float4*>(p.in + (size_t)r * p.k);
            float sum = 0.0f;
            for (uint32_t c = threadIdx.x; c < p.k / 4u; c += blockDim.x) {
                const float4 v = in[c];
                sum = fmaf(v.x, v.x, sum); sum = fmaf(v.y, v.y, sum); sum = fmaf(v.z, v.z, sum); sum = fmaf(v.w, v.w, sum);
            }
            const float total = gemv_block_sum(sum, scratch);
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)p.k), p.eps)));
            if (p.prologue == kPrologueNorm) { inv1[r] = inv; continue; }
            inv0[r] = inv;
            // r = residual + norm(in) * gamma0; its mean square feeds the second norm.
            const float4* res = reinterpret_cast<const float4*>(p.residual + (size_t)r * p.k);
            const float4* g0 = reinterpret_cast<const float4*>(p.gamma0);
            float4* res_out = reinterpret_cast<float4*>(p.residual_out + (size_t)r * p.k);
            float sum2 = 0.0f;
            for (uint32_t c = threadIdx.x; c < p.k / 4u; c += blockDim.x) {
                const float4 v = in[c], a = res[c], gm = g0[c];
                float4 o;
                o.x = __fadd_rn(a.x, __fmul_rn(__fmul_rn(v.x, inv), gm.x));
                o.y = __fadd_rn(a.y, __fmul_rn(__fmul_rn(v.y, inv), gm.y));
                o.z = __fadd_rn(a.z, __fmul_rn(__fmul_rn(v.z, inv), gm.z));
                o.w = __fadd_rn(a.w, __fmul_rn(__fmul_rn(v.w, inv), gm.w));
                sum2 = fmaf(o.x, o.x, sum2); sum2 = fmaf(o.y, o.y, sum2); sum2 = fmaf(o.z, o.z, sum2); sum2 = fmaf(o.w, o.w, sum2);
                if (blockIdx.x == 0) res_out[c] = o;
            }
            const float total2 = gemv_block_sum(sum2, scratch);
            inv1[r] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total2, (float)p.k), p.eps)));
        }
    }
    const uint32_t quads = slice / 4u;      // a multiple of 32: whole warps stay together
    for (uint32_t q = threadIdx.x; q < (uint32_t)ROWS * quads; q += blockDim.x) {
        const uint32_t r = q / quads, o4 = q % quads, o = o4 * 4u;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (o < count) {
            const size_t gi = (size_t)r * p.k + first + o;
            const uint32_t c = first + o;
            float i0 = 1.0f, i1 = 1.0f;
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) if (rr == (int)r) { i0 = inv0[rr]; i1 = inv1[rr]; }
            const float4 in = *reinterpret_cast<const float4*>(p.in + gi);
            if (p.prologue == kProloguePlain) v = in;
            else if (p.prologue == kPrologueNorm) {
                const float4 gm = *reinterpret_cast<const float4*>(p.gamma1 + c);
                v.x = __fmul_rn(__fmul_rn(in.x, i1), gm.x); v.y = __fmul_rn(__fmul_rn(in.y, i1), gm.y);
                v.z = __fmul_rn(__fmul_rn(in.z, i1), gm.z); v.w = __fmul_rn(__fmul_rn(in.w, i1), gm.w);
            } else if (p.prologue == kPrologueAddNorm) {
                const float4 a = *reinterpret_cast<const float4*>(p.residual + gi);
                const float4 g0 = *reinterpret_cast<const float4*>(p.gamma0 + c);
                const float4 g1 = *reinterpret_cast<const float4*>(p.gamma1 + c);
                v.x = __fmul_rn(__fmul_rn(__fadd_rn(a.x, __fmul_rn(__fmul_rn(in.x, i0), g0.x)), i1), g1.x);
                v.y = __fmul_rn(__fmul_rn(__fadd_rn(a.y, __fmul_rn(__fmul_rn(in.y, i0), g0.y)), i1), g1.y);
                v.z = __fmul_rn(__fmul_rn(__fadd_rn(a.z, __fmul_rn(__fmul_rn(in.z, i0), g0.z)), i1), g1.z);
                v.w = __fmul_rn(__fmul_rn(__fadd_rn(a.w, __fmul_rn(__fmul_rn(in.w, i0), g0.w)), i1), g1.w);
            } else {
                const float4 up = *reinterpret_cast<const float4*>(p.residual + gi);
                v.x = __fmul_rn(gelu_tanh_exact(in.x), up.x); v.y = __fmul_rn(gelu_tanh_exact(in.y), up.y);
                v.z = __fmul_rn(gelu_tanh_exact(in.z), up.z); v.w = __fmul_rn(gelu_tanh_exact(in.w), up.w);
            }
        }
        uint32_t b0[3], b1[3];
        split_bf16x3(v.x, v.z, b0);
        split_bf16x3(v.y, v.w, b1);
        const uint32_t g2 = o4 >> 3, parity = (o4 >> 2) & 1u, t = o4 & 3u;
        uint8_t* dst = frags + ((size_t)g2 * NCP * 4u + t) * 16u + parity * 8u;
#pragma unroll
        for (int i = 0; i < 3; ++i) *reinterpret_cast<uint2*>(dst + (3u * r + i) * 64u) = make_uint2(b0[i], b1[i]);
        if (r == 0) {
#pragma unroll
            for (uint32_t n = 3u * ROWS; n < NCP; ++n) *reinterpret_cast<uint2*>(dst + n * 64u) = make_uint2(0u, 0u);
        }
        float s = (v.x + v.y) + (v.z + v.w);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (t == 0u) sums[r * (slice / 16u) + (o4 >> 2)] = s;
    }
}

template <int ROWS>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
    constexpr int NT = (3 * ROWS + 7) / 8;
    constexpr uint32_t NCP = gemv_fragment_columns(ROWS);
    constexpr uint32_t FRAG_STRIDE = NCP * 64u;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[kGemvWarps];
    const GemvSmemLayout lay = gemv_smem_layout(ROWS, p.chunk_units, p.unit_elems, p.slot_bytes, p.table_bytes);
    const uint32_t slice = p.chunk_units * p.unit_elems;
    uint8_t* frags = smem;
    float* sums = reinterpret_cast<float*>(smem + lay.frag_bytes);
    uint8_t* ring_base = smem + lay.frag_bytes + lay.sums_bytes;
    uint8_t* table_base = ring_base + lay.ring_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(table_base + lay.table_bytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint8_t* ring = ring_base + warp * (kGemvSlots * p.slot_bytes);
    uint8_t* table = table_base + warp * p.table_bytes;
    uint64_t* bar = bars + warp * kGemvSlots;

    // This CTA's K chunk and this warp's sequence of column pairs (over all matrices).
    const uint32_t chunk = blockIdx.x % p.chunks;
    const uint32_t group_ctas = gridDim.x / p.chunks;
    const uint32_t first_unit = chunk * p.chunk_units;
    const uint32_t chunk_count = min(p.chunk_units, p.units - first_unit);
    const uint32_t stride = group_ctas * kGemvWarps;
    const uint32_t first_pair = (blockIdx.x / p.chunks) * kGemvWarps + warp;
    const uint32_t my_items = first_pair < p.total_pairs ? (p.total_pairs - first_pair + stride - 1u) / stride : 0u;

    auto matrix_of = [&](uint32_t pair) -> uint32_t {
        uint32_t m = 0;
        if (p.matrices > 1u && pair >= p.m[1].first_pair) m = 1;
        if (p.matrices > 2u && pair >= p.m[2].first_pair) m = 2;
        return m;
    };

    if (lane == 0) {
        for (int s = 0; s < kGemvSlots; ++s) mbar_init(&bar[s], 1);
        fence_barrier_init();
    }
    __syncwarp();

    // Producer cursor (lane 0): the next pair row to request, walking items then units.
    uint32_t prod_item = 0, prod_unit = 0, prod_slot = 0, prod_bytes = 0;
    const uint8_t* prod_src = nullptr;
    auto issue_next = [&]() {   // lane 0 only
        if (prod_item >= my_items) return;
        if (prod_unit == 0u) {
            const uint32_t pair = first_pair + prod_item * stride;
            const GemvMatrix& mat = p.m[matrix_of(pair)];
            prod_bytes = pair_row_bytes((int)mat.dtype);
            prod_src = mat.weight + ((size_t)(pair - mat.first_pair) * p.units + first_unit) * prod_bytes;
        }
        mbar_expect_tx(&bar[prod_slot], prod_bytes);
        bulk_load(ring + prod_slot * p.slot_bytes, prod_src, prod_bytes, &bar[prod_slot]);
        prod_src += prod_bytes;
        prod_slot = prod_slot + 1u == (uint32_t)kGemvSlots ? 0u : prod_slot + 1u;
        if (++prod_unit == chunk_count) { prod_unit = 0; ++prod_item; }
    };
    // Weights do not depend on the previous kernel: start streaming before waiting for it.
    if (lane == 0)
        for (int j = 0; j < kGemvSlots; ++j) issue_next();

    pdl_wait();
    stage_activations<ROWS>(p, first_unit * p.unit_elems, chunk_count * p.unit_elems, slice, frags, sums, scratch);
    __syncthreads();
    pdl_launch_dependents();

    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint8_t* my_frag = frags + ((g & (NCP - 1u)) * 4u + t) * 16u;
    const uint32_t sums_stride = slice / 16u;
    const uint32_t quad_base = lane & ~3u;

    f32x2 accA[NT], accB[NT];
    float macc[ROWS];
    bool failed = false;
    uint32_t slot = 0, phase = 0;
    for (uint32_t item = 0; item < my_items && !failed; ++item) {
        const uint32_t pair = first_pair + item * stride;
        const GemvMatrix& mat = p.m[matrix_of(pair)];
        const uint32_t dtype = mat.dtype;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { accA[nt] = 0ull; accB[nt] = 0ull; }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) macc[r] = 0.0f;
        for (uint32_t u = 0; u < chunk_count; ++u) {
            if (!mbar_wait(&bar[slot], phase)) { failed = true; break; }
            const uint8_t* row = ring + slot * p.slot_bytes;
            if (dtype == GF_Q4_K)
                pair_row_q4k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                    table, lane, accA, accB, macc);
            else if (dtype == GF_Q6_K)
                pair_row_q6k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                    table, lane, accA, accB, macc);
            else
                pair_row_q80<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 4u * FRAG_STRIDE, sums + u * 8u, sums_stride,
                                                    table, lane, accA, accB, macc);
            __syncwarp();   // every lane has finished reading this slot and the scale table
            if (lane == 0) issue_next();
            if (++slot == (uint32_t)kGemvSlots) { slot = 0; phase ^= 1u; }
        }
        if (failed) break;
        // Row r is the sum of B columns 3r, 3r+1, 3r+2 (held by quad lanes (n % 8) / 2 of n-tile
        // n / 8), minus the correction dot product of its column.
        const float offset = dtype == GF_Q4_K ? 1.0f : dtype == GF_Q6_K ? kQ6Offset : kQ80Offset;
        float totalA[ROWS], totalB[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float partA[3], partB[3];
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int n = 3 * r + i, nt = n / 8, holder = (n % 8) / 2;
                const float2 a = unpack2(accA[nt]), b = unpack2(accB[nt]);
                partA[i] = __shfl_sync(0xffffffffu, (n & 1) ? a.y : a.x, quad_base + holder);
                partB[i] = __shfl_sync(0xffffffffu, (n & 1) ? b.y : b.x, quad_base + holder);
            }
            float m = macc[r];
            m += __shfl_xor_sync(0xffffffffu, m, 16);
            const float mA = __shfl_sync(0xffffffffu, m, g), mB = __shfl_sync(0xffffffffu, m, g + 8u);
            totalA[r] = __fsub_rn(__fadd_rn(__fadd_rn(partA[0], partA[1]), partA[2]), __fmul_rn(offset, mA));
            totalB[r] = __fsub_rn(__fadd_rn(__fadd_rn(partB[0], partB[1]), partB[2]), __fmul_rn(offset, mB));
        }
        const uint32_t local_pair = pair - mat.first_pair;
        const uint32_t columnA = local_pair * 16u + g, columnB = columnA + 8u;
        if (p.chunks == 1u) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (t == (uint32_t)(r & 3)) {
                    if (columnA < mat.n) mat.out[(size_t)r * mat.n + columnA] = totalA[r];
                    if (columnB < mat.n) mat.out[(size_t)r * mat.n + columnB] = totalB[r];
                }
            continue;
        }
        // Split K: park this chunk's partial sums; the warp that arrives last for the pair adds
        // all chunks in chunk order (so the result does not depend on arrival order).
        const size_t width = (size_t)p.total_pairs * 16u;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (t == (uint32_t)(r & 3)) {
                float* dst = p.partial + ((size_t)chunk * ROWS + r) * width + (size_t)pair * 16u;
                dst[g] = totalA[r];
                dst[g + 8u] = totalB[r];
            }
        __threadfence();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atomicAdd(&p.counters[pair], 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == p.chunks - 1u) {
            __threadfence();
            for (uint32_t idx = lane; idx < (uint32_t)ROWS * 16u; idx += 32u) {
                const uint32_t r = idx >> 4, col = idx & 15u;
                float sum = 0.0f;
                for (uint32_t c = 0; c < p.chunks; ++c)
                    sum += __ldcg(&p.partial[((size_t)c * ROWS + r) * width + (size_t)pair * 16u + col]);
                const uint32_t out_column = local_pair * 16u + col;
                if (out_column < mat.n) mat.out[(size_t)r * mat.n + out_column] = sum;
            }
            if (lane == 0) p.counters[pair] = 0u;
        }
    }
    if (failed) {
        // Give outstanding copies a bounded chance to land before the shared memory is released.
        for (int s = 0; s < kGemvSlots; ++s) mbar_wait(&bar[s], 0);
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
struct GemvPlan { uint32_t units, unit_elems, total_pairs, chunks, chunk_units, grid, smem, slot_bytes, table_bytes; };

int gemv_plan(const GemvLaunch& launch, GemvPlan& plan);
// Split-K scratch of one launch: `partial` bytes of sums, and one arrival counter per column pair.
// Counters must be zero before a launch and are left zero by it; they must not share memory
// with any launch's partial sums.
size_t gemv_partial_bytes(const GemvLaunch& launch);
size_t gemv_counter_bytes(const GemvLaunch& launch);
int gemv_launch(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                cudaStream_t stream, bool programmatic);

}  // namespace gf
