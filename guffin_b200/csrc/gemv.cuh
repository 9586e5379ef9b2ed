// Weight-streaming dequant-GEMV core for Q4_K / Q6_K / Q8_0, rows M <= 4.
//
// Work decomposition: an item is (column pair of 16 outputs, K chunk).  A CTA is bound to one
// K chunk and stages that slice of the activation rows in shared memory once; each of its
// warps then streams whole items through a private ring of shared-memory slots filled by
// one-shot TMA bulk copies (cp.async.bulk + mbarrier), so no block-level synchronisation
// happens while weights stream.
//
// Arithmetic: the quantised codes are small integers, so the products run on the integer tensor
// cores.  One logic instruction turns four packed nibbles into four u8 elements of the A operand
// of mma.m16n8k32 (16 output columns x 32 K positions; Q8_0 bytes are the operand as they are).
// The activations become block fixed point: every 256 consecutive elements of a row share a
// power-of-two scale, each element is a 31-bit integer of that scale, and its four signed bytes
// are four columns of the s8 B operand.  Integer accumulation is exact; the integer group scales
// of Q4_K / Q6_K are applied with integer multiply-adds, and one conversion per 256-element block
// (per 32-element block for Q8_0) brings the sum back to f32, where it meets the block's f16
// scale and the activation scale.  The result differs from exact arithmetic by the 2^-30
// quantisation of the activations and one f32 rounding per block, which is tighter than an f32
// multiply-add chain.  The Q4_K minima and the Q6_K offset of 32 reduce to one dot product per
// column with per-group activation sums, taken while the scales are decoded.
//
// Row r's arithmetic does not depend on how many rows are computed beside it (its four B
// columns are independent of the others), and partial sums of different K chunks are added in
// chunk order, so results are reproducible and row-count invariant.
#pragma once

#include "common.cuh"

namespace gf {

constexpr int kGemvWarps = 16;       // warps per CTA; one CTA per SM
constexpr int kGemvSlots = 2;        // ring depth per warp; a slot holds `slot_units` consecutive pair rows of an item
constexpr uint32_t kGemvSmemLimit = 225u * 1024u;    // dynamic part; the static arrays take the rest of the 227 KB
constexpr int kGemvMaxMatrices = 3;

// How the activation rows are produced from global memory before the weights are applied.
enum GemvPrologue : uint32_t {
    kProloguePlain = 0,      // xs = in
    kPrologueNorm = 1,       // xs = rmsnorm(in; gamma1)
    kPrologueAddNorm = 2,    // r = residual + rmsnorm(in; gamma0) -> residual_out;  xs = rmsnorm(r; gamma1)
                             // (`residual` is read before the dependency wait: a launch that directly follows its
                             //  writer under programmatic dependent launch must not be given it)
    kPrologueGeglu = 3,      // xs = gelu_tanh(in) * residual
    kPrologueMerge = 4,      // xs = the attention output merged from partition results: `in` holds [row][head][32][256]
                             // unnormalised outputs, `residual` the (maximum, sum) pair of every slot (empty: sum 0)
};

constexpr int kGemvMaxShards = 8;

struct GemvMatrix {
    const uint8_t* weight;   // streaming layout
    float* out;              // [rows][n]
    uint32_t n, pairs, dtype, first_pair;
};

struct WeightStreamParams {
    GemvMatrix m[kGemvMaxMatrices];
    uint32_t matrices, total_pairs;
    uint32_t k, units, unit_elems;
    uint32_t active_rows;                 // rows that exist; the kernel instance may be compiled for more
    uint32_t chunks, chunk_units;         // K chunks spread over CTAs (hand-over through L2), K units per chunk
    uint32_t intra, staged_units;         // K chunks spread over the warps of one CTA (1 = none; hand-over in shared
                                          // memory, `chunks` is then 1); K units of the activation slice a CTA stages
    uint32_t slot_bytes, slot_units;      // ring slot size; pair rows (K units) copied and consumed per slot
    uint32_t grid;                        // CTAs that take part (the launch's grid; a pass kernel's CTAs beyond it idle)
    uint32_t wait_limit;                  // polls before a wait for weights gives up (kMbarWaitLimit)
    uint32_t overstate;                   // bytes the launch's very first copy claims beyond what it brings (0; a testing build's fault seam)
    uint32_t prologue;
    const float *in, *residual, *gamma0, *gamma1;
    float* residual_out;
    float eps;
    // Optional head epilogue of a fused Q/K/V launch (matrix 0 = Q, 1 = K, 2 = V, 256 columns per
    // head): the warp that completes a head's last column pair applies the per-head RMSNorm and
    // the NEOX rotation and writes the rotated query (f32) or the private K/V row of the cache.
    struct HeadEpilogue {
        const float *q_norm, *k_norm;        // [256] or null
        float* q_out;                        // [rows][heads * 256]
        void *private_k, *private_v;         // [rows][kv_heads * 256] in the cache type
        const float2* rotation;              // [table_rows][128] (cos, sin) of position * scale / base^(2i/256)
        const uint32_t* base_position;
        uint32_t* status;
        uint32_t* head_counters;             // [heads + 2 * kv_heads], zero between launches
        uint32_t enabled, table_rows, kv_f16;
        float eps;
        uint32_t row_base;                   // rows ahead of row 0 of this launch in the pass (the second half of a 5..8-row pass: 4)
    } heads;
    float* partial;            // [chunks][rows][total_pairs * 16] when chunks > 1
    uint32_t* counters;        // [total_pairs] arrival counts, zero between launches
    int* error_flag;           // set to 1 when a bounded wait gives up
    // Tensor-parallel shards (the TP instantiation only; both off when their count is 0).  A shard's O and down
    // projections hold partial sums of the hidden rows.  The producing launch mirrors every output value it writes
    // into each peer GPU's arena as an 8-byte (value, stamp) pair -- one plain store over NVLink, the stamp naming
    // the pass and the projection -- and the consuming launch reads its input as the sum of all shards' parts in
    // shard order (so every shard holds the same bits), polling each peer's pairs until they carry the stamp it
    // expects.  No fence, flag or extra launch: a value is usable the moment it lands.  The polls are bounded.
    struct Scatter {
        uint2* out[kGemvMaxShards - 1];          // matrix 0's output [rows][n] as stamped pairs in each peer's arena
        const uint32_t* tick;                    // this GPU's pass counter
        uint32_t count, site;                    // peers; which projection of the pass (1 ..)
    } scatter;
    struct Gather {
        const uint2* parts[kGemvMaxShards];      // the peers' stamped parts in this GPU's arena, by shard (own entry unused)
        const float* own;                        // this shard's part
        const uint32_t* tick;
        uint32_t count, self, site;              // shards; this shard's index; the producing projection
        uint32_t wait_limit;                     // polls before a wait for a peer's value gives up
    } gather;
};

// Columns of the B operand kept per 32-element group: four signed bytes per row, in whole n-tiles
// of eight (one row uses half a tile).
__host__ __device__ constexpr uint32_t gemv_fragment_columns(uint32_t rows) {
    return rows == 1u ? 4u : ((4u * rows + 7u) / 8u) * 8u;
}
// Bytes between the B registers of consecutive 32-element groups: 32 per column plus 32 of padding,
// so that the lanes of a warp that quantise eight consecutive groups at once store to different
// banks (without it the groups are a multiple of 128 bytes apart and collide eight ways).
__host__ __device__ constexpr uint32_t gemv_fragment_stride(uint32_t rows) { return gemv_fragment_columns(rows) * 32u + 32u; }

struct GemvSmemLayout {
    uint32_t frag_bytes, sums_bytes, scale_bytes, ring_bytes, staging_bytes, total;
};
// Shared-memory meeting place of the warps that split K inside a CTA: [warp][row][16 columns] f32.
__host__ __device__ constexpr uint32_t gemv_meeting_bytes(uint32_t rows) { return (uint32_t)kGemvWarps * rows * 16u * 4u; }
// Ring, its barriers and the per-warp cursor records (the size of WeightCursor, checked where it is defined).
constexpr uint32_t kGemvCursorBytes = 96u;
__host__ __device__ constexpr uint32_t gemv_ring_bytes(uint32_t slot_bytes) {
    return (uint32_t)kGemvWarps * kGemvSlots * slot_bytes + (uint32_t)kGemvWarps * kGemvSlots * 8u + (uint32_t)kGemvWarps * kGemvCursorBytes;
}

// [ring | barriers | cursors | fragments | sums | scales | meeting]
__host__ __device__ inline GemvSmemLayout gemv_smem_layout(uint32_t rows, uint32_t chunk_units, uint32_t unit_elems,
                                                           uint32_t slot_bytes, bool meeting = false) {
    GemvSmemLayout s;
    const uint32_t slice = chunk_units * unit_elems, padded = (slice + 255u) & ~255u;
    s.frag_bytes = (padded / 32u) * gemv_fragment_stride(rows);
    s.sums_bytes = rows * (padded / 16u) * 4u;
    s.scale_bytes = ((rows * (padded / 256u) * 4u) + 15u) & ~15u;
    s.ring_bytes = gemv_ring_bytes(slot_bytes);
    s.staging_bytes = s.frag_bytes + s.sums_bytes + s.scale_bytes + (meeting ? gemv_meeting_bytes(rows) : 0u);
    s.total = s.ring_bytes + s.staging_bytes + 64u;
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

// A constant the compiler cannot fold into an immediate (a logic instruction encodes only one).
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
// Byte K of v as an unsigned / sign-extended 32-bit integer: one byte-permute instruction.
template <uint32_t K>
__device__ __forceinline__ int byte_u(uint32_t v) { return (int)__byte_perm(v, 0u, 0x4440u + K); }
template <uint32_t K>
__device__ __forceinline__ int byte_s(uint32_t v) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(v), "r"(0u), "n"(((K | 8u) << 12) | ((K | 8u) << 8) | ((K | 8u) << 4) | K));
    return (int)r;
}

// Integer tensor-core products, s32 accumulation.  Lane (g, t), g = lane / 4, t = lane % 4.
// k32: A registers are (row g, k 4t..4t+3), (row g+8, same k), (row g, k 16+4t..), (row g+8, same);
// B registers are (k 4t..4t+3, column g), (k 16+4t.., column g).  k16: the first two A registers
// and the first B register.  C/D are (row g, columns 2t, 2t+1), (row g+8, columns 2t, 2t+1).
__device__ __forceinline__ void mma_u8s8_k32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
__device__ __forceinline__ void mma_s8s8_k32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %8, %9, %10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Per-lane context of the consumer loops.
struct GemvLane {
    uint32_t lane, g, t;
    f32x2 digit_weight;       // (256^i0, 256^i1): weights of the two B columns this lane's C registers hold
};

// Adds the integer sums of one activation block to the f32 accumulators.  sums = (row g: columns
// 2t, 2t+1; row g+8: the same); block_scale = the activation block's power of two for this lane's
// row; dA / dB = the f16 block scales of output columns g / g + 8.
__device__ __forceinline__ void fold_block(const int (&sums)[4], float block_scale, float dA, float dB,
                                           const GemvLane& L, f32x2& accA, f32x2& accB) {
    const f32x2 w = mul2(pack2f(block_scale, block_scale), L.digit_weight);
    accA = fma2(mul2(pack2f(dA, dA), w), pack2f(__int2float_rn(sums[0]), __int2float_rn(sums[1])), accA);
    accB = fma2(mul2(pack2f(dB, dB), w), pack2f(__int2float_rn(sums[2]), __int2float_rn(sums[3])), accB);
}

// ---- one pair row (16 columns x one K unit) of each format.  `row` points at the pair row in
// shared memory, `frag` at this lane's B registers of the unit's first 32-element group, `sums`
// at the unit's first per-16 activation sum of row 0, `scales` at the unit's activation block
// scales of this lane's rows.  Everything a lane needs about its two output columns (g and g + 8)
// it decodes itself from the pair row, so the warp never synchronises inside a pair row.
// accA / accB are (columns 2t, 2t+1 of the B operand) for output column g / g + 8; maccA / maccB
// collect this lane's share (a quarter of the scale groups) of the correction dot product of
// those columns.  FRAG_STRIDE = bytes between consecutive 32-element groups of B registers;
// n-tile nt starts 256 bytes further.

template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q4k(const uint8_t* row, const uint8_t* frag, const float* sums,
                                             uint32_t sums_stride, const float* scales, const GemvLane& L,
                                             f32x2 (&accA)[NT], f32x2 (&accB)[NT], float (&maccA)[ROWS], float (&maccB)[ROWS]) {
    // Headers of this lane's two columns: d, dmin and the twelve bytes of 6-bit scales and minima.
    const uint4 hA = *reinterpret_cast<const uint4*>(row + 2048u + L.g * 16u);
    const uint4 hB = *reinterpret_cast<const uint4*>(row + 2048u + (L.g + 8u) * 16u);
    const uint32_t scA[2] = {hA.y & 0x3f3f3f3fu, (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u)};   // groups 0-3, 4-7
    const uint32_t scB[2] = {hB.y & 0x3f3f3f3fu, (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u)};
    {   // Minima of groups 2t, 2t+1 (this lane's share of the correction term) times the groups' activation sums.
        const uint32_t mnA = L.t < 2u ? (hA.z & 0x3f3f3f3fu) : (((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u));
        const uint32_t mnB = L.t < 2u ? (hB.z & 0x3f3f3f3fu) : (((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u));
        const uint32_t shift = (L.t & 1u) * 16u;
        const uint32_t magic = opaque_constant(0x4B000000u);
        const f32x2 neg_bias = pack2f(-8388608.0f, -8388608.0f);
        const float dminA = __half2float(__ushort_as_half((unsigned short)(hA.x >> 16)));
        const float dminB = __half2float(__ushort_as_half((unsigned short)(hB.x >> 16)));
        const float2 mA = unpack2(mul2(pack2f(dminA, dminA), byte_pair<0>(mnA >> shift, magic, neg_bias)));
        const float2 mB = unpack2(mul2(pack2f(dminB, dminB), byte_pair<0>(mnB >> shift, magic, neg_bias)));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4 sm = *reinterpret_cast<const float4*>(sums + r * sums_stride + L.t * 4u);
            const float x0 = sm.x + sm.y, x1 = sm.z + sm.w;
            maccA[r] = fmaf(mA.y, x1, fmaf(mA.x, x0, maccA[r]));
            maccB[r] = fmaf(mB.y, x1, fmaf(mB.x, x0, maccB[r]));
        }
    }
    const float dA = __half2float(__ushort_as_half((unsigned short)(hA.x & 0xffffu)));
    const float dB = __half2float(__ushort_as_half((unsigned short)(hB.x & 0xffffu)));
    // Chunk c = elements 64c .. 64c+63; its low nibbles are group 2c, its high nibbles 2c+1.
    const int zero[4] = {0, 0, 0, 0};
    int total[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[nt][i] = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + c * 512 + L.lane * 16u);
        const uint32_t lo[4] = {w.x & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu};
        const uint32_t hi[4] = {(w.x >> 4) & 0x0f0f0f0fu, (w.z >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu};
        const uint32_t wordA = scA[c >> 1], wordB = scB[c >> 1];
        const int sAl = (c & 1) ? byte_u<2>(wordA) : byte_u<0>(wordA), sAh = (c & 1) ? byte_u<3>(wordA) : byte_u<1>(wordA);
        const int sBl = (c & 1) ? byte_u<2>(wordB) : byte_u<0>(wordB), sBh = (c & 1) ? byte_u<3>(wordB) : byte_u<1>(wordB);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint2 bl = *reinterpret_cast<const uint2*>(frag + (2 * c) * FRAG_STRIDE + nt * 256);
            const uint2 bh = *reinterpret_cast<const uint2*>(frag + (2 * c + 1) * FRAG_STRIDE + nt * 256);
            int cl[4], ch[4];
            mma_u8s8_k32(cl, lo, bl.x, bl.y, zero);
            mma_u8s8_k32(ch, hi, bh.x, bh.y, zero);
            total[nt][0] += sAl * cl[0] + sAh * ch[0];
            total[nt][1] += sAl * cl[1] + sAh * ch[1];
            total[nt][2] += sBl * cl[2] + sBh * ch[2];
            total[nt][3] += sBl * cl[3] + sBh * ch[3];
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) fold_block(total[nt], scales[nt], dA, dB, L, accA[nt], accB[nt]);
}

// Q6_K: code = ql nibble | two qh bits << 4 (0..63), value = code - 32; the offset goes through
// the activation sums.
template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q6k(const uint8_t* row, const uint8_t* frag, const float* sums,
                                             uint32_t sums_stride, const float* scales, const GemvLane& L,
                                             f32x2 (&accA)[NT], f32x2 (&accB)[NT], float (&maccA)[ROWS], float (&maccB)[ROWS]) {
    // The sixteen int8 sub-scales and the f16 scale of this lane's two columns.
    const uint4 scA = *reinterpret_cast<const uint4*>(row + 3072u + L.g * 16u);
    const uint4 scB = *reinterpret_cast<const uint4*>(row + 3072u + (L.g + 8u) * 16u);
    const float dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + 3328u + L.g * 2u)));
    const float dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + 3328u + (L.g + 8u) * 2u)));
    {   // This lane's share of the correction term: d * scale_j * (sum of group j) for groups 4t .. 4t+3.
        const uint32_t wA = L.t == 0u ? scA.x : L.t == 1u ? scA.y : L.t == 2u ? scA.z : scA.w;
        const uint32_t wB = L.t == 0u ? scB.x : L.t == 1u ? scB.y : L.t == 2u ? scB.z : scB.w;
        const uint32_t magic = opaque_constant(0x4B000000u);
        const f32x2 neg_bias = pack2f(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f));   // int8 made unsigned by flipping bit 7
        const f32x2 ddA = pack2f(dA, dA), ddB = pack2f(dB, dB);
        const float2 a01 = unpack2(mul2(ddA, byte_pair<0>(wA ^ 0x80808080u, magic, neg_bias)));
        const float2 a23 = unpack2(mul2(ddA, byte_pair<2>(wA ^ 0x80808080u, magic, neg_bias)));
        const float2 b01 = unpack2(mul2(ddB, byte_pair<0>(wB ^ 0x80808080u, magic, neg_bias)));
        const float2 b23 = unpack2(mul2(ddB, byte_pair<2>(wB ^ 0x80808080u, magic, neg_bias)));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float4 sm = *reinterpret_cast<const float4*>(sums + r * sums_stride + L.t * 4u);
            maccA[r] = fmaf(a23.y, sm.w, fmaf(a23.x, sm.z, fmaf(a01.y, sm.y, fmaf(a01.x, sm.x, maccA[r]))));
            maccB[r] = fmaf(b23.y, sm.w, fmaf(b23.x, sm.z, fmaf(b01.y, sm.y, fmaf(b01.x, sm.x, maccB[r]))));
        }
    }
    // Half h = elements 128h .. 128h+127 = four quarters q of 32; 16-element group (q, s) is scale
    // group 8h + 2q + s.  ql byte l of the half serves quarters 0 (low nibble) and 2 (high nibble),
    // byte 32 + l quarters 1 and 3; qh byte l holds two bits per quarter.
    const int zero[4] = {0, 0, 0, 0};
    int total[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[nt][i] = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 qa = *reinterpret_cast<const uint4*>(row + h * 1536 + L.lane * 16u);
        const uint4 qb = *reinterpret_cast<const uint4*>(row + h * 1536 + 512 + L.lane * 16u);
        const uint4 qh = *reinterpret_cast<const uint4*>(row + h * 1536 + 1024 + L.lane * 16u);
        const uint32_t lowA = h ? scA.z : scA.x, highA = h ? scA.w : scA.y;     // scale bytes 8h..8h+3, 8h+4..8h+7
        const uint32_t lowB = h ? scB.z : scB.x, highB = h ? scB.w : scB.y;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const uint32_t ae = s ? qa.z : qa.x, ao = s ? qa.w : qa.y;
            const uint32_t be = s ? qb.z : qb.x, bo = s ? qb.w : qb.y;
            const uint32_t ha = s ? qh.y : qh.x, hb = s ? qh.w : qh.z;
            uint32_t a[4][2];
            a[0][0] = and_or<0x0f0f0f0fu>(ae, (ha << 4) & 0x30303030u);      a[0][1] = and_or<0x0f0f0f0fu>(be, (hb << 4) & 0x30303030u);
            a[1][0] = and_or<0x0f0f0f0fu>(ao, (ha << 2) & 0x30303030u);      a[1][1] = and_or<0x0f0f0f0fu>(bo, (hb << 2) & 0x30303030u);
            a[2][0] = and_or<0x0f0f0f0fu>(ae >> 4, ha & 0x30303030u);        a[2][1] = and_or<0x0f0f0f0fu>(be >> 4, hb & 0x30303030u);
            a[3][0] = and_or<0x0f0f0f0fu>(ao >> 4, (ha >> 2) & 0x30303030u); a[3][1] = and_or<0x0f0f0f0fu>(bo >> 4, (hb >> 2) & 0x30303030u);
            // Scale group 8h + 2q + s: byte 2q + s of the half's eight.
            int sA[4], sB[4];
            if (s == 0) {
                sA[0] = byte_s<0>(lowA); sA[1] = byte_s<2>(lowA); sA[2] = byte_s<0>(highA); sA[3] = byte_s<2>(highA);
                sB[0] = byte_s<0>(lowB); sB[1] = byte_s<2>(lowB); sB[2] = byte_s<0>(highB); sB[3] = byte_s<2>(highB);
            } else {
                sA[0] = byte_s<1>(lowA); sA[1] = byte_s<3>(lowA); sA[2] = byte_s<1>(highA); sA[3] = byte_s<3>(highA);
                sB[0] = byte_s<1>(lowB); sB[1] = byte_s<3>(lowB); sB[2] = byte_s<1>(highB); sB[3] = byte_s<3>(highB);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t b = *reinterpret_cast<const uint32_t*>(frag + (4 * h + q) * FRAG_STRIDE + nt * 256 + s * 4);
                    int c[4];
                    mma_u8s8_k16(c, a[q][0], a[q][1], b, zero);
                    total[nt][0] += sA[q] * c[0]; total[nt][1] += sA[q] * c[1];
                    total[nt][2] += sB[q] * c[2]; total[nt][3] += sB[q] * c[3];
                }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) fold_block(total[nt], scales[nt], dA, dB, L, accA[nt], accB[nt]);
}

// Q8_0: the int8 codes are the A operand as stored; one f16 scale per 32-element block.
template <int ROWS, int NT, uint32_t FRAG_STRIDE>
__device__ __forceinline__ void pair_row_q80(const uint8_t* row, const uint8_t* frag, const float* scales,
                                             const GemvLane& L, f32x2 (&accA)[NT], f32x2 (&accB)[NT]) {
    const uint2 dhA = *reinterpret_cast<const uint2*>(row + 2048u + L.g * 8u);          // four f16 block scales
    const uint2 dhB = *reinterpret_cast<const uint2*>(row + 2048u + (L.g + 8u) * 8u);
    const int zero[4] = {0, 0, 0, 0};
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + b * 512 + L.lane * 16u);
        const uint32_t a[4] = {w.x, w.z, w.y, w.w};
        const uint32_t rawA = b < 2 ? dhA.x : dhA.y, rawB = b < 2 ? dhB.x : dhB.y;
        const float dA = __half2float(__ushort_as_half((unsigned short)((b & 1) ? rawA >> 16 : rawA & 0xffffu)));
        const float dB = __half2float(__ushort_as_half((unsigned short)((b & 1) ? rawB >> 16 : rawB & 0xffffu)));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint2 bq = *reinterpret_cast<const uint2*>(frag + b * FRAG_STRIDE + nt * 256);
            int c[4];
            mma_s8s8_k32(c, a, bq.x, bq.y, zero);
            fold_block(c, scales[nt], dA, dB, L, accA[nt], accB[nt]);
        }
    }
}

// ---- activation prologue ----

__device__ __forceinline__ float gelu_tanh_exact(float v) {
    const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
}

// Sums over the block of ROWS values per thread; every thread gets the totals (fixed order).
// `scratch` holds kGemvWarps * ROWS floats and must not be reused before the next block barrier.
template <int ROWS>
__device__ __forceinline__ void gemv_block_sums(float (&v)[ROWS], float* scratch) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        v[r] = warp_sum(v[r]);
        if (lane == 0) scratch[r * kGemvWarps + warp] = v[r];
    }
    __syncthreads();
    // Every warp adds the kGemvWarps partial sums of each row the same way: lane w holds warp w's.
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        float part = lane < (uint32_t)kGemvWarps ? scratch[r * kGemvWarps + lane] : 0.0f;
#pragma unroll
        for (int offset = 8; offset > 0; offset >>= 1) part += __shfl_xor_sync(0xffffffffu, part, offset);
        v[r] = __shfl_sync(0xffffffffu, part, 0);
    }
}
// 1 / sqrt(mean square + eps): hardware reciprocal square root plus one Newton step (about one ulp;
// the exact divide and square root sequences cost more than the rest of the prologue).
__device__ __forceinline__ float rms_scale(float sum_of_squares, uint32_t k, float eps) {
    const float a = fmaf(sum_of_squares, 1.0f / (float)k, eps);
    const float y = rsqrtf(a);
    return y * fmaf(-0.5f * a, y * y, 1.5f);
}
__device__ __forceinline__ float sum_squares(const float (&v)[8], float sum) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sum = fmaf(v[i], v[i], sum);
    return sum;
}
__device__ __forceinline__ void load8f(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// Activations written by other CTAs (of the launch ahead, or of an earlier phase of the same pass
// kernel, whose stale copy may still sit in this SM's L1): read from L2.
__device__ __forceinline__ void load8f_cg(const float* p, float (&v)[8]) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// Activations of a launch of its own come through L1 like any other load (nothing on this SM can hold an
// older copy: L1 starts empty with the launch); a phase of a pass kernel reads them from L2.
template <bool FROM_L2>
__device__ __forceinline__ void load8f_act(const float* p, float (&v)[8]) {
    if (FROM_L2) load8f_cg(p, v); else load8f(p, v);
}
// The stamp of projection `site` of the pass the counter names: distinct from the stamp of whatever the same place
// of the arena held before (the previous projection of this pass, or of the pass before).
__device__ __forceinline__ uint32_t shard_stamp(const uint32_t* tick, uint32_t site) { return (__ldcg(tick) << 8) | site; }
// Eight consecutive values of a peer's part: polled until all eight pairs carry `stamp` (8-byte stores arrive whole).
__device__ __forceinline__ void load8f_stamped(const WeightStreamParams& p, const uint2* src, uint32_t stamp, float (&v)[8]) {
    const uint4* quads = reinterpret_cast<const uint4*>(src);
    uint4 q[4];
    for (uint32_t polls = 0;; ++polls) {
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = load_volatile16(quads + i);
        bool landed = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) landed = landed && q[i].y == stamp && q[i].w == stamp;
        if (landed) break;
        // A dead peer costs a wrong pass, never a hung GPU; once one wait has given up the others stop waiting too.
        if (polls > p.gather.wait_limit || ((polls & 255u) == 255u && *reinterpret_cast<volatile int*>(p.error_flag) != 0)) { atomicExch(p.error_flag, 1); break; }
        if (polls > 32u) __nanosleep(100);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(q[i].x); v[2 * i + 1] = __uint_as_float(q[i].z); }
}
// The input rows of a launch: `in`, or on a tensor-parallel shard the sum of every shard's part in shard order.
template <bool FROM_L2, bool TP>
__device__ __forceinline__ void load8f_in(const WeightStreamParams& p, size_t offset, uint32_t stamp, float (&v)[8]) {
    if (TP && p.gather.count != 0u) {
        for (uint32_t s = 0; s < p.gather.count; ++s) {
            float w[8];
            if (s == p.gather.self) load8f_cg(p.gather.own + offset, w);
            else load8f_stamped(p, p.gather.parts[s] + offset, stamp, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = s == 0u ? w[i] : __fadd_rn(v[i], w[i]);
        }
        return;
    }
    load8f_act<FROM_L2>(p.in + offset, v);
}
__device__ __forceinline__ void store8f(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// Four 32-bit integers whose bytes are signed base-256 digits become four words, word i holding
// digit i of the four integers in order: a 4 x 4 byte transpose in eight byte-permutes.
__device__ __forceinline__ void transpose_digits(const uint32_t (&w)[4], uint32_t (&digit)[4]) {
    const uint32_t lo01 = __byte_perm(w[0], w[1], 0x5140u), lo23 = __byte_perm(w[2], w[3], 0x5140u);
    const uint32_t hi01 = __byte_perm(w[0], w[1], 0x7362u), hi23 = __byte_perm(w[2], w[3], 0x7362u);
    digit[0] = __byte_perm(lo01, lo23, 0x5410u); digit[1] = __byte_perm(lo01, lo23, 0x7632u);
    digit[2] = __byte_perm(hi01, hi23, 0x5410u); digit[3] = __byte_perm(hi01, hi23, 0x7632u);
}

// Where the staged activations live in shared memory.
struct GemvStage {
    uint8_t* frags;          // B registers
    float* sums;             // [rows][padded / 16]
    float* block_scales;     // [rows][padded / 256]
    uint32_t* bad_rows;      // bit r: row r holds a non-finite activation
    uint32_t padded;
};

// Turns eight consecutive activations of row r (slice piece `piece`, i.e. slice elements
// 8 * piece .. +7) into B registers.  Must be called by whole warps whose lanes hold consecutive
// pieces of one 256-element block: the warp's largest magnitude fixes the block's power-of-two
// scale 2^(e-156), every element becomes round(x / scale), an integer of at most 2^30, and adding
// 0x00808080 then flipping those bits makes its four bytes signed base-256 digits.  For
// 32-element group G2, B column n = 4 * row + digit and lane position t, the 8 bytes at
// G2 * gemv_fragment_stride + (n * 4 + t) * 8 are the digit bytes of elements 4t..4t+3 and 16+4t..16+4t+3 of
// the group.  Also written: the f32 sum of every 16 consecutive elements, the block scale, and
// the row's flag when an input is not finite (the row then yields NaN).  `store` is false for
// lanes whose piece lies outside the slice (they only take part in the warp exchanges).
template <int ROWS>
__device__ __forceinline__ void quantize_piece(const GemvStage& st, uint32_t r, uint32_t piece, const float (&v)[8], bool store) {
    constexpr uint32_t NCP = gemv_fragment_columns(ROWS);
    const uint32_t lane = threadIdx.x & 31u;
    // Largest magnitude of the warp's 256 elements, as a bit pattern (NaN and infinity sort on top).
    uint32_t top = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) top = max(top, __float_as_uint(v[i]) & 0x7fffffffu);
    top = __reduce_max_sync(0xffffffffu, top);         // one warp-wide integer reduction instruction
    uint32_t e = top >> 23;
    if (e == 255u) { if (lane == 0u) atomicOr(st.bad_rows, 1u << r); e = 254u; }
    e = max(e, 30u);
    const float to_fixed = __uint_as_float((283u - e) << 23);           // 2^(156 - e): |x| < 2^(e-126) -> |x * to_fixed| < 2^30
    float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (!store) return;
    if (lane == 0u) st.block_scales[r * (st.padded / 256u) + (piece >> 5)] = __uint_as_float((e - 29u) << 23);   // 2^(e - 156)
    if ((lane & 1u) == 0u) st.sums[r * (st.padded / 16u) + (piece >> 1)] = s;
    uint32_t words[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int fixed = __float2int_rn(__fmul_rn(v[i], to_fixed));
        words[i] = ((uint32_t)fixed + 0x00808080u) ^ 0x00808080u;
    }
    uint32_t d0[4], d1[4];
    { const uint32_t a[4] = {words[0], words[1], words[2], words[3]}; transpose_digits(a, d0); }
    { const uint32_t a[4] = {words[4], words[5], words[6], words[7]}; transpose_digits(a, d1); }
    // Elements 8*piece .. +7: group G2 = piece / 4, sixteen-half (piece / 2) & 1, positions t = 2 * (piece & 1), +1.
    const uint32_t g2 = piece >> 2, half = (piece >> 1) & 1u, t = (piece & 1u) * 2u;
    uint8_t* dst = st.frags + (size_t)g2 * gemv_fragment_stride(ROWS) + t * 8u + half * 4u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        *reinterpret_cast<uint32_t*>(dst + (4u * r + i) * 32u) = d0[i];
        *reinterpret_cast<uint32_t*>(dst + (4u * r + i) * 32u + 8u) = d1[i];
    }
    if (r == 0) {
#pragma unroll
        for (uint32_t n = 4u * ROWS; n < NCP; ++n) {
            *reinterpret_cast<uint32_t*>(dst + n * 32u) = 0u;
            *reinterpret_cast<uint32_t*>(dst + n * 32u + 8u) = 0u;
        }
    }
}

// What the register-resident prologue can read before the launch ahead has finished: the norm
// weights, and for the residual prologue the residual rows, which were written two or more
// launches back (the block schedule never lets the launch directly ahead write them).
template <int ROWS>
struct GemvEarly {
    float res[ROWS][8], g0[8], g1[8];
    bool cached;
};

// Whether the prologue keeps a row in registers: the norms of prologues 1 and 2 with at most one
// 8-element piece per thread (K <= 8 * block size) and a slice that starts on a 256-element boundary.
template <int ROWS>
__device__ __forceinline__ bool gemv_prologue_cached(const WeightStreamParams& p, uint32_t first) {
    const bool norms = p.prologue == kPrologueNorm || p.prologue == kPrologueAddNorm;
    return ROWS <= 4 && norms && p.k / 8u <= blockDim.x && (first & 255u) == 0u;
}

template <int ROWS, bool PASS>
__device__ __forceinline__ void stage_early(const WeightStreamParams& p, uint32_t first, GemvEarly<ROWS>& early) {
    early.cached = gemv_prologue_cached<ROWS>(p, first);
    if (!early.cached) return;
    const uint32_t piece = threadIdx.x, o = piece * 8u;
#pragma unroll
    for (int i = 0; i < 8; ++i) { early.g0[i] = 0.0f; early.g1[i] = 0.0f; }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) early.res[r][i] = 0.0f;
    if (piece >= p.k / 8u) return;
    if (p.prologue == kPrologueAddNorm) {
        load8f(p.gamma0 + o, early.g0);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if ((uint32_t)r < p.active_rows) load8f_act<PASS>(p.residual + (size_t)r * p.k + o, early.res[r]);
    }
    load8f(p.gamma1 + o, early.g1);
}

// Prologue kPrologueMerge for one 256-element block (one attention head) of row r: lane l first
// weighs partition l from its (maximum, sum) pair, then merges its own eight dimensions over the
// partitions that hold data, eight partitions' loads in flight at a time.  Whole warps only.
__device__ __forceinline__ void merge_head_piece(const WeightStreamParams& p, uint32_t r, uint32_t element, float (&v)[8]) {
    const uint32_t lane = threadIdx.x & 31u, heads = p.k / 256u, head = element / 256u, d = element % 256u;
    const size_t slot0 = ((size_t)r * heads + head) * 32u;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.residual + (slot0 + lane) * 2u));
    float top = ml.x;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
    const float weight = ml.y != 0.0f ? expf(ml.x - top) : 0.0f;
    const float total = warp_sum(ml.y * weight);
    const uint32_t filled = __ballot_sync(0xffffffffu, ml.y != 0.0f);
    const float* src = p.in + slot0 * 256u + d;
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.0f;
    for (uint32_t base = 0; base < 32u && (filled >> base) != 0u; base += 8u) {
        float4 lo[8], hi[8];
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const bool has = (filled >> (base + j)) & 1u;
            lo[j] = has ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(base + j) * 256u)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            hi[j] = has ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(base + j) * 256u + 4u)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const float f = __shfl_sync(0xffffffffu, weight, base + j);
            a[0] = fmaf(lo[j].x, f, a[0]); a[1] = fmaf(lo[j].y, f, a[1]); a[2] = fmaf(lo[j].z, f, a[2]); a[3] = fmaf(lo[j].w, f, a[3]);
            a[4] = fmaf(hi[j].x, f, a[4]); a[5] = fmaf(hi[j].y, f, a[5]); a[6] = fmaf(hi[j].z, f, a[6]); a[7] = fmaf(hi[j].w, f, a[7]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = a[i] / total;
}

// Produces this CTA's K slice [first, first + count) of the activation rows in shared memory.
// The RMS norms of prologues 1 and 2 need the whole row, so every CTA recomputes them from global
// memory (a few tens of KB out of L2).  In the register-resident case everything a thread needs
// of the launch ahead's output is loaded once and kept in registers through both norms (the rest
// came in with stage_early); otherwise the row is re-read for each pass.
template <int ROWS, bool PASS, bool TP = false>
__device__ __forceinline__ void stage_activations(const WeightStreamParams& p, uint32_t first, uint32_t count,
                                                  const GemvStage& st, float* scratch, GemvEarly<ROWS>& early, uint32_t stamp = 0u) {
    const bool norms = p.prologue == kPrologueNorm || p.prologue == kPrologueAddNorm;
    const uint32_t row_pieces = p.k / 8u;
    if (early.cached) {
        const uint32_t piece = threadIdx.x;
        const bool live = piece < row_pieces;
        const uint32_t o = piece * 8u;
        float x[ROWS][8];
        float (&res)[ROWS][8] = early.res;
        float (&g0)[8] = early.g0;
        float (&g1)[8] = early.g1;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) x[r][i] = 0.0f;
        if (live) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if ((uint32_t)r < p.active_rows) load8f_in<PASS, TP>(p, (size_t)r * p.k + o, stamp, x[r]);
        }
        float ss[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) ss[r] = sum_squares(x[r], 0.0f);
        gemv_block_sums<ROWS>(ss, scratch);
        if (p.prologue == kPrologueAddNorm) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float inv = rms_scale(ss[r], p.k, p.eps);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[r][i] = __fadd_rn(res[r][i], __fmul_rn(__fmul_rn(x[r][i], inv), g0[i]));
                // Every block holds the whole row: each writes the pieces that fall to it, so none straggles.
                if (live && piece % p.grid == blockIdx.x && (uint32_t)r < p.active_rows) store8f(p.residual_out + (size_t)r * p.k + o, x[r]);
                ss[r] = sum_squares(x[r], 0.0f);
            }
            gemv_block_sums<ROWS>(ss, scratch + kGemvWarps * ROWS);
        }
        const bool inside = live && o >= first && o < first + count;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float inv = rms_scale(ss[r], p.k, p.eps);
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(x[r][i], inv), g1[i]);
            quantize_piece<ROWS>(st, r, (o - first) / 8u, v, inside);
        }
        return;
    }
    float inv0[ROWS], inv1[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { inv0[r] = 1.0f; inv1[r] = 1.0f; }
    if (norms) {
        float ss[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            ss[r] = 0.0f;
            for (uint32_t c = threadIdx.x; c < row_pieces && (uint32_t)r < p.active_rows; c += blockDim.x) {
                float x[8];
                load8f_in<PASS, TP>(p, (size_t)r * p.k + c * 8u, stamp, x);
                ss[r] = sum_squares(x, ss[r]);
            }
        }
        gemv_block_sums<ROWS>(ss, scratch);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) (p.prologue == kPrologueNorm ? inv1[r] : inv0[r]) = rms_scale(ss[r], p.k, p.eps);
        if (p.prologue == kPrologueAddNorm) {
            // r = residual + norm(in) * gamma0; its mean square feeds the second norm.
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                ss[r] = 0.0f;
                for (uint32_t c = threadIdx.x; c < row_pieces && (uint32_t)r < p.active_rows; c += blockDim.x) {
                    float x[8], a[8], gm[8];
                    load8f_in<PASS, TP>(p, (size_t)r * p.k + c * 8u, stamp, x);
                    load8f_act<PASS>(p.residual + (size_t)r * p.k + c * 8u, a);
                    load8f(p.gamma0 + c * 8u, gm);
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(a[i], __fmul_rn(__fmul_rn(x[i], inv0[r]), gm[i]));
                    ss[r] = sum_squares(x, ss[r]);
                    if (c % p.grid == blockIdx.x) store8f(p.residual_out + (size_t)r * p.k + c * 8u, x);
                }
            }
            gemv_block_sums<ROWS>(ss, scratch + kGemvWarps * ROWS);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) inv1[r] = rms_scale(ss[r], p.k, p.eps);
        }
    }
    const uint32_t pieces = st.padded / 8u;      // a multiple of 32: whole warps stay together
    for (uint32_t q = threadIdx.x; q < (uint32_t)ROWS * pieces; q += blockDim.x) {
        const uint32_t r = q / pieces, piece = q % pieces, o = piece * 8u;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        if (p.prologue == kPrologueMerge) {
            // A warp holds one 256-element block of one row (slices start on head boundaries).
            if ((o & ~255u) < count && r < p.active_rows) merge_head_piece(p, r, first + o, v);
        } else if (o < count && r < p.active_rows) {
            const size_t gi = (size_t)r * p.k + first + o;
            const uint32_t c = first + o;
            float i0 = 1.0f, i1 = 1.0f;
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) if (rr == (int)r) { i0 = inv0[rr]; i1 = inv1[rr]; }
            load8f_in<PASS, TP>(p, gi, stamp, v);
            if (p.prologue == kPrologueNorm) {
                float gm[8];
                load8f(p.gamma1 + c, gm);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], i1), gm[i]);
            } else if (p.prologue == kPrologueAddNorm) {
                float a[8], gm0[8], gm1[8];
                load8f_act<PASS>(p.residual + gi, a);
                load8f(p.gamma0 + c, gm0);
                load8f(p.gamma1 + c, gm1);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[i] = __fmul_rn(__fmul_rn(__fadd_rn(a[i], __fmul_rn(__fmul_rn(v[i], i0), gm0[i])), i1), gm1[i]);
            } else if (p.prologue == kPrologueGeglu) {
                float up[8];
                load8f_act<PASS>(p.residual + gi, up);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(gelu_tanh_exact(v[i]), up[i]);
            }
        }
        quantize_piece<ROWS>(st, r, piece, v, true);
    }
}

// Status bit of a non-finite binary16 K/V value (the reference's validation word, metal_kernels.mm:2484).
constexpr uint32_t kGemvStatusKvNonFinite = 8u;
// Status bit of a pass whose committed position plus row lies beyond the tabulated rotations.
constexpr uint32_t kGemvStatusBadPosition = 16u;

// One finished head (256 output columns starting at `column0` of matrix `which`: 0 = Q, 1 = K,
// 2 = V) of every active row: RMSNorm with the head's weights, NEOX rotation by the tabulated
// (cos, sin) of the row's position, and the store the block schedule wants -- rotated queries in
// f32, K and V rounded to the cache type in the private rows.  Lane l owns elements 4l..4l+3 and
// 128+4l..128+4l+3, i.e. four rotation pairs.  The caller has made the head's values visible
// (fence after the last arrival).
template <int ROWS>
__device__ __forceinline__ void finish_head(const WeightStreamParams& p, const GemvMatrix& mat, uint32_t which, uint32_t head, uint32_t lane) {
    const WeightStreamParams::HeadEpilogue& e = p.heads;
    const uint32_t base = *e.base_position + e.row_base;
    const float* gamma = which == 0u ? e.q_norm : which == 1u ? e.k_norm : nullptr;
    // The finished values of the first two rows are requested together (the verify pass has two).
    const uint32_t rows = min(p.active_rows, (uint32_t)ROWS);
    float4 early_a[2], early_b[2];
#pragma unroll
    for (uint32_t i = 0; i < 2u; ++i) {
        const float* src = mat.out + (size_t)min(i, rows - 1u) * mat.n + head * 256u;
        early_a[i] = __ldcg(reinterpret_cast<const float4*>(src + 4u * lane));
        early_b[i] = __ldcg(reinterpret_cast<const float4*>(src + 128u + 4u * lane));
    }
    for (uint32_t r = 0; r < rows; ++r) {
        float4 a, b;
        if (r < 2u) { a = r == 0u ? early_a[0] : early_a[1]; b = r == 0u ? early_b[0] : early_b[1]; }
        else {
            const float* src = mat.out + (size_t)r * mat.n + head * 256u;
            a = __ldcg(reinterpret_cast<const float4*>(src + 4u * lane));
            b = __ldcg(reinterpret_cast<const float4*>(src + 128u + 4u * lane));
        }
        float first[4] = {a.x, a.y, a.z, a.w}, second[4] = {b.x, b.y, b.z, b.w};
        if (which != 2u) {
            if (gamma) {
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) sum = fmaf(first[j], first[j], fmaf(second[j], second[j], sum));
                sum = warp_sum(sum);
                const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, 256.0f), e.eps)));
                const float4 ga = *reinterpret_cast<const float4*>(gamma + 4u * lane);
                const float4 gb = *reinterpret_cast<const float4*>(gamma + 128u + 4u * lane);
                const float g0[4] = {ga.x, ga.y, ga.z, ga.w}, g1[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    first[j] = __fmul_rn(__fmul_rn(first[j], inv), g0[j]);
                    second[j] = __fmul_rn(__fmul_rn(second[j], inv), g1[j]);
                }
            }
            // A position past the rotation table (the device position word drifted from the host's) is reported, not read.
            uint32_t table_row = base + r;
            if (table_row >= e.table_rows) { if (lane == 0) atomicOr(e.status, kGemvStatusBadPosition); table_row = e.table_rows - 1u; }
            const float4* rot = reinterpret_cast<const float4*>(e.rotation + (size_t)table_row * 128u + 4u * lane);
            const float4 r01 = rot[0], r23 = rot[1];            // (cos, sin) of pairs 4l, 4l+1 and 4l+2, 4l+3
            const float cs[4] = {r01.x, r01.z, r23.x, r23.z}, sn[4] = {r01.y, r01.w, r23.y, r23.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float r0 = __fsub_rn(__fmul_rn(first[j], cs[j]), __fmul_rn(second[j], sn[j]));
                const float r1 = __fadd_rn(__fmul_rn(first[j], sn[j]), __fmul_rn(second[j], cs[j]));
                first[j] = r0; second[j] = r1;
            }
        }
        if (which == 0u) {
            float* dst = e.q_out + (size_t)r * mat.n + head * 256u;
            *reinterpret_cast<float4*>(dst + 4u * lane) = make_float4(first[0], first[1], first[2], first[3]);
            *reinterpret_cast<float4*>(dst + 128u + 4u * lane) = make_float4(second[0], second[1], second[2], second[3]);
            continue;
        }
        const size_t o = (size_t)r * mat.n + head * 256u;
        if (e.kv_f16) {
            __half* dst = static_cast<__half*>(which == 1u ? e.private_k : e.private_v) + o;
            __half2 lo[2], hi[2];
            bool finite = true;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                lo[j] = __halves2half2(__float2half_rn(first[2 * j]), __float2half_rn(first[2 * j + 1]));
                hi[j] = __halves2half2(__float2half_rn(second[2 * j]), __float2half_rn(second[2 * j + 1]));
                const float2 fl = __half22float2(lo[j]), fh = __half22float2(hi[j]);
                finite &= isfinite(fl.x) && isfinite(fl.y) && isfinite(fh.x) && isfinite(fh.y);
            }
            *reinterpret_cast<uint2*>(dst + 4u * lane) = make_uint2(*reinterpret_cast<uint32_t*>(&lo[0]), *reinterpret_cast<uint32_t*>(&lo[1]));
            *reinterpret_cast<uint2*>(dst + 128u + 4u * lane) = make_uint2(*reinterpret_cast<uint32_t*>(&hi[0]), *reinterpret_cast<uint32_t*>(&hi[1]));
            if (!finite) atomicOr(e.status, kGemvStatusKvNonFinite);
        } else {
            float* dst = static_cast<float*>(which == 1u ? e.private_k : e.private_v) + o;
            *reinterpret_cast<float4*>(dst + 4u * lane) = make_float4(first[0], first[1], first[2], first[3]);
            *reinterpret_cast<float4*>(dst + 128u + 4u * lane) = make_float4(second[0], second[1], second[2], second[3]);
        }
    }
}

// Counts a finished column pair of a fused Q/K/V launch; the warp that completes a head (16 pairs)
// finishes it.  The pair's outputs must already be written by this warp.
template <int ROWS>
__device__ __forceinline__ void head_pair_done(const WeightStreamParams& p, const GemvMatrix& mat, uint32_t which, uint32_t local_pair, uint32_t lane) {
    const uint32_t head = local_pair >> 4;
    const uint32_t slot = (which == 0u ? 0u : which == 1u ? p.m[0].n / 256u : p.m[0].n / 256u + p.m[1].n / 256u) + head;
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(&p.heads.head_counters[slot], 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived != 15u) return;
    __threadfence();
    finish_head<ROWS>(p, mat, which, head, lane);
    if (lane == 0) p.heads.head_counters[slot] = 0u;
}

// ---- the weight ring of a warp and the cursor that fills it --------------------------------
//
// Issue number k of a warp uses slot k % kGemvSlots and barrier parity (k / kGemvSlots) % 2.  The
// cursor (lane 0) walks the warp's items in the order the consumer meets them; inside a pass kernel
// it carries on into the next phase's items as soon as the current phase's are all requested, so
// weights of the next matrix arrive while the CTA waits for that phase's activations.

// One warp's share of a launch (or of a phase of a pass kernel).
struct WarpShare {
    uint32_t chunk, first_unit, chunk_count, pair_slot, stride, first_pair, unit_base, my_items;
};
__device__ __forceinline__ WarpShare warp_share(const WeightStreamParams& p, uint32_t block, uint32_t warp) {
    WarpShare w;
    const bool intra = p.intra > 1u;
    // With K split inside the CTA, warp w takes K chunk w % intra of the column pairs of slot w / intra.
    w.chunk = intra ? warp % p.intra : block % p.chunks;
    const uint32_t group_ctas = intra ? p.grid : p.grid / p.chunks;
    w.first_unit = w.chunk * p.chunk_units;
    w.chunk_count = min(p.chunk_units, p.units - w.first_unit);
    const uint32_t pair_slots = intra ? (uint32_t)kGemvWarps / p.intra : (uint32_t)kGemvWarps;
    w.pair_slot = intra ? warp / p.intra : warp;
    w.stride = group_ctas * pair_slots;
    w.first_pair = (intra ? block : block / p.chunks) * pair_slots + w.pair_slot;
    w.unit_base = intra ? w.first_unit : 0u;          // of this warp's chunk inside the staged slice
    w.my_items = (block < p.grid && w.first_pair < p.total_pairs) ? (p.total_pairs - w.first_pair + w.stride - 1u) / w.stride : 0u;
    return w;
}
__device__ __forceinline__ uint32_t matrix_of_pair(const WeightStreamParams& p, uint32_t pair) {
    uint32_t m = 0;
    if (p.matrices > 1u && pair >= p.m[1].first_pair) m = 1;
    if (p.matrices > 2u && pair >= p.m[2].first_pair) m = 2;
    return m;
}

// Ring slot of a pass kernel: two Q4_K / Q8_0 pair rows or one Q6_K pair row.
constexpr uint32_t kPassSlotBytes = 4608u;

// The cursor's phase-level state inside a pass kernel, one record per warp in shared memory (only lane 0
// touches it, and only when it starts a new item): which phase the cursor is in and this warp's share
// of it.  A single launch needs none of it: its parameters and the warp's share are at hand.
struct WeightCursor {
    const WeightStreamParams* phase;     // null when nothing is left
    const WeightStreamParams* last;      // last streaming phase of the pass kernel's table
    uint32_t phase_stride;               // bytes between consecutive table entries
    uint32_t stride, first_unit, chunk_count;      // of this warp's share of `phase`
};

// A warp's ring: the slots, and the cursor's state in registers (meaningful in lane 0).
struct WeightRing {
    uint8_t* slots;          // this warp's kGemvSlots slots
    uint64_t* bars;          // and their barriers
    WeightCursor* cursor;
    uint32_t slot_bytes;
    uint32_t consumed;       // copies consumed so far (the same in every lane)
    uint32_t issued;         // copies requested so far
    const uint8_t* src;      // next bytes of the item being requested
    uint32_t units_left;     // K units of that item not yet requested (0: start the next item)
    uint32_t row_bytes, slot_units;
    uint32_t items_left;     // items of the cursor's launch / phase not yet started
    uint32_t next_pair;      // column pair of the next item
};

// Pair rows one slot carries for a matrix of `dtype`.
template <bool PASS>
__device__ __forceinline__ uint32_t ring_slot_units(const WeightStreamParams& p, uint32_t dtype) {
    return PASS ? (dtype == (uint32_t)GF_Q6_K ? 1u : 2u) : p.slot_units;
}

// A table entry holds the parameters of a streaming phase when its first word is kPhaseStream.
constexpr uint32_t kPhaseStream = 1u;
__device__ __forceinline__ const WeightStreamParams* phase_stream_params(const uint8_t* entry) {
    return reinterpret_cast<const WeightStreamParams*>(entry + 16u);
}

__device__ __forceinline__ void cursor_enter(WeightRing& ring, const WeightStreamParams* phase, uint32_t block, uint32_t warp) {
    WeightCursor& c = *ring.cursor;
    c.phase = phase;
    if (phase == nullptr) { ring.items_left = 0; return; }
    const WarpShare w = warp_share(*phase, block, warp);
    ring.items_left = w.my_items; ring.next_pair = w.first_pair;
    c.stride = w.stride; c.first_unit = w.first_unit; c.chunk_count = w.chunk_count;
}

// Points the cursor at the warp's next item of launch / phase `p` (lane 0 only).
template <bool PASS>
__device__ __forceinline__ void ring_take_item(WeightRing& ring, const WeightStreamParams& p, uint32_t stride, uint32_t first_unit,
                                               uint32_t chunk_count) {
    const uint32_t pair = ring.next_pair;
    ring.next_pair += stride;
    --ring.items_left;
    const GemvMatrix& mat = p.m[matrix_of_pair(p, pair)];
    ring.row_bytes = pair_row_bytes((int)mat.dtype);
    ring.slot_units = ring_slot_units<PASS>(p, mat.dtype);
    ring.src = mat.weight + ((size_t)(pair - mat.first_pair) * p.units + first_unit) * ring.row_bytes;
    ring.units_left = chunk_count;
}

// Requests the next slot-full of pair rows (lane 0 only).  `p` and `w` are the launch's parameters and
// the warp's share of it; a pass kernel's cursor uses its own record instead, since it may be a phase ahead.
template <bool PASS>
__device__ __forceinline__ void ring_issue(WeightRing& ring, const WeightStreamParams& p, const WarpShare& w, uint32_t block, uint32_t warp) {
    if (ring.units_left == 0u) {
        if (!PASS) {
            if (ring.items_left == 0u) return;
            ring_take_item<false>(ring, p, w.stride, w.first_unit, w.chunk_count);
        } else {
            WeightCursor& c = *ring.cursor;
            while (ring.items_left == 0u) {
                if (c.phase == nullptr) return;
                if (c.phase == c.last) { c.phase = nullptr; return; }
                // On to the next streaming phase of the table.
                const uint8_t* entry = reinterpret_cast<const uint8_t*>(c.phase) - 16u;
                const uint8_t* last_entry = reinterpret_cast<const uint8_t*>(c.last) - 16u;
                const WeightStreamParams* next = nullptr;
                while (entry != last_entry) {
                    entry += c.phase_stride;
                    if (*reinterpret_cast<const uint32_t*>(entry) == kPhaseStream) { next = phase_stream_params(entry); break; }
                }
                cursor_enter(ring, next, block, warp);
            }
            ring_take_item<true>(ring, *c.phase, c.stride, c.first_unit, c.chunk_count);
        }
    }
    const uint32_t count = min(ring.slot_units, ring.units_left), bytes = count * ring.row_bytes;
    const uint32_t slot = ring.issued % (uint32_t)kGemvSlots;
    const uint32_t claimed = (!PASS && ring.issued == 0u && block == 0u && warp == 0u) ? bytes + p.overstate : bytes;
    mbar_expect_tx(&ring.bars[slot], claimed);
    bulk_load(ring.slots + slot * ring.slot_bytes, ring.src, bytes, &ring.bars[slot]);
    ring.src += bytes;
    ++ring.issued;
    ring.units_left -= count;
}

// Gives outstanding copies a bounded chance to land before the shared memory is released (lane 0).
__device__ __forceinline__ void ring_drain(WeightRing& ring, uint32_t limit = kMbarWaitLimit) {
    for (uint32_t k = ring.consumed; k < ring.issued; ++k)
        mbar_wait(&ring.bars[k % (uint32_t)kGemvSlots], (k / (uint32_t)kGemvSlots) & 1u, limit);
}

// Shared-memory carve-up of a streaming phase: [ring | barriers | cursors | fragments | sums | scales | meeting].
struct StreamSmem {
    uint8_t* ring; uint64_t* bars; WeightCursor* cursors; uint8_t* staging;
};
static_assert(sizeof(WeightCursor) <= kGemvCursorBytes, "cursor record outgrew its shared-memory slot");
__host__ __device__ constexpr uint32_t stream_smem_fixed(uint32_t slot_bytes) { return gemv_ring_bytes(slot_bytes); }
__device__ __forceinline__ StreamSmem stream_smem(uint8_t* smem, uint32_t slot_bytes) {
    StreamSmem s;
    s.ring = smem;
    s.bars = reinterpret_cast<uint64_t*>(smem + (uint32_t)kGemvWarps * kGemvSlots * slot_bytes);
    s.cursors = reinterpret_cast<WeightCursor*>(s.bars + kGemvWarps * kGemvSlots);     // kGemvCursorBytes apart
    s.staging = smem + stream_smem_fixed(slot_bytes);
    return s;
}

// One streaming launch, or one streaming phase of a pass kernel (PASS): stages this CTA's slice of the
// activation rows once `dependency()` says the producer's outputs are visible, then every warp walks
// its items.  `dependency` is called by every thread of the CTA exactly once and returns false when
// the wait gave up; `scratch` holds 2 * kGemvWarps * ROWS floats, `bad_rows` one word that the caller has
// zeroed ahead of a block barrier.  Returns false
// when a bounded wait gave up somewhere in this CTA (the error word is set by the caller).
template <int ROWS, bool PASS, typename Dependency>
__device__ __forceinline__ bool stream_phase(const WeightStreamParams& p, const StreamSmem& sm, WeightRing& ring_state,
                                             float* scratch, uint32_t* bad_rows, Dependency&& dependency) {
    // The ring is worked on in registers and handed back at the end (a pass kernel calls this through a
    // function boundary, where the caller's copy lives in local memory).
    struct RingScope {
        WeightRing& home; WeightRing ring;
        __device__ explicit RingScope(WeightRing& h) : home(h), ring(h) {}
        __device__ ~RingScope() { home = ring; }
    } scope(ring_state);
    WeightRing& ring = scope.ring;
    constexpr int NT = (4 * ROWS + 7) / 8;
    constexpr uint32_t NCP = gemv_fragment_columns(ROWS);
    constexpr uint32_t FRAG_STRIDE = gemv_fragment_stride(ROWS);
    const bool intra = p.intra > 1u;
    const GemvSmemLayout lay = gemv_smem_layout(ROWS, p.staged_units, p.unit_elems, ring.slot_bytes);
    const uint32_t slice = p.staged_units * p.unit_elems, padded = (slice + 255u) & ~255u;
    uint8_t* frags = sm.staging;
    float* sums = reinterpret_cast<float*>(sm.staging + lay.frag_bytes);
    float* block_scales = reinterpret_cast<float*>(sm.staging + lay.frag_bytes + lay.sums_bytes);
    float* meeting = reinterpret_cast<float*>(sm.staging + lay.frag_bytes + lay.sums_bytes + lay.scale_bytes);   // only laid out when K is split inside the CTA

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const bool member = blockIdx.x < p.grid;            // a pass kernel's CTAs beyond the phase's grid only keep the barriers company
    const WarpShare w = warp_share(p, blockIdx.x, warp);
    const uint32_t chunk = w.chunk, first_unit = w.first_unit, chunk_count = w.chunk_count, pair_slot = w.pair_slot;
    const uint32_t stride = w.stride, first_pair = w.first_pair, unit_base = w.unit_base, my_items = w.my_items;

    GemvEarly<ROWS> early_inputs;
    early_inputs.cached = false;
    if (member) stage_early<ROWS, PASS>(p, intra ? 0u : first_unit * p.unit_elems, early_inputs);

    if (!dependency()) return false;
    if (member) {
        const GemvStage stage{frags, sums, block_scales, bad_rows, padded};
        stage_activations<ROWS, PASS>(p, intra ? 0u : first_unit * p.unit_elems, intra ? p.k : chunk_count * p.unit_elems, stage, scratch, early_inputs);
    }
    __syncthreads();
    if (!PASS) pdl_launch_dependents();
    if (!member) return true;

    GemvLane L;
    L.lane = lane; L.g = lane >> 2; L.t = lane & 3u;
    // This lane's C registers hold B columns 2t, 2t+1 of every n-tile: digits (2t) % 4 and the next
    // one of row (8 * nt + 2t) / 4.
    L.digit_weight = (L.t & 1u) ? pack2f(65536.0f, 16777216.0f) : pack2f(1.0f, 256.0f);
    const uint8_t* my_frag = frags + ((L.g & (NCP - 1u)) * 4u + L.t) * 8u;
    const uint32_t sums_stride = padded / 16u, scales_stride = padded / 256u;
    uint32_t my_row[NT];      // the activation row whose digits this lane's C registers of n-tile nt hold
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) my_row[nt] = min(2u * nt + (L.t >> 1), (uint32_t)ROWS - 1u);
    const uint32_t quad_base = lane & ~3u;
    const uint32_t bad = *bad_rows;

    f32x2 accA[NT], accB[NT];
    float maccA[ROWS], maccB[ROWS];
    bool failed = false;
    for (uint32_t item = 0; item < my_items && (!failed || intra); ++item) {
        const uint32_t pair = first_pair + item * stride;
        const uint32_t which = matrix_of_pair(p, pair);
        const GemvMatrix& mat = p.m[which];
        const uint32_t dtype = mat.dtype;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { accA[nt] = 0ull; accB[nt] = 0ull; }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) { maccA[r] = 0.0f; maccB[r] = 0.0f; }
        const uint32_t row_bytes = pair_row_bytes((int)dtype);
        const uint32_t slot_units = ring_slot_units<PASS>(p, dtype);
        for (uint32_t u0 = 0; u0 < chunk_count && !failed; u0 += slot_units) {
            const uint32_t slot = ring.consumed % (uint32_t)kGemvSlots;
            if (!mbar_wait(&ring.bars[slot], (ring.consumed / (uint32_t)kGemvSlots) & 1u, p.wait_limit)) { failed = true; break; }
            const uint32_t count = min(slot_units, chunk_count - u0);
            for (uint32_t j = 0; j < count; ++j) {
                const uint32_t u = unit_base + u0 + j;
                const uint8_t* row = ring.slots + slot * ring.slot_bytes + j * row_bytes;
                float scales[NT];
                if (dtype == GF_Q4_K) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + u];
                    pair_row_q4k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                        scales, L, accA, accB, maccA, maccB);
                } else if (dtype == GF_Q6_K) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + u];
                    pair_row_q6k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                        scales, L, accA, accB, maccA, maccB);
                } else {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + (u >> 1)];
                    pair_row_q80<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 4u * FRAG_STRIDE, scales, L, accA, accB);
                }
            }
            __syncwarp();   // every lane has finished reading this slot
            ++ring.consumed;
            if (lane == 0) ring_issue<PASS>(ring, p, w, blockIdx.x, warp);
        }
        if (failed && !intra) break;      // inside a CTA the other chunks' warps wait at the meeting barrier
        // Row r is the sum of B columns 4r .. 4r+3 (digit 0 first; held by quad lanes (n % 8) / 2 of
        // n-tile n / 8), minus the correction dot product of its column.
        const float offset = dtype == GF_Q4_K ? 1.0f : dtype == GF_Q6_K ? 32.0f : 0.0f;
        float totalA[ROWS], totalB[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float partA[4], partB[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int n = 4 * r + i, nt = n / 8, holder = (n % 8) / 2;
                const float2 a = unpack2(accA[nt]), b = unpack2(accB[nt]);
                partA[i] = __shfl_sync(0xffffffffu, (n & 1) ? a.y : a.x, quad_base + holder);
                partB[i] = __shfl_sync(0xffffffffu, (n & 1) ? b.y : b.x, quad_base + holder);
            }
            float mA = maccA[r], mB = maccB[r];      // quad lanes hold the shares of different groups
            mA += __shfl_xor_sync(0xffffffffu, mA, 1); mB += __shfl_xor_sync(0xffffffffu, mB, 1);
            mA += __shfl_xor_sync(0xffffffffu, mA, 2); mB += __shfl_xor_sync(0xffffffffu, mB, 2);
            totalA[r] = __fsub_rn(__fadd_rn(__fadd_rn(__fadd_rn(partA[0], partA[1]), partA[2]), partA[3]), __fmul_rn(offset, mA));
            totalB[r] = __fsub_rn(__fadd_rn(__fadd_rn(__fadd_rn(partB[0], partB[1]), partB[2]), partB[3]), __fmul_rn(offset, mB));
            if ((bad >> r) & 1u) totalA[r] = totalB[r] = __int_as_float(0x7fc00000);
        }
        const uint32_t local_pair = pair - mat.first_pair;
        const uint32_t columnA = local_pair * 16u + L.g, columnB = columnA + 8u;
        if (intra) {
            // K split inside the CTA: the chunks' partial sums meet in shared memory; the warp of chunk 0
            // adds them in chunk order and carries on as if it had computed the whole column pair.
            float* mine = meeting + (size_t)warp * ROWS * 16u;
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (L.t == (uint32_t)(r & 3)) { mine[r * 16 + L.g] = totalA[r]; mine[r * 16 + L.g + 8u] = totalB[r]; }
            asm volatile("bar.sync %0, %1;" ::"r"(1u + pair_slot), "r"(p.intra * 32u) : "memory");
            if (chunk == 0u) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (L.t == (uint32_t)(r & 3)) {
                        float a = 0.0f, b = 0.0f;
                        for (uint32_t c = 0; c < p.intra; ++c) {
                            const float* theirs = meeting + (size_t)(warp + c) * ROWS * 16u;
                            a += theirs[r * 16 + L.g];
                            b += theirs[r * 16 + L.g + 8u];
                        }
                        totalA[r] = a; totalB[r] = b;
                    }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1u + pair_slot), "r"(p.intra * 32u) : "memory");   // the meeting place is free again
            if (chunk != 0u) continue;
        }
        if (p.chunks == 1u) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (L.t == (uint32_t)(r & 3) && (uint32_t)r < p.active_rows) {
                    if (columnA < mat.n) mat.out[(size_t)r * mat.n + columnA] = totalA[r];
                    if (columnB < mat.n) mat.out[(size_t)r * mat.n + columnB] = totalB[r];
                }
            if (p.heads.enabled) head_pair_done<ROWS>(p, mat, which, local_pair, lane);
            continue;
        }
        // Split K: park this chunk's partial sums; the warp that arrives last for the pair adds
        // all chunks in chunk order (so the result does not depend on arrival order).
        const size_t width = (size_t)p.total_pairs * 16u;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (L.t == (uint32_t)(r & 3)) {
                float* dst = p.partial + ((size_t)chunk * ROWS + r) * width + (size_t)pair * 16u;
                dst[L.g] = totalA[r];
                dst[L.g + 8u] = totalB[r];
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
                if (out_column < mat.n && r < p.active_rows) mat.out[(size_t)r * mat.n + out_column] = sum;
            }
            if (lane == 0) p.counters[pair] = 0u;
            if (p.heads.enabled) head_pair_done<ROWS>(p, mat, which, local_pair, lane);
        }
    }
    return !failed;
}

// Sets up this warp's ring over the CTA's shared memory: barriers initialised, the cursor at the warp's
// first item of `first` (a single launch: last == first, and the cursor lives in registers alone), the
// first copies requested.  Contains a block barrier.
template <bool PASS>
__device__ __forceinline__ WeightRing ring_open(const StreamSmem& sm, uint32_t slot_bytes, const WeightStreamParams* first,
                                                const WeightStreamParams* last, uint32_t phase_stride) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    WeightRing ring;
    ring.slots = sm.ring + warp * (kGemvSlots * slot_bytes);
    ring.bars = sm.bars + warp * kGemvSlots;
    ring.slot_bytes = slot_bytes;
    ring.cursor = sm.cursors + warp;
    ring.consumed = 0; ring.issued = 0;
    ring.src = nullptr; ring.units_left = 0; ring.row_bytes = 0; ring.slot_units = 1;
    ring.items_left = 0; ring.next_pair = 0;
    WarpShare w = {};
    if (!PASS) {
        w = warp_share(*first, blockIdx.x, warp);
        ring.items_left = w.my_items; ring.next_pair = w.first_pair;
    }
    if (lane == 0) {
        for (int s = 0; s < kGemvSlots; ++s) mbar_init(&ring.bars[s], 1);
        fence_barrier_init();
        if (PASS) {
            WeightCursor& c = *ring.cursor;
            c.last = last; c.phase_stride = phase_stride;
            cursor_enter(ring, first, blockIdx.x, warp);
        }
    }
    __syncthreads();
    // Weights do not depend on anything computed on the device: start streaming at once.
    if (lane == 0 && first != nullptr)
        for (int j = 0; j < kGemvSlots; ++j) ring_issue<PASS>(ring, *first, w, blockIdx.x, warp);
    return ring;
}

// The launch of its own: one matrix set per kernel, the schedule replayed as a CUDA graph.  Its body is
// kept apart from stream_phase (the pass kernel's phase) although the two decompose and compute alike:
// with everything a launch needs in the constant bank and in registers this form measured 2.3 % faster
// over a 12B pass than the shared one.
// TP: the instantiation tensor-parallel shards launch (WeightStreamParams::scatter / gather); the plain one carries none of it.
// `again`: the second half of a 5..8-row launch (weight_stream_pair_kernel) -- the CTA's staging area and the
// warps' barriers are taken over from the first half; `last`: no half follows (the next launch may start its prologue).
template <int ROWS, bool TP>
__device__ __forceinline__ void weight_stream_body(const WeightStreamParams& p, const bool again, const bool last, uint32_t& ring_slot, uint32_t& ring_phase) {
    constexpr int NT = (4 * ROWS + 7) / 8;
    constexpr uint32_t NCP = gemv_fragment_columns(ROWS);
    constexpr uint32_t FRAG_STRIDE = gemv_fragment_stride(ROWS);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * kGemvWarps * ROWS];
    __shared__ uint32_t bad_rows;
    const bool intra = p.intra > 1u;
    const GemvSmemLayout lay = gemv_smem_layout(ROWS, p.staged_units, p.unit_elems, p.slot_bytes);
    const uint32_t slots_bytes = (uint32_t)kGemvWarps * kGemvSlots * p.slot_bytes;
    const uint32_t slice = p.staged_units * p.unit_elems, padded = (slice + 255u) & ~255u;
    uint8_t* frags = smem;
    float* sums = reinterpret_cast<float*>(smem + lay.frag_bytes);
    float* block_scales = reinterpret_cast<float*>(smem + lay.frag_bytes + lay.sums_bytes);
    uint8_t* ring_base = smem + lay.frag_bytes + lay.sums_bytes + lay.scale_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_base + slots_bytes);
    float* meeting = reinterpret_cast<float*>(bars + kGemvWarps * kGemvSlots);      // only laid out when K is split inside the CTA

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint8_t* ring = ring_base + warp * (kGemvSlots * p.slot_bytes);
    uint64_t* bar = bars + warp * kGemvSlots;

    // This CTA's K chunk and this warp's sequence of column pairs (over all matrices).
    // With K split inside the CTA, warp w takes K chunk w % intra of the column pairs of slot w / intra.
    const uint32_t chunk = intra ? warp % p.intra : blockIdx.x % p.chunks;
    const uint32_t group_ctas = intra ? gridDim.x : gridDim.x / p.chunks;
    const uint32_t first_unit = chunk * p.chunk_units;
    const uint32_t chunk_count = min(p.chunk_units, p.units - first_unit);
    const uint32_t pair_slots = intra ? (uint32_t)kGemvWarps / p.intra : (uint32_t)kGemvWarps;
    const uint32_t pair_slot = intra ? warp / p.intra : warp;
    const uint32_t stride = group_ctas * pair_slots;
    const uint32_t first_pair = (intra ? blockIdx.x : blockIdx.x / p.chunks) * pair_slots + pair_slot;
    const uint32_t unit_base = intra ? first_unit : 0u;          // of this warp's chunk inside the staged slice
    const uint32_t my_items = first_pair < p.total_pairs ? (p.total_pairs - first_pair + stride - 1u) / stride : 0u;

    auto matrix_of = [&](uint32_t pair) -> uint32_t {
        uint32_t m = 0;
        if (p.matrices > 1u && pair >= p.m[1].first_pair) m = 1;
        if (p.matrices > 2u && pair >= p.m[2].first_pair) m = 2;
        return m;
    };

    if (again) __syncthreads();          // every warp has finished reading the first half's staged rows
    if (threadIdx.x == 0) bad_rows = 0u;
    if (lane == 0 && !again) {           // the second half carries on in the ring where the first stopped
        for (int s = 0; s < kGemvSlots; ++s) mbar_init(&bar[s], 1);
        fence_barrier_init();
    }
    __syncthreads();

    // Producer cursor (lane 0): the next slot-full of pair rows to request, walking items then units.
    uint32_t prod_item = 0, prod_unit = 0, prod_slot = ring_slot, prod_bytes = 0;
    bool first_copy = blockIdx.x == 0u && warp == 0u && !again;
    const uint8_t* prod_src = nullptr;
    auto issue_next = [&]() {   // lane 0 only
        if (prod_item >= my_items) return;
        if (prod_unit == 0u) {
            const uint32_t pair = first_pair + prod_item * stride;
            const GemvMatrix& mat = p.m[matrix_of(pair)];
            prod_bytes = pair_row_bytes((int)mat.dtype);
            prod_src = mat.weight + ((size_t)(pair - mat.first_pair) * p.units + first_unit) * prod_bytes;
        }
        const uint32_t count = min(p.slot_units, chunk_count - prod_unit), bytes = count * prod_bytes;
        mbar_expect_tx(&bar[prod_slot], first_copy ? bytes + p.overstate : bytes);      // overstate: 0 outside a testing build's fault seam
        first_copy = false;
        bulk_load(ring + prod_slot * p.slot_bytes, prod_src, bytes, &bar[prod_slot]);
        prod_src += bytes;
        prod_slot = prod_slot + 1u == (uint32_t)kGemvSlots ? 0u : prod_slot + 1u;
        prod_unit += count;
        if (prod_unit == chunk_count) { prod_unit = 0; ++prod_item; }
    };
    // Weights do not depend on the previous kernel: start streaming before waiting for it.
    if (lane == 0)
        for (int j = 0; j < kGemvSlots; ++j) issue_next();

    GemvEarly<ROWS> early_inputs;
    stage_early<ROWS, false>(p, intra ? 0u : first_unit * p.unit_elems, early_inputs);

    pdl_wait();
    const uint32_t gather_stamp = TP && p.gather.count != 0u ? shard_stamp(p.gather.tick, p.gather.site) : 0u;
    const uint32_t scatter_stamp = TP && p.scatter.count != 0u ? shard_stamp(p.scatter.tick, p.scatter.site) : 0u;
    const GemvStage stage{frags, sums, block_scales, &bad_rows, padded};
    stage_activations<ROWS, false, TP>(p, intra ? 0u : first_unit * p.unit_elems, intra ? p.k : chunk_count * p.unit_elems, stage, scratch, early_inputs,
                                       gather_stamp);
    __syncthreads();
    if (last) pdl_launch_dependents();

    GemvLane L;
    L.lane = lane; L.g = lane >> 2; L.t = lane & 3u;
    // This lane's C registers hold B columns 2t, 2t+1 of every n-tile: digits (2t) % 4 and the next
    // one of row (8 * nt + 2t) / 4.
    L.digit_weight = (L.t & 1u) ? pack2f(65536.0f, 16777216.0f) : pack2f(1.0f, 256.0f);
    const uint8_t* my_frag = frags + ((L.g & (NCP - 1u)) * 4u + L.t) * 8u;
    const uint32_t sums_stride = padded / 16u, scales_stride = padded / 256u;
    uint32_t my_row[NT];      // the activation row whose digits this lane's C registers of n-tile nt hold
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) my_row[nt] = min(2u * nt + (L.t >> 1), (uint32_t)ROWS - 1u);
    const uint32_t quad_base = lane & ~3u;
    const uint32_t bad = bad_rows;

    f32x2 accA[NT], accB[NT];
    float maccA[ROWS], maccB[ROWS];
    bool failed = false;
    uint32_t slot = ring_slot, phase = ring_phase;
    for (uint32_t item = 0; item < my_items && (!failed || intra); ++item) {
        const uint32_t pair = first_pair + item * stride;
        const GemvMatrix& mat = p.m[matrix_of(pair)];
        const uint32_t dtype = mat.dtype;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { accA[nt] = 0ull; accB[nt] = 0ull; }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) { maccA[r] = 0.0f; maccB[r] = 0.0f; }
        const uint32_t row_bytes = pair_row_bytes((int)dtype);
        for (uint32_t u0 = 0; u0 < chunk_count && !failed; u0 += p.slot_units) {
            if (!mbar_wait(&bar[slot], phase, p.wait_limit)) { failed = true; break; }
            const uint32_t count = min(p.slot_units, chunk_count - u0);
            for (uint32_t j = 0; j < count; ++j) {
                const uint32_t u = unit_base + u0 + j;
                const uint8_t* row = ring + slot * p.slot_bytes + j * row_bytes;
                float scales[NT];
                if (dtype == GF_Q4_K) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + u];
                    pair_row_q4k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                        scales, L, accA, accB, maccA, maccB);
                } else if (dtype == GF_Q6_K) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + u];
                    pair_row_q6k<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 8u * FRAG_STRIDE, sums + u * 16u, sums_stride,
                                                        scales, L, accA, accB, maccA, maccB);
                } else {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) scales[nt] = block_scales[my_row[nt] * scales_stride + (u >> 1)];
                    pair_row_q80<ROWS, NT, FRAG_STRIDE>(row, my_frag + (size_t)u * 4u * FRAG_STRIDE, scales, L, accA, accB);
                }
            }
            __syncwarp();   // every lane has finished reading this slot
            if (lane == 0) issue_next();
            if (++slot == (uint32_t)kGemvSlots) { slot = 0; phase ^= 1u; }
        }
        if (failed && !intra) break;      // inside a CTA the other chunks' warps wait at the meeting barrier
        // Row r is the sum of B columns 4r .. 4r+3 (digit 0 first; held by quad lanes (n % 8) / 2 of
        // n-tile n / 8), minus the correction dot product of its column.
        const float offset = dtype == GF_Q4_K ? 1.0f : dtype == GF_Q6_K ? 32.0f : 0.0f;
        float totalA[ROWS], totalB[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float partA[4], partB[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int n = 4 * r + i, nt = n / 8, holder = (n % 8) / 2;
                const float2 a = unpack2(accA[nt]), b = unpack2(accB[nt]);
                partA[i] = __shfl_sync(0xffffffffu, (n & 1) ? a.y : a.x, quad_base + holder);
                partB[i] = __shfl_sync(0xffffffffu, (n & 1) ? b.y : b.x, quad_base + holder);
            }
            float mA = maccA[r], mB = maccB[r];      // quad lanes hold the shares of different groups
            mA += __shfl_xor_sync(0xffffffffu, mA, 1); mB += __shfl_xor_sync(0xffffffffu, mB, 1);
            mA += __shfl_xor_sync(0xffffffffu, mA, 2); mB += __shfl_xor_sync(0xffffffffu, mB, 2);
            totalA[r] = __fsub_rn(__fadd_rn(__fadd_rn(__fadd_rn(partA[0], partA[1]), partA[2]), partA[3]), __fmul_rn(offset, mA));
            totalB[r] = __fsub_rn(__fadd_rn(__fadd_rn(__fadd_rn(partB[0], partB[1]), partB[2]), partB[3]), __fmul_rn(offset, mB));
            if ((bad >> r) & 1u) totalA[r] = totalB[r] = __int_as_float(0x7fc00000);
        }
        const uint32_t local_pair = pair - mat.first_pair;
        const uint32_t columnA = local_pair * 16u + L.g, columnB = columnA + 8u;
        if (intra) {
            // K split inside the CTA: the chunks' partial sums meet in shared memory; the warp of chunk 0
            // adds them in chunk order and carries on as if it had computed the whole column pair.
            float* mine = meeting + (size_t)warp * ROWS * 16u;
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (L.t == (uint32_t)(r & 3)) { mine[r * 16 + L.g] = totalA[r]; mine[r * 16 + L.g + 8u] = totalB[r]; }
            asm volatile("bar.sync %0, %1;" ::"r"(1u + pair_slot), "r"(p.intra * 32u) : "memory");
            if (chunk == 0u) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (L.t == (uint32_t)(r & 3)) {
                        float a = 0.0f, b = 0.0f;
                        for (uint32_t c = 0; c < p.intra; ++c) {
                            const float* theirs = meeting + (size_t)(warp + c) * ROWS * 16u;
                            a += theirs[r * 16 + L.g];
                            b += theirs[r * 16 + L.g + 8u];
                        }
                        totalA[r] = a; totalB[r] = b;
                    }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1u + pair_slot), "r"(p.intra * 32u) : "memory");   // the meeting place is free again
            if (chunk != 0u) continue;
        }
        if (p.chunks == 1u) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (L.t == (uint32_t)(r & 3) && (uint32_t)r < p.active_rows) {
                    if (columnA < mat.n) mat.out[(size_t)r * mat.n + columnA] = totalA[r];
                    if (columnB < mat.n) mat.out[(size_t)r * mat.n + columnB] = totalB[r];
                    if (TP)
                        for (uint32_t s = 0; s < p.scatter.count; ++s) {
                            if (columnA < mat.n) p.scatter.out[s][(size_t)r * mat.n + columnA] = make_uint2(__float_as_uint(totalA[r]), scatter_stamp);
                            if (columnB < mat.n) p.scatter.out[s][(size_t)r * mat.n + columnB] = make_uint2(__float_as_uint(totalB[r]), scatter_stamp);
                        }
                }
            if (p.heads.enabled) head_pair_done<ROWS>(p, mat, matrix_of(pair), local_pair, lane);
            continue;
        }
        // Split K: park this chunk's partial sums; the warp that arrives last for the pair adds
        // all chunks in chunk order (so the result does not depend on arrival order).
        const size_t width = (size_t)p.total_pairs * 16u;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (L.t == (uint32_t)(r & 3)) {
                float* dst = p.partial + ((size_t)chunk * ROWS + r) * width + (size_t)pair * 16u;
                dst[L.g] = totalA[r];
                dst[L.g + 8u] = totalB[r];
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
                if (out_column < mat.n && r < p.active_rows) {
                    mat.out[(size_t)r * mat.n + out_column] = sum;
                    if (TP)
                        for (uint32_t s = 0; s < p.scatter.count; ++s)
                            p.scatter.out[s][(size_t)r * mat.n + out_column] = make_uint2(__float_as_uint(sum), scatter_stamp);
                }
            }
            if (lane == 0) p.counters[pair] = 0u;
            if (p.heads.enabled) head_pair_done<ROWS>(p, mat, matrix_of(pair), local_pair, lane);
        }
    }
    if (failed) {
        // Give outstanding copies a bounded chance to land before the shared memory is released.
        if (lane == 0) atomicExch(p.error_flag, 1);
        for (int s = 0; s < kGemvSlots; ++s) mbar_wait(&bar[s], 0, p.wait_limit);
    }
    ring_slot = slot;
    ring_phase = phase;
}

template <int ROWS, bool TP = false>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) weight_stream_kernel(const __grid_constant__ WeightStreamParams p) {
    uint32_t slot = 0, phase = 0;
    weight_stream_body<ROWS, TP>(p, false, true, slot, phase);
}

// Five to eight rows: the four-row body twice in one launch, rows 0..3 with `first` and the rest with `second`
// (the same launch with every row pointer moved on by four rows, and counters and partial sums of its own).  The
// weights are streamed once per half -- the second time mostly out of L2 -- and a row's sums are those of the
// four-row instance, product for product; the eight-row instance this replaces ran at 1.4 TB/s against the
// four-row one's 3.4 (its accumulators spilled), so two halves are faster than one whole.
template <bool TP = false>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) weight_stream_pair_kernel(const __grid_constant__ WeightStreamParams first,
                                                                                const __grid_constant__ WeightStreamParams second) {
    uint32_t slot = 0, phase = 0;          // where the warp's weight ring stands
    weight_stream_body<4, TP>(first, false, false, slot, phase);
    weight_stream_body<4, TP>(second, true, true, slot, phase);
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
    // Head epilogue of a fused Q/K/V launch (see WeightStreamParams::HeadEpilogue); off when rotation is null.
    struct Heads {
        const float *q_norm = nullptr, *k_norm = nullptr;
        float* q_out = nullptr;
        void *private_k = nullptr, *private_v = nullptr;
        const float2* rotation = nullptr;
        const uint32_t* base_position = nullptr;
        uint32_t* status = nullptr;
        uint32_t* head_counters = nullptr;
        uint32_t table_rows = 0;
        int kv_f16 = 0;
        uint32_t row_base = 0;               // rows of the pass ahead of this launch's row 0
    } heads;
    uint32_t instance = 0;                   // kernel instance to plan for (0: the one `rows` names)
    // Shard exchange of a tensor-parallel plan (see WeightStreamParams): off when the counts are 0.
    WeightStreamParams::Scatter scatter = {};
    WeightStreamParams::Gather gather = {};
};
struct GemvPlan { uint32_t units, unit_elems, total_pairs, chunks, chunk_units, grid, smem, slot_bytes, slot_units, intra, staged_units; };

int gemv_plan(const GemvLaunch& launch, GemvPlan& plan);
// Split-K scratch of one launch: `partial` bytes of sums, and one arrival counter per column pair.
// Counters must be zero before a launch and are left zero by it; they must not share memory
// with any launch's partial sums.
size_t gemv_partial_bytes(const GemvLaunch& launch);
size_t gemv_counter_bytes(const GemvLaunch& launch);
int gemv_launch(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                cudaStream_t stream, bool programmatic);
// The kernel parameters and decomposition gemv_launch would use, without launching (the phases of a pass kernel).
int gemv_prepare(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                 WeightStreamParams& params, GemvPlan& plan);

}  // namespace gf
