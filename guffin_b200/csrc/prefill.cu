// Prefill GEMM on tcgen05 / TMEM and the elementwise steps around it (see prefill.cuh).
#include "prefill.cuh"
#include "ops.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace gf {

namespace {

constexpr uint32_t kStages = 3;                                         // shared-memory stages of 64 K elements
constexpr uint32_t kAhead = 2;                                          // stages the activation copies run ahead of the dequantisation
constexpr uint32_t kWeightBufs = 3;                                     // K units of packed weights in shared memory (two in flight)
constexpr uint32_t kPairs = kPrefillTile / 16u;                         // column pairs (16 columns) per CTA
constexpr uint32_t kMaxPairRow = 3360u;                                 // Q6_K
constexpr uint32_t kWeightBufBytes = kPairs * kMaxPairRow;
constexpr uint32_t kAStageBytes = kPrefillBlockBytes;                   // 256 rows x 64 K bf16
constexpr uint32_t kAHalfBytes = kPrefillHalf * kPrefillBlockK * 2u;    // the rows of one accumulator
constexpr uint32_t kBStageBytes = kPrefillTile * kPrefillBlockK * 2u;   // 128 columns x 64 K bf16
constexpr uint32_t kOffA = 0u, kOffB = kStages * kAStageBytes, kOffW = kOffB + kStages * kBStageBytes;
constexpr uint32_t kOffBars = kOffW + kWeightBufs * kWeightBufBytes;
constexpr uint32_t kDequantWarps = 16;                                  // warps 0..15 dequantise; warp 16 requests copies and issues the products
constexpr uint32_t kBarCount = 2u * kWeightBufs + 3u * kStages + 1u;    // weights full / free, per stage: activations landed, weights written, stage free; all done
constexpr uint32_t kPrefillSmemBytes = kOffBars + kBarCount * 8u + 16u;
static_assert(kPrefillSmemBytes <= 227u * 1024u - 1024u, "the GEMM's stages do not fit in one SM's shared memory");

// ---- tcgen05 wrappers (sm_100a PTX) ----
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Makes this thread's shared-memory stores visible to the tensor core's (asynchronous-proxy) reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory operand descriptor, K-major, no swizzle: start address, 128 bytes between the two
// core matrices of a 16-element K step, 1024 bytes between groups of eight rows, descriptor version 1.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
    return (uint64_t)((smem_address >> 4) & 0x3fffu) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor: f32 accumulator, bf16 x bf16, both operands K-major, M = 128, N = kPrefillTile.
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | ((kPrefillTile >> 3) << 17) | ((kPrefillHalf >> 4) << 24);
constexpr uint32_t kTmemColumns = 2u * kPrefillTile;                    // one accumulator of kPrefillTile columns per half of the rows

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstruction), "r"(accumulate) : "memory");
}
// The barrier receives one arrival once every tensor-core operation issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive columns of 32-bit accumulators: thread l of the warp gets lane (base + l).
__device__ __forceinline__ void tmem_load_32(uint32_t address, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t bf16_pair(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// Four consecutive K elements of column n of the B stage, starting at k (a multiple of four).
__device__ __forceinline__ void store_b4(uint8_t* stage, uint32_t n, uint32_t k, const float (&v)[4]) {
    uint8_t* dst = stage + (n >> 3) * 1024u + (k >> 3) * 128u + (n & 7u) * 16u + (k & 7u) * 2u;
    *reinterpret_cast<uint2*>(dst) = make_uint2(bf16_pair(v[0], v[1]), bf16_pair(v[2], v[3]));
}
__device__ __forceinline__ float half_bits(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }
__device__ __forceinline__ uint32_t byte_of(uint32_t word, uint32_t i) { return (word >> (8u * i)) & 0xffu; }

// ---- dequantisation of one column of one lane slot (column g + 8 * col of a column pair) for one block of
// 64 K elements: the reference's values exactly (quantization.cpp:457,517,590), then rounded to bf16.  `row`
// is the pair row (streaming layout, common.cuh), `n` the column inside the CTA tile.  A code byte becomes
// a float by a byte permute into the mantissa of 2^23 and one exact subtraction.

__device__ __forceinline__ float code_float(uint32_t word, uint32_t i, float bias) {      // byte i of word, minus (bias - 2^23)
    return __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + i)), bias);
}

// The same two values at a time with the packed f32x2 instructions (each half rounds like the scalar
// instruction, so the values are bit for bit those of the scalar form): typedef and helpers as in gemv.cuh.
typedef unsigned long long pf2;
__device__ __forceinline__ pf2 pf2_make(float lo, float hi) {
    pf2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ pf2 pf2_mul(pf2 a, pf2 b) { pf2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ pf2 pf2_add(pf2 a, pf2 b) { pf2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ uint32_t pf2_bf16(pf2 v) {              // both halves rounded to bf16, low half in the low 16 bits
    uint32_t lo, hi, r;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "r"(hi), "r"(lo));
    return r;
}
// Bytes i and i + 1 of `word` as floats, minus (bias - 2^23) each; neg_bias = {-bias, -bias}.
__device__ __forceinline__ pf2 code_pair(uint32_t word, uint32_t i, pf2 neg_bias) {
    pf2 raw;
    asm("mov.b64 %0, {%1, %2};" : "=l"(raw) : "r"(__byte_perm(word, 0x4B000000u, 0x7540u + i)), "r"(__byte_perm(word, 0x4B000000u, 0x7541u + i)));
    return pf2_add(raw, neg_bias);
}
// Four consecutive K elements of column n of the B stage from two packed pairs.
__device__ __forceinline__ void store_b4_pairs(uint8_t* stage, uint32_t n, uint32_t k, pf2 v01, pf2 v23) {
    uint8_t* dst = stage + (n >> 3) * 1024u + (k >> 3) * 128u + (n & 7u) * 16u + (k & 7u) * 2u;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pf2_bf16(v01), pf2_bf16(v23));
}

__device__ __forceinline__ void dequant_q4k(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t col, uint32_t n, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint2 words = *reinterpret_cast<const uint2*>(row + sub * 512u + lane * 16u + col * 8u);      // this column's {w0, w1}
    const uint4 h = *reinterpret_cast<const uint4*>(row + 2048u + (g + 8u * col) * 16u);
    const float d = half_bits(h.x & 0xffffu), dmin = half_bits(h.x >> 16);
    // 6-bit scales and minima of groups 2 * sub (low nibbles) and 2 * sub + 1 (high nibbles).
    const uint32_t scales = sub < 2u ? (h.y & 0x3f3f3f3fu) : ((h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u));
    const uint32_t minima = sub < 2u ? (h.z & 0x3f3f3f3fu) : (((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u));
    const uint32_t first = (sub & 1u) * 2u;
    const pf2 neg_bias = pf2_make(-8388608.0f, -8388608.0f);
#pragma unroll
    for (uint32_t nib = 0; nib < 2u; ++nib) {
        const float ds = __fmul_rn(d, (float)byte_of(scales, first + nib));
        const float dm = __fmul_rn(dmin, (float)byte_of(minima, first + nib));
        const pf2 ds2 = pf2_make(ds, ds), neg_dm2 = pf2_make(-dm, -dm);       // d * sc * q - dmin * mn, each step rounded once
#pragma unroll
        for (uint32_t w = 0; w < 2u; ++w) {
            const uint32_t codes = ((w == 0u ? words.x : words.y) >> (4u * nib)) & 0x0f0f0f0fu;
            const pf2 v01 = pf2_add(pf2_mul(ds2, code_pair(codes, 0u, neg_bias)), neg_dm2);
            const pf2 v23 = pf2_add(pf2_mul(ds2, code_pair(codes, 2u, neg_bias)), neg_dm2);
            store_b4_pairs(stage, n, 32u * nib + 16u * w + 4u * t, v01, v23);
        }
    }
}

__device__ __forceinline__ void dequant_q6k(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t col, uint32_t n, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u, half = sub >> 1, upper = sub & 1u;       // quarters 2 * upper, 2 * upper + 1 of the half
    const uint32_t column = g + 8u * col;
    const uint4 ql = *reinterpret_cast<const uint4*>(row + half * 1536u + col * 512u + lane * 16u);      // {s0 even, s0 odd, s1 even, s1 odd}
    const uint2 qh = *reinterpret_cast<const uint2*>(row + half * 1536u + 1024u + lane * 16u + col * 8u);      // {s0, s1}
    const float d = half_bits(*reinterpret_cast<const unsigned short*>(row + 3328u + column * 2u));
    const uint8_t* scale_bytes = row + 3072u + column * 16u;
#pragma unroll
    for (uint32_t s = 0; s < 2u; ++s) {
        const uint32_t even = s ? ql.z : ql.x, odd = s ? ql.w : ql.y, high = s ? qh.y : qh.x;
#pragma unroll
        for (uint32_t qq = 0; qq < 2u; ++qq) {
            const uint32_t quarter = 2u * upper + qq;
            const float ds = __fmul_rn(d, (float)(int)(signed char)scale_bytes[8u * half + 2u * quarter + s]);
            const uint32_t codes = (((qq ? odd : even) >> (4u * upper)) & 0x0f0f0f0fu) | (((high >> (2u * quarter)) & 0x03030303u) << 4);
            const pf2 ds2 = pf2_make(ds, ds), neg_bias = pf2_make(-(8388608.0f + 32.0f), -(8388608.0f + 32.0f));
            store_b4_pairs(stage, n, 32u * qq + 16u * s + 4u * t, pf2_mul(ds2, code_pair(codes, 0u, neg_bias)),
                           pf2_mul(ds2, code_pair(codes, 2u, neg_bias)));
        }
    }
}

__device__ __forceinline__ void dequant_q80(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t col, uint32_t n, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u, column = g + 8u * col;
#pragma unroll
    for (uint32_t bb = 0; bb < 2u; ++bb) {
        const uint32_t block = 2u * sub + bb;
        const uint2 words = *reinterpret_cast<const uint2*>(row + block * 512u + lane * 16u + col * 8u);      // this column's {w0, w1}
        const float d = half_bits(*reinterpret_cast<const unsigned short*>(row + 2048u + column * 8u + block * 2u));
#pragma unroll
        for (uint32_t w = 0; w < 2u; ++w) {
            const uint32_t codes = (w == 0u ? words.x : words.y) ^ 0x80808080u;        // int8 + 128
            const pf2 d2 = pf2_make(d, d), neg_bias = pf2_make(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f));
            store_b4_pairs(stage, n, 32u * bb + 16u * w + 4u * t, pf2_mul(d2, code_pair(codes, 0u, neg_bias)),
                           pf2_mul(d2, code_pair(codes, 2u, neg_bias)));
        }
    }
}

// Bounded wait that also gives up as soon as another warp of the CTA has.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, const volatile uint32_t* abort) {
    for (uint32_t spin = 0; spin < kMbarWaitLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 63u && *abort != 0u) return false;
    }
    return false;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// C[128, 128-column tile] = A[128, K] x deq(W)^T.  Grid: (tiles over all matrices of the launch, K splits);
// split s handles its share of the K units and writes its own [128][n] partial result.
//
// Warp-specialised, no block-wide barrier in the loop.  Warps 0..15 dequantise: two warps share a column pair
// of the tile, a lane takes one column of one lane slot; for every 64-element K block they wait until the
// stage is free, write their part of the bf16 weight tile and arrive on the stage's "written" barrier.  One
// thread of warp 17 requests the copies (packed weights two K units ahead, activation blocks two stages
// ahead); one thread of warp 16, once a stage's activations have landed and its weights are written, issues
// the four tensor-core products of the stage; their completion frees the stage.  (With one thread doing
// both, its serial waits, copy requests and issues took longer per stage than the dequantisation.)  Every wait is bounded and gives up
// early once any warp has; the CTA always reaches the end, releases its tensor memory and sets the error word.
__global__ void __launch_bounds__(kPrefillThreads, 1) prefill_gemm_kernel(const __grid_constant__ PrefillGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint64_t* weight_full = bars;                                  // [kWeightBufs]  packed weights of a K unit landed (bytes)
    uint64_t* weight_free = bars + kWeightBufs;                    // [kWeightBufs]  all dequantising warps are done with the unit
    uint64_t* a_full = bars + 2 * kWeightBufs;                     // [kStages]      activation block landed (bytes)
    uint64_t* b_full = a_full + kStages;                           // [kStages]      all dequantising warps have written the stage
    uint64_t* stage_free = b_full + kStages;                       // [kStages]      the stage's products have finished
    uint64_t* done_bar = stage_free + kStages;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const volatile uint32_t* abort = &abort_flag;

    uint32_t which = 0;
    if (p.matrices > 1u && blockIdx.x >= p.m[1].first_tile) which = 1;
    if (p.matrices > 2u && blockIdx.x >= p.m[2].first_tile) which = 2;
    const PrefillMatrix& mat = p.m[which];
    const uint32_t tile = blockIdx.x - mat.first_tile, dtype = mat.dtype;
    const uint32_t row_bytes = pair_row_bytes((int)dtype), subs = p.unit_elems / kPrefillBlockK;
    const uint8_t* weights = mat.weight + (size_t)tile * kPairs * p.units * row_bytes;      // pair rows of pair i start i * units * row_bytes further
    // This split's K units and the activation blocks that go with them.
    const uint32_t unit_begin = (uint32_t)((uint64_t)p.units * blockIdx.y / gridDim.y);
    const uint32_t unit_count = (uint32_t)((uint64_t)p.units * (blockIdx.y + 1u) / gridDim.y) - unit_begin;
    const uint32_t steps = unit_count * subs;
    const uint8_t* blocks = p.a + (size_t)unit_begin * subs * kPrefillBlockBytes;

    if (tid == 0) {
        abort_flag = 0u;
        for (uint32_t i = 0; i < kWeightBufs; ++i) { mbar_init(&weight_full[i], 1); mbar_init(&weight_free[i], kDequantWarps); }
        for (uint32_t i = 0; i < kStages; ++i) { mbar_init(&a_full[i], 1); mbar_init(&b_full[i], kDequantWarps); mbar_init(&stage_free[i], 1); }
        mbar_init(done_bar, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kTmemColumns);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    bool ok = true;

    if (warp == kDequantWarps + 1u) {
        // The copy warp: packed weights two K units ahead, activation blocks kAhead stages ahead.
        if (lane == 0) {
            uint32_t requested_units = 0, requested_blocks = 0;
            auto request_weights = [&](uint32_t j) {          // j counts this split's units
                requested_units = j + 1u;
                uint64_t* bar = &weight_full[j % kWeightBufs];
                uint8_t* dst = smem + kOffW + (j % kWeightBufs) * kWeightBufBytes;
                mbar_expect_tx(bar, kPairs * row_bytes);
                for (uint32_t i = 0; i < kPairs; ++i)
                    bulk_load(dst + i * row_bytes, weights + ((size_t)i * p.units + unit_begin + j) * row_bytes, row_bytes, bar);
            };
            auto request_block = [&](uint32_t step) {         // the stage must be free
                requested_blocks = step + 1u;
                const uint32_t stage = step % kStages;
                mbar_expect_tx(&a_full[stage], p.halves * kAHalfBytes);          // rows 0-127 lie in the block's first half
                bulk_load(smem + kOffA + stage * kAStageBytes, blocks + (size_t)step * kPrefillBlockBytes, p.halves * kAHalfBytes, &a_full[stage]);
            };
            for (uint32_t j = 0; j < 2u && j < unit_count; ++j) request_weights(j);
            for (uint32_t step = 0; step < kAhead && step < steps; ++step) request_block(step);
            for (uint32_t step = 0; step < steps && ok; ++step) {
                const uint32_t j = step / subs;
                if (step % subs == 0u && j + 2u < unit_count) {
                    // The buffer two units on held unit j - 1: every dequantising warp must be done with it.
                    if (j >= 1u && !wait_or_abort(&weight_free[(j + 2u) % kWeightBufs], ((j - 1u) / kWeightBufs) & 1u, abort)) { ok = false; break; }
                    request_weights(j + 2u);
                }
                if (step + kAhead < steps) {
                    const uint32_t next = step + kAhead, next_use = next / kStages;
                    if (next_use > 0u && !wait_or_abort(&stage_free[next % kStages], (next_use - 1u) & 1u, abort)) { ok = false; break; }
                    request_block(next);
                }
            }
            // Whether this warp gave up or another did: copies already requested get a bounded chance to
            // land before the shared memory is released (after a clean run every copy has been consumed).
            if (!ok || !wait_or_abort(done_bar, 0u, abort)) {
                ok = false;
                abort_flag = 1u;
                for (uint32_t j = 0; j < unit_count; ++j) {
                    if (j + kWeightBufs < requested_units) continue;
                    if (j >= requested_units) break;
                    mbar_wait(&weight_full[j % kWeightBufs], (j / kWeightBufs) & 1u, 1u << 16);
                }
                for (uint32_t step = 0; step < steps; ++step) {
                    if (step + kStages < requested_blocks) continue;
                    if (step >= requested_blocks) break;
                    mbar_wait(&a_full[step % kStages], (step / kStages) & 1u, 1u << 16);
                }
            }
        }
    } else if (warp == kDequantWarps) {
        // The issuing warp: once a stage's activations have landed and its weights are written, the four
        // tensor-core products of the stage; their completion frees the stage.
        if (lane == 0) {
            for (uint32_t step = 0; step < steps && ok; ++step) {
                const uint32_t stage = step % kStages, use = step / kStages;
                if (!wait_or_abort(&a_full[stage], use & 1u, abort) || !wait_or_abort(&b_full[stage], use & 1u, abort)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_address = smem_u32(smem + kOffA + stage * kAStageBytes), b_address = smem_u32(smem + kOffB + stage * kBStageBytes);
                for (uint32_t h = 0; h < p.halves; ++h)
#pragma unroll
                    for (uint32_t kk = 0; kk < kPrefillBlockK / 16u; ++kk)
                        mma_bf16(tmem + h * kPrefillTile, operand_descriptor(a_address + h * kAHalfBytes + kk * 256u),
                                 operand_descriptor(b_address + kk * 256u), (step | kk) != 0u ? 1u : 0u);
                mma_commit(&stage_free[stage]);
            }
            if (ok) mma_commit(done_bar);
            else abort_flag = 1u;
        }
    } else {
        // Dequantisation: warp w takes column pair w % 8 of the tile and the column g + 8 * (w / 8) of each lane slot.
        const uint32_t my_pair = warp % kPairs, column_half = warp / kPairs, my_column = my_pair * 16u + (lane >> 2) + 8u * column_half;
        uint32_t step = 0;
        for (uint32_t j = 0; j < unit_count && ok; ++j) {
            if (!wait_or_abort(&weight_full[j % kWeightBufs], (j / kWeightBufs) & 1u, abort)) { ok = false; break; }
            const uint8_t* pair_row = smem + kOffW + (j % kWeightBufs) * kWeightBufBytes + my_pair * row_bytes;
            for (uint32_t sub = 0; sub < subs; ++sub, ++step) {
                const uint32_t stage = step % kStages, use = step / kStages;
                if (use > 0u && !wait_or_abort(&stage_free[stage], (use - 1u) & 1u, abort)) { ok = false; break; }
                uint8_t* b_stage = smem + kOffB + stage * kBStageBytes;
                if (dtype == GF_Q4_K) dequant_q4k(pair_row, sub, lane, column_half, my_column, b_stage);
                else if (dtype == GF_Q6_K) dequant_q6k(pair_row, sub, lane, column_half, my_column, b_stage);
                else dequant_q80(pair_row, sub, lane, column_half, my_column, b_stage);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&b_full[stage]);
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&weight_free[j % kWeightBufs]);
        }
        if (!ok && lane == 0) abort_flag = 1u;
        if (ok && !wait_or_abort(done_bar, 0u, abort)) { ok = false; if (lane == 0) abort_flag = 1u; }
    }
    const bool failed = __syncthreads_or(ok ? 0 : 1) != 0;
    if (!failed && warp < kDequantWarps) {
        tc_fence_after_sync();
        // Warp w reads accumulator lanes 32 * (w % 4) .. +31 (its quarter of a half's rows) and a quarter of the columns.
        const uint32_t column0 = (warp >> 2) * (kPrefillTile / 4u);
        for (uint32_t h = 0; h < p.halves; ++h) {
            const uint32_t row = h * kPrefillHalf + (warp & 3u) * 32u + lane;
            float* out = mat.out + (size_t)blockIdx.y * kPrefillRows * mat.n + (size_t)row * mat.n + (size_t)tile * kPrefillTile + column0;
            float v[32];
            tmem_load_32(tmem + (((warp & 3u) * 32u) << 16) + h * kPrefillTile + column0, v);
#pragma unroll
            for (uint32_t i = 0; i < 32u; i += 4u)
                *reinterpret_cast<float4*>(out + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        tc_fence_before_sync();
    } else if (failed && tid == 0) {
        atomicExch(p.error_flag, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemColumns);
}

// ---- elementwise steps.  A thread handles eight consecutive K elements of one row: two 16-byte loads per
// input and one 16-byte store of eight bf16 into the tile-major operand.

__device__ __forceinline__ float block_total(float v, float* scratch) {
    v = warp_sum(v);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < blockDim.x / 32u; ++w) total += scratch[w];      // the same order in every thread
    __syncthreads();
    return total;
}

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store_a8(uint8_t* a, uint32_t row, uint32_t k, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(a + tile_major_offset(row, k)) =
        make_uint4(bf16_pair(v[0], v[1]), bf16_pair(v[2], v[3]), bf16_pair(v[4], v[5]), bf16_pair(v[6], v[7]));
}

constexpr uint32_t kNormPieces = 8;       // 8-element pieces a thread keeps in registers: rows of up to 16384 values

// One block per row.  x is the sum of `splits` partial results laid [split][128][k] (added in split order).
// Rows beyond `rows` (up to 128) are written as zeros so that the GEMM's unused rows are defined.
__global__ void __launch_bounds__(256) prefill_norm_kernel(const float* __restrict__ x, uint32_t splits, const float* __restrict__ residual,
                                                           const float* __restrict__ gamma0, const float* __restrict__ gamma1,
                                                           float* __restrict__ residual_out, uint8_t* __restrict__ a_out,
                                                           uint32_t rows, uint32_t k, float eps, int mode) {
    __shared__ float scratch[8];
    const uint32_t row = blockIdx.x, pieces = k / 8u;
    if (row >= rows) {
        const float zero[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (a_out) for (uint32_t piece = threadIdx.x; piece < pieces; piece += blockDim.x) store_a8(a_out, row, piece * 8u, zero);
        return;
    }
    float v[kNormPieces][8];
    float sum = 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < kNormPieces; ++j) {
        const uint32_t piece = threadIdx.x + j * 256u;
        if (piece >= pieces) break;
        load8(x + (size_t)row * k + piece * 8u, v[j]);
        for (uint32_t split = 1; split < splits; ++split) {
            float more[8];
            load8(x + ((size_t)split * kPrefillRows + row) * k + piece * 8u, more);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] += more[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sum = fmaf(v[j][i], v[j][i], sum);
    }
    float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(block_total(sum, scratch), (float)k), eps)));
    if (mode == 1) {
        float sum2 = 0.0f;
#pragma unroll
        for (uint32_t j = 0; j < kNormPieces; ++j) {
            const uint32_t piece = threadIdx.x + j * 256u;
            if (piece >= pieces) break;
            float r[8], g[8];
            load8(residual + (size_t)row * k + piece * 8u, r);
            load8(gamma0 + piece * 8u, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[j][i] = __fadd_rn(r[i], __fmul_rn(__fmul_rn(v[j][i], inv), g[i]));
                sum2 = fmaf(v[j][i], v[j][i], sum2);
            }
            *reinterpret_cast<float4*>(residual_out + (size_t)row * k + piece * 8u) = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
            *reinterpret_cast<float4*>(residual_out + (size_t)row * k + piece * 8u + 4u) = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
        }
        if (!gamma1 || !a_out) return;
        inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(block_total(sum2, scratch), (float)k), eps)));
    }
#pragma unroll
    for (uint32_t j = 0; j < kNormPieces; ++j) {
        const uint32_t piece = threadIdx.x + j * 256u;
        if (piece >= pieces) break;
        float g[8], out[8];
        load8(gamma1 + piece * 8u, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = __fmul_rn(__fmul_rn(v[j][i], inv), g[i]);
        store_a8(a_out, row, piece * 8u, out);
    }
}

// Eight values of row `row` starting at element `at`, summed over `splits` partial results laid [split][128][k].
__device__ __forceinline__ void load8_summed(const float* x, uint32_t splits, uint32_t row, uint32_t k, uint32_t at, float (&v)[8]) {
    load8(x + (size_t)row * k + at, v);
    for (uint32_t split = 1; split < splits; ++split) {
        float more[8];
        load8(x + ((size_t)split * kPrefillRows + row) * k + at, more);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += more[i];
    }
}

// Grid (128 rows, pieces / 256).  gate and up are sums of `splits` partial results.
__global__ void __launch_bounds__(256) prefill_geglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, uint32_t splits,
                                                            uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x, piece = blockIdx.y * blockDim.x + threadIdx.x;
    if (piece >= k / 8u) return;
    float out[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (row < rows) {
        float g[8], u[8];
        load8_summed(gate, splits, row, k, piece * 8u, g);
        load8_summed(up, splits, row, k, piece * 8u, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float v = g[i];
            const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
            out[i] = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner))), u[i]);
        }
    }
    store_a8(a_out, row, piece * 8u, out);
}

// In-place sum of K-split partial results, for up to three matrices: x[0][row][:] += x[1..][row][:].
struct ReduceSet { float* x[3]; uint32_t n[3]; uint32_t count, splits; };
__global__ void __launch_bounds__(256) prefill_reduce_kernel(ReduceSet set, uint32_t rows) {
    const uint32_t row = blockIdx.x;
    if (row >= rows) return;
    for (uint32_t m = 0; m < set.count; ++m) {
        const uint32_t n = set.n[m];
        for (uint32_t piece = blockIdx.y * blockDim.x + threadIdx.x; piece < n / 8u; piece += gridDim.y * blockDim.x) {
            float v[8];
            load8_summed(set.x[m], set.splits, row, n, piece * 8u, v);
            float* dst = set.x[m] + (size_t)row * n + piece * 8u;
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}

__global__ void __launch_bounds__(256) prefill_pack_kernel(const float* __restrict__ x, uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x, piece = blockIdx.y * blockDim.x + threadIdx.x;
    if (piece >= k / 8u) return;
    float out[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (row < rows) load8(x + (size_t)row * k + piece * 8u, out);
    store_a8(a_out, row, piece * 8u, out);
}

// ---- attention of a prompt chunk over a binary16 cache ------------------------------------------------
//
// Online-softmax GQA for up to 128 rows at once, both contractions on the tensor cores
// (mma.sync.m16n8k16, f16 operands, f32 accumulation), operands straight from global memory in 16-byte
// pieces -- no shared memory.  The sixteen rows of an MMA tile are (prompt row, query head) pairs of one KV
// head: 16 / G prompt rows x G heads.  A block is four pairs of warps on the same sixteen queries.  The pairs
// take the tiles of sixteen cached rows in turn (pair q the tiles q, q + 4, ...) and are merged at the end
// through shared memory; inside a pair both warps compute the scores of a tile and each accumulates one half
// of the 256 output dimensions.
// The contraction index of a product may be permuted as long as both operands agree, so a lane reads
// whole 16-byte pieces: for the scores, dimensions 32c + 8t .. +7 of its query rows and of cached row g
// serve k-steps 2c and 2c + 1; for the outputs, dimensions 8g .. 8g + 7 (of each group of 64) of cached
// rows 2t, 2t+1, 2t+8, 2t+9 are paired across rows by byte permutes, and column g of output tile j of the
// group stands for dimension 8g + j.  (flash prefill attention of the reference: metal_kernels.mm:2596-2798.)

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t half_pair(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t word_at(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

constexpr uint32_t kAttentionPairs = 4;                   // warp pairs of a block, each on every fourth tile of cached rows

template <int G>
__global__ void __launch_bounds__(64 * kAttentionPairs) prefill_attention_kernel(AttentionParams p) {
    constexpr uint32_t kRows = 16u / G;                   // prompt rows per block
    __shared__ float merge_m[kAttentionPairs][16], merge_l[kAttentionPairs][16];
    __shared__ float merge_acc[2][2][64][32];             // [slot][half][accumulator word][lane]
    const uint32_t kvh = blockIdx.x, first_row = blockIdx.y * kRows;
    const uint32_t warp = threadIdx.x >> 5, half = warp & 1u, pair = warp >> 1;
    const uint32_t lane = threadIdx.x & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t base = *p.base_position;
    const uint32_t kv_width = p.kv_heads * 256u;
    const __half* ring_k = static_cast<const __half*>(p.ring_k);
    const __half* ring_v = static_cast<const __half*>(p.ring_v);
    const __half* priv_k = static_cast<const __half*>(p.private_k);
    const __half* priv_v = static_cast<const __half*>(p.private_v);

    // This lane's two query rows of the tile (m = g and g + 8): prompt row and head, and what they may see.
    uint32_t low[2], high[2];
    bool live[2];
    const float* query[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint32_t m = g + 8u * i, row = first_row + m / G, head = kvh * G + m % G;
        live[i] = row < p.rows;
        const uint32_t position = base + row;
        low[i] = live[i] ? ((p.window != 0u && position + 1u > p.window) ? position + 1u - p.window : 0u) : 1u;
        high[i] = live[i] ? position : 0u;
        query[i] = p.q + ((size_t)min(row, p.rows - 1u) * p.heads + head) * 256u;
    }
    // A registers of the scores: qa[c][i] = dimensions 32c + 8t .. +7 of query row i, scaled, as four f16 pairs.
    uint4 qa[8][2];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 x = *reinterpret_cast<const float4*>(query[i] + 32 * c + 8 * t);
            const float4 y = *reinterpret_cast<const float4*>(query[i] + 32 * c + 8 * t + 4);
            qa[c][i] = live[i] ? make_uint4(half_pair(x.x * p.scale, x.y * p.scale), half_pair(x.z * p.scale, x.w * p.scale),
                                            half_pair(y.x * p.scale, y.y * p.scale), half_pair(y.z * p.scale, y.w * p.scale))
                               : make_uint4(0u, 0u, 0u, 0u);
        }
    float acc[16][4];                                     // output tiles (J, j) of this warp's two groups of 64 dimensions
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    // Cached rows the block's queries can see: from the first row's window start to the last row itself.
    const uint32_t last_row = min(first_row + kRows, p.rows) - 1u;
    const uint32_t first_position = (p.window != 0u && base + first_row + 1u > p.window) ? base + first_row + 1u - p.window : 0u;
    const uint32_t end_position = base + last_row + 1u;
    auto row_pointer = [&](uint32_t position, const __half* ring, const __half* priv) -> const __half* {
        position = min(position, end_position - 1u);
        return position < base ? ring + (size_t)(position & p.ring_mask) * kv_width + kvh * 256u
                               : priv + (size_t)(position - base) * kv_width + kvh * 256u;
    };
    for (uint32_t tile = first_position + 16u * pair; tile < end_position; tile += 16u * kAttentionPairs) {
        // Scores of sixteen cached rows: two n-tiles of eight.
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            s[n][0] = 0.0f; s[n][1] = 0.0f; s[n][2] = 0.0f; s[n][3] = 0.0f;
            const __half* key = row_pointer(tile + 8u * n + g, ring_k, priv_k);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 kb = __ldcg(reinterpret_cast<const uint4*>(key + 32 * c + 8 * t));
                mma_f16(s[n], qa[c][0].x, qa[c][1].x, qa[c][0].y, qa[c][1].y, kb.x, kb.y);
                mma_f16(s[n], qa[c][0].z, qa[c][1].z, qa[c][0].w, qa[c][1].w, kb.z, kb.w);
            }
        }
        // s[n] = (row g: keys 2t, 2t+1), (row g + 8: keys 2t, 2t+1) of n-tile n.
        float m_new[2] = {m_run[0], m_run[1]};
        bool visible[2][2][2];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t position = tile + 8u * n + 2u * t + e;
                    float& v = s[n][2 * i + e];
                    if (p.softcap > 0.0f) v = tanhf(v / p.softcap) * p.softcap;
                    visible[n][i][e] = position >= low[i] && position <= high[i];
                    if (visible[n][i][e]) m_new[i] = fmaxf(m_new[i], v);
                }
        uint32_t pa[2][2];                                // A registers of the outputs: [n-tile][row i] = weights of keys 2t, 2t+1
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
            const float corr = m_run[i] == -INFINITY ? 0.0f : expf(m_run[i] - m_new[i]);
            float sum = 0.0f;
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const float w0 = visible[n][i][0] ? expf(s[n][2 * i] - m_new[i]) : 0.0f;
                const float w1 = visible[n][i][1] ? expf(s[n][2 * i + 1] - m_new[i]) : 0.0f;
                sum += w0 + w1;
                pa[n][i] = half_pair(w0, w1);
            }
            l_run[i] = l_run[i] * corr + sum;
            m_run[i] = m_new[i];
#pragma unroll
            for (int o = 0; o < 16; ++o) { acc[o][2 * i] *= corr; acc[o][2 * i + 1] *= corr; }
        }
        // Outputs: this warp's half of the dimensions, J = 2 * half, 2 * half + 1.
        const __half* value[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) value[u] = row_pointer(tile + 2u * t + (u & 1) + 8u * (u >> 1), ring_v, priv_v);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            const uint32_t J = 2u * half + jj;
            uint4 vr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) vr[u] = __ldcg(reinterpret_cast<const uint4*>(value[u] + 64u * J + 8u * g));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(word_at(vr[0], j >> 1), word_at(vr[1], j >> 1), sel);
                const uint32_t b1 = __byte_perm(word_at(vr[2], j >> 1), word_at(vr[3], j >> 1), sel);
                mma_f16(acc[jj * 8 + j], pa[0][0], pa[0][1], pa[1][0], pa[1][1], b0, b1);
            }
        }
    }
    // l over the four lanes that share a row.
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    // Merge of the pairs: every pair rescales its sums to the common maximum and the common denominator, then
    // pairs 2 and 3 hand their sums to pairs 0 and 1, and pair 1 hands the result to pair 0.
    if (half == 0u && t == 0u) {
#pragma unroll
        for (int i = 0; i < 2; ++i) { merge_m[pair][g + 8 * i] = m_run[i]; merge_l[pair][g + 8 * i] = l_run[i]; }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float top = -INFINITY;
#pragma unroll
        for (uint32_t q = 0; q < kAttentionPairs; ++q) top = fmaxf(top, merge_m[q][g + 8 * i]);
        float denominator = 0.0f;
#pragma unroll
        for (uint32_t q = 0; q < kAttentionPairs; ++q) {
            const float mq = merge_m[q][g + 8 * i];
            if (mq != -INFINITY) denominator += merge_l[q][g + 8 * i] * expf(mq - top);
        }
        const float factor = (m_run[i] == -INFINITY || denominator == 0.0f) ? 0.0f : expf(m_run[i] - top) / denominator;
#pragma unroll
        for (int o = 0; o < 16; ++o) { acc[o][2 * i] *= factor; acc[o][2 * i + 1] *= factor; }
    }
    if (pair >= 2u) {
#pragma unroll
        for (int o = 0; o < 16; ++o)
#pragma unroll
            for (int e = 0; e < 4; ++e) merge_acc[pair - 2u][half][o * 4 + e][lane] = acc[o][e];
    }
    __syncthreads();
    if (pair < 2u) {
#pragma unroll
        for (int o = 0; o < 16; ++o)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[o][e] += merge_acc[pair][half][o * 4 + e][lane];
    }
    __syncthreads();
    if (pair == 1u) {
#pragma unroll
        for (int o = 0; o < 16; ++o)
#pragma unroll
            for (int e = 0; e < 4; ++e) merge_acc[0][half][o * 4 + e][lane] = acc[o][e];
    }
    __syncthreads();
    if (pair != 0u) return;
#pragma unroll
    for (int o = 0; o < 16; ++o)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[o][e] += merge_acc[0][half][o * 4 + e][lane];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!live[i]) continue;
        const uint32_t m = g + 8u * i, row = first_row + m / G, head = kvh * G + m % G;
        float* out = p.out + ((size_t)row * p.heads + head) * 256u;
        const float inv = 1.0f;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // Columns 2t and 2t + 1 of output tile (J, j) stand for dimensions 64J + 8 * (2t) + j and 64J + 8 * (2t + 1) + j.
                const uint32_t J = 2u * half + jj;
                out[64u * J + 16u * t + j] = acc[jj * 8 + j][2 * i] * inv;
                out[64u * J + 16u * t + 8u + j] = acc[jj * 8 + j][2 * i + 1] * inv;
            }
    }
}

}  // namespace

int launch_prefill_gemm(const PrefillGemmLaunch& launch, int* error_flag, cudaStream_t stream) {
    if (launch.count == 0 || launch.count > 3 || !launch.a || !error_flag) return fail(GF_ERR_INVALID, "prefill GEMM: bad launch");
    PrefillGemmParams p = {};
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < launch.count; ++i) {
        const auto& m = launch.matrices[i];
        if (m.dtype != GF_Q4_K && m.dtype != GF_Q6_K && m.dtype != GF_Q8_0) return fail(GF_ERR_INVALID, "prefill GEMM: unsupported weight dtype %d", m.dtype);
        if (!m.packed || !m.out || m.n == 0 || m.n % kPrefillTile) return fail(GF_ERR_INVALID, "prefill GEMM: N must be a positive multiple of %u", kPrefillTile);
        const uint32_t unit = unit_elements(m.dtype);
        if (p.unit_elems && p.unit_elems != unit) return fail(GF_ERR_INVALID, "prefill GEMM: Q8_0 and K-quant matrices cannot share a launch");
        p.unit_elems = unit;
        p.m[i] = PrefillMatrix{static_cast<const uint8_t*>(m.packed), m.out, (uint32_t)m.n, (uint32_t)m.dtype, tiles};
        tiles += (uint32_t)(m.n / kPrefillTile);
    }
    if (launch.k == 0 || launch.k % p.unit_elems) return fail(GF_ERR_INVALID, "prefill GEMM: K must be a positive multiple of %u", p.unit_elems);
    p.matrices = launch.count;
    p.tiles = tiles;
    p.k = (uint32_t)launch.k;
    p.units = (uint32_t)(launch.k / p.unit_elems);
    if (launch.splits == 0 || launch.splits > p.units) return fail(GF_ERR_INVALID, "prefill GEMM: K splits must be between 1 and the number of K units");
    p.a = static_cast<const uint8_t*>(launch.a);
    p.error_flag = error_flag;
    if (launch.rows == 0 || launch.rows > kPrefillRows) return fail(GF_ERR_INVALID, "prefill GEMM: rows outside [1, %u]", kPrefillRows);
    p.halves = prefill_padded_rows(launch.rows) / kPrefillHalf;
    static std::once_flag once[64];
    int device = 0;
    cudaGetDevice(&device);
    cudaError_t attr_error = cudaSuccess;
    std::call_once(once[device & 63], [&] {
        attr_error = cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrefillSmemBytes);
    });
    GF_CUDA(attr_error);
    prefill_gemm_kernel<<<dim3(tiles, launch.splits), kPrefillThreads, kPrefillSmemBytes, stream>>>(p);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

uint32_t prefill_gemm_splits(uint64_t n, uint64_t k, int dtype) {
    // CTAs run one per SM, wave after wave: a launch costs ceil(tiles * splits / SMs) waves of 1 / splits of the
    // whole K each.  Take the split with the least time; ties go to fewer splits.
    const uint32_t tiles = (uint32_t)(n / kPrefillTile), units = (uint32_t)(k / unit_elements(dtype)), sms = (uint32_t)sm_count();
    if (tiles >= sms) return 1;         // every SM already has a tile: more CTAs only add partial results
    uint32_t best = 1;
    double best_cost = 1e30;
    for (uint32_t splits = 1; splits <= kPrefillMaxSplits && splits <= units; ++splits) {
        const uint32_t waves = (tiles * splits + sms - 1u) / sms;
        const double cost = (double)waves * ((double)((units + splits - 1u) / splits) + 0.5);      // half a unit of set-up and epilogue per CTA
        if (cost < best_cost - 1e-9) { best_cost = cost; best = splits; }
    }
    return best;
}

int launch_prefill_norm(const float* x, uint32_t splits, const float* residual, const float* gamma0, const float* gamma1,
                        float* residual_out, void* a_out, uint32_t rows, uint32_t k, float eps, int mode, cudaStream_t stream) {
    if (!x || splits == 0 || rows == 0 || rows > kPrefillRows || k == 0 || k % 8u || k > kNormPieces * 256u * 8u
        || (mode == 0 && (!gamma1 || !a_out)) || (mode == 1 && (!residual || !gamma0 || !residual_out)))
        return fail(GF_ERR_INVALID, "prefill norm: bad arguments");
    const uint32_t blocks = a_out ? prefill_padded_rows(rows) : rows;
    prefill_norm_kernel<<<blocks, 256, 0, stream>>>(x, splits, residual, gamma0, gamma1, residual_out, static_cast<uint8_t*>(a_out), rows, k, eps, mode);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_reduce(float* const* x, const uint64_t* n, uint32_t count, uint32_t splits, uint32_t rows, cudaStream_t stream) {
    if (!x || !n || count == 0 || count > 3 || splits == 0 || rows == 0 || rows > kPrefillRows) return fail(GF_ERR_INVALID, "prefill reduce: bad arguments");
    if (splits == 1) return GF_OK;
    ReduceSet set = {};
    for (uint32_t i = 0; i < count; ++i) { set.x[i] = x[i]; set.n[i] = (uint32_t)n[i]; }
    set.count = count; set.splits = splits;
    prefill_reduce_kernel<<<dim3(rows, 2), 256, 0, stream>>>(set, rows);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_geglu(const float* gate, const float* up, uint32_t splits, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!gate || !up || !a_out || splits == 0 || rows == 0 || rows > kPrefillRows || k % 8u) return fail(GF_ERR_INVALID, "prefill GeGLU: bad arguments");
    prefill_geglu_kernel<<<dim3(prefill_padded_rows(rows), (k / 8u + 255u) / 256u), 256, 0, stream>>>(gate, up, splits, static_cast<uint8_t*>(a_out), rows, k);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

bool prefill_attention_supported(const AttentionParams& p) {
    const uint32_t group = p.kv_heads ? p.heads / p.kv_heads : 0u;
    return p.kv_f16 && p.head_dim == 256u && p.kv_heads != 0u && p.heads % p.kv_heads == 0u && (group == 1u || group == 2u || group == 4u);
}

int launch_prefill_attention(const AttentionParams& p, cudaStream_t stream) {
    if (!prefill_attention_supported(p) || p.rows == 0 || p.rows > kPrefillRows) return fail(GF_ERR_INVALID, "prefill attention: unsupported shape");
    const uint32_t group = p.heads / p.kv_heads, rows_per_block = 16u / group;
    const dim3 grid(p.kv_heads, (p.rows + rows_per_block - 1u) / rows_per_block);
    if (group == 1u) prefill_attention_kernel<1><<<grid, 64 * kAttentionPairs, 0, stream>>>(p);
    else if (group == 2u) prefill_attention_kernel<2><<<grid, 64 * kAttentionPairs, 0, stream>>>(p);
    else prefill_attention_kernel<4><<<grid, 64 * kAttentionPairs, 0, stream>>>(p);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_pack(const float* x, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!x || !a_out || rows == 0 || rows > kPrefillRows || k % 8u) return fail(GF_ERR_INVALID, "prefill pack: bad arguments");
    prefill_pack_kernel<<<dim3(prefill_padded_rows(rows), (k / 8u + 255u) / 256u), 256, 0, stream>>>(x, static_cast<uint8_t*>(a_out), rows, k);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_prefill_workspace_bytes(uint64_t k) { return tile_major_bytes(k); }

int gf_prefill_attention(const float* q_dev, const void* ring_k_dev, const void* ring_v_dev, const void* private_k_dev,
                         const void* private_v_dev, float* out_dev, const uint32_t* base_position_dev, uint32_t rows,
                         uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t ring_rows, uint32_t window, float scale,
                         float softcap, void* stream) {
    if (!q_dev || !ring_k_dev || !ring_v_dev || !private_k_dev || !private_v_dev || !out_dev || !base_position_dev || rows == 0
        || rows > kPrefillRows || ring_rows == 0 || (ring_rows & (ring_rows - 1u)))
        return fail(GF_ERR_INVALID, "gf_prefill_attention: bad arguments (ring rows must be a power of two, rows at most %u)", kPrefillRows);
    const uintptr_t pointers = reinterpret_cast<uintptr_t>(q_dev) | reinterpret_cast<uintptr_t>(ring_k_dev) | reinterpret_cast<uintptr_t>(ring_v_dev)
        | reinterpret_cast<uintptr_t>(private_k_dev) | reinterpret_cast<uintptr_t>(private_v_dev) | reinterpret_cast<uintptr_t>(out_dev);
    if (pointers & 15u) return fail(GF_ERR_INVALID, "gf_prefill_attention: device pointers must be 16-byte aligned");
    AttentionParams p;
    p.q = q_dev; p.ring_k = ring_k_dev; p.ring_v = ring_v_dev; p.private_k = private_k_dev; p.private_v = private_v_dev;
    p.out = out_dev; p.partial_out = nullptr; p.partial_ml = nullptr; p.counters = nullptr;
    p.base_position = base_position_dev;
    p.rows = rows; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.ring_mask = ring_rows - 1u; p.window = window; p.target_parts = 1; p.scale = scale; p.softcap = softcap; p.kv_f16 = 1;
    return launch_prefill_attention(p, as_stream(stream));
}

int gf_prefill_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev, uint32_t rows, uint64_t k, uint64_t n,
                      void* workspace_dev, void* stream) {
    if (!packed_dev || !x_dev || !y_dev || !workspace_dev || rows == 0 || rows > kPrefillRows)
        return fail(GF_ERR_INVALID, "gf_prefill_matmul: null buffer or rows outside [1, %u]", kPrefillRows);
    if ((reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(workspace_dev)) & 15u)
        return fail(GF_ERR_INVALID, "gf_prefill_matmul: y and the workspace must be 16-byte aligned");
    static int* flags[64] = {nullptr};
    int device = 0;
    GF_CUDA(cudaGetDevice(&device));
    device &= 63;
    if (!flags[device]) {
        GF_CUDA(cudaMalloc(&flags[device], sizeof(int)));
        GF_CUDA(cudaMemset(flags[device], 0, sizeof(int)));
    }
    cudaStream_t s = as_stream(stream);
    const int status = launch_prefill_pack(x_dev, workspace_dev, rows, (uint32_t)k, s);
    if (status != GF_OK) return status;
    PrefillGemmLaunch launch;
    launch.matrices[0] = {dtype, packed_dev, y_dev, n};
    launch.count = 1;
    launch.k = k;
    launch.a = workspace_dev;
    launch.rows = rows;
    const int launched = launch_prefill_gemm(launch, flags[device], s);
    if (launched != GF_OK) return launched;
    int value = 0;
    GF_CUDA(cudaMemcpyAsync(&value, flags[device], sizeof(int), cudaMemcpyDeviceToHost, s));
    GF_CUDA(cudaStreamSynchronize(s));
    if (value != 0) {
        cudaMemsetAsync(flags[device], 0, sizeof(int), s);
        return fail(GF_ERR_TIMEOUT, "gf_prefill_matmul: a bounded wait gave up");
    }
    return GF_OK;
}

}  // extern "C"
