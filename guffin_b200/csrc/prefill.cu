// Prefill GEMM on tcgen05 / TMEM and the elementwise steps around it (see prefill.cuh).
#include "prefill.cuh"
#include "ops.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace gf {

namespace {

constexpr uint32_t kStages = 4;                                         // shared-memory stages of 64 K elements
constexpr uint32_t kAhead = 2;                                          // stages the activation copies run ahead of the dequantisation
constexpr uint32_t kWeightBufs = 3;                                     // K units of packed weights in shared memory (two in flight)
constexpr uint32_t kPairs = kPrefillTile / 16u;                         // column pairs (16 columns) per CTA
constexpr uint32_t kMaxPairRow = 3360u;                                 // Q6_K
constexpr uint32_t kWeightBufBytes = kPairs * kMaxPairRow;
constexpr uint32_t kAStageBytes = kPrefillBlockBytes;                   // 128 rows x 64 K bf16
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
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | ((kPrefillTile >> 3) << 17) | ((kPrefillRows >> 4) << 24);

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

__device__ __forceinline__ void dequant_q4k(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t col, uint32_t n, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint2 words = *reinterpret_cast<const uint2*>(row + sub * 512u + lane * 16u + col * 8u);      // this column's {w0, w1}
    const uint4 h = *reinterpret_cast<const uint4*>(row + 2048u + (g + 8u * col) * 16u);
    const float d = half_bits(h.x & 0xffffu), dmin = half_bits(h.x >> 16);
    // 6-bit scales and minima of groups 2 * sub (low nibbles) and 2 * sub + 1 (high nibbles).
    const uint32_t scales = sub < 2u ? (h.y & 0x3f3f3f3fu) : ((h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u));
    const uint32_t minima = sub < 2u ? (h.z & 0x3f3f3f3fu) : (((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u));
    const uint32_t first = (sub & 1u) * 2u;
#pragma unroll
    for (uint32_t nib = 0; nib < 2u; ++nib) {
        const float ds = __fmul_rn(d, (float)byte_of(scales, first + nib));
        const float dm = __fmul_rn(dmin, (float)byte_of(minima, first + nib));
#pragma unroll
        for (uint32_t w = 0; w < 2u; ++w) {
            const uint32_t codes = ((w == 0u ? words.x : words.y) >> (4u * nib)) & 0x0f0f0f0fu;
            float v[4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) v[i] = __fsub_rn(__fmul_rn(ds, code_float(codes, i, 8388608.0f)), dm);
            store_b4(stage, n, 32u * nib + 16u * w + 4u * t, v);
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
            float v[4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) v[i] = __fmul_rn(ds, code_float(codes, i, 8388608.0f + 32.0f));
            store_b4(stage, n, 32u * qq + 16u * s + 4u * t, v);
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
            float v[4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) v[i] = __fmul_rn(d, code_float(codes, i, 8388608.0f + 128.0f));
            store_b4(stage, n, 32u * bb + 16u * w + 4u * t, v);
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
// thread of warp 16 requests the copies (packed weights two K units ahead, activation blocks two stages
// ahead) and, once a stage's activations have landed and its weights are written, issues the four
// tensor-core products of the stage; their completion frees the stage.  Every wait is bounded and gives up
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
    if (warp == 0) tmem_alloc(&tmem_slot, kPrefillTile);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    bool ok = true;

    if (warp == kDequantWarps) {
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
                mbar_expect_tx(&a_full[stage], kAStageBytes);
                bulk_load(smem + kOffA + stage * kAStageBytes, blocks + (size_t)step * kPrefillBlockBytes, kAStageBytes, &a_full[stage]);
            };
            for (uint32_t j = 0; j < 2u && j < unit_count; ++j) request_weights(j);
            for (uint32_t step = 0; step < kAhead && step < steps; ++step) request_block(step);
            for (uint32_t step = 0; step < steps && ok; ++step) {
                const uint32_t stage = step % kStages, use = step / kStages, j = step / subs;
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
                if (!wait_or_abort(&a_full[stage], use & 1u, abort) || !wait_or_abort(&b_full[stage], use & 1u, abort)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_address = smem_u32(smem + kOffA + stage * kAStageBytes), b_address = smem_u32(smem + kOffB + stage * kBStageBytes);
#pragma unroll
                for (uint32_t kk = 0; kk < kPrefillBlockK / 16u; ++kk)
                    mma_bf16(tmem, operand_descriptor(a_address + kk * 256u), operand_descriptor(b_address + kk * 256u),
                             (step | kk) != 0u ? 1u : 0u);
                mma_commit(&stage_free[stage]);
            }
            if (ok) mma_commit(done_bar);
            else {
                abort_flag = 1u;
                // Copies already requested get a bounded chance to land before the shared memory is released.
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
        // Warp w reads accumulator lanes 32 * (w % 4) .. +31 (its quarter of the rows) and a quarter of the columns.
        const uint32_t row = (warp & 3u) * 32u + lane, column0 = (warp >> 2) * (kPrefillTile / 4u);
        float* out = mat.out + (size_t)blockIdx.y * kPrefillRows * mat.n + (size_t)row * mat.n + (size_t)tile * kPrefillTile + column0;
        float v[32];
        tmem_load_32(tmem + (((warp & 3u) * 32u) << 16) + column0, v);
#pragma unroll
        for (uint32_t i = 0; i < 32u; i += 4u)
            *reinterpret_cast<float4*>(out + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        tc_fence_before_sync();
    } else if (failed && tid == 0) {
        atomicExch(p.error_flag, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kPrefillTile);
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

// Grid (128 rows, pieces / 256).
__global__ void __launch_bounds__(256) prefill_geglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                            uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x, piece = blockIdx.y * blockDim.x + threadIdx.x;
    if (piece >= k / 8u) return;
    float out[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (row < rows) {
        float g[8], u[8];
        load8(gate + (size_t)row * k + piece * 8u, g);
        load8(up + (size_t)row * k + piece * 8u, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float v = g[i];
            const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
            out[i] = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner))), u[i]);
        }
    }
    store_a8(a_out, row, piece * 8u, out);
}

__global__ void __launch_bounds__(256) prefill_pack_kernel(const float* __restrict__ x, uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x, piece = blockIdx.y * blockDim.x + threadIdx.x;
    if (piece >= k / 8u) return;
    float out[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (row < rows) load8(x + (size_t)row * k + piece * 8u, out);
    store_a8(a_out, row, piece * 8u, out);
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
    // A narrow output leaves most SMs without a tile: cut K so that about one wave of CTAs runs.
    const uint32_t tiles = (uint32_t)(n / kPrefillTile), units = (uint32_t)(k / unit_elements(dtype));
    uint32_t splits = tiles ? (uint32_t)sm_count() / tiles : 1u;
    splits = splits < 1u ? 1u : splits > kPrefillMaxSplits ? kPrefillMaxSplits : splits;
    return splits > units ? units : splits;
}

int launch_prefill_norm(const float* x, uint32_t splits, const float* residual, const float* gamma0, const float* gamma1,
                        float* residual_out, void* a_out, uint32_t rows, uint32_t k, float eps, int mode, cudaStream_t stream) {
    if (!x || splits == 0 || rows == 0 || rows > kPrefillRows || k == 0 || k % 8u || k > kNormPieces * 256u * 8u
        || (mode == 0 && (!gamma1 || !a_out)) || (mode == 1 && (!residual || !gamma0 || !residual_out)))
        return fail(GF_ERR_INVALID, "prefill norm: bad arguments");
    const uint32_t blocks = a_out ? kPrefillRows : rows;
    prefill_norm_kernel<<<blocks, 256, 0, stream>>>(x, splits, residual, gamma0, gamma1, residual_out, static_cast<uint8_t*>(a_out), rows, k, eps, mode);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_geglu(const float* gate, const float* up, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!gate || !up || !a_out || rows == 0 || rows > kPrefillRows || k % 8u) return fail(GF_ERR_INVALID, "prefill GeGLU: bad arguments");
    prefill_geglu_kernel<<<dim3(kPrefillRows, (k / 8u + 255u) / 256u), 256, 0, stream>>>(gate, up, static_cast<uint8_t*>(a_out), rows, k);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_pack(const float* x, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!x || !a_out || rows == 0 || rows > kPrefillRows || k % 8u) return fail(GF_ERR_INVALID, "prefill pack: bad arguments");
    prefill_pack_kernel<<<dim3(kPrefillRows, (k / 8u + 255u) / 256u), 256, 0, stream>>>(x, static_cast<uint8_t*>(a_out), rows, k);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_prefill_workspace_bytes(uint64_t k) { return tile_major_bytes(k); }

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

