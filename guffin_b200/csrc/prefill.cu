// Prefill GEMM on tcgen05 / TMEM and the elementwise steps around it (see prefill.cuh).
#include "prefill.cuh"
#include "ops.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace gf {

namespace {

constexpr uint32_t kStages = 4;                                         // shared-memory stages of 64 K elements
constexpr uint32_t kPairs = kPrefillTile / 16u;                         // column pairs (16 columns) per CTA
constexpr uint32_t kMaxPairRow = 3360u;                                 // Q6_K
constexpr uint32_t kWeightBufBytes = kPairs * kMaxPairRow;
constexpr uint32_t kAStageBytes = kPrefillBlockBytes;                   // 128 rows x 64 K bf16
constexpr uint32_t kBStageBytes = kPrefillTile * kPrefillBlockK * 2u;   // 128 columns x 64 K bf16
constexpr uint32_t kOffA = 0u, kOffB = kStages * kAStageBytes, kOffW = kOffB + kStages * kBStageBytes;
constexpr uint32_t kOffBars = kOffW + 2u * kWeightBufBytes;
constexpr uint32_t kBarCount = 2u + 2u * kStages + 1u;                  // weights x2, activations x stages, mma x stages, all done
constexpr uint32_t kPrefillSmemBytes = kOffBars + kBarCount * 8u + 16u;

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

// ---- dequantisation of one lane slot (columns g and g + 8 of one column pair) for one block of 64 K
// elements, with the reference's rounding (quantization.cpp:457,517,590), then bf16.  `row` is the pair row
// (streaming layout, common.cuh), `n0` the pair's first column inside the CTA tile.

__device__ __forceinline__ void dequant_q4k(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t n0, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint4 words = *reinterpret_cast<const uint4*>(row + sub * 512u + lane * 16u);      // {A.w0, A.w1, B.w0, B.w1}
#pragma unroll
    for (uint32_t col = 0; col < 2u; ++col) {
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
                const uint32_t word = col == 0u ? (w == 0u ? words.x : words.y) : (w == 0u ? words.z : words.w);
                float v[4];
#pragma unroll
                for (uint32_t i = 0; i < 4u; ++i) {
                    const uint32_t q = (byte_of(word, i) >> (4u * nib)) & 15u;
                    v[i] = __fsub_rn(__fmul_rn(ds, (float)q), dm);
                }
                store_b4(stage, n0 + g + 8u * col, 32u * nib + 16u * w + 4u * t, v);
            }
        }
    }
}

__device__ __forceinline__ void dequant_q6k(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t n0, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u, half = sub >> 1, upper = sub & 1u;       // quarters 2 * upper, 2 * upper + 1 of the half
    const uint4 ql[2] = {*reinterpret_cast<const uint4*>(row + half * 1536u + lane * 16u),
                         *reinterpret_cast<const uint4*>(row + half * 1536u + 512u + lane * 16u)};
    const uint4 qh = *reinterpret_cast<const uint4*>(row + half * 1536u + 1024u + lane * 16u);      // {A.s0, A.s1, B.s0, B.s1}
#pragma unroll
    for (uint32_t col = 0; col < 2u; ++col) {
        const uint32_t column = g + 8u * col;
        const float d = half_bits(*reinterpret_cast<const unsigned short*>(row + 3328u + column * 2u));
        const uint8_t* scale_bytes = row + 3072u + column * 16u;
#pragma unroll
        for (uint32_t s = 0; s < 2u; ++s) {
            const uint32_t even = s ? ql[col].z : ql[col].x, odd = s ? ql[col].w : ql[col].y;
            const uint32_t high = col == 0u ? (s ? qh.y : qh.x) : (s ? qh.w : qh.z);
#pragma unroll
            for (uint32_t qq = 0; qq < 2u; ++qq) {
                const uint32_t quarter = 2u * upper + qq;
                const uint32_t low_word = qq ? odd : even;
                const float ds = __fmul_rn(d, (float)(int)(signed char)scale_bytes[8u * half + 2u * quarter + s]);
                float v[4];
#pragma unroll
                for (uint32_t i = 0; i < 4u; ++i) {
                    const uint32_t low = (byte_of(low_word, i) >> (4u * upper)) & 15u;
                    const uint32_t top = (byte_of(high, i) >> (2u * quarter)) & 3u;
                    v[i] = __fmul_rn(ds, (float)((int)(low | (top << 4)) - 32));
                }
                store_b4(stage, n0 + column, 32u * qq + 16u * s + 4u * t, v);
            }
        }
    }
}

__device__ __forceinline__ void dequant_q80(const uint8_t* row, uint32_t sub, uint32_t lane, uint32_t n0, uint8_t* stage) {
    const uint32_t g = lane >> 2, t = lane & 3u;
#pragma unroll
    for (uint32_t bb = 0; bb < 2u; ++bb) {
        const uint32_t block = 2u * sub + bb;
        const uint4 words = *reinterpret_cast<const uint4*>(row + block * 512u + lane * 16u);      // {A.w0, A.w1, B.w0, B.w1}
#pragma unroll
        for (uint32_t col = 0; col < 2u; ++col) {
            const uint32_t column = g + 8u * col;
            const float d = half_bits(*reinterpret_cast<const unsigned short*>(row + 2048u + column * 8u + block * 2u));
#pragma unroll
            for (uint32_t w = 0; w < 2u; ++w) {
                const uint32_t word = col == 0u ? (w == 0u ? words.x : words.y) : (w == 0u ? words.z : words.w);
                float v[4];
#pragma unroll
                for (uint32_t i = 0; i < 4u; ++i) v[i] = __fmul_rn(d, (float)(int)(signed char)byte_of(word, i));
                store_b4(stage, n0 + column, 32u * bb + 16u * w + 4u * t, v);
            }
        }
    }
}

// C[128, 128-column tile] = A[128, K] x deq(W)^T.  Grid: one CTA per tile over all matrices of the launch.
// Thread 0 requests the copies (weights a K unit ahead, one activation block per stage) and issues the
// tensor-core operations; all 256 threads dequantise: warp w owns column pair w of the tile, a lane one
// lane slot of its pair rows.  Every wait is bounded; a wait that gives up sets the error word, and the
// CTA still releases its tensor memory before it returns.
__global__ void __launch_bounds__(kPrefillThreads, 1) prefill_gemm_kernel(const __grid_constant__ PrefillGemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t tmem_slot;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint64_t* weight_bar = bars;                       // [2]
    uint64_t* a_bar = bars + 2;                        // [kStages]
    uint64_t* mma_bar = bars + 2 + kStages;            // [kStages]
    uint64_t* done_bar = bars + 2 + 2 * kStages;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    uint32_t which = 0;
    if (p.matrices > 1u && blockIdx.x >= p.m[1].first_tile) which = 1;
    if (p.matrices > 2u && blockIdx.x >= p.m[2].first_tile) which = 2;
    const PrefillMatrix& mat = p.m[which];
    const uint32_t tile = blockIdx.x - mat.first_tile, dtype = mat.dtype;
    const uint32_t row_bytes = pair_row_bytes((int)dtype), subs = p.unit_elems / kPrefillBlockK;
    const uint8_t* weights = mat.weight + (size_t)tile * kPairs * p.units * row_bytes;      // pair rows of pair i start i * units * row_bytes further

    if (tid == 0) {
        for (uint32_t i = 0; i < kBarCount; ++i) mbar_init(&bars[i], 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kPrefillTile);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;

    auto request_weights = [&](uint32_t unit) {       // thread 0
        uint64_t* bar = &weight_bar[unit & 1u];
        uint8_t* dst = smem + kOffW + (unit & 1u) * kWeightBufBytes;
        mbar_expect_tx(bar, kPairs * row_bytes);
        for (uint32_t i = 0; i < kPairs; ++i)
            bulk_load(dst + i * row_bytes, weights + ((size_t)i * p.units + unit) * row_bytes, row_bytes, bar);
    };
    if (tid == 0) request_weights(0);

    // A wait that gives up is agreed on by the whole CTA at the next block barrier, so that every thread
    // leaves the loops at the same place.
    bool failed = false;
    uint32_t step = 0;                                 // stages used so far
    for (uint32_t unit = 0; unit < p.units && !failed; ++unit) {
        bool bad = !mbar_wait(&weight_bar[unit & 1u], (unit >> 1) & 1u);
        // The other weight buffer was last read while unit - 1 was dequantised, which ended with a block barrier.
        if (tid == 0 && !bad && unit + 1u < p.units) request_weights(unit + 1u);
        const uint8_t* pair_row = smem + kOffW + (unit & 1u) * kWeightBufBytes + warp * row_bytes;
        for (uint32_t sub = 0; sub < subs; ++sub, ++step) {
            const uint32_t stage = step % kStages, use = step / kStages;
            // The stage's previous tensor-core reads must be over before it is overwritten.
            if (!bad && use > 0u && !mbar_wait(&mma_bar[stage], (use - 1u) & 1u)) bad = true;
            uint8_t* a_stage = smem + kOffA + stage * kAStageBytes;
            uint8_t* b_stage = smem + kOffB + stage * kBStageBytes;
            if (!bad) {
                if (tid == 0) {
                    mbar_expect_tx(&a_bar[stage], kAStageBytes);
                    bulk_load(a_stage, p.a + (size_t)(unit * subs + sub) * kPrefillBlockBytes, kAStageBytes, &a_bar[stage]);
                }
                if (dtype == GF_Q4_K) dequant_q4k(pair_row, sub, lane, warp * 16u, b_stage);
                else if (dtype == GF_Q6_K) dequant_q6k(pair_row, sub, lane, warp * 16u, b_stage);
                else dequant_q80(pair_row, sub, lane, warp * 16u, b_stage);
                fence_async_smem();
                if (tid == 0 && !mbar_wait(&a_bar[stage], use & 1u)) bad = true;
            }
            failed = __syncthreads_or(bad ? 1 : 0) != 0;
            if (failed) break;
            if (tid == 0) {
                tc_fence_after_sync();
                const uint32_t a_address = smem_u32(a_stage), b_address = smem_u32(b_stage);
#pragma unroll
                for (uint32_t kk = 0; kk < kPrefillBlockK / 16u; ++kk)
                    mma_bf16(tmem, operand_descriptor(a_address + kk * 256u), operand_descriptor(b_address + kk * 256u),
                             (step | kk) != 0u ? 1u : 0u);
                mma_commit(&mma_bar[stage]);
            }
        }
    }
    if (!failed) {
        if (tid == 0) mma_commit(done_bar);
        if (!mbar_wait(done_bar, 0u)) failed = true;
    }
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    if (!failed) {
        tc_fence_after_sync();
        // Warp w reads accumulator lanes 32 * (w % 4) .. +31 (its quarter of the rows) and half of the columns.
        const uint32_t row = (warp & 3u) * 32u + lane, column0 = (warp >> 2) * (kPrefillTile / 2u);
        float* out = mat.out + (size_t)row * mat.n + (size_t)tile * kPrefillTile + column0;
#pragma unroll
        for (uint32_t c = 0; c < kPrefillTile / 2u; c += 32u) {
            float v[32];
            tmem_load_32(tmem + (((warp & 3u) * 32u) << 16) + column0 + c, v);
#pragma unroll
            for (uint32_t i = 0; i < 32u; i += 4u)
                *reinterpret_cast<float4*>(out + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        tc_fence_before_sync();
    } else if (tid == 0) {
        atomicExch(p.error_flag, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kPrefillTile);
}

// ---- elementwise steps: one block per row, 256 threads ----

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

__device__ __forceinline__ void store_a(uint8_t* a, uint32_t row, uint32_t k, float value) {
    *reinterpret_cast<__nv_bfloat16*>(a + tile_major_offset(row, k)) = __float2bfloat16_rn(value);
}

// Rows beyond `rows` (up to 128) are written as zeros so that the GEMM's unused rows are defined.
__global__ void __launch_bounds__(256) prefill_norm_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                                                           const float* __restrict__ gamma0, const float* __restrict__ gamma1,
                                                           float* __restrict__ residual_out, uint8_t* __restrict__ a_out,
                                                           uint32_t rows, uint32_t k, float eps, int mode) {
    __shared__ float scratch[8];
    const uint32_t row = blockIdx.x;
    if (row >= rows) {
        if (a_out) for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) store_a(a_out, row, i, 0.0f);
        return;
    }
    const float* in = x + (size_t)row * k;
    float sum = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) sum = fmaf(in[i], in[i], sum);
    float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(block_total(sum, scratch), (float)k), eps)));
    if (mode == 0) {
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) store_a(a_out, row, i, __fmul_rn(__fmul_rn(in[i], inv), gamma1[i]));
        return;
    }
    float sum2 = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        const float r = __fadd_rn(residual[(size_t)row * k + i], __fmul_rn(__fmul_rn(in[i], inv), gamma0[i]));
        residual_out[(size_t)row * k + i] = r;
        sum2 = fmaf(r, r, sum2);
    }
    if (!gamma1 || !a_out) return;
    inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(block_total(sum2, scratch), (float)k), eps)));
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x)
        store_a(a_out, row, i, __fmul_rn(__fmul_rn(residual_out[(size_t)row * k + i], inv), gamma1[i]));
}

__global__ void __launch_bounds__(256) prefill_geglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                            uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        float value = 0.0f;
        if (row < rows) {
            const float v = gate[(size_t)row * k + i];
            const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
            value = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner))), up[(size_t)row * k + i]);
        }
        store_a(a_out, row, i, value);
    }
}

__global__ void __launch_bounds__(256) prefill_pack_kernel(const float* __restrict__ x, uint8_t* __restrict__ a_out, uint32_t rows, uint32_t k) {
    const uint32_t row = blockIdx.x;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) store_a(a_out, row, i, row < rows ? x[(size_t)row * k + i] : 0.0f);
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
    prefill_gemm_kernel<<<tiles, kPrefillThreads, kPrefillSmemBytes, stream>>>(p);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_norm(const float* x, const float* residual, const float* gamma0, const float* gamma1, float* residual_out,
                        void* a_out, uint32_t rows, uint32_t k, float eps, int mode, cudaStream_t stream) {
    if (!x || rows == 0 || rows > kPrefillRows || k == 0 || (mode == 0 && (!gamma1 || !a_out))
        || (mode == 1 && (!residual || !gamma0 || !residual_out)))
        return fail(GF_ERR_INVALID, "prefill norm: bad arguments");
    const uint32_t blocks = a_out ? kPrefillRows : rows;
    prefill_norm_kernel<<<blocks, 256, 0, stream>>>(x, residual, gamma0, gamma1, residual_out, static_cast<uint8_t*>(a_out), rows, k, eps, mode);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_geglu(const float* gate, const float* up, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!gate || !up || !a_out || rows == 0 || rows > kPrefillRows) return fail(GF_ERR_INVALID, "prefill GeGLU: bad arguments");
    prefill_geglu_kernel<<<kPrefillRows, 256, 0, stream>>>(gate, up, static_cast<uint8_t*>(a_out), rows, k);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int launch_prefill_pack(const float* x, void* a_out, uint32_t rows, uint32_t k, cudaStream_t stream) {
    if (!x || !a_out || rows == 0 || rows > kPrefillRows) return fail(GF_ERR_INVALID, "prefill pack: bad arguments");
    prefill_pack_kernel<<<kPrefillRows, 256, 0, stream>>>(x, static_cast<uint8_t*>(a_out), rows, k);
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

