// Decode pass kernel (see pass.cuh).
#include "pass.cuh"
#include "attention.cuh"
#include "embedding.cuh"

#include <algorithm>
#include <cstddef>
#include <mutex>

namespace gf {

static_assert(offsetof(PassPhase, stream) == 16, "phase_stream_params() expects the streaming parameters at byte 16");

// ---- grid-wide barrier: one counter that only ever grows.  A launch is told the value the counter has
// when it starts (`base`: every earlier launch's arrivals, which the host can count because every CTA
// arrives exactly once per barrier); barrier b of the launch, between its phases b and b + 1, is passed
// once the counter has reached base + (b + 1) * gridDim.x.  Comparisons are modulo 2^32.  Thread 0
// polls; the block barrier hands the outcome to the other threads (the scheme of a cooperative grid
// sync, with a limit on the polls).
__device__ __forceinline__ uint32_t load_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool grid_wait(const uint32_t* arrived, uint32_t target, const int* error_flag, uint32_t poll_limit,
                                          uint32_t* outcome) {
    if (threadIdx.x == 0) {
        uint32_t ok = 0;
        for (uint32_t spin = 0; spin < poll_limit; ++spin) {
            if ((int32_t)(load_acquire(arrived) - target) >= 0) { ok = 1; break; }
            if ((spin & 31u) == 31u && *reinterpret_cast<const volatile int*>(error_flag) != 0) break;   // another CTA gave up
        }
        *outcome = ok;
    }
    __syncthreads();
    return *outcome != 0;
}

// Arrival of a CTA whose threads have all passed a block barrier: the release orders every write of
// the CTA's phase before the count; nothing is waited for.
__device__ __forceinline__ void grid_arrive(uint32_t* arrived) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(arrived) : "memory");
}

// The 16 warps of the CTA as one attention block (two warps per tile of cached rows).
template <typename Dependency>
struct PassBlock {
    Dependency& wait;
    __device__ __forceinline__ uint32_t tid() const { return threadIdx.x; }
    __device__ __forceinline__ uint32_t threads() const { return blockDim.x; }
    __device__ __forceinline__ void sync() const { __syncthreads(); }
    __device__ __forceinline__ bool dependency() const { return wait(); }
};

// The phase bodies are separate functions (not inlined): each gets the whole register budget of a
// 512-thread CTA to itself, and what the phase loop keeps across a call is a handful of words.
template <int G, int R, typename Dependency>
__device__ __noinline__ bool attention_phase_instance(const AttentionParams& p, uint8_t* staging, Dependency& dependency) {
    auto& sm = *reinterpret_cast<AttentionMmaSmem<kAttentionMmaWarps, G * R>*>(staging);
    const uint32_t groups = (p.rows + R - 1u) / R;
    const uint32_t kvh = blockIdx.x % p.kv_heads, rest = blockIdx.x / p.kv_heads;
    const uint32_t part = rest % p.target_parts, group = rest / p.target_parts;
    bool waited = false, ok = true;
    if (group < groups) {
        const PassBlock<Dependency> block{dependency};
        ok = attention_mma_body<G, R, 2, false, false>(p, kvh, part, group, sm, block, waited);
    }
    if (!waited) ok = dependency();
    return ok;
}

template <int ROWS, typename Dependency>
__device__ __forceinline__ bool attention_phase(const PassPhase& phase, uint8_t* staging, Dependency& dependency) {
    const AttentionParams& p = phase.attention;
    const uint32_t group = phase.attention_group;
    if (ROWS == 1) {
        if (group == 1u) return attention_phase_instance<1, 1>(p, staging, dependency);
        if (group == 2u) return attention_phase_instance<2, 1>(p, staging, dependency);
        return attention_phase_instance<4, 1>(p, staging, dependency);
    }
    if (group == 1u) return attention_phase_instance<1, 2>(p, staging, dependency);
    if (group == 2u) return attention_phase_instance<2, 2>(p, staging, dependency);
    return attention_phase_instance<4, 1>(p, staging, dependency);
}

template <int ROWS, typename Dependency>
__device__ __noinline__ bool stream_phase_call(const WeightStreamParams& p, const StreamSmem& sm, WeightRing& ring, float* scratch,
                                               uint32_t* bad_rows, Dependency& dependency) {
    return stream_phase<ROWS, true>(p, sm, ring, scratch, bad_rows, dependency);
}

// 16-byte asynchronous global -> shared copy (the next phase's table entry travels while this phase runs).
__device__ __forceinline__ void copy_async_16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

constexpr uint32_t kPhaseChunks = (uint32_t)(sizeof(PassPhase) / 16u);
static_assert(sizeof(PassPhase) % 16u == 0, "table entries are copied 16 bytes at a time");

template <int ROWS>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) decode_pass_kernel(const PassPhase* __restrict__ table, uint32_t count,
                                                                         uint32_t first_stream, uint32_t last_stream,
                                                                         uint32_t* arrived, uint32_t base, int* error_flag,
                                                                         uint32_t poll_limit, uint32_t skip_arrival) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * kGemvWarps * ROWS];
    __shared__ uint32_t bad_rows, wait_outcome;
    // The running phase's parameters are read from shared memory (two entries: the current one and the
    // next one on its way); only the ring's cursor, which runs ahead, reads the table itself.
    __shared__ __align__(16) uint8_t entries[2][sizeof(PassPhase)];
    if (threadIdx.x < kPhaseChunks) copy_async_16(entries[0] + threadIdx.x * 16u, reinterpret_cast<const uint8_t*>(table) + threadIdx.x * 16u);
    copy_async_wait();
    const StreamSmem sm = stream_smem(smem, kPassSlotBytes);
    if (threadIdx.x == 0) bad_rows = 0u;
    // The ring's cursor starts at the first streaming phase of the launch and ends with the last one.
    const bool streams = first_stream < count;
    WeightRing ring = ring_open<true>(sm, kPassSlotBytes, streams ? &table[first_stream].stream : nullptr,
                                      streams ? &table[last_stream].stream : nullptr, (uint32_t)sizeof(PassPhase));   // ends with a block barrier

    bool ok = true;
    for (uint32_t ph = 0; ph < count; ++ph) {
        const PassPhase& phase = *reinterpret_cast<const PassPhase*>(entries[ph & 1u]);
        if (ph + 1u < count && threadIdx.x < kPhaseChunks)
            copy_async_16(entries[(ph + 1u) & 1u] + threadIdx.x * 16u, reinterpret_cast<const uint8_t*>(&table[ph + 1u]) + threadIdx.x * 16u);
        // What phase ph reads was written before barrier ph - 1; the launch's first phase follows stream order.
        auto dependency = [&]() -> bool {
            if (ph == 0u) return true;
            return grid_wait(arrived, base + ph * gridDim.x, error_flag, poll_limit, &wait_outcome);
        };
        if (phase.kind == kPhaseStream) {
            ok = stream_phase_call<ROWS>(phase.stream, sm, ring, scratch, &bad_rows, dependency);
        } else if (phase.kind == kPhaseAttention) {
            ok = attention_phase<ROWS>(phase, sm.staging, dependency);
        } else {
            ok = dependency();
            if (ok) {
                const EmbeddingPhase& e = phase.embedding;
                embedding_rows(e.dtype, e.packed, e.k, e.vocab, e.tokens, e.rows, e.scale, e.out, e.status,
                               blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
            }
        }
        copy_async_wait();            // this thread's piece of the next entry has landed; the barrier below publishes it
        // The CTA agrees on the outcome, then arrives (the last phase needs no barrier behind it).
        ok = __syncthreads_or(ok ? 0 : 1) == 0;
        if (!ok) break;
        if (threadIdx.x == 0) bad_rows = 0u;          // for the next streaming phase; ordered by its dependency barrier
        if (threadIdx.x == 0 && ph + 1u < count && !(blockIdx.x == 0u && ph == skip_arrival)) grid_arrive(arrived);
    }
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);          // first, so that the other CTAs stop polling at once
        if ((threadIdx.x & 31u) == 0u) ring_drain(ring);
    }
}

// ------------------------------------------------------------------------------------------ host

static uint32_t attention_smem_bytes(uint32_t queries) {
    switch (queries) {
        case 1: return (uint32_t)sizeof(AttentionMmaSmem<kAttentionMmaWarps, 1>);
        case 2: return (uint32_t)sizeof(AttentionMmaSmem<kAttentionMmaWarps, 2>);
        default: return (uint32_t)sizeof(AttentionMmaSmem<kAttentionMmaWarps, 4>);
    }
}

bool pass_attention_supported(const AttentionParams& p, uint32_t rows, uint32_t& group, uint32_t& rows_per_block, uint32_t& target_parts) {
    if (!p.kv_f16 || p.head_dim != 256u || p.kv_heads == 0 || p.heads % p.kv_heads || rows == 0 || rows > kPassMaxRows) return false;
    group = p.heads / p.kv_heads;
    if (group != 1u && group != 2u && group != 4u) return false;
    rows_per_block = group == 4u ? 1u : rows;            // at most four query vectors per block
    const uint32_t groups = (rows + rows_per_block - 1u) / rows_per_block;
    const uint32_t per_pair = (uint32_t)sm_count() / (p.kv_heads * groups);        // about one virtual block per CTA
    if (per_pair == 0) return false;
    target_parts = std::min<uint32_t>(per_pair, (uint32_t)kMaxAttentionPartitions);
    return true;
}

uint32_t pass_smem_bytes(const PassPhase* table, uint32_t count, uint32_t rows) {
    uint32_t staging = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const PassPhase& phase = table[i];
        if (phase.kind == kPhaseStream) {
            const WeightStreamParams& p = phase.stream;
            staging = std::max(staging, gemv_smem_layout(rows, p.staged_units, p.unit_elems, kPassSlotBytes, p.intra > 1u).staging_bytes);
        } else if (phase.kind == kPhaseAttention) {
            staging = std::max(staging, attention_smem_bytes(phase.attention_group * phase.attention_rows));
        }
    }
    const uint32_t total = gemv_ring_bytes(kPassSlotBytes) + staging + 64u;
    return total <= kGemvSmemLimit ? total : 0u;
}

template <int ROWS>
static int launch_pass_instance(const PassLaunch& launch, cudaStream_t stream) {
    static std::once_flag once[64];
    int device = 0;
    cudaGetDevice(&device);
    cudaError_t attr_error = cudaSuccess;
    std::call_once(once[device & 63], [&] {
        attr_error = cudaFuncSetAttribute(decode_pass_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvSmemLimit);
    });
    GF_CUDA(attr_error);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)sm_count());       // one CTA per SM: its blocks wait on one another, so all must be resident
    config.blockDim = dim3(kGemvWarps * 32);
    config.dynamicSmemBytes = launch.smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeCooperative;      // the launch fails instead of starting if the grid cannot be co-resident
    attribute.val.cooperative = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    GF_CUDA(cudaLaunchKernelEx(&config, decode_pass_kernel<ROWS>, launch.table_dev + launch.first, launch.count,
                               launch.first_stream, launch.last_stream, launch.arrived_dev, launch.base, launch.error_flag,
                               launch.poll_limit, launch.skip_arrival));
    return GF_OK;
}

// Two pass kernels must never be resident together: each wants every SM, and two half-resident grids
// would wait on each other's missing CTAs until their polls run out.  Launches on one stream are
// ordered anyway; a launch on another stream of the same device first waits for the previous pass
// kernel (an event recorded behind every launch).
struct PassOrder { std::mutex guard; cudaEvent_t last = nullptr; bool any = false; };
static PassOrder g_pass_order[64];

int launch_pass(const PassLaunch& launch, cudaStream_t stream) {
    if (!launch.table_dev || launch.count == 0 || !launch.arrived_dev || !launch.error_flag || launch.smem_bytes == 0)
        return fail(GF_ERR_INVALID, "decode pass: incomplete launch description");
    if (launch.rows != 1 && launch.rows != 2)
        return fail(GF_ERR_INVALID, "decode pass: rows=%u has no kernel instance (1 or 2)", launch.rows);
    int device = 0;
    GF_CUDA(cudaGetDevice(&device));
    PassOrder& order = g_pass_order[device & 63];
    std::lock_guard<std::mutex> lock(order.guard);
    if (!order.last) GF_CUDA(cudaEventCreateWithFlags(&order.last, cudaEventDisableTiming));
    if (order.any) GF_CUDA(cudaStreamWaitEvent(stream, order.last, 0));       // a no-op behind a launch on the same stream
#ifdef GF_TESTING
    PassLaunch armed = launch;
    if (testing_fault().kind == 2) {
        armed.poll_limit = testing_fault().limit;
        armed.skip_arrival = 1;
        testing_fault().kind = 0;
    }
    const int status = armed.rows == 1 ? launch_pass_instance<1>(armed, stream) : launch_pass_instance<2>(armed, stream);
#else
    const int status = launch.rows == 1 ? launch_pass_instance<1>(launch, stream) : launch_pass_instance<2>(launch, stream);
#endif
    if (status != GF_OK) return status;
    GF_CUDA(cudaEventRecord(order.last, stream));
    order.any = true;
    return GF_OK;
}

}  // namespace gf
