// Shared device/host helpers for the sm_100a decode kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/guffin_b200.h"

namespace gf {

// Last error text for gf_last_error(); set by every failing entry point.
void set_error(const char* format, ...);
int fail(int status, const char* format, ...);
int check_cuda(cudaError_t error, const char* what);

#define GF_CUDA(call)                                                        \
    do {                                                                     \
        const int gf_status_ = ::gf::check_cuda((call), #call);              \
        if (gf_status_ != GF_OK) return gf_status_;                          \
    } while (0)

inline cudaStream_t as_stream(void* stream) { return static_cast<cudaStream_t>(stream); }

#ifdef GF_TESTING
// Host-side fault seam of the testing build (never compiled into the shipped library; the reference keeps
// its seams behind LOCAL_GGUF_ENGINE_TESTING the same way, tests/support/target_verifier_test_hooks.cpp).
// A one-shot request that the next prepared launch consumes.  kind 1: a weight-streaming launch overstates
// the byte count its first copy expects by 16 and gives up after `limit` polls -- every copy still lands,
// the wait runs out, nothing faults.  kind 2: one CTA of the next decode pass kernel leaves out one barrier
// arrival and every CTA's poll gives up after `limit` reads.
struct TestingFault { int kind = 0; uint32_t limit = 0; };
TestingFault& testing_fault();
#endif

int sm_count();

// ---- block geometry (GGUF type ids: 8 = Q8_0, 12 = Q4_K, 14 = Q6_K)
__host__ __device__ inline uint32_t block_elements(int dtype) { return dtype == GF_Q8_0 ? 32u : 256u; }
__host__ __device__ inline uint32_t block_bytes(int dtype) {
    return dtype == GF_Q8_0 ? 34u : dtype == GF_Q4_K ? 144u : 210u;
}
// The streaming layout groups 16 output columns (two column tiles of 8) over one K "unit":
// 256 elements for the K-quants, 128 elements (four blocks) for Q8_0.  One group is a "pair row".
__host__ __device__ inline uint32_t unit_elements(int dtype) { return dtype == GF_Q8_0 ? 128u : 256u; }
__host__ __device__ inline uint32_t unit_native_bytes(int dtype) {
    return dtype == GF_Q8_0 ? 136u : dtype == GF_Q4_K ? 144u : 210u;
}
__host__ __device__ inline uint32_t pair_row_bytes(int dtype) { return 16u * unit_native_bytes(dtype); }

// Where byte `native` (offset inside one column's native unit) of column `c16` of a group lives
// inside the group's pair row.  The quantised codes are laid out in tensor-core fragment order:
// lane (g, t) of a warp (g = lane / 4, t = lane % 4) feeds rows g (column g) and g + 8 (column
// g + 8) of a 16 x 16 A operand whose sixteen K positions are sixteen consecutive elements,
// lane t supplying elements 4t .. 4t+3, and it finds every word it needs for one loop body in
// 16 consecutive bytes at lane * 16 of a 512-byte plane:
//   Q4_K (2304 B): plane c (64-element chunk c)      = words {A.w0, A.w1, B.w0, B.w1}, A/B = column g / g+8,
//                  w = which 16 of the chunk's 32 code bytes; then header[16][16] (d, dmin, scales)
//   Q6_K (3360 B): per 128-element half h three planes: column g's ql words {s0 even, s0 odd, s1 even, s1 odd},
//                  the same for column g+8, and qh words {A.s0, A.s1, B.s0, B.s1} (s = which 16 of 32 bytes,
//                  even / odd = ql bytes 0-31 / 32-63 of the half); then scales[16][16], d[16][2]
//   Q8_0 (2176 B): plane b (32-element block b)      = words {A.w0, A.w1, B.w0, B.w1}; then d[16][4][2]
// Only 16-bit words move (all fields are 2-byte aligned in the native blocks), so the mapping is a
// bijection and unpacking restores the native payload byte for byte.
__host__ __device__ inline uint32_t packed_offset(int dtype, uint32_t c16, uint32_t native) {
    const uint32_t g = c16 & 7u, tb = c16 >> 3;
    if (dtype == GF_Q4_K) {
        if (native < 16u) return 2048u + c16 * 16u + native;
        const uint32_t o = native - 16u, word = o >> 2, c = word >> 3, w = (word >> 2) & 1u, t = word & 3u;
        return c * 512u + (g * 4u + t) * 16u + (tb * 2u + w) * 4u + (o & 3u);
    }
    if (dtype == GF_Q6_K) {
        if (native < 128u) {
            const uint32_t word = native >> 2, h = word >> 4, odd = (word >> 3) & 1u, s = (word >> 2) & 1u, t = word & 3u;
            return h * 1536u + tb * 512u + (g * 4u + t) * 16u + (2u * s + odd) * 4u + (native & 3u);
        }
        if (native < 192u) {
            const uint32_t o = native - 128u, word = o >> 2, h = word >> 3, s = (word >> 2) & 1u, t = word & 3u;
            return h * 1536u + 1024u + (g * 4u + t) * 16u + (tb * 2u + s) * 4u + (o & 3u);
        }
        if (native < 208u) return 3072u + c16 * 16u + (native - 192u);
        return 3328u + c16 * 2u + (native - 208u);
    }
    const uint32_t b = native / 34u, o = native % 34u;
    if (o < 2u) return 2048u + c16 * 8u + b * 2u + o;
    const uint32_t q = o - 2u, word = q >> 2, w = word >> 2, t = word & 3u;
    return b * 512u + (g * 4u + t) * 16u + (tb * 2u + w) * 4u + (q & 3u);
}

#ifdef __CUDACC__
// ---- mbarrier / bulk-copy PTX (sm_90+ instructions, compiled for sm_100a)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: gives up after a fixed number of polls so a lost copy can never hang the GPU.
constexpr uint32_t kMbarWaitLimit = 1u << 24;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kMbarWaitLimit) {
    for (uint32_t spin = 0; spin < limit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// One contiguous global -> shared copy through the TMA engine (both addresses 16-byte aligned,
// size a multiple of 16); completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its prologue, and
// wait for everything the previous kernel wrote.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// One 16-byte load that is never served from a stale L1 line: two (value, stamp) pairs of a shard exchange, each
// pair read whole (the pairs are written by 8-byte stores).
__device__ __forceinline__ uint4 load_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}
// Butterfly reduction of eight per-lane column sums: afterwards lane (4*c') with
// c' = bit-reversed column holds the warp total of that column; returns it for lanes
// whose low two bits are zero.  column_of_lane() gives the column such a lane holds.
__device__ __forceinline__ float reduce_columns8(float (&acc)[8], uint32_t lane) {
    float v4[4], v2[2];
    const bool b16 = lane & 16u, b8 = lane & 8u, b4 = lane & 4u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float keep = b16 ? acc[i + 4] : acc[i];
        const float send = b16 ? acc[i] : acc[i + 4];
        v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float keep = b8 ? v4[i + 2] : v4[i];
        const float send = b8 ? v4[i] : v4[i + 2];
        v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float keep = b4 ? v2[1] : v2[0];
    const float send = b4 ? v2[0] : v2[1];
    float v = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}
__device__ __forceinline__ uint32_t column_of_lane(uint32_t lane) {
    return ((lane & 16u) ? 4u : 0u) | ((lane & 8u) ? 2u : 0u) | ((lane & 4u) ? 1u : 0u);
}

#endif

}  // namespace gf
