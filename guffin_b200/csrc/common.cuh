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

int sm_count();

// ---- block geometry (GGUF type ids: 8 = Q8_0, 12 = Q4_K, 14 = Q6_K)
__host__ __device__ inline uint32_t block_elements(int dtype) { return dtype == GF_Q8_0 ? 32u : 256u; }
__host__ __device__ inline uint32_t block_bytes(int dtype) {
    return dtype == GF_Q8_0 ? 34u : dtype == GF_Q4_K ? 144u : 210u;
}
// The streaming layout groups 8 output columns over one K "unit": 256 elements for the
// K-quants, 128 elements (four blocks) for Q8_0.
__host__ __device__ inline uint32_t unit_elements(int dtype) { return dtype == GF_Q8_0 ? 128u : 256u; }
__host__ __device__ inline uint32_t unit_row_bytes(int dtype) {
    return dtype == GF_Q8_0 ? 1088u : dtype == GF_Q4_K ? 1152u : 1680u;
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 24); ++spin)
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
