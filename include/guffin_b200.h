/*
 * guffin_b200 -- C ABI of the B200 (sm_100a) backend for the Gemma decode hot path.
 *
 * This is the boundary a host engine binds instead of the reference's Metal command encoder
 * (src/tensor/backends/metal/metal_command_context.hpp:54-369) and its Metal drafter
 * (include/local_gguf_engine/engine/gemma3_draft.hpp:30-105).  Plain pointers and sizes only.
 *
 * Conventions
 *  - Every function returns GF_OK (0) or a negative status; gf_last_error() gives the text.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Kernels never
 *    allocate; callers own every buffer.  Pointers named *_dev are device pointers.
 *  - A context (stream + its buffers) is used from one thread at a time
 *    (target_verifier.hpp:363-365 states the same contract).
 *  - Weight matrices are logically [K, N]: output column n owns K/block consecutive GGUF
 *    blocks (src/tensor/backends/cpu_backend.cpp:49-53).
 */
#ifndef GUFFIN_B200_H
#define GUFFIN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GF_API __attribute__((visibility("default")))

enum {
    GF_OK = 0,
    GF_ERR_INVALID = -1,      /* std::invalid_argument in the reference (shape / extent) */
    GF_ERR_STATE = -2,        /* std::logic_error (state machine) */
    GF_ERR_CUDA = -3,         /* BackendError{metal_execution_failed} */
    GF_ERR_UNAVAILABLE = -4,  /* BackendError{unavailable_metal_device} */
    GF_ERR_NUMERIC = -5,      /* std::overflow_error: non-finite F16 K/V, poisoned plan */
    GF_ERR_TIMEOUT = -6       /* a bounded device-side wait gave up */
};

/* GGUF tensor type ids (include/local_gguf_engine/tensor/dtype.hpp:9-15). */
enum { GF_F32 = 0, GF_F16 = 1, GF_Q8_0 = 8, GF_Q4_K = 12, GF_Q6_K = 14 };

GF_API const char* gf_last_error(void);
GF_API const char* gf_version(void);

/* ---- device, memory, streams: replaces metal_backend.hpp:17-51 / metal_buffer.hpp:48-84 ---- */
GF_API int gf_device_count(int* count);             /* tensor_backend_is_available (tensor/backend.hpp:10) */
GF_API int gf_set_device(int device);
GF_API int gf_memory_info(size_t* free_bytes, size_t* total_bytes);   /* metal_backend.hpp memory_info */
GF_API int gf_malloc(void** out_dev, size_t bytes);                   /* allocate_backend_buffer */
GF_API int gf_free(void* ptr_dev);
GF_API int gf_host_alloc(void** out_host, size_t bytes);              /* pinned staging */
GF_API int gf_host_free(void* ptr_host);
GF_API int gf_memset(void* dst_dev, int value, size_t bytes, void* stream);
GF_API int gf_upload(void* dst_dev, const void* src_host, size_t bytes, void* stream);    /* copy_tensor_to_backend */
GF_API int gf_download(void* dst_host, const void* src_dev, size_t bytes, void* stream);  /* copy_tensor_from_backend */
GF_API int gf_copy(void* dst_dev, const void* src_dev, size_t bytes, void* stream);
GF_API int gf_stream_create(void** out_stream);
GF_API int gf_stream_destroy(void* stream);
GF_API int gf_stream_synchronize(void* stream);     /* MetalCommandContext::wait_until_completed */

/* ---- weight preparation: replaces repack_kquant_weight_columns8 / restore_native_kquant_weight
 * (src/tensor/kquant_packing.cpp:154,250).  The streaming layout keeps every bit of the native
 * blocks: 8 output columns x one K unit (256 elements; 128 for Q8_0) per contiguous 16-byte
 * aligned group, missing columns zero-filled.  K must be a multiple of the unit. ---- */
GF_API size_t gf_packed_weight_bytes(int dtype, uint64_t k, uint64_t n);
GF_API int gf_pack_weight(int dtype, const void* native_dev, uint64_t k, uint64_t n,
                          void* packed_dev, void* stream);
GF_API int gf_unpack_weight(int dtype, const void* packed_dev, uint64_t k, uint64_t n,
                            void* native_dev, void* stream);

/* ---- dequantisation: Q8_0/Q4_K/Q6_K BlockView::dequantized_value
 * (src/tensor/quantization.cpp:457,517,590), bit-exact, native block order. ---- */
GF_API int gf_dequantize(int dtype, const void* native_dev, uint64_t block_count, float* out_dev,
                         void* stream);

/* ---- quantised GEMV / small-M GEMM: MetalCommandContext::encode_verifier_matmul
 * (metal_command_context.hpp:94-101; kernels metal_kernels.mm:551-986) and the CPU reference
 * matmul_f32_quantized_gguf_weight (cpu_backend.cpp:301-323).
 * y[m, n] = sum_k x[m, k] * deq(W)[n, k], rows m <= GF_MAX_ROWS, f32 accumulate.  Each row's
 * result is identical whether computed alone or beside other rows.
 * `workspace_dev` holds split-K partial sums (gf_matmul_workspace_bytes); it may be NULL when
 * that size is 0. ---- */
#define GF_MAX_ROWS 4
GF_API size_t gf_matmul_workspace_bytes(int dtype, uint32_t rows, uint64_t k, uint64_t n);
GF_API int gf_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev,
                     uint32_t rows, uint64_t k, uint64_t n, void* workspace_dev, void* stream);
/* Reads and clears the device error word the streaming kernels set when a bounded wait gives
 * up (GF_ERR_TIMEOUT); synchronises `stream`.  The analogue of reading the command buffer's
 * status after wait_until_completed (metal_command_context.mm:2316-2344). */
GF_API int gf_matmul_check(void* stream);
/* Same product from HOST buffers through an internal context: uploads x, runs, downloads y.
 * `packed_dev` stays device-resident (weights are uploaded once at load time). */
GF_API int gf_matmul_host(int dtype, const void* packed_dev, const float* x_host, float* y_host,
                          uint32_t rows, uint64_t k, uint64_t n);

#ifdef __cplusplus
}
#endif
#endif
