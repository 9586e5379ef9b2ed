// Device, memory and stream entry points of the C ABI, and the shared error text.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace gf {

static thread_local char g_error[512] = "";

void set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
}

int fail(int status, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
    return status;
}

int check_cuda(cudaError_t error, const char* what) {
    if (error == cudaSuccess) return GF_OK;
    set_error("CUDA error %d (%s) in %s", static_cast<int>(error), cudaGetErrorString(error), what);
    return GF_ERR_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            count = 148;
        cached[device] = count;
    }
    return cached[device];
}

}  // namespace gf

using namespace gf;

extern "C" {

const char* gf_last_error(void) { return g_error; }
const char* gf_version(void) { return "guffin_b200 0.1 (sm_100a)"; }

int gf_device_count(int* count) {
    if (!count) return fail(GF_ERR_INVALID, "gf_device_count: null output");
    *count = 0;
    const cudaError_t error = cudaGetDeviceCount(count);
    if (error != cudaSuccess) {
        *count = 0;
        return fail(GF_ERR_UNAVAILABLE, "no CUDA device: %s", cudaGetErrorString(error));
    }
    return GF_OK;
}

int gf_set_device(int device) { GF_CUDA(cudaSetDevice(device)); return GF_OK; }

int gf_memory_info(size_t* free_bytes, size_t* total_bytes) {
    if (!free_bytes || !total_bytes) return fail(GF_ERR_INVALID, "gf_memory_info: null output");
    GF_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
    return GF_OK;
}

int gf_malloc(void** out_dev, size_t bytes) {
    if (!out_dev) return fail(GF_ERR_INVALID, "gf_malloc: null output");
    *out_dev = nullptr;
    GF_CUDA(cudaMalloc(out_dev, bytes == 0 ? 16 : bytes));
    return GF_OK;
}

int gf_free(void* ptr_dev) { GF_CUDA(cudaFree(ptr_dev)); return GF_OK; }

int gf_host_alloc(void** out_host, size_t bytes) {
    if (!out_host) return fail(GF_ERR_INVALID, "gf_host_alloc: null output");
    *out_host = nullptr;
    GF_CUDA(cudaHostAlloc(out_host, bytes == 0 ? 16 : bytes, cudaHostAllocDefault));
    return GF_OK;
}

int gf_host_free(void* ptr_host) { GF_CUDA(cudaFreeHost(ptr_host)); return GF_OK; }

int gf_memset(void* dst_dev, int value, size_t bytes, void* stream) {
    GF_CUDA(cudaMemsetAsync(dst_dev, value, bytes, as_stream(stream)));
    return GF_OK;
}

int gf_upload(void* dst_dev, const void* src_host, size_t bytes, void* stream) {
    GF_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return GF_OK;
}

int gf_download(void* dst_host, const void* src_dev, size_t bytes, void* stream) {
    GF_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return GF_OK;
}

int gf_copy(void* dst_dev, const void* src_dev, size_t bytes, void* stream) {
    GF_CUDA(cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return GF_OK;
}

int gf_stream_create(void** out_stream) {
    if (!out_stream) return fail(GF_ERR_INVALID, "gf_stream_create: null output");
    cudaStream_t stream = nullptr;
    GF_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    *out_stream = stream;
    return GF_OK;
}

int gf_stream_destroy(void* stream) { GF_CUDA(cudaStreamDestroy(as_stream(stream))); return GF_OK; }

int gf_stream_synchronize(void* stream) { GF_CUDA(cudaStreamSynchronize(as_stream(stream))); return GF_OK; }

int gf_event_create(void** out_event) {
    if (!out_event) return fail(GF_ERR_INVALID, "gf_event_create: null output");
    cudaEvent_t event = nullptr;
    GF_CUDA(cudaEventCreate(&event));
    *out_event = event;
    return GF_OK;
}

int gf_event_destroy(void* event) { GF_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event))); return GF_OK; }

int gf_event_record(void* event, void* stream) {
    GF_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)));
    return GF_OK;
}

int gf_event_synchronize(void* event) { GF_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event))); return GF_OK; }

int gf_event_elapsed_ms(void* start, void* end, float* out_ms) {
    if (!out_ms) return fail(GF_ERR_INVALID, "gf_event_elapsed_ms: null output");
    GF_CUDA(cudaEventElapsedTime(out_ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
    return GF_OK;
}

}  // extern "C"

#ifdef GF_TESTING
namespace gf {
TestingFault& testing_fault() {
    static TestingFault fault;
    return fault;
}
}  // namespace gf

// Testing build only (absent from include/guffin_b200.h): arms the one-shot fault described in common.cuh.
extern "C" GF_API int gf_testing_arm_fault(int kind, uint32_t limit) {
    if (kind < 0 || kind > 2 || (kind != 0 && limit == 0)) return gf::fail(GF_ERR_INVALID, "gf_testing_arm_fault: bad request");
    gf::testing_fault().kind = kind;
    gf::testing_fault().limit = limit;
    return GF_OK;
}
#endif
