// Host side of the streaming dequant-GEMV: decomposition plan, launch, C entry points.
#include "gemv.cuh"

#include <mutex>

namespace gf {

constexpr uint32_t kMaxDynamicSmem = 227u * 1024u;

int gemv_plan(int dtype, uint32_t rows, uint64_t k, uint64_t n, GemvPlan& plan) {
    if (dtype != GF_Q8_0 && dtype != GF_Q4_K && dtype != GF_Q6_K)
        return fail(GF_ERR_INVALID, "gf_matmul: unsupported weight dtype %d", dtype);
    if (rows == 0 || rows > GF_MAX_ROWS) return fail(GF_ERR_INVALID, "gf_matmul: rows=%u outside [1, %d]", rows, GF_MAX_ROWS);
    const uint32_t unit = unit_elements(dtype);
    if (k == 0 || n == 0 || k % unit != 0 || k > (1ull << 24) || n > (1ull << 28))
        return fail(GF_ERR_INVALID, "gf_matmul: K=%llu must be a positive multiple of %u and N=%llu positive",
                    (unsigned long long)k, unit, (unsigned long long)n);
    plan.units = (uint32_t)(k / unit);
    plan.tiles = (uint32_t)((n + 7u) / 8u);
    const uint32_t sms = (uint32_t)sm_count();
    double best = -1.0;
    plan.chunks = 0;
    for (uint32_t chunks = 1; chunks <= 64 && chunks <= plan.units && chunks <= sms; ++chunks) {
        const uint32_t chunk_units = (plan.units + chunks - 1u) / chunks;
        if ((chunks - 1u) * chunk_units >= plan.units) continue;          // an empty last chunk
        if (chunk_units > (uint32_t)kGemvMaxChunkUnits) continue;
        if (gemv_smem_layout(dtype, (int)rows, chunk_units).total > kMaxDynamicSmem) continue;
        const uint32_t group_ctas = sms / chunks;
        const uint32_t group_warps = group_ctas * kGemvWarps;
        const uint32_t rounds = (plan.tiles + group_warps - 1u) / group_warps;
        // Share of the machine's warp-slots doing useful work; ties go to fewer chunks.
        double efficiency = (double)plan.tiles / ((double)rounds * group_warps) * (double)(group_ctas * chunks) / sms;
        efficiency -= 0.002 * chunks;
        if (efficiency > best) {
            best = efficiency;
            plan.chunks = chunks;
            plan.chunk_units = chunk_units;
            plan.grid = group_ctas * chunks;
        }
    }
    if (plan.chunks == 0) return fail(GF_ERR_INVALID, "gf_matmul: no decomposition fits K=%llu rows=%u", (unsigned long long)k, rows);
    plan.smem = gemv_smem_layout(dtype, (int)rows, plan.chunk_units).total;
    return GF_OK;
}

template <int DTYPE, int ROWS>
static int launch_instance(const GemvParams& p, const GemvPlan& plan, cudaStream_t stream, bool programmatic) {
    static std::once_flag once[64];
    int device = 0;
    cudaGetDevice(&device);
    cudaError_t attr_error = cudaSuccess;
    std::call_once(once[device & 63], [&] {
        attr_error = cudaFuncSetAttribute(gemv_kernel<DTYPE, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kMaxDynamicSmem);
    });
    GF_CUDA(attr_error);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(plan.grid);
    config.blockDim = dim3(kGemvWarps * 32);
    config.dynamicSmemBytes = plan.smem;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = programmatic ? 1 : 0;
    GF_CUDA(cudaLaunchKernelEx(&config, gemv_kernel<DTYPE, ROWS>, p));
    return GF_OK;
}

template <int DTYPE>
static int launch_rows(uint32_t rows, const GemvParams& p, const GemvPlan& plan, cudaStream_t stream, bool programmatic) {
    switch (rows) {
        case 1: return launch_instance<DTYPE, 1>(p, plan, stream, programmatic);
        case 2: return launch_instance<DTYPE, 2>(p, plan, stream, programmatic);
        case 3: return launch_instance<DTYPE, 3>(p, plan, stream, programmatic);
        default: return launch_instance<DTYPE, 4>(p, plan, stream, programmatic);
    }
}

int gemv_launch(int dtype, const void* packed, const float* x, float* y, uint32_t rows, uint64_t k, uint64_t n,
                void* workspace, int* error_flag, cudaStream_t stream, bool programmatic) {
    GemvPlan plan;
    int status = gemv_plan(dtype, rows, k, n, plan);
    if (status != GF_OK) return status;
    if (!packed || !x || !y || !error_flag) return fail(GF_ERR_INVALID, "gf_matmul: null buffer");
    if (plan.chunks > 1 && !workspace) return fail(GF_ERR_INVALID, "gf_matmul: this shape needs a split-K workspace");
    GemvParams p;
    p.weight = static_cast<const uint8_t*>(packed);
    p.x = x;
    p.out = plan.chunks > 1 ? static_cast<float*>(workspace) : y;
    p.k = (uint32_t)k;
    p.n = (uint32_t)n;
    p.units = plan.units;
    p.tiles = plan.tiles;
    p.chunks = plan.chunks;
    p.chunk_units = plan.chunk_units;
    p.error_flag = error_flag;
    if (dtype == GF_Q4_K) status = launch_rows<GF_Q4_K>(rows, p, plan, stream, programmatic);
    else if (dtype == GF_Q6_K) status = launch_rows<GF_Q6_K>(rows, p, plan, stream, programmatic);
    else status = launch_rows<GF_Q8_0>(rows, p, plan, stream, programmatic);
    if (status != GF_OK) return status;
    if (plan.chunks > 1) {
        const uint32_t elements = rows * (uint32_t)n;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((elements + 255u) / 256u);
        config.blockDim = dim3(256);
        config.stream = stream;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute.val.programmaticStreamSerializationAllowed = 1;
        config.attrs = &attribute;
        config.numAttrs = programmatic ? 1 : 0;
        GF_CUDA(cudaLaunchKernelEx(&config, gemv_reduce_kernel, (const float*)workspace, y, plan.chunks, elements));
    }
    return GF_OK;
}

// Process-wide error word for the plain entry points (one per device).
static int* device_error_flag() {
    static int* flags[64] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
    device &= 63;
    if (!flags[device]) {
        if (cudaMalloc(&flags[device], sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(flags[device], 0, sizeof(int));
    }
    return flags[device];
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_matmul_workspace_bytes(int dtype, uint32_t rows, uint64_t k, uint64_t n) {
    GemvPlan plan;
    if (gemv_plan(dtype, rows, k, n, plan) != GF_OK) return 0;
    return plan.chunks > 1 ? (size_t)plan.chunks * rows * n * sizeof(float) : 0;
}

int gf_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev, uint32_t rows, uint64_t k,
              uint64_t n, void* workspace_dev, void* stream) {
    GemvPlan plan;
    const int status = gemv_plan(dtype, rows, k, n, plan);   // argument errors come before any GPU work
    if (status != GF_OK) return status;
    int* flag = device_error_flag();
    if (!flag) return fail(GF_ERR_CUDA, "gf_matmul: cannot allocate the device error word");
    return gemv_launch(dtype, packed_dev, x_dev, y_dev, rows, k, n, workspace_dev, flag, as_stream(stream), false);
}

int gf_matmul_check(void* stream) {
    int* flag = device_error_flag();
    if (!flag) return fail(GF_ERR_CUDA, "gf_matmul_check: no device");
    int value = 0;
    GF_CUDA(cudaMemcpyAsync(&value, flag, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)));
    GF_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (value != 0) {
        cudaMemsetAsync(flag, 0, sizeof(int), as_stream(stream));
        return fail(GF_ERR_TIMEOUT, "a weight-streaming wait gave up (bounded mbarrier wait)");
    }
    return GF_OK;
}

int gf_matmul_host(int dtype, const void* packed_dev, const float* x_host, float* y_host, uint32_t rows,
                   uint64_t k, uint64_t n) {
    GemvPlan plan;
    int status = gemv_plan(dtype, rows, k, n, plan);
    if (status != GF_OK) return status;
    if (!x_host || !y_host) return fail(GF_ERR_INVALID, "gf_matmul_host: null host buffer");
    // Per-thread scratch grown on demand; the timed path reuses it, so no allocation per call.
    struct Scratch { float* x = nullptr; float* y = nullptr; void* ws = nullptr; size_t xb = 0, yb = 0, wb = 0; int device = -1; };
    static thread_local Scratch s;
    int device = 0;
    GF_CUDA(cudaGetDevice(&device));
    if (s.device != device) { s = Scratch(); s.device = device; }
    const size_t xb = (size_t)rows * k * 4, yb = (size_t)rows * n * 4;
    const size_t wb = plan.chunks > 1 ? (size_t)plan.chunks * rows * n * 4 : 0;
    if (xb > s.xb) { cudaFree(s.x); GF_CUDA(cudaMalloc(&s.x, xb)); s.xb = xb; }
    if (yb > s.yb) { cudaFree(s.y); GF_CUDA(cudaMalloc(&s.y, yb)); s.yb = yb; }
    if (wb > s.wb) { cudaFree(s.ws); GF_CUDA(cudaMalloc(&s.ws, wb)); s.wb = wb; }
    GF_CUDA(cudaMemcpyAsync(s.x, x_host, xb, cudaMemcpyHostToDevice, nullptr));
    status = gf_matmul(dtype, packed_dev, s.x, s.y, rows, k, n, s.ws, nullptr);
    if (status != GF_OK) return status;
    GF_CUDA(cudaMemcpyAsync(y_host, s.y, yb, cudaMemcpyDeviceToHost, nullptr));
    GF_CUDA(cudaStreamSynchronize(nullptr));
    return GF_OK;
}

}  // extern "C"
