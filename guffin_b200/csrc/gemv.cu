// Host side of the streaming dequant-GEMV: decomposition plan, launch, C entry points.
#include "gemv.cuh"

#include <algorithm>
#include <mutex>

namespace gf {

// The kernel is compiled for 1, 2, 3, 4 and 8 rows; 5 to 7 rows run the eight-row instance.
#define GF_TRY_STATUS(expr) do { const int gf_s_ = (expr); if (gf_s_ != GF_OK) return gf_s_; } while (0)

// Five to eight rows run as two halves of the four-row instance in one launch (weight_stream_pair_kernel).
static uint32_t instance_rows(uint32_t rows) { return rows <= 4u ? rows : 4u; }
static uint32_t launch_halves(uint32_t rows) { return rows <= 4u ? 1u : 2u; }
static uint32_t planned_instance(const GemvLaunch& launch) { return launch.instance ? launch.instance : instance_rows(launch.rows); }

static uint32_t max_chunk_units(uint32_t rows, uint32_t unit_elems, uint32_t slot_bytes) {
    uint32_t best = 0;
    for (uint32_t cu = 1; cu <= 64u; ++cu)
        if (gemv_smem_layout(rows, cu, unit_elems, slot_bytes).total <= kGemvSmemLimit) best = cu;
    return best;
}

int gemv_plan(const GemvLaunch& launch, GemvPlan& plan) {
    if (launch.count == 0 || launch.count > (uint32_t)kGemvMaxMatrices) return fail(GF_ERR_INVALID, "gf_matmul: 1..3 matrices per launch");
    if (launch.rows == 0 || launch.rows > GF_MAX_ROWS) return fail(GF_ERR_INVALID, "gf_matmul: rows=%u outside [1, %d]", launch.rows, GF_MAX_ROWS);
    plan.total_pairs = 0;
    plan.unit_elems = 0;
    plan.slot_bytes = 0;
    for (uint32_t i = 0; i < launch.count; ++i) {
        const int dtype = launch.matrices[i].dtype;
        if (dtype != GF_Q8_0 && dtype != GF_Q4_K && dtype != GF_Q6_K) return fail(GF_ERR_INVALID, "gf_matmul: unsupported weight dtype %d", dtype);
        const uint32_t unit = unit_elements(dtype);
        if (plan.unit_elems && plan.unit_elems != unit) return fail(GF_ERR_INVALID, "gf_matmul: Q8_0 and K-quant matrices cannot share a launch");
        plan.unit_elems = unit;
        if (launch.matrices[i].n == 0 || launch.matrices[i].n > (1ull << 28)) return fail(GF_ERR_INVALID, "gf_matmul: N must be positive");
        plan.total_pairs += (uint32_t)((launch.matrices[i].n + 15u) / 16u);
        plan.slot_bytes = std::max(plan.slot_bytes, pair_row_bytes(dtype));     // one pair row; scaled below
    }
    // Two pair rows per slot (one copy, one wait for both) unless a Q6_K row makes that too large.
    plan.slot_units = plan.slot_bytes <= 2304u ? 2u : 1u;
    plan.slot_bytes *= plan.slot_units;
    if (launch.k == 0 || launch.k % plan.unit_elems != 0 || launch.k > (1ull << 24))
        return fail(GF_ERR_INVALID, "gf_matmul: K=%llu must be a positive multiple of %u", (unsigned long long)launch.k, plan.unit_elems);
    plan.units = (uint32_t)(launch.k / plan.unit_elems);
    const uint32_t limit = max_chunk_units(planned_instance(launch), plan.unit_elems, plan.slot_bytes);
    if (limit == 0) return fail(GF_ERR_INVALID, "gf_matmul: no decomposition fits");
    const uint32_t slots = (uint32_t)sm_count();           // one CTA per SM
    // Critical path of a warp, in pair rows: rounds x (units per item + per-item overhead); the
    // split-K hand-over (fence, arrival count, re-read of the partial sums) costs about four more.
    // Ties go to fewer chunks.
    double best = 1e30;
    plan.chunks = 0;
    for (uint32_t chunks = 1; chunks <= 64u && chunks <= plan.units && chunks <= slots; ++chunks) {
        const uint32_t chunk_units = (plan.units + chunks - 1u) / chunks;
        if ((chunks - 1u) * chunk_units >= plan.units) continue;          // an empty last chunk
        if (chunk_units > limit) continue;
        if (launch.prologue == kPrologueMerge && (chunk_units * plan.unit_elems) % 256u) continue;   // slices start on head boundaries
        const uint32_t group_ctas = slots / chunks;
        const uint32_t group_warps = group_ctas * kGemvWarps;
        const uint32_t rounds = (plan.total_pairs + group_warps - 1u) / group_warps;
        const double cost = (double)rounds * ((double)chunk_units + 2.0) + (chunks > 1u ? 4.0 : 0.0);
        if (cost < best - 1e-9) {
            best = cost;
            plan.chunks = chunks;
            plan.chunk_units = chunk_units;
            plan.grid = group_ctas * chunks;
        }
    }
    if (plan.chunks == 0) return fail(GF_ERR_INVALID, "gf_matmul: no decomposition fits K=%llu rows=%u", (unsigned long long)launch.k, launch.rows);
    plan.intra = 1;
    plan.staged_units = plan.chunk_units;
    // K split over the warps of one CTA instead: the partial sums then meet in shared memory, which
    // costs about half a pair row, but every CTA stages the whole activation row, so it must fit beside
    // the ring.  Not with the partition-merge prologue, whose cost grows with the staged slice.  Whether
    // K is split this way, and where, is decided for the four-row instance, so that every row count
    // adds the same partial sums in the same order: an instance too large for it (eight rows) takes
    // the same chunks across CTAs.
    const bool whole_row_fits = gemv_smem_layout(4u, plan.units, plan.unit_elems, plan.slot_bytes, true).total <= kGemvSmemLimit;
    if (whole_row_fits && launch.prologue != kPrologueMerge) {
        uint32_t inside_best = 0, units_best = 0;
        for (uint32_t inside = 2; inside <= (uint32_t)kGemvWarps && inside <= plan.units; inside *= 2u) {
            const uint32_t chunk_units = (plan.units + inside - 1u) / inside;
            if ((inside - 1u) * chunk_units >= plan.units) continue;
            const uint32_t pair_slots = (uint32_t)kGemvWarps / inside;
            const uint32_t rounds = (plan.total_pairs + slots * pair_slots - 1u) / (slots * pair_slots);
            const double cost = (double)rounds * ((double)chunk_units + 2.0) + 0.5;
            if (cost < best - 1e-9) { best = cost; inside_best = inside; units_best = chunk_units; }
        }
        if (inside_best != 0u) {
            const uint32_t pair_slots = (uint32_t)kGemvWarps / inside_best;
            if (planned_instance(launch) <= 4u) {
                plan.chunks = 1;
                plan.intra = inside_best;
                plan.chunk_units = units_best;
                plan.staged_units = plan.units;
                plan.grid = std::min(slots, (plan.total_pairs + pair_slots - 1u) / pair_slots);
            } else if (units_best <= limit && inside_best <= slots) {
                plan.chunks = inside_best;
                plan.chunk_units = units_best;
                plan.staged_units = units_best;
                plan.grid = slots / inside_best * inside_best;
            }
        }
    }
    plan.smem = gemv_smem_layout(planned_instance(launch), plan.staged_units, plan.unit_elems, plan.slot_bytes, plan.intra > 1u).total;
    return GF_OK;
}

static size_t counters_bytes(const GemvPlan& plan) { return ((size_t)plan.total_pairs * 4u + 255u) & ~(size_t)255u; }

// Partial sums of one half of a launch (the whole launch up to four rows).
static size_t half_partial_bytes(const GemvPlan& plan, const GemvLaunch& launch) {
    return (((size_t)plan.chunks * planned_instance(launch) * plan.total_pairs * 16u * sizeof(float)) + 255u) & ~(size_t)255u;
}

size_t gemv_partial_bytes(const GemvLaunch& launch) {
    GemvPlan plan;
    if (gemv_plan(launch, plan) != GF_OK || plan.chunks == 1) return 0;
    return half_partial_bytes(plan, launch) * launch_halves(launch.rows);
}

size_t gemv_counter_bytes(const GemvLaunch& launch) {
    GemvPlan plan;
    if (gemv_plan(launch, plan) != GF_OK || plan.chunks == 1) return 0;
    return counters_bytes(plan) * launch_halves(launch.rows);
}

template <int ROWS, bool TP = false>
static int launch_instance(const WeightStreamParams& p, const GemvPlan& plan, cudaStream_t stream, bool programmatic) {
    static std::once_flag once[64];
    int device = 0;
    cudaGetDevice(&device);
    cudaError_t attr_error = cudaSuccess;
    std::call_once(once[device & 63], [&] {
        attr_error = cudaFuncSetAttribute(weight_stream_kernel<ROWS, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvSmemLimit);
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
    GF_CUDA(cudaLaunchKernelEx(&config, weight_stream_kernel<ROWS, TP>, p));
    return GF_OK;
}

int gemv_prepare(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                 WeightStreamParams& p, GemvPlan& plan) {
    const int status = gemv_plan(launch, plan);
    if (status != GF_OK) return status;
    if ((!launch.in && launch.gather.count == 0u) || !error_flag) return fail(GF_ERR_INVALID, "gf_matmul: null buffer");
    if (launch.gather.count > (uint32_t)kGemvMaxShards || launch.scatter.count >= (uint32_t)kGemvMaxShards
        || (launch.gather.count != 0u && (launch.prologue != kPrologueAddNorm || !launch.gather.own || !launch.gather.tick || launch.gather.self >= launch.gather.count))
        || (launch.scatter.count != 0u && (launch.count != 1u || !launch.scatter.tick || launch.scatter.site == 0u || launch.scatter.site > 255u)))
        return fail(GF_ERR_INVALID, "gf_matmul: bad shard exchange");
    // The activation prologue reads four floats at a time.
    auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0u; };
    if (!aligned(launch.in) || !aligned(launch.residual) || !aligned(launch.gamma0) || !aligned(launch.gamma1) || !aligned(launch.residual_out))
        return fail(GF_ERR_INVALID, "gf_matmul: activation, residual and norm-weight pointers must be 16-byte aligned");
    if ((launch.prologue == kPrologueNorm && !launch.gamma1)
        || (launch.prologue == kPrologueAddNorm && (!launch.gamma0 || !launch.gamma1 || !launch.residual || !launch.residual_out))
        || (launch.prologue == kPrologueGeglu && !launch.residual)
        || (launch.prologue == kPrologueMerge && (!launch.residual || launch.k % 256u)) || launch.prologue > kPrologueMerge)
        return fail(GF_ERR_INVALID, "gf_matmul: prologue operands missing");
    p = WeightStreamParams{};
    uint32_t first = 0;
    for (uint32_t i = 0; i < launch.count; ++i) {
        const GemvMatrixDesc& d = launch.matrices[i];
        if (!d.packed || !d.out) return fail(GF_ERR_INVALID, "gf_matmul: null buffer");
        p.m[i].weight = static_cast<const uint8_t*>(d.packed);
        p.m[i].out = d.out;
        p.m[i].n = (uint32_t)d.n;
        p.m[i].pairs = (uint32_t)((d.n + 15u) / 16u);
        p.m[i].dtype = (uint32_t)d.dtype;
        p.m[i].first_pair = first;
        first += p.m[i].pairs;
    }
    p.matrices = launch.count;
    p.total_pairs = plan.total_pairs;
    p.k = (uint32_t)launch.k;
    p.units = plan.units;
    p.unit_elems = plan.unit_elems;
    p.active_rows = launch.rows;
    p.chunks = plan.chunks;
    p.chunk_units = plan.chunk_units;
    p.intra = plan.intra;
    p.staged_units = plan.staged_units;
    p.slot_bytes = plan.slot_bytes;
    p.slot_units = plan.slot_units;
    p.grid = plan.grid;
    p.wait_limit = kMbarWaitLimit;
    p.overstate = 0;
#ifdef GF_TESTING
    if (testing_fault().kind == 1) {
        p.wait_limit = testing_fault().limit;
        p.overstate = 16;
        testing_fault().kind = 0;
    }
#endif
    p.prologue = launch.prologue;
    p.in = launch.in; p.residual = launch.residual; p.gamma0 = launch.gamma0; p.gamma1 = launch.gamma1;
    p.residual_out = launch.residual_out;
    p.eps = launch.eps;
    p.error_flag = error_flag;
    p.scatter = launch.scatter;
    p.gather = launch.gather;
    if (launch.heads.rotation) {
        const GemvLaunch::Heads& h = launch.heads;
        if (launch.count != 3 || !h.q_out || !h.private_k || !h.private_v || !h.base_position || !h.status || !h.head_counters
            || launch.matrices[0].n % 256u || launch.matrices[1].n % 256u || launch.matrices[2].n != launch.matrices[1].n)
            return fail(GF_ERR_INVALID, "gf_matmul: the head epilogue needs Q, K and V matrices of 256-column heads and its buffers");
        p.heads.q_norm = h.q_norm; p.heads.k_norm = h.k_norm; p.heads.q_out = h.q_out;
        p.heads.private_k = h.private_k; p.heads.private_v = h.private_v; p.heads.rotation = h.rotation;
        p.heads.base_position = h.base_position; p.heads.status = h.status; p.heads.head_counters = h.head_counters;
        p.heads.enabled = 1u; p.heads.table_rows = h.table_rows; p.heads.kv_f16 = h.kv_f16 ? 1u : 0u;
        p.heads.eps = launch.eps;
        p.heads.row_base = h.row_base;
    }
    if (plan.chunks > 1) {
        const size_t need = half_partial_bytes(plan, launch);
        if (!counters || !partial || partial_bytes < need) return fail(GF_ERR_INVALID, "gf_matmul: this shape needs a %zu-byte split-K workspace", need);
        p.counters = counters;
        p.partial = partial;
    }
    return GF_OK;
}

// Rows 4.. of a 5..8-row launch as a launch of their own: every row pointer moved on by four rows.
static GemvLaunch second_half(const GemvLaunch& launch) {
    GemvLaunch h = launch;
    const size_t k = launch.k, skip = 4;
    h.rows = launch.rows - 4u;
    h.instance = 4;
    if (launch.prologue == kPrologueMerge) {          // [row][head][32 partitions][256] outputs and [..][32] (maximum, sum) pairs
        const size_t heads = k / 256u;
        h.in = launch.in + skip * heads * 32u * 256u;
        h.residual = launch.residual + skip * heads * 32u * 2u;
    } else {
        if (h.in) h.in += skip * k;
        if (h.residual) h.residual += skip * k;
    }
    if (h.residual_out) h.residual_out += skip * k;
    for (uint32_t i = 0; i < launch.count; ++i) h.matrices[i].out += skip * launch.matrices[i].n;
    if (launch.heads.rotation) {
        const size_t element = launch.heads.kv_f16 ? 2u : 4u;
        h.heads.q_out += skip * launch.matrices[0].n;
        h.heads.private_k = static_cast<uint8_t*>(launch.heads.private_k) + skip * launch.matrices[1].n * element;
        h.heads.private_v = static_cast<uint8_t*>(launch.heads.private_v) + skip * launch.matrices[1].n * element;
        h.heads.head_counters += (launch.matrices[0].n + 2u * launch.matrices[1].n) / 256u;      // arrival counts of its own
        h.heads.row_base = launch.heads.row_base + 4u;
    }
    for (uint32_t g = 0; g < launch.scatter.count; ++g) h.scatter.out[g] += skip * launch.matrices[0].n;
    if (launch.gather.count) {
        for (uint32_t s = 0; s < launch.gather.count; ++s) h.gather.parts[s] += skip * k;
        h.gather.own += skip * k;
    }
    return h;
}

template <bool TP>
static int launch_pair(const WeightStreamParams& first, const WeightStreamParams& second, const GemvPlan& plan, cudaStream_t stream, bool programmatic) {
    static std::once_flag once[64];
    int device = 0;
    cudaGetDevice(&device);
    cudaError_t attr_error = cudaSuccess;
    std::call_once(once[device & 63], [&] {
        attr_error = cudaFuncSetAttribute(weight_stream_pair_kernel<TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvSmemLimit);
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
    GF_CUDA(cudaLaunchKernelEx(&config, weight_stream_pair_kernel<TP>, first, second));
    return GF_OK;
}

int gemv_launch(const GemvLaunch& launch, uint32_t* counters, float* partial, size_t partial_bytes, int* error_flag,
                cudaStream_t stream, bool programmatic) {
    WeightStreamParams p;
    GemvPlan plan;
    if (launch.rows > 4u && launch.rows <= GF_MAX_ROWS && launch.instance == 0u) {
        // Two halves of the four-row instance in one launch, each with arrival counts and partial sums of its own.
        GemvLaunch front = launch;
        front.rows = 4;
        front.instance = 4;
        const GemvLaunch back = second_half(launch);
        WeightStreamParams q;
        GemvPlan plan_back;
        GF_TRY_STATUS(gemv_prepare(front, counters, partial, partial_bytes, error_flag, p, plan));
        const size_t counter_words = plan.chunks > 1u ? counters_bytes(plan) / sizeof(uint32_t) : 0u;
        const size_t half_bytes = plan.chunks > 1u ? half_partial_bytes(plan, front) : 0u;
        GF_TRY_STATUS(gemv_prepare(back, counters ? counters + counter_words : nullptr,
                                   partial ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(partial) + half_bytes) : nullptr,
                                   partial_bytes >= half_bytes ? partial_bytes - half_bytes : 0u, error_flag, q, plan_back));
        if (plan_back.grid != plan.grid || plan_back.smem != plan.smem || plan_back.chunks != plan.chunks || plan_back.intra != plan.intra)
            return fail(GF_ERR_CUDA, "gf_matmul: the two halves of a launch were planned differently");
        if (p.scatter.count != 0u || p.gather.count != 0u) return launch_pair<true>(p, q, plan, stream, programmatic);
        return launch_pair<false>(p, q, plan, stream, programmatic);
    }
    const int status = gemv_prepare(launch, counters, partial, partial_bytes, error_flag, p, plan);
    if (status != GF_OK) return status;
    if (p.scatter.count != 0u || p.gather.count != 0u)        // a tensor-parallel shard's exchange rides on the launch
        switch (launch.rows) {
            case 1: return launch_instance<1, true>(p, plan, stream, programmatic);
            case 2: return launch_instance<2, true>(p, plan, stream, programmatic);
            case 3: return launch_instance<3, true>(p, plan, stream, programmatic);
            case 4: return launch_instance<4, true>(p, plan, stream, programmatic);
            default: return fail(GF_ERR_INVALID, "gf_matmul: no instance for %u rows", launch.rows);
        }
    switch (launch.rows) {
        case 1: return launch_instance<1>(p, plan, stream, programmatic);
        case 2: return launch_instance<2>(p, plan, stream, programmatic);
        case 3: return launch_instance<3>(p, plan, stream, programmatic);
        case 4: return launch_instance<4>(p, plan, stream, programmatic);
        default: return fail(GF_ERR_INVALID, "gf_matmul: no instance for %u rows", launch.rows);
    }
}

static GemvLaunch single(int dtype, const void* packed, const float* x, float* y, uint32_t rows, uint64_t k, uint64_t n) {
    GemvLaunch launch;
    launch.matrices[0] = GemvMatrixDesc{dtype, packed, y, n};
    launch.count = 1;
    launch.k = k;
    launch.rows = rows;
    launch.in = x;
    return launch;
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
    const GemvLaunch launch = single(dtype, reinterpret_cast<const void*>(1), nullptr, reinterpret_cast<float*>(1), rows, k, n);
    return gemv_counter_bytes(launch) + gemv_partial_bytes(launch);
}

int gf_matmul(int dtype, const void* packed_dev, const float* x_dev, float* y_dev, uint32_t rows, uint64_t k,
              uint64_t n, void* workspace_dev, void* stream) {
    const GemvLaunch launch = single(dtype, packed_dev ? packed_dev : reinterpret_cast<const void*>(1), x_dev, y_dev ? y_dev : reinterpret_cast<float*>(1), rows, k, n);
    GemvPlan plan;
    const int status = gemv_plan(launch, plan);      // argument errors come before any GPU work
    if (status != GF_OK) return status;
    if (!packed_dev || !x_dev || !y_dev) return fail(GF_ERR_INVALID, "gf_matmul: null buffer");
    int* flag = device_error_flag();
    if (!flag) return fail(GF_ERR_CUDA, "gf_matmul: cannot allocate the device error word");
    const size_t bytes = gemv_partial_bytes(launch);
    if (bytes && !workspace_dev) return fail(GF_ERR_INVALID, "gf_matmul: this shape needs a split-K workspace");
    // The arrival counters at the head of the workspace must start at zero.
    const size_t counters = gemv_counter_bytes(launch);          // both halves' of a 5..8-row launch
    if (bytes) GF_CUDA(cudaMemsetAsync(workspace_dev, 0, counters, as_stream(stream)));
    return gemv_launch(launch, static_cast<uint32_t*>(workspace_dev),
                       reinterpret_cast<float*>(static_cast<uint8_t*>(workspace_dev) + counters), bytes, flag,
                       as_stream(stream), false);
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
    const size_t wb = gf_matmul_workspace_bytes(dtype, rows, k, n);
    GemvPlan plan;
    int status = gemv_plan(single(dtype, reinterpret_cast<const void*>(1), nullptr, reinterpret_cast<float*>(1), rows, k, n), plan);
    if (status != GF_OK) return status;
    if (!x_host || !y_host) return fail(GF_ERR_INVALID, "gf_matmul_host: null host buffer");
    // Per-thread scratch grown on demand; the timed path reuses it, so no allocation per call.
    struct Scratch { float* x = nullptr; float* y = nullptr; void* ws = nullptr; size_t xb = 0, yb = 0, wb = 0; int device = -1; };
    static thread_local Scratch s;
    int device = 0;
    GF_CUDA(cudaGetDevice(&device));
    if (s.device != device) { s = Scratch(); s.device = device; }
    const size_t xb = (size_t)rows * k * 4, yb = (size_t)rows * n * 4;
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

// ------------------------------------------------------------------------------------------
// gf_matmul_static: the same product with its split-K scratch in a fixed device array.
//
// Some callers may not allocate device memory at the moment they need a projection: a decode
// loop that must not hit cudaMalloc's implicit device-wide synchronisation, a host process whose
// HBM has been handed out completely to its own pools, or a plugin that is only ever given
// the buffers it reads and writes.  For them the scratch the kernel needs (arrival counters
// and per-chunk partial sums) and the error word live in this translation unit's static
// device storage, which every GPU that loads the library holds until the process exits.
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) int g_static_error_flag[64];

struct StaticScratch { unsigned char* scratch = nullptr; int* error_flag = nullptr; };

// In host code the array names above are host-side stand-ins, not device addresses; the
// device address comes from cudaGetSymbolAddress, once per device, with that device current.
int static_scratch_for_current_device(StaticScratch& out) {
    static StaticScratch per_device[64];
    static std::mutex guard;
    int device = 0;
    GF_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(GF_ERR_INVALID, "gf_matmul_static: device index %d out of range", device);
    std::lock_guard<std::mutex> lock(guard);
    StaticScratch& slot = per_device[device];
    if (!slot.scratch) {
        void* scratch = nullptr;
        void* flag = nullptr;
        GF_CUDA(cudaGetSymbolAddress(&scratch, g_static_scratch));
        GF_CUDA(cudaGetSymbolAddress(&flag, g_static_error_flag));
        slot.scratch = static_cast<unsigned char*>(scratch);
        slot.error_flag = static_cast<int*>(flag);
    }
    out = slot;
    return GF_OK;
}

}  // namespace

extern "C" {

size_t gf_matmul_static_capacity(void) { return kStaticScratchBytes; }

int gf_matmul_static(int dtype, const void* packed_dev, const float* x_dev, float* y_dev, uint32_t rows, uint64_t k,
                     uint64_t n, void* stream) {
    const GemvLaunch launch = single(dtype, packed_dev ? packed_dev : reinterpret_cast<const void*>(1), x_dev,
                                     y_dev ? y_dev : reinterpret_cast<float*>(1), rows, k, n);
    GemvPlan plan;
    const int status = gemv_plan(launch, plan);
    if (status != GF_OK) return status;
    const size_t counters = gemv_counter_bytes(launch), partial = gemv_partial_bytes(launch);
    if (counters + partial > kStaticScratchBytes)
        return fail(GF_ERR_INVALID,
                    "gf_matmul_static: this shape needs %zu bytes of split-K scratch but the built-in array holds %zu; "
                    "use gf_matmul with a caller-provided workspace",
                    counters + partial, (size_t)kStaticScratchBytes);
    if (!packed_dev || !x_dev || !y_dev) return fail(GF_ERR_INVALID, "gf_matmul_static: null buffer");
    StaticScratch device;
    const int setup = static_scratch_for_current_device(device);
    if (setup != GF_OK) return setup;
    cudaStream_t s = as_stream(stream);
    // The array keeps whatever the previous call left: the arrival counters must start at zero,
    // the partial sums are fully overwritten before they are read.  The error word is NOT cleared
    // here: a wait that gave up in an earlier call stays visible until gf_matmul_static_check reads it.
    if (counters) GF_CUDA(cudaMemsetAsync(device.scratch, 0, counters, s));
    return gemv_launch(launch, reinterpret_cast<uint32_t*>(device.scratch), reinterpret_cast<float*>(device.scratch + counters),
                       partial, device.error_flag, s, false);
}

int gf_matmul_static_check(void* stream) {
    StaticScratch device;
    const int setup = static_scratch_for_current_device(device);
    if (setup != GF_OK) return setup;
    cudaStream_t s = as_stream(stream);
    int value = 0;
    // The word lives in the library's static device storage: read through its symbol address, nothing is allocated.
    GF_CUDA(cudaMemcpyAsync(&value, device.error_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    GF_CUDA(cudaStreamSynchronize(s));
    if (value != 0) {
        GF_CUDA(cudaMemsetAsync(device.error_flag, 0, sizeof(int), s));
        // A call that was cut short leaves its arrival counters half way; the next call zeroes the ones it uses.
        return fail(GF_ERR_TIMEOUT, "gf_matmul_static: a weight-streaming wait gave up (bounded mbarrier wait); y is incomplete");
    }
    return GF_OK;
}

}  // extern "C"
