// Candidate selection: the output-head epilogue.  From a full row of logits keep the best
// `retain` (= top_k + unique history tokens) pairs ordered by (logit descending, token
// ascending), then append the logits of the history tokens, so the host sampler never reads
// the 262k-wide row.  Contract of token_candidate_{tile,merge,finalize}_f32_kernel
// (metal_kernels.mm:3444-3589) and of better_logit_candidate (sampling.cpp:25-30).
#include "ops.cuh"

namespace gf {

constexpr uint32_t kTile = 2048;             // logits sorted per block
constexpr uint32_t kMaxRetain = 320;         // token_sampler_max_base_candidates
constexpr uint32_t kMaxHistory = 64;
constexpr uint32_t kMaxCandidates = 384;

struct SelectionRequest {                    // one per row, device resident
    uint32_t retain;                         // top_k + history_count, 1..320
    uint32_t history_count;                  // 0..64
    uint32_t history[kMaxHistory];
};
struct CandidateResult {                     // TokenCandidateResult (metal_kernels.mm:72-76)
    uint32_t status;
    uint32_t count;
    struct { uint32_t token; float logit; } candidates[kMaxCandidates];
};

// Sort key: ascending u64 order == (logit descending, token ascending).
__device__ __forceinline__ uint64_t make_key(float logit, uint32_t token) {
    uint32_t bits = logit == 0.0f ? 0u : __float_as_uint(logit);       // -0 and +0 compare equal
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);         // monotone in the float order
    return ((uint64_t)(~bits) << 32) | token;
}
__device__ __forceinline__ float key_logit(uint64_t key) {
    uint32_t bits = ~(uint32_t)(key >> 32);
    bits = (bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits;
    return __uint_as_float(bits);
}
constexpr uint64_t kPadKey = ~0ull;

__device__ __forceinline__ float transform(float logit, float softcap) {
    return softcap == 0.0f ? logit : __fmul_rn(softcap, tanhf(logit / softcap));
}

// Ascending bitonic sort of kTile keys by 1024 threads.
__device__ __forceinline__ void bitonic_sort(uint64_t* keys) {
    for (uint32_t width = 2; width <= kTile; width <<= 1) {
        for (uint32_t stride = width >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const uint32_t t = threadIdx.x;
            const uint32_t lo = 2u * t - (t & (stride - 1u));      // index with the `stride` bit clear
            const uint32_t hi = lo + stride;
            const bool ascending = (lo & width) == 0u;
            const uint64_t a = keys[lo], b = keys[hi];
            if ((a > b) == ascending) { keys[lo] = b; keys[hi] = a; }
        }
    }
    __syncthreads();
}

// Ascending bitonic sort of the first n keys (n a power of two <= kTile) by the first n / 2 threads.
__device__ __forceinline__ void bitonic_sort_prefix(uint64_t* keys, uint32_t n) {
    for (uint32_t width = 2; width <= n; width <<= 1) {
        for (uint32_t stride = width >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const uint32_t t = threadIdx.x;
            if (t < n / 2u) {
                const uint32_t lo = 2u * t - (t & (stride - 1u));
                const uint32_t hi = lo + stride;
                const bool ascending = (lo & width) == 0u;
                const uint64_t a = keys[lo], b = keys[hi];
                if ((a > b) == ascending) { keys[lo] = b; keys[hi] = a; }
            }
        }
    }
    __syncthreads();
}
__device__ __forceinline__ uint32_t next_pow2_u32(uint32_t v) { return v <= 1u ? 1u : 1u << (32 - __clz(v - 1u)); }

__global__ void __launch_bounds__(1024) candidate_tile_kernel(const float* __restrict__ logits, uint32_t vocab,
                                                              float softcap, const SelectionRequest* __restrict__ requests,
                                                              uint64_t* __restrict__ runs, CandidateResult* results) {
    __shared__ uint64_t keys[kTile];
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t tile = blockIdx.x, row = blockIdx.y, tiles = gridDim.x;
    const uint32_t retain = min(requests[row].retain, kMaxRetain);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t token = tile * kTile + threadIdx.x + j * 1024u;
        uint64_t key = kPadKey;
        if (token < vocab) {
            const float v = transform(logits[(size_t)row * vocab + token], softcap);
            if (isfinite(v)) key = make_key(v, token);
            else atomicOr(&results[row].status, 1u);
        }
        keys[threadIdx.x + j * 1024u] = key;
    }
    bitonic_sort(keys);
    for (uint32_t i = threadIdx.x; i < retain; i += blockDim.x)
        runs[((size_t)row * tiles + tile) * kMaxRetain + i] = keys[i];
}

__global__ void __launch_bounds__(1024) candidate_merge_kernel(const float* __restrict__ logits, uint32_t vocab,
                                                               float softcap, const SelectionRequest* __restrict__ requests,
                                                               const uint64_t* __restrict__ runs, uint32_t tiles,
                                                               CandidateResult* results) {
    __shared__ uint64_t keys[kTile];
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t row = blockIdx.x;
    const SelectionRequest& request = requests[row];
    const uint32_t retain = min(request.retain, kMaxRetain);
    const uint32_t history_count = min(request.history_count, kMaxHistory);
    if (request.retain == 0u || request.retain > kMaxRetain || request.history_count > kMaxHistory) {
        if (threadIdx.x == 0) atomicOr(&results[row].status, kStatusBadRequest);
    }
    const uint32_t total = tiles * retain;            // run entries, flattened tile-major
    __shared__ uint32_t survivors;
    bool merged = false;
    if (retain > 0u && tiles >= retain && tiles <= kTile) {
        // The `retain`-th best of the tiles' best keys bounds the answer from below: at least
        // `retain` keys (those heads) are that good, so nothing worse can be in the result.
        // Usually only about two `retain` run entries pass, and one small sort finishes the job.
        const uint32_t heads = next_pow2_u32(tiles);
        for (uint32_t i = threadIdx.x; i < heads; i += blockDim.x)
            keys[i] = i < tiles ? runs[((size_t)row * tiles + i) * kMaxRetain] : kPadKey;
        if (threadIdx.x == 0) survivors = 0u;
        bitonic_sort_prefix(keys, heads);
        const uint64_t bound = keys[retain - 1u];
        __syncthreads();
        for (uint32_t flat = threadIdx.x; flat < total; flat += blockDim.x) {
            const uint64_t key = runs[((size_t)row * tiles + flat / retain) * kMaxRetain + flat % retain];
            if (key <= bound) {
                const uint32_t slot = atomicAdd(&survivors, 1u);
                if (slot < kTile) keys[slot] = key;
            }
        }
        __syncthreads();
        const uint32_t count = survivors;
        if (count <= kTile) {
            const uint32_t padded = next_pow2_u32(max(count, retain));
            for (uint32_t i = count + threadIdx.x; i < padded; i += blockDim.x) keys[i] = kPadKey;
            bitonic_sort_prefix(keys, padded);
            merged = true;
        }
        __syncthreads();
    }
    if (!merged) {
        const uint32_t fresh = kTile - retain;            // new entries admitted per round
        for (uint32_t i = threadIdx.x; i < retain; i += blockDim.x) keys[i] = kPadKey;
        for (uint32_t first = 0; first < total || first == 0; first += fresh) {
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < fresh; i += blockDim.x) {
                const uint32_t flat = first + i;
                uint64_t key = kPadKey;
                if (flat < total) key = runs[((size_t)row * tiles + flat / retain) * kMaxRetain + flat % retain];
                keys[retain + i] = key;
            }
            bitonic_sort(keys);
        }
    }
    CandidateResult& result = results[row];
    for (uint32_t i = threadIdx.x; i < retain; i += blockDim.x) {
        const uint64_t key = keys[i];
        result.candidates[i].token = key == kPadKey ? 0xffffffffu : (uint32_t)key;
        result.candidates[i].logit = key == kPadKey ? -INFINITY : key_logit(key);
    }
    for (uint32_t i = threadIdx.x; i < history_count; i += blockDim.x) {
        const uint32_t token = request.history[i];
        if (token >= vocab) {
            atomicOr(&result.status, kStatusBadRequest);
            result.candidates[retain + i].token = 0xffffffffu;
            result.candidates[retain + i].logit = -INFINITY;
        } else {
            const float v = transform(logits[(size_t)row * vocab + token], softcap);
            if (!isfinite(v)) atomicOr(&result.status, 1u);
            result.candidates[retain + i].token = token;
            result.candidates[retain + i].logit = v;
        }
    }
    if (threadIdx.x == 0) result.count = retain + history_count;
}

// Selection requests written on the device: the role of gd_requests (src/engine/gemma3_draft.mm:396-400),
// which fills VerifierDeviceSelectionRow (target_verifier.hpp:114-121) from the sampler's history row and
// the drafted tokens, and of the resolve step of encode_verifier_selection_requests.  `base` is
// { top_k, window_limit, count, tokens[64] }: the repetition window as the host sampler holds it,
// oldest first.  Row i of `chain` (the root, then the drafted tokens, in device memory) gets the request
// of the context "window, then chain[0..i]": the window slides over the appended tokens, then its
// distinct tokens in order of first appearance are the history, and retain = top_k + their number --
// what Sampler::request_after builds on the host.  One thread per row.
struct RequestBase { uint32_t top_k, window_limit, count, tokens[kMaxHistory]; };

__global__ void request_rows_kernel(const RequestBase* __restrict__ base, uint32_t root, const uint32_t* __restrict__ chain,
                                    uint32_t first_row, uint32_t row_count, SelectionRequest* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t row = first_row + blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= first_row + row_count) return;
    const uint32_t limit = min(base->window_limit, kMaxHistory), held = min(base->count, limit);
    SelectionRequest request;
    request.history_count = 0;
    if (limit != 0u) {
        // The window after the slide: the last `limit` of (held tokens, then chain[0..row]).
        const uint32_t appended = row + 1u, total = held + appended;
        const uint32_t skip = total > limit ? total - limit : 0u;
        for (uint32_t i = skip; i < total; ++i) {
            const uint32_t token = i < held ? base->tokens[i] : (i == held ? root : chain[i - held]);
            bool seen = false;
            for (uint32_t j = 0; j < request.history_count; ++j) seen |= request.history[j] == token;
            if (!seen) request.history[request.history_count++] = token;
        }
    }
    request.retain = base->top_k + request.history_count;
    for (uint32_t j = request.history_count; j < kMaxHistory; ++j) request.history[j] = 0u;
    out[row] = request;
}

size_t request_base_bytes() { return sizeof(RequestBase); }

// Rows [first_row, first_row + row_count) of `requests_dev` from the base window at `base_dev`; chain[0] is
// taken from `root` (the host knows it), chain[i > 0] from `chain_dev[i]`.
int launch_request_rows(const void* base_dev, uint32_t root, const uint32_t* chain_dev, uint32_t first_row, uint32_t row_count,
                        void* requests_dev, cudaStream_t stream) {
    if (!base_dev || !chain_dev || !requests_dev || row_count == 0 || first_row + row_count > GF_MAX_ROWS)
        return fail(GF_ERR_INVALID, "selection request rows: bad arguments");
    return launch_kernel(request_rows_kernel, dim3(1), dim3(32), 0, stream, false, static_cast<const RequestBase*>(base_dev), root,
                         chain_dev, first_row, row_count, static_cast<SelectionRequest*>(requests_dev));
}

size_t candidates_workspace_bytes(uint32_t rows, uint32_t vocab) {
    const uint32_t tiles = (vocab + kTile - 1u) / kTile;
    return (size_t)rows * tiles * kMaxRetain * sizeof(uint64_t);
}

int launch_candidates(const float* logits, uint32_t rows, uint32_t vocab, float softcap, const void* requests,
                      void* workspace, void* results, cudaStream_t stream, bool pdl) {
    const uint32_t tiles = (vocab + kTile - 1u) / kTile;
    GF_CUDA(cudaMemsetAsync(results, 0, (size_t)rows * sizeof(CandidateResult), stream));
    int status = launch_kernel(candidate_tile_kernel, dim3(tiles, rows), dim3(1024), 0, stream, false, logits, vocab,
                               softcap, static_cast<const SelectionRequest*>(requests), static_cast<uint64_t*>(workspace),
                               static_cast<CandidateResult*>(results));
    if (status != GF_OK) return status;
    return launch_kernel(candidate_merge_kernel, dim3(rows), dim3(1024), 0, stream, pdl, logits, vocab, softcap,
                         static_cast<const SelectionRequest*>(requests), static_cast<const uint64_t*>(workspace), tiles,
                         static_cast<CandidateResult*>(results));
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_token_candidates_workspace_bytes(uint32_t rows, uint32_t vocab) { return candidates_workspace_bytes(rows, vocab); }
size_t gf_selection_request_bytes(void) { return sizeof(SelectionRequest); }
size_t gf_candidate_result_bytes(void) { return sizeof(CandidateResult); }

size_t gf_selection_base_bytes(void) { return request_base_bytes(); }

int gf_selection_requests(const void* base_dev, uint32_t root, const uint32_t* chain_dev, uint32_t rows, void* requests_dev,
                          void* stream) {
    return launch_request_rows(base_dev, root, chain_dev, 0, rows, requests_dev, as_stream(stream));
}

int gf_token_candidates(const float* logits_dev, uint32_t rows, uint32_t vocab, float softcap, const void* requests_dev,
                        void* workspace_dev, void* results_dev, void* stream) {
    if (!logits_dev || !requests_dev || !workspace_dev || !results_dev || rows == 0 || vocab == 0 || softcap < 0.0f)
        return fail(GF_ERR_INVALID, "gf_token_candidates: bad arguments");
    return launch_candidates(logits_dev, rows, vocab, softcap, requests_dev, workspace_dev, results_dev, as_stream(stream), false);
}

}  // extern "C"
