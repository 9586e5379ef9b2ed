// Device sampler of the drafter: builds the exact proposal law the acceptance test needs.
//
// Contract of the reference's compact path (src/engine/gemma3_draft.mm:191-203,237-294): scores
// are the logits after repetition penalty and temperature; the support is every token whose
// score reaches the top_k-th best (ties at the cut-off survive); inside it the ascending-tail
// top-p rule and min-p suppress tokens; F32 exp weights are accumulated in token-id order and
// turned into an integer CDF with total exactly 2^32; the drafted token is the bin holding the
// 32-bit proposal word.  The bins, not an idealised softmax, are the law q that the lossless
// acceptance test divides by, so the sampler and the receipt can never disagree.
// A support of more than 256 tokens is reported as status 20; the caller then builds the law over
// the whole vocabulary from the same scores (draft_full.cu), as it does from the start when top_k is
// disabled or above 64.
#include "ops.cuh"

namespace gf {

size_t candidates_workspace_bytes(uint32_t rows, uint32_t vocab);
int launch_candidates(const float* logits, uint32_t rows, uint32_t vocab, float softcap, const void* requests,
                      void* workspace, void* results, cudaStream_t stream, bool pdl);

constexpr uint32_t kDraftSupportMax = 256;

struct DraftPair { uint32_t token; float score; };

struct DraftReceipt {                 // read back by the host for gather()
    uint32_t status;                  // 0 ok; 10/11 non-finite logit/score; 12 empty; 13 bad total; 15 CDF did not close; 20 support > 256
    uint32_t count;                   // support size (tokens may carry zero mass)
    uint32_t token;                   // drafted token
    uint32_t word;                    // the proposal word that selected it
    uint32_t ids[kDraftSupportMax];   // ascending token ids
    uint64_t cdf[kDraftSupportMax + 1];
};

struct CandidateHead {                // leading fields of the candidate result row
    uint32_t status, count;
    struct { uint32_t token; float logit; } candidates[384];
};

__global__ void __launch_bounds__(256) draft_process_kernel(const float* __restrict__ logits, uint32_t vocab, float temperature,
                                                            float penalty, const uint32_t* __restrict__ history,
                                                            uint32_t history_count, const uint32_t* __restrict__ history_count_dev,
                                                            float* __restrict__ scores,
                                                            DraftReceipt* receipt, uint32_t* support_count) {
    __shared__ uint32_t hist[64];
    pdl_wait();
    pdl_launch_dependents();
    if (history_count_dev) history_count = min(*history_count_dev, 64u);       // a request row written on the device
    const bool penalise = penalty != 1.0f && history_count != 0u;
    if (penalise) {
        for (uint32_t i = threadIdx.x; i < history_count && i < 64u; i += blockDim.x) hist[i] = history[i];
        __syncthreads();
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) { *support_count = 0u; }
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        float score = logits[i];
        if (!isfinite(score)) { atomicMax(&receipt->status, 10u); score = 0.0f; }
        if (penalise) {
            bool seen = false;
            for (uint32_t h = 0; h < history_count && h < 64u; ++h) seen |= hist[h] == i;
            if (seen) score = score < 0.0f ? __fmul_rn(score, penalty) : __fdiv_rn(score, penalty);
        }
        if (temperature > 0.0f) score = __fdiv_rn(score, temperature);
        if (!isfinite(score)) { atomicMax(&receipt->status, 11u); score = 0.0f; }
        scores[i] = score;
    }
}

__global__ void __launch_bounds__(256) draft_collect_kernel(const float* __restrict__ scores, uint32_t vocab,
                                                            const CandidateHead* best, uint32_t top_k, int greedy,
                                                            DraftPair* support, uint32_t* support_count) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t have = min(best->count, top_k);
    const float cutoff = have ? best->candidates[have - 1u].logit : INFINITY;
    // A greedy drafter puts all mass on the argmax, the lowest token id among exact ties (the step CDF
    // of gd_cdf, gemma3_draft.mm:372-381).
    const uint32_t only = greedy && have ? best->candidates[0].token : 0xffffffffu;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float s = scores[i];
        if (greedy ? i == only : s >= cutoff) {
            const uint32_t slot = atomicAdd(support_count, 1u);
            if (slot < kDraftSupportMax) support[slot] = DraftPair{i, s};
        }
    }
}

__device__ __forceinline__ bool draft_better(DraftPair a, DraftPair b) {
    return a.score > b.score || (a.score == b.score && a.token < b.token);
}

template <typename Less>
__device__ __forceinline__ void bitonic256(DraftPair* values, Less less) {
    const uint32_t t = threadIdx.x;
    for (uint32_t width = 2; width <= 256u; width <<= 1) {
        for (uint32_t stride = width >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const uint32_t other = t ^ stride;
            if (other > t) {
                const bool ascending = (t & width) == 0u;
                const DraftPair a = values[t], b = values[other];
                if (ascending ? less(b, a) : less(a, b)) { values[t] = b; values[other] = a; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256) draft_law_kernel(const DraftPair* __restrict__ support, const uint32_t* support_count,
                                                        float top_p, float min_p, uint32_t word, DraftReceipt* receipt,
                                                        uint32_t* out_token_a, uint32_t* out_token_b) {
    __shared__ DraftPair values[256];
    __shared__ float weights[256];
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t t = threadIdx.x;
    const uint32_t n = *support_count;
    if (t == 0) { receipt->word = word; receipt->count = min(n, kDraftSupportMax); }
    if (n > kDraftSupportMax) { if (t == 0) atomicMax(&receipt->status, 20u); return; }
    if (n == 0u) { if (t == 0) atomicMax(&receipt->status, 12u); return; }
    values[t] = t < n ? support[t] : DraftPair{0xffffffffu, -INFINITY};
    bitonic256(values, draft_better);                                   // best first
    weights[t] = t < n ? expf(values[t].score - values[0].score) : 0.0f;
    __syncthreads();
    if (t == 0) {
        // Ascending-tail nucleus: a token survives while the mass of itself and everything worse
        // exceeds 1 - top_p; min-p compares its weight with the best token's (weight 1).
        float total = 0.0f, tail = 0.0f;
        for (uint32_t j = n; j > 0; --j) total += weights[j - 1];
        for (uint32_t j = n; j > 0; --j) {
            const uint32_t i = j - 1;
            tail += weights[i];
            const bool keep = i == 0 || ((top_p >= 1.0f || tail / total > 1.0f - top_p) && (min_p <= 0.0f || weights[i] >= min_p));
            if (!keep) values[i].score = -INFINITY;
        }
    }
    __syncthreads();
    bitonic256(values, [](DraftPair a, DraftPair b) { return a.token < b.token; });   // token-id order
    if (t == 0) {
        float maximum = -INFINITY;
        for (uint32_t i = 0; i < n; ++i) maximum = fmaxf(maximum, values[i].score);
        float total = 0.0f;
        for (uint32_t i = 0; i < n; ++i) { weights[i] = expf(values[i].score - maximum); total += weights[i]; }
        if (!(total > 0.0f) || !isfinite(total)) { atomicMax(&receipt->status, 13u); return; }
        float prefix = 0.0f;
        uint64_t last = 0;
        receipt->cdf[0] = 0;
        uint32_t chosen = 0xffffffffu;
        for (uint32_t i = 0; i < n; ++i) {
            receipt->ids[i] = values[i].token;
            prefix += weights[i];
            const float scaled = fminf(fmaxf((prefix / total) * 4294967296.0f, 0.0f), 4294967296.0f);
            const uint64_t next = (uint64_t)scaled;
            receipt->cdf[i + 1] = next;
            if (next < last) atomicMax(&receipt->status, 14u);
            if ((uint64_t)word >= last && (uint64_t)word < next) chosen = values[i].token;
            last = next;
        }
        if (last != 4294967296ull) atomicMax(&receipt->status, 15u);
        receipt->token = chosen;
        if (chosen != 0xffffffffu) {
            if (out_token_a) *out_token_a = chosen;
            if (out_token_b) *out_token_b = chosen;
        }
    }
}

size_t draft_full_workspace_bytes(uint32_t vocab);
int launch_draft_law_full(float* scores, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                          uint32_t word, void* workspace, void* receipt_dev, bool keep_status, uint32_t* out_token_a,
                          uint32_t* out_token_b, cudaStream_t stream);
int launch_draft_gather_full(void* workspace, uint32_t vocab, const uint32_t* tokens_host, uint32_t count, uint64_t* intervals_host,
                             cudaStream_t stream);

static size_t compact_workspace_bytes(uint32_t vocab) {
    const size_t bytes = (size_t)vocab * 4 + candidates_workspace_bytes(1, vocab) + 264 + 3080 + kDraftSupportMax * sizeof(DraftPair) + 64
                         + 64 * 4 + 256;
    return (bytes + 255u) & ~(size_t)255u;
}
// The compact sampler's scratch, then the full-vocabulary law's (sorted keys, prefix sums, the CDF).
size_t draft_sampler_workspace_bytes(uint32_t vocab) { return compact_workspace_bytes(vocab) + draft_full_workspace_bytes(vocab); }

// The compact law serves a tempered drafter with 1 <= top_k <= 64 (Impl::sample's `compact`,
// gemma3_draft.mm:1022-1024); a greedy drafter is a point mass and takes the same kernels.
bool draft_law_is_compact(float temperature, uint32_t top_k) { return temperature == 0.0f || (top_k >= 1u && top_k <= 64u); }

// Lays the scratch out inside one allocation and runs the five launches.
// `history_request_dev` (optional): a selection request row in device memory ({ retain, count, tokens[64] })
// whose history replaces history_host -- the drafter then penalises drafts the host has not seen yet.
int launch_draft_sample(const float* logits, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                        float penalty, const uint32_t* history_host, uint32_t history_count, uint32_t word,
                        void* workspace, void* receipt_dev, uint32_t* out_token_a, uint32_t* out_token_b,
                        cudaStream_t stream, const uint32_t* history_request_dev) {
    if (!logits || !workspace || !receipt_dev || vocab == 0 || history_count > 64u)
        return fail(GF_ERR_INVALID, "draft sampler: bad arguments");
    const bool compact = draft_law_is_compact(temperature, top_k);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    float* scores = reinterpret_cast<float*>(base); base += (size_t)vocab * 4;
    void* cand_ws = base; base += candidates_workspace_bytes(1, vocab);
    uint32_t* request = reinterpret_cast<uint32_t*>(base); base += 264 + 8;
    void* best = base; base += 3080 + 8;
    DraftPair* support = reinterpret_cast<DraftPair*>(base); base += kDraftSupportMax * sizeof(DraftPair);
    uint32_t* support_count = reinterpret_cast<uint32_t*>(base); base += 64;
    uint32_t* history_dev = reinterpret_cast<uint32_t*>(base);
    DraftReceipt* receipt = static_cast<DraftReceipt*>(receipt_dev);
    GF_CUDA(cudaMemsetAsync(receipt, 0, 16, stream));
    const uint32_t effective_k = temperature == 0.0f ? 1u : top_k;      // a greedy drafter puts all mass on the argmax
    const uint32_t request_words[2] = {effective_k, 0u};
    GF_CUDA(cudaMemcpyAsync(request, request_words, 8, cudaMemcpyHostToDevice, stream));
    if (!history_request_dev && history_count && penalty != 1.0f)
        GF_CUDA(cudaMemcpyAsync(history_dev, history_host, history_count * 4u, cudaMemcpyHostToDevice, stream));
    const uint32_t* history_tokens = history_request_dev ? history_request_dev + 2 : history_dev;
    const uint32_t* history_count_dev = history_request_dev ? history_request_dev + 1 : nullptr;
    const uint32_t blocks = min((vocab + 255u) / 256u, 1024u);
    int status = launch_kernel(draft_process_kernel, dim3(blocks), dim3(256), 0, stream, false, logits, vocab, temperature,
                               penalty, history_tokens, history_count, history_count_dev, scores, receipt, support_count);
    if (status != GF_OK) return status;
    if (!compact)       // top_k disabled or above 64: the law over the whole vocabulary
        return launch_draft_law_full(scores, vocab, temperature, top_k, top_p, min_p, word,
                                     static_cast<uint8_t*>(workspace) + compact_workspace_bytes(vocab), receipt_dev, true,
                                     out_token_a, out_token_b, stream);
    status = launch_candidates(scores, 1, vocab, 0.0f, request, cand_ws, best, stream, false);
    if (status != GF_OK) return status;
    status = launch_kernel(draft_collect_kernel, dim3(blocks), dim3(256), 0, stream, false, (const float*)scores, vocab,
                           (const CandidateHead*)best, effective_k, temperature == 0.0f ? 1 : 0, support, support_count);
    if (status != GF_OK) return status;
    return launch_kernel(draft_law_kernel, dim3(1), dim3(256), 0, stream, false, (const DraftPair*)support,
                         (const uint32_t*)support_count, temperature == 0.0f ? 1.0f : top_p, temperature == 0.0f ? 0.0f : min_p,
                         word, receipt, out_token_a, out_token_b);
}

// After a compact receipt reported status 20 (more than 256 tokens reach the top_k cut-off): builds the
// full-vocabulary law from the processed scores the compact pass left in `workspace` -- same logits, same
// proposal word -- and selects the drafted token from it.
int launch_draft_resolve_overflow(uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p, uint32_t word,
                                  void* workspace, void* receipt_dev, uint32_t* out_token_a, uint32_t* out_token_b,
                                  cudaStream_t stream) {
    if (!workspace || !receipt_dev || vocab == 0) return fail(GF_ERR_INVALID, "draft sampler: bad arguments");
    return launch_draft_law_full(static_cast<float*>(workspace), vocab, temperature, top_k, top_p, min_p, word,
                                 static_cast<uint8_t*>(workspace) + compact_workspace_bytes(vocab), receipt_dev, true,
                                 out_token_a, out_token_b, stream);
}

int launch_draft_gather(void* workspace, uint32_t vocab, const uint32_t* tokens_host, uint32_t count, uint64_t* intervals_host,
                        cudaStream_t stream) {
    if (!workspace) return fail(GF_ERR_INVALID, "draft gather: null workspace");
    return launch_draft_gather_full(static_cast<uint8_t*>(workspace) + compact_workspace_bytes(vocab), vocab, tokens_host, count,
                                    intervals_host, stream);
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_draft_receipt_bytes(void) { return sizeof(DraftReceipt); }
size_t gf_draft_sample_workspace_bytes(uint32_t vocab) { return draft_sampler_workspace_bytes(vocab); }

int gf_draft_sample(const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                    float repetition_penalty, const uint32_t* history_host, uint32_t history_count, uint32_t word,
                    void* workspace_dev, void* receipt_dev, uint32_t* out_token_dev, void* stream) {
    return launch_draft_sample(logits_dev, vocab, temperature, top_k, top_p, min_p, repetition_penalty, history_host,
                               history_count, word, workspace_dev, receipt_dev, out_token_dev, nullptr, as_stream(stream), nullptr);
}

int gf_draft_resolve_overflow(uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p, uint32_t word,
                              void* workspace_dev, void* receipt_dev, uint32_t* out_token_dev, void* stream) {
    return launch_draft_resolve_overflow(vocab, temperature, top_k, top_p, min_p, word, workspace_dev, receipt_dev, out_token_dev,
                                         nullptr, as_stream(stream));
}

int gf_draft_gather_full(void* workspace_dev, uint32_t vocab, const uint32_t* tokens_host, uint32_t count,
                         uint64_t* intervals_host, void* stream) {
    return launch_draft_gather(workspace_dev, vocab, tokens_host, count, intervals_host, as_stream(stream));
}

}  // extern "C"
