// The drafter's full-vocabulary proposal law: the law Gemma3DraftPlan uses when the compact support
// would hold more than 256 tokens (more than 216 exact ties at the top_k cut-off), when top_k is 0 or
// above 64, or for a greedy drafter (src/engine/gemma3_draft.mm:295-395, driven by Impl::sample
// :995-1167).  The receipt is a CDF over the whole vocabulary, `vocab + 1` 64-bit bounds with total
// exactly 2^32, that stays on the device; the host reads only the intervals it needs through
// launch_draft_gather_full (the role of Gemma3DraftPlan::gather's non-compact branch, :1528-1581).
//
//   filter (temperature > 0 and top_k, top_p or min_p active): every token sorted by (score
//   descending, token ascending); walking from the worst to the best in blocks of 256 (the order padded
//   at the worst end to a multiple of 256), the F32 weights exp(score - best) of the tokens at or above
//   the top_k-th score are summed in order inside a block and the block totals in block order; a token
//   is dropped when its tail share is <= 1 - top_p or its weight is below min_p; the best token stays.
//   law: maximum of the survivors (lowest id on ties); weights exp(score - maximum) summed in token-id
//   order the same blockwise way; cdf[i] = u64(clamp(sum_before(i) / total * 2^32)), cdf[vocab] = 2^32.
//   greedy: cdf is a step at the argmax.
//
// The sort is a shared-memory bitonic sort of 2048-key tiles followed by rank-counting merges (keys are
// unique: the token id is part of the key), so every sum is formed in one fixed order.
#include "ops.cuh"

#include <utility>

#define GF_TRY(expr) do { const int gf_s_ = (expr); if (gf_s_ != GF_OK) return gf_s_; } while (0)

namespace gf {

constexpr uint32_t kFullTile = 2048;
constexpr uint32_t kFullBlock = 256;          // tokens per prefix block (gd_filter_prefix / gd_prefix)
constexpr uint64_t kFullPadKey = ~0ull;
constexpr uint64_t kMassTotal = 1ull << 32;

struct DraftReceiptHead { uint32_t status, count, token, word; };

// Ascending u64 order == (score descending, token ascending); -0 and +0 tie.
__device__ __forceinline__ uint64_t full_key(float score, uint32_t token) {
    uint32_t bits = score == 0.0f ? 0u : __float_as_uint(score);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return ((uint64_t)(~bits) << 32) | token;
}
__device__ __forceinline__ float full_key_score(uint64_t key) {
    uint32_t bits = ~(uint32_t)(key >> 32);
    bits = (bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits;
    return __uint_as_float(bits);
}

__global__ void __launch_bounds__(1024) full_sort_tile_kernel(const float* __restrict__ scores, uint32_t vocab,
                                                              uint64_t* __restrict__ runs) {
    __shared__ uint64_t keys[kFullTile];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t slot = threadIdx.x + j * 1024u, token = blockIdx.x * kFullTile + slot;
        keys[slot] = token < vocab ? full_key(scores[token], token) : kFullPadKey;
    }
    for (uint32_t width = 2; width <= kFullTile; width <<= 1) {
        for (uint32_t stride = width >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const uint32_t t = threadIdx.x;
            const uint32_t lo = 2u * t - (t & (stride - 1u)), hi = lo + stride;
            const bool ascending = (lo & width) == 0u;
            const uint64_t a = keys[lo], b = keys[hi];
            if ((a > b) == ascending) { keys[lo] = b; keys[hi] = a; }
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) runs[(size_t)blockIdx.x * kFullTile + threadIdx.x + j * 1024u] = keys[threadIdx.x + j * 1024u];
}

// Merges neighbouring sorted runs of `width` keys: an entry's place is its index in its own run plus the
// number of entries of the partner run that go before it (strictly smaller for the left run, smaller or
// equal for the right run, which only matters for the pad keys).
__global__ void __launch_bounds__(256) full_merge_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                                                         uint32_t width, uint32_t total) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const uint32_t run = i / width, index = i % width, pair_base = (run & ~1u) * width;
    const uint32_t partner_base = (run ^ 1u) * width;
    const uint64_t key = in[i];
    if (partner_base >= total) { out[i] = key; return; }
    const uint64_t* partner = in + partner_base;
    const uint32_t partner_count = min(width, total - partner_base);
    const bool left = (run & 1u) == 0u;
    uint32_t low = 0, high = partner_count;
    while (low < high) {
        const uint32_t probe = (low + high) >> 1;
        const uint64_t other = partner[probe];
        if (left ? other < key : other <= key) low = probe + 1u; else high = probe;
    }
    out[pair_base + index + low] = key;
}

// Block g of the ascending walk covers positions 256g .. 256g+255; position i holds rank padded-1-i.
__global__ void __launch_bounds__(256) full_filter_prefix_kernel(const uint64_t* __restrict__ sorted, uint32_t vocab, uint32_t padded,
                                                                 uint32_t top_k, float* __restrict__ prefix, float* __restrict__ totals) {
    __shared__ float weights[kFullBlock];
    const uint32_t i = blockIdx.x * kFullBlock + threadIdx.x, rank = padded - 1u - i;
    const float cutoff = top_k ? full_key_score(sorted[min(top_k, vocab) - 1u]) : -INFINITY;
    const float best = full_key_score(sorted[0]);
    float w = 0.0f;
    if (rank < vocab) {
        const float score = full_key_score(sorted[rank]);
        if (score >= cutoff) w = expf(score - best);
    }
    weights[threadIdx.x] = w;
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < kFullBlock; ++j) { sum += weights[j]; prefix[blockIdx.x * kFullBlock + j] = sum; }
        totals[blockIdx.x] = sum;
    }
}

__global__ void full_offsets_kernel(const float* __restrict__ totals, uint32_t groups, float* __restrict__ offsets,
                                    uint32_t* status, uint32_t code_if_bad) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float sum = 0.0f;
    offsets[0] = 0.0f;
    for (uint32_t g = 0; g < groups; ++g) { sum += totals[g]; offsets[g + 1u] = sum; }
    if (code_if_bad && (!(sum > 0.0f) || !isfinite(sum))) atomicMax(status, code_if_bad);
}

__global__ void __launch_bounds__(256) full_filter_apply_kernel(const uint64_t* __restrict__ sorted, uint32_t vocab, uint32_t padded,
                                                                uint32_t groups, uint32_t top_k, float top_p, float min_p,
                                                                const float* __restrict__ prefix, const float* __restrict__ offsets,
                                                                float* __restrict__ scores) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= padded) return;
    const uint32_t rank = padded - 1u - i;
    if (rank >= vocab) return;
    const uint64_t key = sorted[rank];
    const float score = full_key_score(key), best = full_key_score(sorted[0]);
    const float cutoff = top_k ? full_key_score(sorted[min(top_k, vocab) - 1u]) : -INFINITY;
    bool keep = score >= cutoff;
    const float tail = (offsets[i / kFullBlock] + prefix[i]) / offsets[groups];
    if (top_p < 1.0f && tail <= 1.0f - top_p && rank != 0u) keep = false;
    if (min_p > 0.0f && expf(score - best) < min_p && rank != 0u) keep = false;
    scores[(uint32_t)key] = keep ? score : -INFINITY;
}

// Maximum of the surviving scores per block of 256 tokens, lowest token id on ties.
__global__ void __launch_bounds__(256) full_max_kernel(const float* __restrict__ scores, uint32_t vocab, float* __restrict__ maxima,
                                                       uint32_t* __restrict__ argmax) {
    __shared__ float m[kFullBlock];
    __shared__ uint32_t ids[kFullBlock];
    const uint32_t i = blockIdx.x * kFullBlock + threadIdx.x;
    m[threadIdx.x] = i < vocab ? scores[i] : -INFINITY;
    ids[threadIdx.x] = i;
    __syncthreads();
    for (uint32_t s = kFullBlock / 2u; s; s >>= 1) {
        if (threadIdx.x < s && (m[threadIdx.x + s] > m[threadIdx.x] || (m[threadIdx.x + s] == m[threadIdx.x] && ids[threadIdx.x + s] < ids[threadIdx.x]))) {
            m[threadIdx.x] = m[threadIdx.x + s];
            ids[threadIdx.x] = ids[threadIdx.x + s];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { maxima[blockIdx.x] = m[0]; argmax[blockIdx.x] = ids[0]; }
}

__global__ void full_max_finish_kernel(float* maxima, uint32_t* argmax, uint32_t groups, uint32_t* status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float m = -INFINITY;
    uint32_t id = 0;
    for (uint32_t g = 0; g < groups; ++g)
        if (maxima[g] > m || (maxima[g] == m && argmax[g] < id)) { m = maxima[g]; id = argmax[g]; }
    maxima[groups] = m;
    argmax[groups] = id;
    if (!isfinite(m)) atomicMax(status, 6u);
}

__global__ void __launch_bounds__(256) full_prefix_kernel(const float* __restrict__ scores, uint32_t vocab, uint32_t groups,
                                                          const float* __restrict__ maxima, float* __restrict__ prefix,
                                                          float* __restrict__ totals) {
    __shared__ float weights[kFullBlock];
    const uint32_t i = blockIdx.x * kFullBlock + threadIdx.x;
    const float score = i < vocab ? scores[i] : -INFINITY;
    weights[threadIdx.x] = score > -INFINITY ? expf(score - maxima[groups]) : 0.0f;
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < kFullBlock; ++j) { sum += weights[j]; prefix[blockIdx.x * kFullBlock + j] = sum; }
        totals[blockIdx.x] = sum;
    }
}

__global__ void __launch_bounds__(256) full_cdf_kernel(const float* __restrict__ prefix, const float* __restrict__ offsets,
                                                       const uint32_t* __restrict__ argmax, uint32_t vocab, uint32_t groups, int greedy,
                                                       const uint32_t* status, uint64_t* __restrict__ cdf) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > vocab) return;
    if (*status != 0u) { cdf[i] = 0; return; }
    if (greedy) { cdf[i] = i <= argmax[groups] ? 0ull : kMassTotal; return; }
    if (i == 0u) { cdf[i] = 0; return; }
    if (i == vocab) { cdf[i] = kMassTotal; return; }
    const uint32_t b = i / kFullBlock;
    const float before = (i % kFullBlock == 0u) ? offsets[b] : offsets[b] + prefix[i - 1u];
    cdf[i] = (uint64_t)fminf(fmaxf((before / offsets[groups]) * 4294967296.0f, 0.0f), 4294967296.0f);
}

// The token whose interval holds the proposal word; also checks the CDF is monotone and that no
// suppressed token carries mass (statuses 8 and 9 of gd_select).
__global__ void __launch_bounds__(256) full_select_kernel(const uint64_t* __restrict__ cdf, const float* __restrict__ scores, uint32_t vocab,
                                                          uint32_t word, int greedy, DraftReceiptHead* receipt, uint32_t* out_token_a,
                                                          uint32_t* out_token_b) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vocab || receipt->status != 0u) return;
    const uint64_t begin = cdf[i], end = cdf[i + 1u];
    if (begin > end || end > kMassTotal) atomicMax(&receipt->status, 8u);
    if (begin < end && !greedy && !(scores[i] > -INFINITY)) { atomicMax(&receipt->status, 9u); return; }
    if ((uint64_t)word >= begin && (uint64_t)word < end) {
        receipt->token = i;
        if (out_token_a) *out_token_a = i;
        if (out_token_b) *out_token_b = i;
    }
}

__global__ void full_receipt_init_kernel(DraftReceiptHead* receipt, uint32_t word, int keep_status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (!keep_status || receipt->status == 20u) receipt->status = 0u;
    receipt->count = 0xffffffffu;             // marks a full-vocabulary receipt
    receipt->token = 0xffffffffu;
    receipt->word = word;
}

__global__ void full_gather_kernel(const uint64_t* __restrict__ cdf, uint32_t vocab, const uint32_t* __restrict__ tokens, uint32_t count,
                                   uint64_t* __restrict__ intervals) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t token = tokens[i];
    const bool inside = token < vocab;
    intervals[2u * i] = inside ? cdf[token] : 0ull;
    intervals[2u * i + 1u] = inside ? cdf[token + 1u] : 0ull;
}

static uint32_t full_groups(uint32_t vocab) { return (vocab + kFullBlock - 1u) / kFullBlock; }
static uint32_t full_sorted_capacity(uint32_t vocab) { return (vocab + kFullTile - 1u) / kFullTile * kFullTile; }
static size_t align256(size_t v) { return (v + 255u) & ~(size_t)255u; }

struct FullLayout {
    size_t keys_a, keys_b, prefix, totals, offsets, maxima, argmax, cdf, gather_tokens, gather_out, total;
};
static FullLayout full_layout(uint32_t vocab) {
    const uint32_t groups = full_groups(vocab), capacity = full_sorted_capacity(vocab);
    FullLayout l {};
    size_t at = 0;
    l.keys_a = at; at += align256((size_t)capacity * 8u);
    l.keys_b = at; at += align256((size_t)capacity * 8u);
    l.prefix = at; at += align256((size_t)groups * kFullBlock * 4u);
    l.totals = at; at += align256((size_t)groups * 4u);
    l.offsets = at; at += align256((size_t)(groups + 1u) * 4u);
    l.maxima = at; at += align256((size_t)(groups + 1u) * 4u);
    l.argmax = at; at += align256((size_t)(groups + 1u) * 4u);
    l.cdf = at; at += align256((size_t)(vocab + 1u) * 8u);
    l.gather_tokens = at; at += align256(257u * 4u);
    l.gather_out = at; at += align256(257u * 16u);
    l.total = at;
    return l;
}

size_t draft_full_workspace_bytes(uint32_t vocab) { return full_layout(vocab).total; }

// Builds the full law from processed scores (overwritten by the filter) and selects the drafted token.
// `receipt_dev` receives status / count = 0xffffffff / token / word; the CDF stays in `workspace`.
int launch_draft_law_full(float* scores, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                          uint32_t word, void* workspace, void* receipt_dev, bool keep_status, uint32_t* out_token_a,
                          uint32_t* out_token_b, cudaStream_t stream) {
    if (!scores || !workspace || !receipt_dev || vocab == 0) return fail(GF_ERR_INVALID, "full draft law: null argument");
    const FullLayout l = full_layout(vocab);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    uint64_t* keys_a = reinterpret_cast<uint64_t*>(base + l.keys_a);
    uint64_t* keys_b = reinterpret_cast<uint64_t*>(base + l.keys_b);
    float* prefix = reinterpret_cast<float*>(base + l.prefix);
    float* totals = reinterpret_cast<float*>(base + l.totals);
    float* offsets = reinterpret_cast<float*>(base + l.offsets);
    float* maxima = reinterpret_cast<float*>(base + l.maxima);
    uint32_t* argmax = reinterpret_cast<uint32_t*>(base + l.argmax);
    uint64_t* cdf = reinterpret_cast<uint64_t*>(base + l.cdf);
    DraftReceiptHead* receipt = static_cast<DraftReceiptHead*>(receipt_dev);
    const uint32_t groups = full_groups(vocab), padded = groups * kFullBlock, capacity = full_sorted_capacity(vocab);
    const bool greedy = temperature == 0.0f;
    GF_TRY(launch_kernel(full_receipt_init_kernel, dim3(1), dim3(32), 0, stream, false, receipt, word, keep_status ? 1 : 0));
    if (!greedy && (top_k != 0u || top_p < 1.0f || min_p > 0.0f)) {
        GF_TRY(launch_kernel(full_sort_tile_kernel, dim3(capacity / kFullTile), dim3(1024), 0, stream, false, (const float*)scores, vocab, keys_a));
        uint64_t *in = keys_a, *out = keys_b;
        for (uint32_t width = kFullTile; width < capacity; width *= 2u) {
            GF_TRY(launch_kernel(full_merge_kernel, dim3((capacity + 255u) / 256u), dim3(256), 0, stream, false, (const uint64_t*)in, out, width, capacity));
            std::swap(in, out);
        }
        GF_TRY(launch_kernel(full_filter_prefix_kernel, dim3(groups), dim3(kFullBlock), 0, stream, false, (const uint64_t*)in, vocab, padded, top_k, prefix, totals));
        GF_TRY(launch_kernel(full_offsets_kernel, dim3(1), dim3(32), 0, stream, false, (const float*)totals, groups, offsets, &receipt->status, 0u));
        GF_TRY(launch_kernel(full_filter_apply_kernel, dim3((padded + 255u) / 256u), dim3(256), 0, stream, false, (const uint64_t*)in, vocab, padded,
                             groups, top_k, top_p, min_p, (const float*)prefix, (const float*)offsets, scores));
    }
    GF_TRY(launch_kernel(full_max_kernel, dim3(groups), dim3(kFullBlock), 0, stream, false, (const float*)scores, vocab, maxima, argmax));
    GF_TRY(launch_kernel(full_max_finish_kernel, dim3(1), dim3(32), 0, stream, false, maxima, argmax, groups, &receipt->status));
    if (!greedy) {
        GF_TRY(launch_kernel(full_prefix_kernel, dim3(groups), dim3(kFullBlock), 0, stream, false, (const float*)scores, vocab, groups, (const float*)maxima, prefix, totals));
        GF_TRY(launch_kernel(full_offsets_kernel, dim3(1), dim3(32), 0, stream, false, (const float*)totals, groups, offsets, &receipt->status, 7u));
    }
    GF_TRY(launch_kernel(full_cdf_kernel, dim3((vocab + 256u) / 256u), dim3(256), 0, stream, false, (const float*)prefix, (const float*)offsets,
                         (const uint32_t*)argmax, vocab, groups, greedy ? 1 : 0, (const uint32_t*)&receipt->status, cdf));
    return launch_kernel(full_select_kernel, dim3((vocab + 255u) / 256u), dim3(256), 0, stream, false, (const uint64_t*)cdf, (const float*)scores, vocab, word,
                         greedy ? 1 : 0, receipt, out_token_a, out_token_b);
}

// Reads the CDF intervals of `count` <= 257 tokens: uploads the ids, gathers on the device, downloads
// [begin, end) pairs and synchronises the stream.
int launch_draft_gather_full(void* workspace, uint32_t vocab, const uint32_t* tokens_host, uint32_t count, uint64_t* intervals_host,
                             cudaStream_t stream) {
    if (!workspace || !tokens_host || !intervals_host || count == 0 || count > 257u)
        return fail(GF_ERR_INVALID, "full draft gather: between 1 and 257 tokens");
    const FullLayout l = full_layout(vocab);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    uint32_t* tokens = reinterpret_cast<uint32_t*>(base + l.gather_tokens);
    uint64_t* out = reinterpret_cast<uint64_t*>(base + l.gather_out);
    GF_CUDA(cudaMemcpyAsync(tokens, tokens_host, count * sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
    GF_TRY(launch_kernel(full_gather_kernel, dim3(2), dim3(256), 0, stream, false, (const uint64_t*)(base + l.cdf), vocab, (const uint32_t*)tokens, count, out));
    GF_CUDA(cudaMemcpyAsync(intervals_host, out, (size_t)count * 16u, cudaMemcpyDeviceToHost, stream));
    GF_CUDA(cudaStreamSynchronize(stream));
    return GF_OK;
}

const uint64_t* draft_full_cdf(const void* workspace, uint32_t vocab) {
    return reinterpret_cast<const uint64_t*>(static_cast<const uint8_t*>(workspace) + full_layout(vocab).cdf);
}

}  // namespace gf
