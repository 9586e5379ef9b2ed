// Host sampler C entry points and the H1 draft -> verify -> accept / rollback cycle.
#include "model.cuh"
#include "sampler.hpp"

#include <algorithm>
#include <cstring>
#include <memory>
#include <random>
#include <vector>

namespace gf {

size_t draft_sampler_workspace_bytes(uint32_t vocab);
int launch_draft_sample(const float* logits, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                        float penalty, const uint32_t* history_host, uint32_t history_count, uint32_t word,
                        void* workspace, void* receipt_dev, uint32_t* out_token_a, uint32_t* out_token_b,
                        cudaStream_t stream, const uint32_t* history_request_dev);
size_t request_base_bytes();
int launch_request_rows(const void* base_dev, uint32_t root, const uint32_t* chain_dev, uint32_t first_row, uint32_t row_count,
                        void* requests_dev, cudaStream_t stream);
int launch_draft_resolve_overflow(uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p, uint32_t word,
                                  void* workspace, void* receipt_dev, uint32_t* out_token_a, uint32_t* out_token_b,
                                  cudaStream_t stream);
int launch_draft_gather(void* workspace, uint32_t vocab, const uint32_t* tokens_host, uint32_t count, uint64_t* intervals_host,
                        cudaStream_t stream);

#define GF_TRY(expr) do { const int gf_s_ = (expr); if (gf_s_ != GF_OK) return gf_s_; } while (0)

static SamplerOptions to_options(const gf_sampler_options& o) {
    SamplerOptions s;
    s.temperature = o.temperature; s.top_k = o.top_k; s.top_p = o.top_p; s.min_p = o.min_p;
    s.repetition_penalty = o.repetition_penalty; s.repetition_window = o.repetition_window; s.seed = o.seed;
    return s;
}

// Layouts shared with candidates.cu / draft_sampler.cu.
struct SelectionRequestRow { uint32_t retain, history_count, history[64]; };
struct CandidateRow { uint32_t status, count; TokenLogit candidates[384]; };
struct DraftReceiptRow { uint32_t status, count, token, word, ids[256]; uint64_t cdf[257]; };
struct RequestBaseRow { uint32_t top_k, window_limit, count, tokens[64]; };      // candidates.cu's RequestBase

static SelectionRequestRow to_request(const SelectionHistory& h) {
    SelectionRequestRow r {};
    r.retain = h.top_k + h.count;
    r.history_count = h.count;
    for (uint32_t i = 0; i < h.count; ++i) r.history[i] = h.tokens[i];
    return r;
}

// Looks the prepared target support up in the drafter's receipt (Gemma3DraftPlan::gather,
// gemma3_draft.mm:1528-1581): a token outside the draft support has q = 0.
static void gather(const DraftReceiptRow& receipt, const TokenDistribution& target, GatheredDraft& out) {
    auto interval = [&](uint32_t token, uint64_t& begin, uint64_t& end) {
        const uint32_t* first = receipt.ids;
        const uint32_t* last = receipt.ids + receipt.count;
        const uint32_t* found = std::lower_bound(first, last, token);
        if (found == last || *found != token) { begin = end = 0; return; }
        begin = receipt.cdf[found - first];
        end = receipt.cdf[found - first + 1];
    };
    out = GatheredDraft();
    out.proposal = receipt.token;
    uint64_t begin = 0, end = 0;
    interval(receipt.token, begin, end);
    out.proposal_mass = end - begin;
    out.proposal_cdf_begin = begin;
    out.count = target.count;
    for (uint32_t i = 0; i < target.count; ++i) {
        interval(target.values[i].token, begin, end);
        out.target_mass[i] = end - begin;
    }
}

// Drafts per verification tile of a chain of h <= 7 drafts (at most four tiles): all in one, or the reference's
// conditional partition (make_registered_conditional_chain_schedule, speculative_controller.cpp:596-604, and the
// pairs of chain_chat.mm:78-86 for lengths it does not register).
static uint32_t verification_partition(uint32_t h, bool conditional, uint32_t (&parts)[4]) {
    parts[0] = h; parts[1] = parts[2] = parts[3] = 0;
    if (!conditional || h < 2u) return 1;
    if (h == 3u) { parts[0] = 2; parts[1] = 1; return 2; }
    if (h == 4u) { parts[0] = 2; parts[1] = 2; return 2; }
    if (h == 7u) { parts[0] = 4; parts[1] = 3; return 2; }
    uint32_t count = 0;
    for (uint32_t remaining = h; remaining && count < 4u;) { const uint32_t take = std::min(remaining, 2u); parts[count++] = take; remaining -= take; }
    return count;
}

class H1Engine {
public:
    H1Engine(Model& target, Model* draft, const gf_h1_options& options)
        : target_(target), draft_(draft), options_(options), sampler_(to_options(options.sampler)), schedule_(options.schedule_seed) {}
    ~H1Engine() {
        for (void* ws : draft_ws_) if (ws) cudaFree(ws);
        if (receipt_dev_) cudaFree(receipt_dev_);
        if (base_dev_) cudaFree(base_dev_);
        if (base_host_) cudaFreeHost(base_host_);
        if (results_host_) cudaFreeHost(results_host_);
        if (receipt_host_) cudaFreeHost(receipt_host_);
        for (cudaEvent_t e : step_done_) if (e) cudaEventDestroy(e);
        if (draft_done_) cudaEventDestroy(draft_done_);
    }

    int init() {
        GF_TRY(validate_options(sampler_.options()));
        horizon_ = options_.horizon == 0 ? 1u : options_.horizon;
        if (options_.speculative) {
            if (!draft_) return fail(GF_ERR_INVALID, "speculative decoding needs a drafter plan");
            if (draft_->config().vocab != target_.token_vocab()) return fail(GF_ERR_INVALID, "drafter and target vocabularies differ (direct token ids are required)");
            if (horizon_ > kMaxHorizon) return fail(GF_ERR_INVALID, "horizon %u exceeds %u (a verification pass holds at most %d rows)", horizon_, kMaxHorizon, GF_MAX_ROWS);
            VerifyTile tiles[kMaxTiles];
            const uint32_t tile_count = verification_tiles(horizon_, tiles);
            uint32_t widest = 0;
            for (uint32_t t = 0; t < tile_count; ++t) widest = std::max(widest, tiles[t].rows);
            if (target_.config().row_capacity < widest)
                return fail(GF_ERR_INVALID, "horizon %u needs %u rows per target pass (the plan was built for %u)", horizon_, widest, target_.config().row_capacity);
            if (draft_->config().row_capacity < std::max(2u, horizon_))
                return fail(GF_ERR_INVALID, "horizon %u needs %u rows per drafter pass (the plan was built for %u)", horizon_, std::max(2u, horizon_), draft_->config().row_capacity);
            const size_t ws_bytes = draft_sampler_workspace_bytes(draft_->config().vocab);
            draft_ws_.assign(horizon_, nullptr);
            for (uint32_t j = 0; j < horizon_; ++j) GF_CUDA(cudaMalloc(&draft_ws_[j], ws_bytes));     // one per drafted token: an overflowing step is resolved from its own scores
            GF_CUDA(cudaMalloc(&receipt_dev_, horizon_ * sizeof(DraftReceiptRow)));
            GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&receipt_host_), horizon_ * sizeof(DraftReceiptRow), cudaHostAllocDefault));
            GF_CUDA(cudaEventCreateWithFlags(&draft_done_, cudaEventDisableTiming));
            if (request_base_bytes() != sizeof(RequestBaseRow)) return fail(GF_ERR_STATE, "selection base layouts differ");
            GF_CUDA(cudaMalloc(&base_dev_, sizeof(RequestBaseRow)));
            GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&base_host_), sizeof(RequestBaseRow), cudaHostAllocDefault));
            step_done_.assign(horizon_, nullptr);
            for (uint32_t j = 0; j < horizon_; ++j) GF_CUDA(cudaEventCreateWithFlags(&step_done_[j], cudaEventDisableTiming));
        }
        GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&results_host_), (size_t)(horizon_ + 1u) * sizeof(CandidateRow), cudaHostAllocDefault));
        return GF_OK;
    }

    int prefill(const uint32_t* tokens, uint32_t count) {
        if (!tokens || count == 0) return fail(GF_ERR_INVALID, "empty prompt");
        GF_TRY(target_.reset());
        if (draft_ && options_.speculative) GF_TRY(draft_->reset());
        sampler_ = Sampler(to_options(options_.sampler));
        stats_ = gf_h1_stats();
        records_.clear();
        pending_ = false;
        draft_exhausted_ = false;
        GF_TRY(target_.prefill(tokens, count));
        if (draft_ && options_.speculative) GF_TRY(draft_->prefill(tokens, count));      // the drafter ingests the same prompt
        sampler_.observe(tokens, count);
        // First token: ordinary sample from the prompt's last row.
        const uint32_t last_row = target_.prefill_logits_row();
        const SelectionHistory request = sampler_.request_after(nullptr, 0);
        GF_TRY(select_and_read(request, last_row));
        GF_TRY(sampler_.sample(results_host_[0].candidates, results_host_[0].count, request, root_));
        has_root_ = true;
        first_emitted_ = false;
        return GF_OK;
    }

    int generate(uint32_t max_tokens, uint32_t* out, uint32_t* out_count, uint32_t max_steps = 0xffffffffu) {
        if (!has_root_) return fail(GF_ERR_STATE, "generate needs a prefilled prompt");
        if (!out || !out_count) return fail(GF_ERR_INVALID, "null output");
        uint32_t produced = 0, steps = 0;
        auto emit = [&](uint32_t token) { if (produced < max_tokens) out[produced++] = token; ++stats_.emitted_tokens; };
        if (!first_emitted_ && max_tokens) { emit(root_); first_emitted_ = true; }
        while (produced < max_tokens && steps < max_steps) {
            ++steps;
            const uint32_t room = target_.config().context - target_.position();
            if (room < 2) break;                                            // context exhausted
            // A cycle with h drafts emits up to h + 1 tokens, caches up to h + 1 rows and leaves one more
            // token to be cached later; the drafter caches its pending token, the root and h - 1 drafts.
            uint32_t h = 0;
            if (options_.speculative && !draft_exhausted_) {
                h = horizon_;
                h = std::min(h, max_tokens - produced - 1u);
                h = std::min(h, room - 2u);
                const uint32_t draft_room = draft_->config().context - draft_->position();
                h = draft_room >= 3u ? std::min(h, draft_room - 2u) : 0u;
            }
            if (h >= 1u) {
                uint32_t tokens[kMaxHorizon + 1u];
                uint32_t n = 0;
                const int status = cycle(h, tokens, n);
                if (status != GF_OK) return status;
                for (uint32_t i = 0; i < n; ++i) emit(tokens[i]);
            } else {
                uint32_t token = 0;
                GF_TRY(ordinary_step(token));
                emit(token);
            }
        }
        *out_count = produced;
        return GF_OK;
    }

    const gf_h1_stats& stats() const { return stats_; }
    void reseed_schedule(uint64_t seed) { schedule_.seed(seed); }
    const std::vector<gf_h1_cycle_record>& records() const { return records_; }

private:
    static constexpr uint32_t kMaxHorizon = GF_MAX_ROWS - 1;
    static constexpr uint32_t kMaxTiles = 4;

    // How a cycle's h drafts are verified.  Unconditional: one pass of h + 1 rows.  Conditional
    // (chain_chat.mm:63-88): a cascade of passes, each run only when every draft before it was accepted; a tile
    // tests `edges` drafts with `edges` rows, the last one carries one more row for the token that follows a
    // fully accepted chain.  The partitions are the reference's registered ones
    // (make_registered_conditional_chain_schedule, speculative_controller.cpp:590-623: 3 = 2 + 1, 4 = 2 + 2,
    // 7 = 4 + 3) and its pairs for other lengths.
    struct VerifyTile { uint32_t edges, rows; };
    uint32_t verification_tiles(uint32_t h, VerifyTile (&tiles)[kMaxTiles]) const {
        uint32_t parts[kMaxTiles];
        const uint32_t count = verification_partition(h, options_.conditional != 0, parts);
        for (uint32_t t = 0; t < count; ++t) tiles[t] = VerifyTile{parts[t], parts[t] + (t + 1u == count ? 1u : 0u)};
        return count;
    }

    // Selection for one target row through a single-row request, then readback.
    int select_and_read(const SelectionHistory& request, uint32_t logits_row) {
        // The selection kernels read row `r` of the logits for request r; a lone request for a
        // later row is expressed by padding the earlier rows with cheap greedy requests.
        std::vector<SelectionRequestRow> rows(logits_row + 1u);
        for (uint32_t r = 0; r < logits_row; ++r) { rows[r] = SelectionRequestRow(); rows[r].retain = 1; }
        rows[logits_row] = to_request(request);
        GF_TRY(target_.select(rows.data(), logits_row + 1u));
        std::vector<CandidateRow> results(logits_row + 1u);
        GF_TRY(target_.read_candidates(results.data(), logits_row + 1u));
        results_host_[0] = results[logits_row];
        if (results_host_[0].status) return fail(GF_ERR_NUMERIC, "candidate selection reported status %u", results_host_[0].status);
        return GF_OK;
    }

    // Ordinary decode: one target row, sample, publish (run_gemma3_resident_decode path).
    int ordinary_step(uint32_t& token) {
        const uint32_t r = root_;
        GF_TRY(target_.forward(&r, 1, kForwardLogits));
        const uint32_t suffix[1] = {r};
        const SelectionHistory request = sampler_.request_after(suffix, 1);
        const SelectionRequestRow row = to_request(request);
        GF_TRY(target_.select(&row, 1));
        GF_TRY(target_.publish(1));
        if (draft_ && options_.speculative && !draft_exhausted_) {           // keep the drafter's timeline in step
            uint32_t tokens[2];
            uint32_t rows = 0;
            if (pending_) tokens[rows++] = pending_token_;
            tokens[rows++] = r;
            if (draft_->config().context - draft_->position() < rows) {
                // The drafter's context is full before the target's: decoding goes on without it
                // (generate() no longer speculates once fewer than three drafter rows remain).
                draft_exhausted_ = true;
            } else {
                GF_TRY(draft_->forward(tokens, rows, 0));
                GF_TRY(draft_->publish(rows));
            }
            pending_ = false;
        }
        GF_TRY(target_.read_candidates(results_host_, 1));
        if (results_host_[0].status) return fail(GF_ERR_NUMERIC, "candidate selection reported status %u", results_host_[0].status);
        sampler_.observe(&r, 1);
        const SelectionHistory now = sampler_.request_after(nullptr, 0);
        GF_TRY(sampler_.sample(results_host_[0].candidates, results_host_[0].count, now, token));
        root_ = token;
        ++stats_.ordinary_steps;
        return GF_OK;
    }

    // Drafter steps first..h-1 of a cycle.  Step 0 forwards [pending?, root]; step j > 0 forwards the
    // token step j - 1 drafted, which the sampler left in the drafter's device token buffer.  Each step
    // publishes its rows, samples the next draft into row j + 1 of the target's token buffer and sends
    // its receipt to the host.  `resolve` = step `first` has already run and reported a support larger
    // than the compact law holds: its law is rebuilt over the whole vocabulary from its own scores.
    int draft_steps(uint32_t first, uint32_t h, bool resolve, const uint32_t* words, uint32_t* chain, uint32_t (&draft_position)[kMaxHorizon]) {
        const SamplerOptions& so = sampler_.options();
        const bool penalised = so.repetition_penalty != 1.0f;
        const uint32_t vocab = draft_->config().vocab;
        for (uint32_t j = first; j < h; ++j) {
            uint32_t* next_draft_token = j + 1u < h ? draft_->tokens_dev() : nullptr;
            DraftReceiptRow* receipt = static_cast<DraftReceiptRow*>(receipt_dev_) + j;
            if (j == first && resolve) {
                GF_TRY(launch_draft_resolve_overflow(vocab, so.temperature, so.top_k, so.top_p, so.min_p, words[j], draft_ws_[j], receipt,
                                                     target_.tokens_dev() + j + 1u, next_draft_token, draft_->stream()));
                stats_.sampler_launches += 16;
                ++stats_.full_law_proposals;
            } else {
                uint32_t rows = 1;
                if (j == 0) {
                    uint32_t tokens[2];
                    rows = 0;
                    if (pending_) tokens[rows++] = pending_token_;
                    tokens[rows++] = chain[0];
                    GF_TRY(draft_->forward(tokens, rows, kForwardLogits));
                } else {
                    GF_TRY(draft_->forward(nullptr, 1, kForwardLogits | kForwardDeviceTokens));
                }
                GF_TRY(draft_->publish(rows));
                draft_position[j] = draft_->position();
                // With a repetition penalty the window names the root and the earlier drafts, which only the
                // device knows: row j of the target's request rows is written here, on the device, and the
                // drafter's sampler reads its history from it (the row is also the target's request for row j).
                const uint32_t* history_row = nullptr;
                if (penalised) {
                    GF_TRY(launch_request_rows(base_dev_, chain[0], target_.tokens_dev(), j, 1, target_.requests_dev(), draft_->stream()));
                    history_row = static_cast<const uint32_t*>(target_.requests_dev()) + (size_t)j * (sizeof(SelectionRequestRow) / 4u);
                    stats_.sampler_launches += 1;
                }
                GF_TRY(launch_draft_sample(draft_->logits_dev() + (size_t)(rows - 1u) * vocab, vocab, so.temperature, so.top_k, so.top_p,
                                           so.min_p, so.repetition_penalty, nullptr, 0, words[j], draft_ws_[j],
                                           receipt, target_.tokens_dev() + j + 1u, next_draft_token, draft_->stream(), history_row));
                stats_.sampler_launches += 3;
            }
            GF_CUDA(cudaMemcpyAsync(receipt_host_ + j, receipt, sizeof(DraftReceiptRow), cudaMemcpyDeviceToHost, draft_->stream()));
            GF_CUDA(cudaEventRecord(step_done_[j], draft_->stream()));
        }
        if (penalised) {      // the request of the row behind the last draft
            GF_TRY(launch_request_rows(base_dev_, chain[0], target_.tokens_dev(), h, 1, target_.requests_dev(), draft_->stream()));
            stats_.sampler_launches += 1;
        }
        GF_CUDA(cudaEventRecord(draft_done_, draft_->stream()));
        return GF_OK;
    }

    // Draft masses on the prepared target support.  A compact receipt is searched on the host; a
    // full-vocabulary receipt keeps its CDF on the device and is read through a small gather.
    int gather_step(uint32_t j, const TokenDistribution& target, GatheredDraft& out) {
        const DraftReceiptRow& receipt = receipt_host_[j];
        if (receipt.count != 0xffffffffu) { gather(receipt, target, out); return GF_OK; }
        uint32_t tokens[kSamplerMaxTopK + 1u];
        uint64_t intervals[2u * (kSamplerMaxTopK + 1u)];
        for (uint32_t i = 0; i < target.count; ++i) tokens[i] = target.values[i].token;
        tokens[target.count] = receipt.token;
        GF_TRY(launch_draft_gather(draft_ws_[j], draft_->config().vocab, tokens, target.count + 1u, intervals, draft_->stream()));
        out = GatheredDraft();
        out.proposal = receipt.token;
        out.proposal_cdf_begin = intervals[2u * target.count];
        out.proposal_mass = intervals[2u * target.count + 1u] - intervals[2u * target.count];
        out.count = target.count;
        for (uint32_t i = 0; i < target.count; ++i) out.target_mass[i] = intervals[2u * i + 1u] - intervals[2u * i];
        return GF_OK;
    }

    // One speculative cycle with h >= 1 drafts (ChainChatVerifier::run with one tile of h proposals and
    // h + 1 rows, chain_chat.mm:245-543; h = 1 is the H1 cycle).  On entry root_ is selected but not yet
    // in any cache.
    int cycle(uint32_t h, uint32_t* emitted, uint32_t& emitted_count) {
        const SamplerOptions& so = sampler_.options();
        const bool penalised = so.repetition_penalty != 1.0f;
        uint32_t chain[kMaxHorizon + 1u] = {root_};        // root, then the drafted tokens as the host learns them
        uint32_t words[kMaxHorizon];
        sampler_.preview_proposal_words(words, h);
        uint32_t draft_position[kMaxHorizon] = {};           // the drafter's position after step j
        const uint32_t r = root_;
        uint32_t first = 0;
        bool resolve = false;
        VerifyTile tiles[kMaxTiles];
        const uint32_t tile_count = verification_tiles(h, tiles);
        if (penalised) {      // the sampler's repetition window, for the request rows the device writes
            const std::vector<uint32_t>& window = sampler_.history();
            base_host_->top_k = so.temperature == 0.0f ? 1u : so.top_k;
            base_host_->window_limit = so.repetition_window;
            base_host_->count = (uint32_t)window.size();
            for (size_t i = 0; i < window.size() && i < 64u; ++i) base_host_->tokens[i] = window[i];
            GF_CUDA(cudaMemcpyAsync(base_dev_, base_host_, sizeof(RequestBaseRow), cudaMemcpyHostToDevice, draft_->stream()));
        }
        for (;;) {
            GF_TRY(draft_steps(first, h, resolve, words, chain, draft_position));
            // --- target: verify rows [r, x1 .. xh] in one pass; the drafts never visit the host on this path.
            GF_TRY(target_.set_device_token(0, r));
            GF_CUDA(cudaStreamWaitEvent(target_.stream(), draft_done_, 0));
            GF_TRY(target_.forward(nullptr, tiles[0].rows, kForwardLogits | kForwardDeviceTokens));
            ++stats_.verify_passes;
            if (penalised) {      // every row's request names the drafts before it: the drafter's stream wrote them
                GF_TRY(target_.select_device(tiles[0].rows));
            } else {
                SelectionRequestRow requests[kMaxHorizon + 1u];
                requests[0] = to_request(sampler_.request_after(chain, 1));
                for (uint32_t i = 1; i < tiles[0].rows; ++i) requests[i] = requests[0];
                GF_TRY(target_.select(requests, tiles[0].rows));
            }
            GF_TRY(target_.read_candidates(results_host_, tiles[0].rows));    // the cycle's one synchronisation (one more per further tile)
            GF_CUDA(cudaEventSynchronize(draft_done_));
            // A step whose support outgrew the compact law (status 20) drafted nothing usable: rebuild its
            // law over the whole vocabulary, redo the steps behind it and verify again.  Nothing of the
            // first attempt was published on the target, and no random stream has moved.
            uint32_t overflow = h;
            for (uint32_t j = first; j < h && overflow == h; ++j) if (receipt_host_[j].status == 20u) overflow = j;
            if (overflow == h) break;
            GF_TRY(draft_->truncate(draft_position[overflow]));
            first = overflow;
            resolve = true;
            ++stats_.fallback_cycles;
        }
        for (uint32_t j = 0; j < h; ++j) {
            const DraftReceiptRow& receipt = receipt_host_[j];
            if (receipt.status != 0 || receipt.token >= target_.token_vocab())
                return fail(GF_ERR_NUMERIC, "drafter sampler reported status %u at depth %u", receipt.status, j);
            chain[j + 1u] = receipt.token;
            if (receipt.count == 0xffffffffu && !resolve) ++stats_.full_law_proposals;
        }
        auto check_rows = [&](uint32_t rows) {
            for (uint32_t i = 0; i < rows; ++i)
                if (results_host_[i].status) return fail(GF_ERR_NUMERIC, "candidate selection reported status %u in row %u", results_host_[i].status, i);
            return (int)GF_OK;
        };
        GF_TRY(check_rows(tiles[0].rows));
        ++stats_.cycles;
        stats_.drafted_tokens += h;
        // --- acceptance (host, double precision), draft by draft until the first rejection.
        uint32_t matched = 0;
        uint32_t corrected = 0;
        uint32_t tile = 0, tile_start = 0;                   // the tile whose candidates are on the host, and its first draft
        for (uint32_t i = 0; i < h; ++i) {
            if (i == tile_start + tiles[tile].edges) {
                // Every draft of the tile was accepted: its rows are final, and the next tile's pass runs on the
                // tokens the host now knows (rows chain[i] .., which continue the published cache).
                GF_TRY(target_.publish(tiles[tile].edges));
                tile_start = i;
                ++tile;
                const uint32_t rows = tiles[tile].rows;
                GF_TRY(target_.forward(chain + tile_start, rows, kForwardLogits));
                ++stats_.verify_passes;
                SelectionRequestRow requests[kMaxHorizon + 1u];
                for (uint32_t k = 0; k < rows; ++k)
                    requests[k] = penalised || k == 0 ? to_request(sampler_.request_after(chain, tile_start + k + 1u)) : requests[0];
                GF_TRY(target_.select(requests, rows));
                GF_TRY(target_.read_candidates(results_host_, rows));
                GF_TRY(check_rows(rows));
            }
            const CandidateRow& row = results_host_[i - tile_start];
            const SelectionHistory request = sampler_.request_after(chain, i + 1u);
            TokenDistribution prepared;
            GF_TRY(prepare_distribution(row.candidates, row.count, so, request, prepared));
            GatheredDraft gathered;
            GF_TRY(gather_step(i, prepared, gathered));
            SpeculativeOutcome outcome;
            const int law_status = sampler_.sample_speculative(gathered, row.candidates, row.count, request, outcome);
            if (options_.record_cycles) {
                gf_h1_cycle_record record {};
                record.root = chain[i]; record.proposal = chain[i + 1u]; record.word = words[i]; record.candidate_count = row.count;
                std::memcpy(record.candidates, row.candidates, sizeof(TokenLogit) * row.count);
                record.draft.proposal = gathered.proposal; record.draft.count = gathered.count;
                record.draft.proposal_mass = gathered.proposal_mass; record.draft.proposal_cdf_begin = gathered.proposal_cdf_begin;
                std::memcpy(record.draft.target_mass, gathered.target_mass.data(), sizeof(uint64_t) * 256);
                record.token = outcome.token; record.accepted = outcome.accepted; record.target_draws = outcome.target_draws;
                record.status = law_status; record.depth = i; record.horizon = h;
                if (records_.size() < 65536) records_.push_back(record);
            }
            if (law_status != GF_OK) return law_status;
            bool accepted = outcome.accepted;
            corrected = outcome.token;
            if (options_.forced_schedule) {
                std::bernoulli_distribution coin(options_.forced_accept_probability);
                const bool forced = coin(schedule_);
                if (forced == outcome.accepted) ++stats_.law_agreements;
                if (!forced && outcome.accepted) {
                    // Scheduled rejection of a proposal the law accepted: continue from an ordinary
                    // sample of the same row, so the control flow (one row published, no carry) matches.
                    GF_TRY(sampler_.sample(row.candidates, row.count, request, corrected));
                }
                accepted = forced;
            }
            if (!accepted) break;
            ++matched;
        }
        stats_.accepted_tokens += matched;
        GF_TRY(target_.publish(matched - tile_start + 1u));   // rows behind the first rejection are never published: the rollback
        sampler_.observe(chain, matched + 1u);
        for (uint32_t i = 0; i < matched; ++i) emitted[i] = chain[i + 1u];
        if (matched == h) {
            ++stats_.accepted;
            const SelectionHistory now = sampler_.request_after(nullptr, 0);
            uint32_t next = 0;
            GF_TRY(sampler_.sample(results_host_[h - tile_start].candidates, results_host_[h - tile_start].count, now, next));
            pending_ = true;                              // the last draft is selected but not yet forwarded by the drafter
            pending_token_ = chain[h];
            root_ = next;
            emitted[matched] = next;
        } else {
            ++stats_.rejected;
            // The drafter has cached the root and drafts 1 .. h-1; it keeps the accepted ones.
            if (matched + 1u < h) GF_TRY(draft_->truncate(draft_position[matched]));
            pending_ = false;                             // the rejected draft was never forwarded
            root_ = corrected;
            emitted[matched] = corrected;
        }
        emitted_count = matched + 1u;
        return GF_OK;
    }

    Model& target_;
    Model* draft_;
    gf_h1_options options_;
    Sampler sampler_;
    std::mt19937_64 schedule_;
    gf_h1_stats stats_ {};
    std::vector<gf_h1_cycle_record> records_;
    std::vector<void*> draft_ws_;
    void* receipt_dev_ = nullptr;
    void* base_dev_ = nullptr;
    RequestBaseRow* base_host_ = nullptr;
    CandidateRow* results_host_ = nullptr;
    DraftReceiptRow* receipt_host_ = nullptr;
    cudaEvent_t draft_done_ = nullptr;
    std::vector<cudaEvent_t> step_done_;
    uint32_t horizon_ = 1;
    uint32_t root_ = 0, pending_token_ = 0;
    bool has_root_ = false, pending_ = false, first_emitted_ = false, draft_exhausted_ = false;
};

}  // namespace gf

using namespace gf;

struct gf_sampler { Sampler impl; explicit gf_sampler(const SamplerOptions& o) : impl(o) {} };
struct gf_h1 { H1Engine impl; gf_h1(Model& t, Model* d, const gf_h1_options& o) : impl(t, d, o) {} };

extern "C" {

int gf_sampler_create(const gf_sampler_options* options, gf_sampler** out_sampler) {
    if (!options || !out_sampler) return fail(GF_ERR_INVALID, "gf_sampler_create: null argument");
    const SamplerOptions o = to_options(*options);
    const int status = validate_options(o);
    if (status != GF_OK) return status;
    *out_sampler = new gf_sampler(o);
    return GF_OK;
}
int gf_sampler_destroy(gf_sampler* sampler) { delete sampler; return GF_OK; }
int gf_sampler_observe(gf_sampler* s, const uint32_t* tokens, uint32_t count) {
    if (!s || (!tokens && count)) return fail(GF_ERR_INVALID, "gf_sampler_observe: null argument");
    s->impl.observe(tokens, count);
    return GF_OK;
}
int gf_sampler_preview_proposal_word(const gf_sampler* s, uint32_t* out_word) {
    if (!s || !out_word) return fail(GF_ERR_INVALID, "null argument");
    *out_word = s->impl.preview_proposal_word();
    return GF_OK;
}
int gf_h1_verification_schedule(uint32_t horizon, int conditional, uint32_t* out_drafts, uint32_t* out_rows, uint32_t* out_tiles) {
    if (!out_drafts || !out_rows || !out_tiles || horizon == 0 || horizon > GF_MAX_ROWS - 1) return fail(GF_ERR_INVALID, "a horizon between 1 and %d", GF_MAX_ROWS - 1);
    uint32_t parts[4];
    const uint32_t count = verification_partition(horizon, conditional != 0, parts);
    for (uint32_t t = 0; t < count; ++t) { out_drafts[t] = parts[t]; out_rows[t] = parts[t] + (t + 1u == count ? 1u : 0u); }
    *out_tiles = count;
    return GF_OK;
}
int gf_sampler_preview_proposal_words(const gf_sampler* s, uint32_t count, uint32_t* out_words) {
    if (!s || !out_words || count == 0 || count > 23u) return fail(GF_ERR_INVALID, "between 1 and 23 proposal words");
    s->impl.preview_proposal_words(out_words, count);
    return GF_OK;
}
int gf_sampler_prepare(const gf_sampler* s, const gf_token_logit* candidates, uint32_t count, const uint32_t* suffix,
                       uint32_t suffix_count, uint32_t* out_tokens, double* out_weights, uint32_t* out_count,
                       double* out_total_weight) {
    if (!s || !out_tokens || !out_weights || !out_count || !out_total_weight) return fail(GF_ERR_INVALID, "null argument");
    TokenDistribution d;
    const SelectionHistory request = s->impl.request_after(suffix, suffix_count);
    const int status = prepare_distribution(reinterpret_cast<const TokenLogit*>(candidates), count, s->impl.options(), request, d);
    if (status != GF_OK) return status;
    for (uint32_t i = 0; i < d.count; ++i) { out_tokens[i] = d.values[i].token; out_weights[i] = d.values[i].weight; }
    *out_count = d.count;
    *out_total_weight = d.total_weight;
    return GF_OK;
}
int gf_sampler_sample(gf_sampler* s, const gf_token_logit* candidates, uint32_t count, const uint32_t* suffix,
                      uint32_t suffix_count, uint32_t* out_token) {
    if (!s || !out_token) return fail(GF_ERR_INVALID, "null argument");
    const SelectionHistory request = s->impl.request_after(suffix, suffix_count);
    return s->impl.sample(reinterpret_cast<const TokenLogit*>(candidates), count, request, *out_token);
}
int gf_sampler_sample_speculative(gf_sampler* s, const gf_gathered_draft* draft, const gf_token_logit* candidates,
                                  uint32_t count, const uint32_t* suffix, uint32_t suffix_count, uint32_t* out_token,
                                  int* out_accepted, uint32_t* out_target_draws) {
    if (!s || !draft || !out_token || !out_accepted) return fail(GF_ERR_INVALID, "null argument");
    if (draft->count > kSamplerMaxTopK) return fail(GF_ERR_INVALID, "gathered support exceeds 256");
    GatheredDraft g;
    g.proposal = draft->proposal; g.proposal_mass = draft->proposal_mass; g.proposal_cdf_begin = draft->proposal_cdf_begin;
    g.count = draft->count;
    for (uint32_t i = 0; i < draft->count; ++i) g.target_mass[i] = draft->target_mass[i];
    const SelectionHistory request = s->impl.request_after(suffix, suffix_count);
    SpeculativeOutcome outcome;
    const int status = s->impl.sample_speculative(g, reinterpret_cast<const TokenLogit*>(candidates), count, request, outcome);
    if (status != GF_OK) return status;
    *out_token = outcome.token;
    *out_accepted = outcome.accepted ? 1 : 0;
    if (out_target_draws) *out_target_draws = outcome.target_draws;
    return GF_OK;
}

int gf_h1_create(gf_model* target, gf_model* draft, const gf_h1_options* options, gf_h1** out_engine) {
    if (!target || !options || !out_engine) return fail(GF_ERR_INVALID, "gf_h1_create: null argument");
    std::unique_ptr<gf_h1> engine(new gf_h1(target->impl, draft ? &draft->impl : nullptr, *options));
    const int status = engine->impl.init();
    if (status != GF_OK) return status;
    *out_engine = engine.release();
    return GF_OK;
}
int gf_h1_destroy(gf_h1* engine) { delete engine; return GF_OK; }
int gf_h1_prefill(gf_h1* e, const uint32_t* tokens_host, uint32_t count) {
    return e ? e->impl.prefill(tokens_host, count) : fail(GF_ERR_INVALID, "null engine");
}
int gf_h1_generate(gf_h1* e, uint32_t max_tokens, uint32_t* out_tokens, uint32_t* out_count) {
    return e ? e->impl.generate(max_tokens, out_tokens, out_count) : fail(GF_ERR_INVALID, "null engine");
}
int gf_h1_generate_steps(gf_h1* e, uint32_t steps, uint32_t max_tokens, uint32_t* out_tokens, uint32_t* out_count) {
    return e ? e->impl.generate(max_tokens, out_tokens, out_count, steps) : fail(GF_ERR_INVALID, "null engine");
}
int gf_h1_stats_read(const gf_h1* e, gf_h1_stats* out_stats) {
    if (!e || !out_stats) return fail(GF_ERR_INVALID, "null argument");
    *out_stats = e->impl.stats();
    return GF_OK;
}
int gf_h1_reseed_schedule(gf_h1* e, uint64_t seed) {
    if (!e) return fail(GF_ERR_INVALID, "null engine");
    e->impl.reseed_schedule(seed);
    return GF_OK;
}
uint32_t gf_h1_cycle_record_count(const gf_h1* e) { return e ? (uint32_t)e->impl.records().size() : 0; }
int gf_h1_cycle_record_read(const gf_h1* e, uint32_t index, gf_h1_cycle_record* out_record) {
    if (!e || !out_record || index >= e->impl.records().size()) return fail(GF_ERR_INVALID, "bad record index");
    *out_record = e->impl.records()[index];
    return GF_OK;
}

}  // extern "C"
