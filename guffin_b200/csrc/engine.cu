// Host sampler C entry points and the H1 draft -> verify -> accept / rollback cycle.
#include "model.cuh"
#include "sampler.hpp"

#include <cstring>
#include <memory>
#include <random>
#include <vector>

namespace gf {

size_t draft_sampler_workspace_bytes(uint32_t vocab);
int launch_draft_sample(const float* logits, uint32_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                        float penalty, const uint32_t* history_host, uint32_t history_count, uint32_t word,
                        void* workspace, void* receipt_dev, uint32_t* out_token_a, uint32_t* out_token_b,
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

class H1Engine {
public:
    H1Engine(Model& target, Model* draft, const gf_h1_options& options)
        : target_(target), draft_(draft), options_(options), sampler_(to_options(options.sampler)), schedule_(options.schedule_seed) {}
    ~H1Engine() {
        if (draft_ws_) cudaFree(draft_ws_);
        if (receipt_dev_) cudaFree(receipt_dev_);
        if (results_host_) cudaFreeHost(results_host_);
        if (receipt_host_) cudaFreeHost(receipt_host_);
        if (draft_done_) cudaEventDestroy(draft_done_);
    }

    int init() {
        GF_TRY(validate_options(sampler_.options()));
        if (options_.speculative) {
            if (!draft_) return fail(GF_ERR_INVALID, "speculative decoding needs a drafter plan");
            if (draft_->config().vocab != target_.config().vocab) return fail(GF_ERR_INVALID, "drafter and target vocabularies differ (direct token ids are required)");
            if (target_.config().row_capacity < 2 || draft_->config().row_capacity < 2) return fail(GF_ERR_INVALID, "H1 needs two rows per pass in both plans");
            if (sampler_.options().top_k > 64) return fail(GF_ERR_INVALID, "the compact proposal law supports top_k <= 64");
            GF_CUDA(cudaMalloc(&draft_ws_, draft_sampler_workspace_bytes(draft_->config().vocab)));
            GF_CUDA(cudaMalloc(&receipt_dev_, sizeof(DraftReceiptRow)));
            GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&receipt_host_), sizeof(DraftReceiptRow), cudaHostAllocDefault));
            GF_CUDA(cudaEventCreateWithFlags(&draft_done_, cudaEventDisableTiming));
        }
        GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&results_host_), 2 * sizeof(CandidateRow), cudaHostAllocDefault));
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
            const bool spec = options_.speculative && !draft_exhausted_ && max_tokens - produced >= 2 && room >= 3
                && draft_->config().context - draft_->position() >= 3;
            if (spec) {
                uint32_t tokens[2];
                uint32_t n = 0;
                const int status = cycle(tokens, n);
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

    // One H1 cycle.  On entry root_ is selected but not yet in any cache.
    int cycle(uint32_t (&emitted)[2], uint32_t& emitted_count) {
        const SamplerOptions& so = sampler_.options();
        const uint32_t r = root_;
        const uint32_t word = sampler_.preview_proposal_word();
        // --- drafter: ingest [pending?, r], sample one token from the last row's logits.
        uint32_t draft_tokens[2];
        uint32_t draft_rows = 0;
        if (pending_) draft_tokens[draft_rows++] = pending_token_;
        draft_tokens[draft_rows++] = r;
        GF_TRY(draft_->forward(draft_tokens, draft_rows, kForwardLogits));
        GF_TRY(draft_->publish(draft_rows));
        const SelectionHistory draft_history = sampler_.request_after(&r, 1);     // repetition window incl. the root
        GF_TRY(launch_draft_sample(draft_->logits_dev() + (size_t)(draft_rows - 1u) * draft_->config().vocab,
                                   draft_->config().vocab, so.temperature, so.top_k, so.top_p, so.min_p,
                                   so.repetition_penalty, draft_history.tokens.data(), draft_history.count, word, draft_ws_,
                                   receipt_dev_, target_.tokens_dev() + 1, nullptr, draft_->stream()));
        stats_.sampler_launches += 3;
        GF_CUDA(cudaMemcpyAsync(receipt_host_, receipt_dev_, sizeof(DraftReceiptRow), cudaMemcpyDeviceToHost, draft_->stream()));
        GF_CUDA(cudaEventRecord(draft_done_, draft_->stream()));
        // --- target: verify rows [r, x] in one pass; x never visits the host on this path.
        GF_TRY(target_.set_device_token(0, r));
        GF_CUDA(cudaStreamWaitEvent(target_.stream(), draft_done_, 0));
        GF_TRY(target_.forward(nullptr, 2, kForwardLogits | kForwardDeviceTokens));
        uint32_t x = 0;
        bool have_x = false;
        SelectionRequestRow requests[2];
        {
            const uint32_t suffix0[1] = {r};
            requests[0] = to_request(sampler_.request_after(suffix0, 1));
            if (so.repetition_penalty != 1.0f) {      // row 1's request names x: read it first
                GF_CUDA(cudaEventSynchronize(draft_done_));
                x = receipt_host_->token;
                have_x = true;
                const uint32_t suffix1[2] = {r, x};
                requests[1] = to_request(sampler_.request_after(suffix1, 2));
            } else {
                requests[1] = requests[0];
            }
        }
        GF_TRY(target_.select(requests, 2));
        GF_TRY(target_.read_candidates(results_host_, 2));           // the cycle's one synchronisation
        GF_CUDA(cudaEventSynchronize(draft_done_));
        const DraftReceiptRow& receipt = *receipt_host_;
        if (!have_x) x = receipt.token;
        if (results_host_[0].status || results_host_[1].status)
            return fail(GF_ERR_NUMERIC, "candidate selection reported status %u/%u", results_host_[0].status, results_host_[1].status);
        ++stats_.cycles;
        if (receipt.status != 0 || x >= target_.config().vocab) {
            // No usable proposal law (support overflow or a numeric fault in the drafter): finish
            // the step as ordinary decoding of r from row 0; nothing speculative is published.
            if (receipt.status != 20u) return fail(GF_ERR_NUMERIC, "drafter sampler reported status %u", receipt.status);
            ++stats_.fallback_cycles;
            GF_TRY(target_.publish(1));
            sampler_.observe(&r, 1);
            const SelectionHistory now = sampler_.request_after(nullptr, 0);
            uint32_t token = 0;
            GF_TRY(sampler_.sample(results_host_[0].candidates, results_host_[0].count, now, token));
            pending_ = false;
            root_ = token;
            emitted[0] = token;
            emitted_count = 1;
            return GF_OK;
        }
        // --- acceptance (host, double precision).
        const uint32_t suffix0[1] = {r};
        const SelectionHistory request0 = sampler_.request_after(suffix0, 1);
        TokenDistribution prepared;
        GF_TRY(prepare_distribution(results_host_[0].candidates, results_host_[0].count, so, request0, prepared));
        GatheredDraft gathered;
        gather(receipt, prepared, gathered);
        SpeculativeOutcome outcome;
        const int law_status = sampler_.sample_speculative(gathered, results_host_[0].candidates, results_host_[0].count, request0, outcome);
        if (options_.record_cycles) {
            gf_h1_cycle_record record {};
            record.root = r; record.proposal = x; record.word = word; record.candidate_count = results_host_[0].count;
            std::memcpy(record.candidates, results_host_[0].candidates, sizeof(TokenLogit) * results_host_[0].count);
            record.draft.proposal = gathered.proposal; record.draft.count = gathered.count;
            record.draft.proposal_mass = gathered.proposal_mass; record.draft.proposal_cdf_begin = gathered.proposal_cdf_begin;
            std::memcpy(record.draft.target_mass, gathered.target_mass.data(), sizeof(uint64_t) * 256);
            record.token = outcome.token; record.accepted = outcome.accepted; record.target_draws = outcome.target_draws;
            record.status = law_status;
            if (records_.size() < 65536) records_.push_back(record);
        }
        if (law_status != GF_OK) return law_status;
        bool accepted = outcome.accepted;
        uint32_t corrected = outcome.token;
        if (options_.forced_schedule) {
            std::bernoulli_distribution coin(options_.forced_accept_probability);
            const bool forced = coin(schedule_);
            if (forced == outcome.accepted) ++stats_.law_agreements;
            if (!forced && outcome.accepted) {
                // Scheduled rejection of a proposal the law accepted: continue from an ordinary
                // sample of the same row, so the control flow (one row published, no carry) matches.
                GF_TRY(sampler_.sample(results_host_[0].candidates, results_host_[0].count, request0, corrected));
            }
            accepted = forced;
        }
        if (accepted) {
            ++stats_.accepted;
            GF_TRY(target_.publish(2));                 // both private rows become durable
            const uint32_t observed[2] = {r, x};
            sampler_.observe(observed, 2);
            const SelectionHistory now = sampler_.request_after(nullptr, 0);
            uint32_t next = 0;
            GF_TRY(sampler_.sample(results_host_[1].candidates, results_host_[1].count, now, next));
            pending_ = true;                             // x is selected but not yet forwarded by the drafter
            pending_token_ = x;
            root_ = next;
            emitted[0] = x; emitted[1] = next;
            emitted_count = 2;
        } else {
            ++stats_.rejected;
            GF_TRY(target_.publish(1));                 // row 1 is simply never published: the rollback
            sampler_.observe(&r, 1);
            pending_ = false;                            // the drafter drops its pending token
            root_ = corrected;
            emitted[0] = corrected;
            emitted_count = 1;
        }
        return GF_OK;
    }

    Model& target_;
    Model* draft_;
    gf_h1_options options_;
    Sampler sampler_;
    std::mt19937_64 schedule_;
    gf_h1_stats stats_ {};
    std::vector<gf_h1_cycle_record> records_;
    void *draft_ws_ = nullptr, *receipt_dev_ = nullptr;
    CandidateRow* results_host_ = nullptr;
    DraftReceiptRow* receipt_host_ = nullptr;
    cudaEvent_t draft_done_ = nullptr;
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
