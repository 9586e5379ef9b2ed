// Host-side sampler and lossless acceptance (see sampler.hpp).
#include "sampler.hpp"
#include "common.cuh"

#include <algorithm>
#include <cmath>
#include <limits>

namespace gf {

static bool better(const TokenLogit& a, const TokenLogit& b) {
    return a.logit != b.logit ? a.logit > b.logit : a.token < b.token;
}

int validate_options(const SamplerOptions& o) {
    if (!std::isfinite(o.temperature) || o.temperature < 0.0f) return fail(GF_ERR_INVALID, "sampler options: temperature %g is negative or not finite", (double)o.temperature);
    if (o.top_k == 0 || o.top_k > kSamplerMaxTopK) return fail(GF_ERR_INVALID, "sampler options: top_k outside 1..256");
    if (!std::isfinite(o.top_p) || o.top_p <= 0.0f || o.top_p > 1.0f) return fail(GF_ERR_INVALID, "sampler options: top_p outside (0, 1]");
    if (!std::isfinite(o.min_p) || o.min_p < 0.0f || o.min_p > 1.0f) return fail(GF_ERR_INVALID, "sampler options: min_p outside [0, 1]");
    if (!std::isfinite(o.repetition_penalty) || o.repetition_penalty <= 0.0f) return fail(GF_ERR_INVALID, "sampler options: repetition_penalty must be a positive finite number");
    if (o.repetition_window > kSamplerMaxWindow) return fail(GF_ERR_INVALID, "sampler options: repetition_window above 64");
    return GF_OK;
}

int prepare_distribution(const TokenLogit* compact, uint32_t count, const SamplerOptions& options,
                         const SelectionHistory& request, TokenDistribution& out) {
    if (!compact || count == 0 || count > kSamplerMaxCandidates)
        return fail(GF_ERR_INVALID, "candidate list: expected 1..384 (token, logit) pairs");
    if (request.top_k == 0 || request.top_k > options.top_k || request.count > kSamplerMaxWindow)
        return fail(GF_ERR_INVALID, "candidate list: the selection request that produced it is malformed");
    std::array<TokenLogit, kSamplerMaxCandidates> pool;
    uint32_t n = 0;
    for (uint32_t i = 0; i < count; ++i) {
        if (!std::isfinite(compact[i].logit)) return fail(GF_ERR_INVALID, "candidate list: a logit is NaN or infinite");
        uint32_t j = 0;
        while (j < n && pool[j].token != compact[i].token) ++j;
        if (j == n) pool[n++] = compact[i];
        else if (pool[j].logit != compact[i].logit) return fail(GF_ERR_INVALID, "candidate list: one token appears twice with two logits");
    }
    if (n < request.top_k) return fail(GF_ERR_INVALID, "candidate list: fewer pairs than the requested top_k");
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t* end = request.tokens.data() + request.count;
        if (std::find(request.tokens.data(), end, pool[i].token) != end)
            pool[i].logit = pool[i].logit < 0.0f ? pool[i].logit * options.repetition_penalty
                                                 : pool[i].logit / options.repetition_penalty;
    }
    std::sort(pool.begin(), pool.begin() + n, better);
    n = std::min(n, request.top_k);
    out = TokenDistribution();
    if (options.temperature == 0.0f) {
        out.values[0] = {pool[0].token, 1.0, 1.0};
        out.count = 1;
        out.total_weight = 1.0;
        return GF_OK;
    }
    std::array<double, kSamplerMaxTopK> weights {};
    const float top = pool[0].logit;
    double total = 0.0;
    for (uint32_t i = 0; i < n; ++i) weights[i] = std::exp(static_cast<double>(pool[i].logit - top));
    for (uint32_t i = 0; i < n; ++i) total += weights[i];
    // Nucleus on the un-tempered weights, then min-p relative to the best candidate (weight 1).
    double kept = 0.0;
    uint32_t nucleus = 0;
    do { kept += weights[nucleus++]; } while (nucleus < n && kept / total < static_cast<double>(options.top_p));
    n = nucleus;
    if (options.min_p > 0.0f) {
        uint32_t m = 1;
        while (m < n && weights[m] >= static_cast<double>(options.min_p)) ++m;
        n = m;
    }
    double normalization = 0.0;
    for (uint32_t i = 0; i < n; ++i) {
        weights[i] = std::exp(static_cast<double>(pool[i].logit - top) / static_cast<double>(options.temperature));
        normalization += weights[i];
    }
    if (!std::isfinite(normalization) || normalization <= 0.0) return fail(GF_ERR_NUMERIC, "target law: the weights do not sum to a positive finite number");
    out.count = n;
    out.total_weight = normalization;
    for (uint32_t i = 0; i < n; ++i) out.values[i] = {pool[i].token, weights[i] / normalization, weights[i]};
    return GF_OK;
}

// Compensated (Neumaier) sum of the sampling weights: the normaliser both laws divide by.
static int compensated_total(const TokenDistribution& d, double& total_out) {
    if (d.count == 0 || d.count > kSamplerMaxTopK || !std::isfinite(d.total_weight) || d.total_weight <= 0.0)
        return fail(GF_ERR_INVALID, "target law: empty or oversized support");
    double total = 0.0, correction = 0.0;
    for (uint32_t i = 0; i < d.count; ++i) {
        const double w = d.values[i].weight;
        if (!std::isfinite(w) || w < 0.0) return fail(GF_ERR_INVALID, "target law: a weight is negative or not finite");
        const double sum = total + w;
        correction += total >= w ? (total - sum) + w : (w - sum) + total;
        total = sum;
    }
    total += correction;
    const double tolerance = static_cast<double>(d.count) * std::numeric_limits<double>::epsilon() * total;
    if (!std::isfinite(total) || total <= 0.0 || std::abs(total - d.total_weight) > tolerance)
        return fail(GF_ERR_INVALID, "target law: stored total differs from the sum of its weights");
    total_out = total;
    return GF_OK;
}

int prepare_speculative(const GatheredDraft& draft, const TokenDistribution& target, double& acceptance,
                        TokenDistribution& residual) {
    double normalization = 0.0;
    const int status = compensated_total(target, normalization);
    if (status != GF_OK) return status;
    if (draft.proposal_mass == 0 || draft.proposal_mass > kDraftMassTotal
        || draft.proposal_cdf_begin > kDraftMassTotal - draft.proposal_mass || draft.count != target.count)
        return fail(GF_ERR_INVALID, "draft law: proposal or support size out of range");
    uint64_t gathered = 0;
    bool proposal_in_target = false;
    for (uint32_t i = 0; i < target.count; ++i) {
        if (draft.target_mass[i] > kDraftMassTotal - gathered)
            return fail(GF_ERR_INVALID, "draft law: gathered on a support other than the target's");
        gathered += draft.target_mass[i];
        if (target.values[i].token == draft.proposal) {
            proposal_in_target = true;
            if (draft.target_mass[i] != draft.proposal_mass)
                return fail(GF_ERR_INVALID, "draft law: the proposal's mass and its gathered entry differ");
        }
    }
    if (!proposal_in_target && draft.proposal_mass > kDraftMassTotal - gathered)
        return fail(GF_ERR_INVALID, "draft law: masses add up to more than 2^32");
    // a = min(1, p(x) / q(x)); residual proportional to max(p - q, 0) on the target support,
    // q taken as it is (never renormalised).
    const double two32 = static_cast<double>(kDraftMassTotal);
    const double proposed = static_cast<double>(draft.proposal_mass) / two32;
    acceptance = 0.0;
    residual = TokenDistribution();
    for (uint32_t i = 0; i < target.count; ++i) {
        const double p = target.values[i].weight / normalization;
        if (target.values[i].token == draft.proposal) acceptance = std::min(1.0, p / proposed);
        const double difference = p - static_cast<double>(draft.target_mass[i]) / two32;
        if (difference <= 0.0) continue;
        residual.values[residual.count++] = {target.values[i].token, 0.0, difference};
        residual.total_weight += difference;
    }
    if (residual.count != 0) {
        for (uint32_t i = 0; i < residual.count; ++i) residual.values[i].probability = residual.values[i].weight / residual.total_weight;
    } else if (acceptance < 1.0) {
        return fail(GF_ERR_NUMERIC, "acceptance: a rejection is possible but the residual law is empty");
    }
    return GF_OK;
}

static uint32_t pick(const TokenDistribution& d, double draw) {
    double cumulative = 0.0;
    for (uint32_t i = 0; i < d.count; ++i) {
        cumulative += d.values[i].weight;
        if (draw < cumulative) return d.values[i].token;
    }
    return d.values[d.count - 1].token;
}

static std::mt19937_64 proposal_stream(std::mt19937_64 target) {
    // Domain separation: two draws of a COPY of the target stream seed the proposal stream.
    const uint64_t first = target(), second = target();
    std::seed_seq seed {0x4c475350u, 0x524f5031u, static_cast<uint32_t>(first), static_cast<uint32_t>(first >> 32),
                        static_cast<uint32_t>(second), static_cast<uint32_t>(second >> 32)};
    return std::mt19937_64(seed);
}

Sampler::Sampler(const SamplerOptions& options) : options_(options), rng_(options.seed), proposal_rng_(proposal_stream(rng_)) {}

void Sampler::observe(const uint32_t* tokens, uint32_t count) {
    if (options_.repetition_window == 0) return;
    for (uint32_t i = 0; i < count; ++i) {
        if (history_.size() == options_.repetition_window) history_.erase(history_.begin());
        history_.push_back(tokens[i]);
    }
}

void Sampler::reset_history() { history_.clear(); }

SelectionHistory Sampler::request_after(const uint32_t* suffix, uint32_t suffix_count) const {
    SelectionHistory request;
    request.top_k = options_.temperature == 0.0f ? 1u : options_.top_k;
    if (options_.repetition_penalty == 1.0f || options_.repetition_window == 0) return request;
    std::vector<uint32_t> window(history_);
    for (uint32_t i = 0; i < suffix_count; ++i) {
        if (window.size() == options_.repetition_window) window.erase(window.begin());
        window.push_back(suffix[i]);
    }
    for (uint32_t token : window) {             // chronological, first occurrence wins
        bool seen = false;
        for (uint32_t i = 0; i < request.count; ++i) seen |= request.tokens[i] == token;
        if (!seen) request.tokens[request.count++] = token;
    }
    return request;
}

int Sampler::sample(const TokenLogit* candidates, uint32_t count, const SelectionHistory& request, uint32_t& token) {
    TokenDistribution prepared;
    const int status = prepare_distribution(candidates, count, options_, request, prepared);
    if (status != GF_OK) return status;
    if (greedy()) { token = prepared.values[0].token; return GF_OK; }
    std::uniform_real_distribution<double> distribution(0.0, prepared.total_weight);
    const double draw = distribution(rng_);
    ++draws_;
    token = pick(prepared, draw);
    return GF_OK;
}

uint32_t Sampler::preview_proposal_word() const {
    std::mt19937_64 cursor = proposal_rng_;
    return static_cast<uint32_t>(cursor() >> 32);
}

void Sampler::preview_proposal_words(uint32_t* out, uint32_t count) const {
    std::mt19937_64 cursor = proposal_rng_;
    for (uint32_t i = 0; i < count; ++i) out[i] = static_cast<uint32_t>(cursor() >> 32);
}

int Sampler::sample_speculative(const GatheredDraft& draft, const TokenLogit* candidates, uint32_t count,
                                const SelectionHistory& request, SpeculativeOutcome& out) {
    TokenDistribution target, residual;
    int status = prepare_distribution(candidates, count, options_, request, target);
    if (status != GF_OK) return status;
    double acceptance = 0.0;
    status = prepare_speculative(draft, target, acceptance, residual);
    if (status != GF_OK) return status;
    std::mt19937_64 proposal_cursor = proposal_rng_;
    const uint64_t word = proposal_cursor() >> 32;
    if (word < draft.proposal_cdf_begin || word - draft.proposal_cdf_begin >= draft.proposal_mass)
        return fail(GF_ERR_INVALID, "acceptance: the proposal word falls outside the proposal's CDF interval");
    std::mt19937_64 target_cursor = rng_;
    uint32_t draws = 0;
    double accept_draw = 0.0, residual_draw = 0.0;
    if (!greedy()) {
        std::uniform_real_distribution<double> uniform(0.0, 1.0);
        accept_draw = uniform(target_cursor);
        ++draws;
        if (accept_draw >= acceptance) { residual_draw = uniform(target_cursor); ++draws; }
    }
    if (accept_draw < acceptance) {
        out = {draft.proposal, true, draws};
    } else {
        if (residual.count == 0) return fail(GF_ERR_NUMERIC, "acceptance: rejected with an empty residual law");
        double checked = 0.0;
        status = compensated_total(residual, checked);
        if (status != GF_OK) return status;
        out = {pick(residual, residual_draw * residual.total_weight), false, draws};
    }
    rng_ = target_cursor;
    proposal_rng_ = proposal_cursor;
    draws_ += draws;
    ++proposal_draws_;
    return GF_OK;
}

}  // namespace gf
