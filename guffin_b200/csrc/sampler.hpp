// Host-side token sampler and lossless speculative acceptance, in double precision.
//
// Behavioural mirror of the reference's TokenSampler (src/engine/sampling.cpp): the same
// transform order (dedupe -> repetition penalty -> sort by (logit desc, token asc) -> top-k ->
// top-p on un-tempered weights -> min-p -> temperature), the same two mt19937_64 streams
// (target stream seeded directly, proposal stream domain-separated from two target draws), and
// the same accept / residual law, so that with identical candidates, draft masses and seed the
// decisions are identical.  The CPU stays the authority for token selection, as in the
// reference; the GPU only narrows 262k logits to <= 384 candidates.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <random>
#include <vector>

namespace gf {

constexpr uint32_t kSamplerMaxTopK = 256;           // token_sampler_max_top_k
constexpr uint32_t kSamplerMaxWindow = 64;          // token_sampler_max_repetition_window
constexpr uint32_t kSamplerMaxCandidates = 384;     // token_sampler_max_candidates
constexpr uint64_t kDraftMassTotal = 1ull << 32;    // draft_probability_mass_total

struct TokenLogit { uint32_t token; float logit; };

struct SamplerOptions {                             // TokenSamplerOptions (sampling.hpp:184-196)
    float temperature = 0.0f;
    uint32_t top_k = 40;
    float top_p = 0.95f;
    float min_p = 0.05f;
    float repetition_penalty = 1.0f;
    uint64_t seed = 0;
    uint32_t repetition_window = 64;
};

struct WeightedToken { uint32_t token; double probability; double weight; };
struct TokenDistribution {                          // PreparedTokenDistribution
    std::array<WeightedToken, kSamplerMaxTopK> values {};
    uint32_t count = 0;
    double total_weight = 0.0;
};

struct SelectionHistory {                           // the deduplicated history a selection request carries
    std::array<uint32_t, kSamplerMaxWindow> tokens {};
    uint32_t count = 0;
    uint32_t top_k = 1;
};

struct SpeculativeOutcome { uint32_t token = 0; bool accepted = false; uint32_t target_draws = 0; };

// Draft masses gathered on the prepared target support (GatheredDraftTokenDistribution).
struct GatheredDraft {
    uint32_t proposal = 0;
    uint64_t proposal_mass = 0;
    uint64_t proposal_cdf_begin = 0;
    std::array<uint64_t, kSamplerMaxTopK> target_mass {};
    uint32_t count = 0;
};

int validate_options(const SamplerOptions& options);
int prepare_distribution(const TokenLogit* candidates, uint32_t count, const SamplerOptions& options,
                         const SelectionHistory& request, TokenDistribution& out);
int prepare_speculative(const GatheredDraft& draft, const TokenDistribution& target, double& acceptance,
                        TokenDistribution& residual);

class Sampler {
public:
    explicit Sampler(const SamplerOptions& options);
    const SamplerOptions& options() const { return options_; }
    bool greedy() const { return options_.temperature == 0.0f; }

    // Chronological repetition window, newest last.
    void observe(const uint32_t* tokens, uint32_t count);
    void reset_history();
    // The request for a row whose context is the observed history plus `suffix`.
    SelectionHistory request_after(const uint32_t* suffix, uint32_t suffix_count) const;

    int sample(const TokenLogit* candidates, uint32_t count, const SelectionHistory& request, uint32_t& token);
    uint32_t preview_proposal_word() const;
    // The next `count` proposal words without consuming them (preview_proposal_words, sampling.cpp:62-80).
    void preview_proposal_words(uint32_t* out, uint32_t count) const;
    // Accept/reject `draft.proposal` against the target candidates of the same row; advances both
    // streams only when every check passes (sampling.cpp:896-934).
    int sample_speculative(const GatheredDraft& draft, const TokenLogit* candidates, uint32_t count,
                           const SelectionHistory& request, SpeculativeOutcome& out);
    const std::vector<uint32_t>& history() const { return history_; }      // the repetition window, oldest first
    uint64_t target_draws() const { return draws_; }
    uint64_t proposal_draws() const { return proposal_draws_; }

private:
    SamplerOptions options_;
    std::mt19937_64 rng_, proposal_rng_;
    std::vector<uint32_t> history_;
    uint64_t draws_ = 0, proposal_draws_ = 0;
};

}  // namespace gf
