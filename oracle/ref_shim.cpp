// C entry points over the reference engine's own CPU code, compiled from the reference
// sources where they lie (never copied).  TEST INFRASTRUCTURE ONLY: used to validate the
// C restatement in gf_oracle.c, to generate golden fixtures, and as the timed CPU baseline.
//
// Each function calls the reference symbol named in its comment and does no arithmetic of
// its own beyond marshalling flat arrays into the reference's tensor types.
#include "local_gguf_engine/engine/sampling.hpp"
#include "local_gguf_engine/tensor/f16.hpp"
#include "local_gguf_engine/tensor/kquant_packing.hpp"
#include "local_gguf_engine/tensor/ops/attention.hpp"
#include "local_gguf_engine/tensor/ops/elementwise.hpp"
#include "local_gguf_engine/tensor/ops/normalization.hpp"
#include "local_gguf_engine/tensor/ops/rope.hpp"
#include "local_gguf_engine/tensor/ops/softmax.hpp"
#include "local_gguf_engine/tensor/quantization.hpp"
#include "local_gguf_engine/tensor/tensor.hpp"
#include "backends/cpu_backend.hpp"

#include <cstring>
#include <exception>
#include <span>
#include <vector>

using namespace local_gguf_engine;
using tensor::DType;
using tensor::Shape;
using tensor::TensorDescriptor;
using tensor::TensorStorage;

namespace {

TensorStorage f32_tensor(std::initializer_list<std::uint64_t> dims, const float* data) {
    const auto descriptor = TensorDescriptor::from(Shape::from(dims), DType::f32);
    return TensorStorage::from_bytes(descriptor,
        std::span<const std::uint8_t>(reinterpret_cast<const std::uint8_t*>(data), descriptor.byte_count));
}

TensorStorage weight_tensor(int dtype, const std::uint8_t* data, std::uint64_t k, std::uint64_t n) {
    const auto descriptor = TensorDescriptor::from_quantized_gguf_weight_matrix(
        Shape::from({k, n}), static_cast<DType>(dtype));
    return TensorStorage::from_bytes(descriptor, std::span<const std::uint8_t>(data, descriptor.byte_count));
}

void copy_out(const TensorStorage& storage, float* out) {
    std::memcpy(out, storage.bytes().data(), storage.bytes().size());
}

engine::TokenSamplerOptions sampler_options(float temperature, std::uint32_t top_k, float top_p,
    float min_p, float repetition_penalty, std::uint64_t seed) {
    engine::TokenSamplerOptions options;
    options.temperature = temperature;
    options.top_k = top_k;
    options.top_p = top_p;
    options.min_p = min_p;
    options.repetition_penalty = repetition_penalty;
    options.seed = seed;
    options.repetition_window = 64;
    return options;
}

}  // namespace

extern "C" {

// tensor::f16_bits_to_f32 / f32_to_f16_bits  (src/tensor/f16.cpp)
float ref_f16_to_f32(std::uint16_t bits) { return tensor::f16_bits_to_f32(bits); }
std::uint16_t ref_f32_to_f16(float value) { return tensor::f32_to_f16_bits(value); }

// Q8_0/Q4_K/Q6_K BlockView::dequantized_value  (src/tensor/quantization.cpp)
int ref_dequantize(int dtype, const std::uint8_t* blocks, std::uint64_t block_count, float* out) {
    try {
        const std::uint64_t elements = dtype == 8 ? 32U : 256U;
        const auto storage = weight_tensor(dtype, blocks, elements, block_count);
        for (std::uint64_t block = 0; block < block_count; ++block) {
            for (std::uint64_t e = 0; e < elements; ++e) {
                float value = 0.0F;
                if (dtype == 8) value = tensor::q8_0_block_view(storage, block).dequantized_value(e);
                else if (dtype == 12) value = tensor::q4_k_block_view(storage, block).dequantized_value(e);
                else value = tensor::q6_k_block_view(storage, block).dequantized_value(e);
                out[block * elements + e] = value;
            }
        }
        return 0;
    } catch (const std::exception&) { return -1; }
}

// tensor::quantize_f16_gguf_weight_q8_0  (src/tensor/quantization.cpp:628-673)
int ref_quantize_f16_q8_0(const std::uint16_t* f16, std::uint64_t k, std::uint64_t n, std::uint8_t* out) {
    try {
        const auto descriptor = TensorDescriptor::from(Shape::from({k, n}), DType::f16);
        const auto source = TensorStorage::from_bytes(descriptor,
            std::span<const std::uint8_t>(reinterpret_cast<const std::uint8_t*>(f16), descriptor.byte_count));
        const auto result = tensor::quantize_f16_gguf_weight_q8_0(source.view());
        std::memcpy(out, result.bytes().data(), result.bytes().size());
        return 0;
    } catch (const std::exception&) { return -1; }
}

// tensor::requantize_q6_k_gguf_weight_q4_k  (src/tensor/quantization.cpp:746-800), canonical layout
int ref_requantize_q6k_q4k(const std::uint8_t* q6, std::uint64_t k, std::uint64_t n, std::uint8_t* out) {
    try {
        const auto source = weight_tensor(14, q6, k, n);
        const auto result = tensor::requantize_q6_k_gguf_weight_q4_k(source.view());
        std::memcpy(out, result.bytes().data(), result.bytes().size());
        return 0;
    } catch (const std::exception&) { return -1; }
}

// backends::cpu::matmul_f32_quantized_gguf_weight  (src/tensor/backends/cpu_backend.cpp:301)
int ref_matmul_quantized(int dtype, const float* x, const std::uint8_t* weight, std::uint32_t rows,
    std::uint64_t k, std::uint64_t n, float* out) {
    try {
        const auto left = f32_tensor({rows, k}, x);
        const auto right = weight_tensor(dtype, weight, k, n);
        copy_out(tensor::backends::cpu::matmul_f32_quantized_gguf_weight(left, right), out);
        return 0;
    } catch (const std::exception&) { return -1; }
}

// ops::rms_norm_f32  (src/tensor/ops/normalization.cpp:70)
int ref_rms_norm(const float* x, const float* gamma, std::uint32_t rows, std::uint32_t hidden,
    float eps, float* out) {
    try {
        copy_out(tensor::ops::rms_norm_f32(f32_tensor({rows, hidden}, x), f32_tensor({hidden}, gamma), eps), out);
        return 0;
    } catch (const std::exception&) { return -1; }
}

// ops::gelu_tanh_f32 then ops::multiply_f32  (src/tensor/ops/elementwise.cpp:79)
int ref_gelu_tanh_multiply(const float* gate, const float* up, std::uint64_t count, float* out) {
    try {
        const auto activated = tensor::ops::gelu_tanh_f32(f32_tensor({count}, gate));
        copy_out(tensor::ops::multiply_f32(activated, f32_tensor({count}, up)), out);
        return 0;
    } catch (const std::exception&) { return -1; }
}

// ops::softcap_f32  (src/tensor/ops/elementwise.cpp:96)
int ref_softcap(const float* x, std::uint64_t count, float softcap, float* out) {
    try { copy_out(tensor::ops::softcap_f32(f32_tensor({count}, x), softcap), out); return 0; }
    catch (const std::exception&) { return -1; }
}

// ops::softmax_f32  (src/tensor/ops/softmax.cpp:42)
int ref_softmax(const float* x, std::uint32_t rows, std::uint32_t columns, float* out) {
    try { copy_out(tensor::ops::softmax_f32(f32_tensor({rows, columns}, x)), out); return 0; }
    catch (const std::exception&) { return -1; }
}

// ops::rope_neox_f32_by_heads_with_position_start  (src/tensor/ops/rope.cpp:246); rows take
// consecutive positions and the frequency scale is 1.
int ref_rope_neox(const float* x, std::uint64_t position_start, std::uint32_t rows,
    std::uint32_t heads, std::uint32_t head_dim, float base, float* out) {
    try {
        copy_out(tensor::ops::rope_neox_f32_by_heads_with_position_start(
            f32_tensor({rows, static_cast<std::uint64_t>(heads) * head_dim}, x),
            position_start, heads, head_dim, head_dim, base), out);
        return 0;
    } catch (const std::exception&) { return -1; }
}

// causal_grouped_attention_scores_f32 -> softmax_f32 -> causal_grouped_attention_values_f32
// (src/tensor/ops/attention.cpp:482,550) for one query row at position count-1 over `count` keys.
int ref_attention_row(const float* q, const float* keys, const float* values, std::uint32_t count,
    std::uint32_t heads, std::uint32_t kv_heads, std::uint32_t head_dim, float scale, float softcap,
    float* out) {
    try {
        const std::uint64_t qw = static_cast<std::uint64_t>(heads) * head_dim;
        const std::uint64_t kw = static_cast<std::uint64_t>(kv_heads) * head_dim;
        const auto scores = tensor::ops::causal_grouped_attention_scores_f32(
            f32_tensor({1, qw}, q), f32_tensor({count, kw}, keys), count - 1U, heads, kv_heads,
            head_dim, count, scale, softcap);
        const auto probabilities = tensor::ops::softmax_f32(scores);
        copy_out(tensor::ops::causal_grouped_attention_values_f32(
            probabilities, f32_tensor({count, kw}, values), count - 1U, heads, kv_heads, head_dim, count), out);
        return 0;
    } catch (const std::exception&) { return -1; }
}

struct RefTokenLogit { std::uint32_t token; float logit; };
struct RefProb { std::uint32_t token; double probability; double weight; };

// engine::make_token_selection_request + prepare_token_distribution  (src/engine/sampling.cpp:394).
// `history` is the chronological repetition window. Returns the support size or a negative code.
int ref_prepare_distribution(const RefTokenLogit* candidates, std::uint32_t count, float temperature,
    std::uint32_t top_k, float top_p, float min_p, float repetition_penalty,
    const std::uint32_t* history, std::uint32_t history_count, RefProb* out, double* total_weight) {
    try {
        const auto options = sampler_options(temperature, top_k, top_p, min_p, repetition_penalty, 1U);
        engine::SamplerHistorySnapshot snapshot;
        snapshot.window_limit = 64;
        snapshot = engine::append_sampler_history(snapshot, std::span<const std::uint32_t>(history, history_count));
        const auto request = engine::make_token_selection_request(options, snapshot);
        std::vector<engine::TokenLogit> values(count);
        for (std::uint32_t i = 0; i < count; ++i) values[i] = {candidates[i].token, candidates[i].logit};
        const auto prepared = engine::prepare_token_distribution(values, options, request);
        for (std::uint32_t i = 0; i < prepared.count; ++i)
            out[i] = {prepared.values[i].token, prepared.values[i].probability, prepared.values[i].sampling_weight};
        *total_weight = prepared.total_sampling_weight;
        return static_cast<int>(prepared.count);
    } catch (const std::exception&) { return -1; }
}

// TokenSampler(seed).preview_proposal_words  (src/engine/sampling.cpp:45-79)
int ref_proposal_words(std::uint64_t seed, std::uint32_t count, std::uint32_t* words) {
    try {
        engine::TokenSampler sampler(sampler_options(0.7F, 40, 0.95F, 0.05F, 1.0F, seed));
        const auto preview = sampler.preview_proposal_words(count);
        for (std::uint32_t i = 0; i < count; ++i) words[i] = preview.words[i];
        return 0;
    } catch (const std::exception&) { return -1; }
}

// The reference's RNG stream: mt19937_64(seed) through uniform_real_distribution<double>(a, b)
// exactly as sampling.cpp:841,913 draw it.
void ref_uniform_draws(std::uint64_t seed, double a, double b, std::uint32_t count, double* out) {
    std::mt19937_64 rng(seed);
    for (std::uint32_t i = 0; i < count; ++i) {
        std::uniform_real_distribution<double> distribution(a, b);
        out[i] = distribution(rng);
    }
}

// TokenSamplerFork::sample_speculative with a gathered draft law  (src/engine/sampling.cpp:896-934).
// draft masses are given on the prepared target support (q_mass[i] for the i-th prepared token,
// prepared by this same call's options); the proposal's CDF bin is [cdf_begin, cdf_begin+mass).
// `history` is observed before sampling.  Outputs: token, accepted flag, and how many target
// draws the fork consumed.  Returns 0, or -1 when the reference throws.
int ref_sample_speculative(std::uint64_t seed, float temperature, std::uint32_t top_k, float top_p,
    float min_p, float repetition_penalty, const std::uint32_t* history, std::uint32_t history_count,
    const RefTokenLogit* candidates, std::uint32_t count, std::uint32_t proposal,
    std::uint64_t proposal_mass, std::uint64_t proposal_cdf_begin, const std::uint64_t* q_mass,
    std::uint32_t* token, int* accepted, std::uint64_t* target_draws) {
    try {
        engine::TokenSampler sampler(sampler_options(temperature, top_k, top_p, min_p, repetition_penalty, seed));
        sampler.observe_tokens(std::span<const std::uint32_t>(history, history_count));
        auto fork = sampler.fork();
        std::vector<engine::TokenLogit> values(count);
        for (std::uint32_t i = 0; i < count; ++i) values[i] = {candidates[i].token, candidates[i].logit};
        const auto prepared = fork.prepare_distribution(values);
        engine::DraftProbabilityLeaseOwner owner;
        owner.begin_epoch();
        engine::GatheredDraftTokenDistribution gathered;
        gathered.lease = owner.lease(0);
        gathered.proposal = {proposal, proposal_mass};
        gathered.proposal_cdf_begin = proposal_cdf_begin;
        gathered.count = prepared.count;
        for (std::uint32_t i = 0; i < prepared.count; ++i)
            gathered.target_values[i] = {prepared.values[i].token, q_mass[i]};
        const auto before = fork.checkpoint().draw_count();
        const auto selected = fork.sample_speculative(proposal, gathered, values);
        *token = selected.token;
        *accepted = selected.accepted ? 1 : 0;
        *target_draws = fork.checkpoint().draw_count() - before;
        return 0;
    } catch (const std::exception&) { return -1; }
}

// TokenSampler::sample  (src/engine/sampling.cpp:841-852): one ordinary draw.
int ref_sample(std::uint64_t seed, float temperature, std::uint32_t top_k, float top_p, float min_p,
    float repetition_penalty, const std::uint32_t* history, std::uint32_t history_count,
    const RefTokenLogit* candidates, std::uint32_t count, std::uint32_t* token) {
    try {
        engine::TokenSampler sampler(sampler_options(temperature, top_k, top_p, min_p, repetition_penalty, seed));
        sampler.observe_tokens(std::span<const std::uint32_t>(history, history_count));
        std::vector<engine::TokenLogit> values(count);
        for (std::uint32_t i = 0; i < count; ++i) values[i] = {candidates[i].token, candidates[i].logit};
        *token = sampler.sample(values);
        return 0;
    } catch (const std::exception&) { return -1; }
}

// repack_kquant_weight_columns8 -> restore_native_kquant_weight round trip
// (src/tensor/kquant_packing.cpp:154,250): returns 1 when the restored bytes equal the input.
int ref_columns8_round_trip(int dtype, const std::uint8_t* weight, std::uint64_t k, std::uint64_t n) {
    try {
        const auto native = weight_tensor(dtype, weight, k, n);
        const auto packed = tensor::repack_kquant_weight_columns8(native.view());
        const auto restored = tensor::restore_native_kquant_weight(packed.view());
        return restored.bytes().size() == native.bytes().size()
            && std::memcmp(restored.bytes().data(), native.bytes().data(), native.bytes().size()) == 0 ? 1 : 0;
    } catch (const std::exception&) { return -1; }
}

}  // extern "C"
