// TEST INFRASTRUCTURE ONLY.  Drives the library's block-schedule operators through the reference's own
// command-context interface (cuda_command_context.cpp) with the inputs and pass criteria of the reference's
// operator tests in tests/tensor/gemma3_metal_tests.cpp:
//   * native_q6_embedding_and_head (:511-552): a tied Q6_K table gathered with a token offset and scaled by
//     sqrt(hidden) within 2e-6 of the reference's own block decode, and the same table as the output head within
//     3e-5 of a double-precision dot product of the decoded weights;
//   * head_norm_and_scaled_rope (:554-633): per-head RMS norm within 6e-7, the half-split rotation at positions
//     1, 1024, 32769 and 131071 under both frequency policies inside the reference's phase-error bound, the
//     F32 key store equal to the query rotation bit for bit, the F32 value store lossless, and binary16 keys
//     rounded only after the F32 rotation;
//   * native_half_cache_cast_rounding (:87-128): the 28 pinned binary16 round-to-nearest-even cases (signed
//     zeros, both tie parities, the subnormal boundary, overflow) through an unrotated cache store;
//   * half_cache_numerical_status (:130-160): a non-finite binary16 K or V sets the status bit, a later finite
//     store keeps it, earlier bits survive, and the check costs no dispatch;
//   * uncapped_candidate_selection (:1112-1142): ordering, deterministic ties, exact logits and the history
//     token's pair for a 1025-entry row, then the greedy request.
// Prints one line per section and "OK <checks>"; exits non-zero on the first failure.
#include "tensor/backends/metal/metal_command_context.hpp"

#include "tensor_test_support.hpp"
#include "test_support.hpp"

#include "local_gguf_engine/engine/gemma2_metal_plan.hpp"
#include "local_gguf_engine/engine/sampling.hpp"
#include "local_gguf_engine/tensor/backend.hpp"
#include "local_gguf_engine/tensor/backend_buffer.hpp"
#include "local_gguf_engine/tensor/quantization.hpp"

#include <array>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <span>
#include <vector>

using namespace local_gguf_engine;
using namespace local_gguf_engine::tensor;
using local_gguf_engine::tensor::backends::metal::MetalCommandContext;
using runtime::BackendKind;
using tests::expect;
using tests::expect_close;

namespace {

std::uint64_t checks = 0;

BackendBuffer buffer(std::initializer_list<std::uint64_t> shape, DType dtype = DType::f32) {
    return allocate_backend_buffer(TensorDescriptor::from(Shape::from(shape), dtype), BackendKind::metal);
}
BackendBuffer upload(std::uint32_t rows, std::uint32_t columns, const std::vector<float>& data) {
    return copy_tensor_to_backend(tests::tensor_f32_matrix(rows, columns, data), BackendKind::metal);
}
std::vector<float> values(const BackendBuffer& input) {
    const auto copied = copy_tensor_from_backend(input);
    std::vector<float> result(copied.bytes().size() / sizeof(float));
    std::memcpy(result.data(), copied.bytes().data(), copied.bytes().size());
    return result;
}
std::vector<std::uint16_t> half_bits(const BackendBuffer& input) {
    const auto copied = copy_tensor_from_backend(input);
    expect(copied.descriptor().dtype == DType::f16, "half readback requires F16 storage");
    std::vector<std::uint16_t> result(copied.descriptor().element_count);
    std::memcpy(result.data(), copied.bytes().data(), copied.bytes().size());
    return result;
}
// 32-bit words in an F32-typed buffer, written the way the reference stages ids and positions.
BackendBuffer words(std::span<const std::uint32_t> source) {
    auto result = buffer({source.size()});
    MetalCommandContext staging("staging", false, true);
    staging.write_u32s(result, 0U, source);
    return result;
}
// The activation pattern of the reference's Metal tests (gemma3_metal_tests.cpp:67-74).
std::vector<float> pattern(std::size_t count, float scale) {
    std::vector<float> result(count);
    for (std::size_t i = 0; i < count; ++i)
        result[i] = std::sin(static_cast<float>(i % 8191U) * 0.071F) * scale + std::cos(static_cast<float>(i % 997U) * 0.027F) * scale * 0.37F;
    return result;
}

void q6_embedding_and_head() {
    constexpr std::uint32_t hidden = 3840U, vocabulary = 7U, rows = 3U;
    const auto weight = tests::tensor_q6_k_stress_gguf_weight_matrix(hidden, vocabulary, 137U);
    const auto resident = copy_tensor_to_backend(weight, BackendKind::metal);
    const std::array<std::uint32_t, 4> ids {6U, 2U, 0U, 5U};
    const auto tokens = words(ids);
    const auto embeddings = buffer({rows, hidden});
    const float scale = std::sqrt(static_cast<float>(hidden));
    MetalCommandContext command("tied Q6 embedding and head", false, true);
    command.encode_embedding(tokens, resident, embeddings, scale, 1U, rows);       // ids[1..3]
    static_cast<void>(command.commit_and_wait());
    const auto gathered = values(embeddings);
    for (std::uint32_t row = 0U; row < rows; ++row)
        for (std::uint32_t column = 0U; column < hidden; ++column) {
            const auto block = q6_k_block_view(weight, ids[row + 1U] * (hidden / 256U) + column / 256U);
            expect_close(gathered[row * hidden + column], block.dequantized_value(column % 256U) * scale, 2.0e-6F,
                "Q6 embedding uses every signed scale and high-bit group");
            ++checks;
        }
    const auto input_values = pattern(4U * hidden, 0.03F);
    const auto input = upload(4U, hidden, input_values);
    const auto logits = buffer({rows, vocabulary});
    command.restart();
    command.encode_target_head_rows(input, 1U, resident, logits, rows);
    static_cast<void>(command.commit_and_wait());
    const auto head = values(logits);
    for (std::uint32_t row = 0U; row < rows; ++row)
        for (std::uint32_t token = 0U; token < vocabulary; ++token) {
            double sum = 0.0;
            for (std::uint32_t column = 0U; column < hidden; ++column)
                sum += static_cast<double>(input_values[(row + 1U) * hidden + column])
                    * q6_k_block_view(weight, token * (hidden / 256U) + column / 256U).dequantized_value(column % 256U);
            expect_close(head[row * vocabulary + token], static_cast<float>(sum), 3.0e-5F, "Q6 output head agrees with the decoded dot product");
            ++checks;
        }
    std::printf("Q6_K embedding gather (offset 1, 3 rows) and tied head: inside the reference's tolerances\n");
}

void head_norm_and_rope() {
    constexpr std::uint32_t rows = 4U, heads = 3U, dimension = 256U;
    auto input_values = pattern(rows * heads * dimension, 1.3F);
    for (std::uint32_t row = 0U; row < rows; ++row)
        for (std::uint32_t head = 0U; head < heads; ++head)
            for (std::uint32_t column = 0U; column < dimension; ++column) input_values[(row * heads + head) * dimension + column] *= static_cast<float>(head + 1U);
    auto weights = pattern(dimension, 0.2F);
    for (auto& w : weights) w += 0.7F;
    weights[19] = -0.25F;
    const std::array<std::uint32_t, rows> position_values {1U, 1024U, 32769U, 131071U};
    const auto positions = words(position_values);
    const auto input = upload(rows, heads * dimension, input_values);
    const auto weight = upload(1U, dimension, weights);
    const auto normalized = buffer({rows, heads * dimension});
    const auto output = buffer({rows, heads * dimension});
    const auto value_values = pattern(rows * heads * dimension, 0.07F);
    const auto value = upload(rows, heads * dimension, value_values);
    const auto stored_key = buffer({rows, heads, dimension}), stored_value = buffer({rows, heads, dimension});
    const auto half_key = buffer({rows, heads, dimension}, DType::f16), half_value = buffer({rows, heads, dimension}, DType::f16);
    constexpr float epsilon = 1.0e-6F;
    for (const auto frequency : std::array<std::array<float, 2>, 2> {{{10000.0F, 1.0F}, {1000000.0F, 0.125F}}}) {
        MetalCommandContext command("per-head normalization and position policy", false, true);
        command.encode_head_rms_norm(input, weight, normalized, epsilon, rows, heads, dimension);
        command.encode_memory_barrier();
        command.encode_verifier_rope(normalized, positions, output, rows, heads, dimension, dimension, frequency[0], frequency[1]);
        command.encode_verifier_kv_store(normalized, value, positions, stored_key, stored_value, rows, heads, dimension, dimension, frequency[0], frequency[1]);
        command.encode_memory_barrier();
        // V = the F32 query rotation: equal binary16 outputs show that keys are narrowed after the rotation.
        command.encode_verifier_kv_store(normalized, output, positions, half_key, half_value, rows, heads, dimension, dimension, frequency[0], frequency[1]);
        static_cast<void>(command.commit_and_wait());
        const auto norm = values(normalized), rotated = values(output);
        expect(values(stored_key) == rotated, "query and key use identical half-split rotation arithmetic");
        expect(values(stored_value) == value_values, "the F32 value store does not narrow");
        expect(half_bits(half_key) == half_bits(half_value), "binary16 keys are rounded only after the F32 rotation");
        checks += 3U;
        for (std::uint32_t row = 0U; row < rows; ++row)
            for (std::uint32_t head = 0U; head < heads; ++head) {
                const auto offset = (row * heads + head) * dimension;
                double squares = 0.0;
                for (std::uint32_t column = 0U; column < dimension; ++column) squares += static_cast<double>(input_values[offset + column]) * input_values[offset + column];
                const double factor = 1.0 / std::sqrt(squares / dimension + epsilon);
                for (std::uint32_t column = 0U; column < dimension; ++column) {
                    expect_close(norm[offset + column], static_cast<float>(input_values[offset + column] * factor * weights[column]), 6.0e-7F,
                        "independent per-head RMS denominator");
                    ++checks;
                }
                for (std::uint32_t pair = 0U; pair < dimension / 2U; ++pair) {
                    const double angle = static_cast<double>(position_values[row])
                        * std::pow(static_cast<double>(frequency[0]), -static_cast<double>(2U * pair) / dimension) * frequency[1];
                    const float a = norm[offset + pair], b = norm[offset + pair + dimension / 2U];
                    // The reference's bound: four relative F32 rounding units of phase, propagated through the rotation.
                    const auto tolerance = static_cast<float>(4.0 * std::numeric_limits<float>::epsilon() * std::abs(angle) * (std::abs(a) + std::abs(b)) + 2.0e-6);
                    expect_close(rotated[offset + pair], static_cast<float>(a * std::cos(angle) - b * std::sin(angle)), tolerance,
                        "first rotation component at a high logical position");
                    expect_close(rotated[offset + pair + dimension / 2U], static_cast<float>(a * std::sin(angle) + b * std::cos(angle)), tolerance,
                        "second rotation component at a high logical position");
                    checks += 2U;
                }
            }
        std::printf("head norm + rotation, base %.0f scale %.3f, positions 1 / 1024 / 32769 / 131071: inside the reference's bounds\n", frequency[0], frequency[1]);
    }
}

void half_cache_rounding() {
    struct Case { float input; std::uint16_t bits; };
    // IEEE binary16 nearest-even results stated independently of any conversion routine (gemma3_metal_tests.cpp:92-108).
    const std::array cases {
        Case {0.0F, 0x0000U}, Case {-0.0F, 0x8000U}, Case {1.0F, 0x3c00U}, Case {-1.0F, 0xbc00U},
        Case {1.0F + 0x1p-11F, 0x3c00U}, Case {-1.0F - 0x1p-11F, 0xbc00U}, Case {1.0F + 0x1.8p-10F, 0x3c02U}, Case {-1.0F - 0x1.8p-10F, 0xbc02U},
        Case {std::nextafter(1.0F + 0x1p-11F, 0.0F), 0x3c00U}, Case {std::nextafter(1.0F + 0x1p-11F, 2.0F), 0x3c01U},
        Case {0x1p-24F, 0x0001U}, Case {-0x1p-24F, 0x8001U}, Case {0x1p-25F, 0x0000U}, Case {-0x1p-25F, 0x8000U},
        Case {0x1.8p-24F, 0x0002U}, Case {-0x1.8p-24F, 0x8002U}, Case {0x1p-14F - 0x1p-24F, 0x03ffU}, Case {0x1p-14F - 0x1p-25F, 0x0400U},
        Case {0x1p-14F, 0x0400U}, Case {-0x1p-14F, 0x8400U}, Case {65504.0F, 0x7bffU}, Case {-65504.0F, 0xfbffU},
        Case {65519.0F, 0x7bffU}, Case {-65519.0F, 0xfbffU}, Case {65520.0F, 0x7c00U}, Case {-65520.0F, 0xfc00U},
        Case {65536.0F, 0x7c00U}, Case {-65536.0F, 0xfc00U},
    };
    constexpr std::uint32_t width = 256U;
    std::vector<float> input(width);
    for (std::size_t i = 0; i < input.size(); ++i) input[i] = cases[i % cases.size()].input;
    const auto raw = upload(1U, width, input);
    const auto key = buffer({1U, width}, DType::f16), value = buffer({1U, width}, DType::f16);
    const std::array<std::uint32_t, 1> position {0U};
    const auto positions = words(position);
    MetalCommandContext command("binary16 cache narrowing", false, true);
    command.encode_verifier_kv_store(raw, raw, positions, key, value, 1U, 1U, width, 0U, 10000.0F);     // rotation off isolates the narrowing
    static_cast<void>(command.commit_and_wait());
    const auto keys = half_bits(key), vals = half_bits(value);
    for (std::size_t i = 0; i < input.size(); ++i) {
        expect(keys[i] == cases[i % cases.size()].bits && vals[i] == cases[i % cases.size()].bits,
            "K/V narrowing must implement the pinned binary16 rounding at case " + std::to_string(i % cases.size()));
        ++checks;
    }
    std::printf("binary16 cache narrowing: 28 pinned cases x K and V\n");
}

void half_cache_status() {
    constexpr std::uint32_t width = 256U;
    constexpr std::uint32_t nonfinite = 8U;       // the reference's verifier_kv_nonfinite_status (metal_kernels.mm:2484)
    const auto key = buffer({1U, width}, DType::f16), value = buffer({1U, width}, DType::f16);
    const auto status = buffer({1U});
    const std::array<std::uint32_t, 1> position {0U};
    const auto positions = words(position);
    std::vector<float> finite(width, 0.25F);
    finite[3U] = 65519.0F;            // rounds to the largest finite half: not an overflow
    finite[4U] = -65519.0F;
    finite[5U] = 0x1p-24F;
    const auto finite_raw = upload(1U, width, finite);
    for (const auto fault : {0U, 1U, 2U, 3U, 4U}) {
        auto raw_values = finite;
        if (fault == 1U || fault == 3U) raw_values[19U] = 65520.0F;
        if (fault == 2U) raw_values[19U] = std::numeric_limits<float>::quiet_NaN();
        if (fault == 4U) raw_values[19U] = -std::numeric_limits<float>::infinity();
        const auto changed = upload(1U, width, raw_values);
        const auto& raw_key = fault == 1U || fault == 4U ? changed : finite_raw;
        const auto& raw_value = fault == 2U || fault == 3U ? changed : finite_raw;
        MetalCommandContext command("checked half-cache numerical status", false, true);
        command.write_u32(status, 5U);
        command.encode_verifier_kv_store(raw_key, raw_value, positions, key, value, 1U, 1U, width, 0U, 10000.0F, 1.0F, &status);
        command.encode_memory_barrier();
        // A later finite layer must not clear the first layer's bit.
        command.encode_verifier_kv_store(finite_raw, finite_raw, positions, key, value, 1U, 1U, width, 0U, 10000.0F, 1.0F, &status);
        const auto stats = command.commit_and_wait();
        expect(command.read_verifier_status(status) == (5U | (fault == 0U ? 0U : nonfinite)),
            "checked half stores report non-finite K/V and keep earlier status bits");
        expect(stats.compute_dispatch_count == 2U, "the numerical check adds no dispatch");
        checks += 2U;
    }
    const auto half_status = buffer({2U}, DType::f16);
    for (const auto* bad : {&half_status}) {
        MetalCommandContext command("invalid status word", false, true);
        bool rejected = false;
        try {
            command.encode_verifier_kv_store(finite_raw, finite_raw, positions, key, key, 1U, 1U, width, 0U, 10000.0F, 1.0F, bad);
        } catch (const std::invalid_argument&) { rejected = true; }
        expect(rejected && command.commit_and_wait().compute_dispatch_count == 0U, "an invalid status word fails before dispatch");
        ++checks;
    }
    std::printf("binary16 cache status word: overflow, NaN and infinity in K or V, sticky, no extra dispatch\n");
}

void candidate_selection() {
    constexpr std::uint32_t vocabulary = 1025U;
    std::vector<float> logits(vocabulary, -2.0F);
    logits[1000] = 101.0F; logits[1001] = 101.0F; logits[1010] = 100.0F; logits[7] = -99.75F;
    const auto input = upload(1U, vocabulary, logits);
    const engine::Gemma2MetalSelectionWorkspace workspace {
        buffer({2U * 3U * engine::token_sampler_max_candidates}), buffer({2U * 3U * engine::token_sampler_max_candidates}),
        buffer({2U * (2U + 2U * engine::token_sampler_max_candidates)}), buffer({2U * engine::token_sampler_max_repetition_window}),
    };
    MetalCommandContext command("uncapped selection", false, true);
    engine::TokenSelectionRequest request;
    request.top_k = 2U; request.base_candidate_count = 3U;
    request.history_token_count = 1U; request.history_token_ids[0] = 7U;
    static_cast<void>(command.encode_token_candidates(input, workspace, request, 0.0F));
    static_cast<void>(command.commit_and_wait());
    auto result = command.read_token_candidates(workspace);
    expect(result.count == 4U && result.values[0].token == 1000U && result.values[1].token == 1001U,
        "the compact selector keeps ordering and deterministic ties");
    ++checks;
    for (std::uint32_t i = 0U; i < result.count; ++i) {
        expect(result.values[i].logit == logits[result.values[i].token], "selected logits keep their values exactly");
        ++checks;
    }
    request = {};
    command.restart();
    static_cast<void>(command.encode_token_candidates(input, workspace, request, 0.0F));
    static_cast<void>(command.commit_and_wait());
    result = command.read_token_candidates(workspace);
    expect(result.count == 1U && result.values[0].token == 1000U && result.values[0].logit == 101.0F, "the greedy request uses the same tie and logit policy");
    ++checks;
    std::printf("candidate selection over 1025 logits: ties, exact logits, history pair, greedy\n");
}

}  // namespace

int main() {
    try {
        expect(tensor_backend_is_available(BackendKind::metal), "no device backend");
        q6_embedding_and_head();
        head_norm_and_rope();
        half_cache_rounding();
        half_cache_status();
        candidate_selection();
    } catch (const std::exception& error) {
        std::printf("FAILED: %s\n", error.what());
        return 1;
    }
    std::printf("OK %llu checks\n", static_cast<unsigned long long>(checks));
    return 0;
}
