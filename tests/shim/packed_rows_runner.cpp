// TEST INFRASTRUCTURE ONLY.  Drives the library through the reference's own command-context interface
// (cuda_command_context.cpp) with the reference's own test inputs and pass criteria: the packed-row
// part of hybrid_prefill_preserves_native_precision (tests/tensor/gemma3_metal_tests.cpp:1144-1366) --
// for the projection widths of the 12B model and both K-quant formats,
//   * a row's result is the same bits whether it is computed alone (encode_target_head_rows) or beside
//     one to seven other rows (encode_verifier_matmul with row counts 1, 2, 3, 4, 5, 7, 8);
//   * every result lies inside the reference's packed-reduction envelope around an independently decoded
//     double-precision dot product (operations = K / 32 + 32, :1268-1273);
//   * the adversarial Q4_K scale/minimum cancellation case (:1291-1365) stays finite, row-count
//     invariant and inside the same envelope.
// Weights come from the reference's stress generators, activations from its `pattern`, decoded weights
// from its block views.  Prints one line per case and "OK <checks>"; exits non-zero on the first failure.
#include "tensor/backends/metal/metal_command_context.hpp"

#include "tensor_test_support.hpp"
#include "test_support.hpp"

#include "local_gguf_engine/tensor/backend.hpp"
#include "local_gguf_engine/tensor/backend_buffer.hpp"
#include "local_gguf_engine/tensor/quantization.hpp"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <vector>

using namespace local_gguf_engine;
using namespace local_gguf_engine::tensor;
using local_gguf_engine::tensor::backends::metal::MetalCommandContext;
using runtime::BackendKind;
using tests::expect;
using tests::expect_close;

namespace {

std::uint64_t checks = 0;

BackendBuffer buffer(std::initializer_list<std::uint64_t> shape) {
    return allocate_backend_buffer(TensorDescriptor::from(Shape::from(shape), DType::f32), BackendKind::metal);
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
// The activation pattern of the reference's Metal tests (gemma3_metal_tests.cpp:67-74).
std::vector<float> pattern(std::size_t count, float scale) {
    std::vector<float> result(count);
    for (std::size_t i = 0; i < count; ++i)
        result[i] = std::sin(static_cast<float>(i % 8191U) * 0.071F) * scale + std::cos(static_cast<float>(i % 997U) * 0.027F) * scale * 0.37F;
    return result;
}
float envelope(std::uint32_t width, double absolute_sum) {
    const double operations = static_cast<double>(width / 32U + 32U);
    const double rounding = operations * std::numeric_limits<float>::epsilon();
    return static_cast<float>(rounding / (1.0 - rounding) * absolute_sum + 1.0e-6);
}

void projection_rows() {
    constexpr std::uint32_t rows = 8U;
    constexpr std::array<std::uint32_t, 7> row_counts {1U, 2U, 3U, 4U, 5U, 7U, 8U};
    for (const auto [width, columns] : std::array {std::array {3840U, 37U}, std::array {4096U, 37U}, std::array {15360U, 37U},
             std::array {256U, 63U}, std::array {256U, 64U}, std::array {256U, 65U}, std::array {256U, 129U}}) {
        const auto input_values = pattern(std::size_t(rows) * width, 0.027F);
        const auto input = upload(rows, width, input_values);
        for (const auto dtype : {DType::q4_k, DType::q6_k}) {
            const auto host_weight = dtype == DType::q4_k ? tests::tensor_q4_k_stress_gguf_weight_matrix(width, columns, 51U)
                                                          : tests::tensor_q6_k_stress_gguf_weight_matrix(width, columns, 71U);
            const auto weight = copy_tensor_to_backend(host_weight, BackendKind::metal);
            MetalCommandContext command("packed-row projection parity", false, true);
            // Every row alone.
            std::vector<std::vector<float>> alone;
            for (std::uint32_t row = 0U; row < rows; ++row) {
                const auto single = buffer({1U, columns});
                command.restart();
                command.encode_target_head_rows(input, row, weight, single, 1U);
                static_cast<void>(command.commit_and_wait());
                alone.push_back(values(single));
            }
            for (const auto count : row_counts) {
                const auto output = buffer({count, columns});
                command.restart();
                command.encode_verifier_matmul(input, weight, output, count);
                static_cast<void>(command.commit_and_wait());
                const auto batch = values(output);
                for (std::uint32_t row = 0U; row < count; ++row) {
                    expect(std::equal(alone[row].begin(), alone[row].end(), batch.begin() + std::size_t(row) * columns),
                        "verifier batches retain exact packed arithmetic for every row count");
                    ++checks;
                }
            }
            for (const auto row : {0U, 1U, 2U, 7U}) {
                for (std::uint32_t column = 0U; column < columns; ++column) {
                    double reference = 0.0, absolute_sum = 0.0;
                    for (std::uint32_t inner = 0U; inner < width; ++inner) {
                        const auto block = column * (width / 256U) + inner / 256U;
                        const float decoded = dtype == DType::q4_k ? q4_k_block_view(host_weight, block).dequantized_value(inner % 256U)
                                                                   : q6_k_block_view(host_weight, block).dequantized_value(inner % 256U);
                        const double product = static_cast<double>(input_values[std::size_t(row) * width + inner]) * decoded;
                        reference += product;
                        absolute_sum += std::abs(product);
                    }
                    expect_close(alone[row][column], static_cast<float>(reference), envelope(width, absolute_sum),
                        "native packed F32 projection agrees with independent decoded dot product");
                    ++checks;
                }
            }
            std::printf("projection %s K=%u N=%u: rows 1-8 invariant, inside the envelope\n", dtype == DType::q4_k ? "Q4_K" : "Q6_K", width, columns);
        }
    }
}

void q4_cancellation() {
    constexpr std::uint32_t rows = 5U, columns = 3U;
    for (const auto width : {3840U, 15360U}) {
        auto input_values = pattern(std::size_t(rows) * width, 0.027F);
        for (std::size_t i = 0U; i < input_values.size(); ++i) {
            input_values[i] += float(i % 11U + 1U) * 0x1p-20F;
            if ((i / 16U) % 2U != 0U) input_values[i] = -input_values[i];
        }
        const auto input = upload(rows, width, input_values);
        auto host_weight = tests::tensor_q4_k_stress_gguf_weight_matrix(width, columns, 0U);
        auto bytes = host_weight.mutable_bytes();
        const auto blocks = width / 256U;
        for (std::uint32_t column = 0U; column < columns; ++column) {
            for (std::uint32_t block = 0U; block < blocks; ++block) {
                // d = 1365/4096, dmin = (1364 or 1366)/4096, every group scale 1 and minimum 13, every code 13:
                // each weight is +-13/4096, the small difference of two terms about 1365 times larger.
                auto* packed = bytes.data() + (std::size_t(column) * blocks + block) * 144U;
                packed[0] = 0x55U; packed[1] = 0x35U;
                packed[2] = (column + block) % 2U == 0U ? 0x54U : 0x56U;
                packed[3] = 0x35U;
                for (std::uint32_t group = 0U; group < 4U; ++group) { packed[4U + group] = 1U; packed[8U + group] = 13U; packed[12U + group] = 0xd1U; }
                std::fill(packed + 16U, packed + 144U, std::uint8_t {0xddU});
            }
        }
        const auto weight = copy_tensor_to_backend(host_weight, BackendKind::metal);
        MetalCommandContext command("Q4 scale/min cancellation", false, true);
        for (std::uint32_t count = 1U; count <= rows; ++count) {
            const auto output = buffer({count, columns});
            const auto single = buffer({1U, columns});
            command.restart();
            command.encode_verifier_matmul(input, weight, output, count);
            command.encode_target_head_rows(input, count - 1U, weight, single, 1U);
            static_cast<void>(command.commit_and_wait());
            const auto actual = values(output), scalar = values(single);
            for (std::uint32_t column = 0U; column < columns; ++column) {
                const std::uint32_t row = count - 1U;
                double reference = 0.0, absolute_sum = 0.0;
                for (std::uint32_t inner = 0U; inner < width; ++inner) {
                    const double decoded = (column + inner / 256U) % 2U == 0U ? 13.0 / 4096.0 : -13.0 / 4096.0;
                    const double product = double(input_values[std::size_t(row) * width + inner]) * decoded;
                    reference += product;
                    absolute_sum += std::abs(product);
                }
                const auto value = actual[std::size_t(row) * columns + column];
                expect(std::isfinite(value), "Q4 cancellation must produce finite results");
                expect(value == scalar[column], "Q4 cancellation changed ordinary/verifier arithmetic");
                expect_close(value, static_cast<float>(reference), envelope(width, absolute_sum),
                    "Q4 scale/min cancellation agrees with independently retained dense weights");
                checks += 3U;
            }
        }
        std::printf("cancellation K=%u: finite, invariant, inside the envelope\n", width);
    }
}

}  // namespace

int main() {
    try {
        expect(tensor_backend_is_available(BackendKind::metal), "no device backend");
        projection_rows();
        q4_cancellation();
    } catch (const std::exception& error) {
        std::printf("FAILED: %s\n", error.what());
        return 1;
    }
    std::printf("OK %llu checks\n", static_cast<unsigned long long>(checks));
    return 0;
}
