// TEST INFRASTRUCTURE ONLY -- nothing under guffin_b200/ includes or links this file.
//
// The reference's GPU seam, implemented over the C ABI of include/guffin_b200.h and compiled against
// the reference's own headers (their location comes from the build recipe, never from this file):
//   * the backend-buffer factories the reference defines in src/tensor/backend_buffer.mm
//     (include/local_gguf_engine/tensor/backend_buffer.hpp:17-68), over gf_malloc / gf_upload /
//     gf_download;
//   * the methods of class MetalCommandContext that the packed-row projection tests call
//     (src/tensor/backends/metal/metal_command_context.hpp:54-369): construction, restart, write_u32s,
//     encode_verifier_matmul, encode_target_head_rows, encode_gelu_tanh_multiply,
//     commit / wait_until_completed / commit_and_wait;
//   * the operator methods the reference's tensor tests drive one by one: encode_embedding, encode_rms_norm,
//     encode_rms_norm_add, encode_head_rms_norm, encode_verifier_rope, encode_verifier_kv_store (with its
//     numerical status word), read_verifier_status, encode_token_candidates / read_token_candidates;
//   * availability (src/tensor/backends/metal_backend.hpp: is_available, unavailable_reason).
// A maintainer porting the engine would grow this file into the real CUDA command context; here it
// proves that the reference's portable C++ drives the library through its own interface.
//
// Status codes of the C ABI become the exception types the reference's callers expect.
#include "tensor/backends/metal/metal_command_context.hpp"
#include "tensor/backends/metal_backend.hpp"

#include "local_gguf_engine/runtime/backend_error.hpp"
#include "local_gguf_engine/tensor/backend.hpp"

#include "guffin_b200.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>
#include <stdexcept>
#include <string>

namespace local_gguf_engine::tensor {

namespace {

using runtime::BackendError;
using runtime::BackendErrorCode;
using runtime::BackendKind;

// The reference's BackendKind has two members; its GPU member names the device backend here.
constexpr BackendKind device_kind = BackendKind::metal;

void check(int status) {
    if (status == GF_OK) return;
    const std::string message = gf_last_error();
    switch (status) {
        case GF_ERR_INVALID: throw std::invalid_argument(message);
        case GF_ERR_STATE: throw std::logic_error(message);
        case GF_ERR_NUMERIC: throw std::overflow_error(message);
        case GF_ERR_UNAVAILABLE: throw BackendError(BackendErrorCode::unavailable_metal_device, device_kind, message);
        default: throw BackendError(BackendErrorCode::metal_execution_failed, device_kind, message);
    }
}

int gguf_type(DType dtype) {
    switch (dtype) {
        case DType::f32: return GF_F32;
        case DType::f16: return GF_F16;
        case DType::q8_0: return GF_Q8_0;
        case DType::q4_k: return GF_Q4_K;
        case DType::q6_k: return GF_Q6_K;
    }
    throw std::invalid_argument("unknown tensor dtype");
}

class DeviceStorage final : public detail::BackendBufferStorage {
public:
    explicit DeviceStorage(const TensorDescriptor& descriptor) : descriptor_(descriptor) {
        check(gf_malloc(&data_, std::max<std::size_t>(descriptor.byte_count, 16U)));
    }
    ~DeviceStorage() override {
        if (packed_) gf_free(packed_);
        if (data_) gf_free(data_);
    }
    [[nodiscard]] BackendKind backend() const noexcept override { return device_kind; }
    [[nodiscard]] const TensorDescriptor& descriptor() const noexcept override { return descriptor_; }
    [[nodiscard]] void* data() const noexcept { return data_; }

    // A quantised GGUF weight matrix [K, N] in the library's streaming layout, made on first use and kept
    // (the reference repacks weights once at load the same way, kquant_packing.cpp).
    [[nodiscard]] const void* packed_weight() const {
        std::lock_guard<std::mutex> lock(guard_);
        if (!packed_) {
            const auto k = descriptor_.shape.dimension(0), n = descriptor_.shape.dimension(1);
            const auto bytes = gf_packed_weight_bytes(gguf_type(descriptor_.dtype), k, n);
            if (bytes == 0) check(GF_ERR_INVALID);
            check(gf_malloc(&packed_, bytes));
            check(gf_pack_weight(gguf_type(descriptor_.dtype), data_, k, n, packed_, nullptr));
            check(gf_stream_synchronize(nullptr));
        }
        return packed_;
    }

private:
    TensorDescriptor descriptor_;
    void* data_ = nullptr;
    mutable void* packed_ = nullptr;
    mutable std::mutex guard_;
};

const DeviceStorage& device_storage(const BackendBuffer& buffer) {
    const auto* storage = dynamic_cast<const DeviceStorage*>(&backend_buffer_storage(buffer));
    if (!storage) throw std::invalid_argument("buffer does not live on the device backend");
    return *storage;
}

void require_device(BackendKind backend) {
    if (backend != device_kind)
        throw BackendError(BackendErrorCode::unsupported_backend, backend, "this build binds the device backend only");
}

}  // namespace

// ---- backend_buffer.hpp:17-68 ----

detail::BackendBufferStorage::~BackendBufferStorage() = default;

BackendBuffer detail::make_backend_buffer(std::shared_ptr<BackendBufferStorage> storage) { return BackendBuffer(std::move(storage)); }

BackendBuffer::BackendBuffer(std::shared_ptr<detail::BackendBufferStorage> storage) : storage_(std::move(storage)) {}
runtime::BackendKind BackendBuffer::backend() const noexcept { return storage_->backend(); }
const TensorDescriptor& BackendBuffer::descriptor() const noexcept { return storage_->descriptor(); }

BackendBuffer copy_tensor_to_backend(const TensorStorage& storage, runtime::BackendKind backend) {
    require_device(backend);
    auto device = std::make_shared<DeviceStorage>(storage.descriptor());
    check(gf_upload(device->data(), storage.bytes().data(), storage.bytes().size(), nullptr));
    check(gf_stream_synchronize(nullptr));
    return BackendBuffer(std::move(device));
}

BackendBuffer copy_tensor_view_to_backend(const TensorView& view, runtime::BackendKind backend) {
    require_device(backend);
    auto device = std::make_shared<DeviceStorage>(view.descriptor());
    check(gf_upload(device->data(), view.bytes().data(), view.bytes().size(), nullptr));
    check(gf_stream_synchronize(nullptr));
    return BackendBuffer(std::move(device));
}

BackendBuffer allocate_backend_buffer(const TensorDescriptor& descriptor, runtime::BackendKind backend) {
    require_device(backend);
    auto device = std::make_shared<DeviceStorage>(descriptor);
    check(gf_memset(device->data(), 0, std::max<std::size_t>(descriptor.byte_count, 16U), nullptr));
    check(gf_stream_synchronize(nullptr));
    return BackendBuffer(std::move(device));
}

TensorStorage copy_tensor_from_backend(const BackendBuffer& buffer) {
    const auto& device = device_storage(buffer);
    auto host = TensorStorage::allocate(device.descriptor());
    check(gf_download(host.mutable_bytes().data(), device.data(), host.mutable_bytes().size(), nullptr));
    check(gf_stream_synchronize(nullptr));
    return host;
}

const detail::BackendBufferStorage& backend_buffer_storage(const BackendBuffer& buffer) noexcept { return *buffer.storage_; }

// ---- metal_backend.hpp: availability ----

namespace backends::metal {

bool is_available() noexcept {
    int count = 0;
    return gf_device_count(&count) == GF_OK && count > 0;
}

std::string unavailable_reason() { return is_available() ? std::string() : std::string("no CUDA device is visible"); }

// ---- metal_command_context.hpp:54-369 (the part the projection tests drive) ----

struct MetalCommandContext::Impl {
    std::string label;
    void* stream = nullptr;
    void* workspace = nullptr;
    std::size_t workspace_bytes = 0;
    bool committed = false;
    MetalCommandStats stats;
    void* spare_status = nullptr;                       // where unobserved device status bits go
    // Selection results of the library, keyed by the reference workspace they were encoded for.
    struct Selection { void* requests = nullptr; void* results = nullptr; void* workspace = nullptr; std::size_t workspace_bytes = 0; };
    std::map<const void*, Selection> selections;

    void encoding() const {
        if (committed) throw std::logic_error("the command has been committed: restart it first");
    }
    std::uint32_t* status_word() {
        if (!spare_status) { check(gf_malloc(&spare_status, 16U)); check(gf_memset(spare_status, 0, 16U, stream)); }
        return static_cast<std::uint32_t*>(spare_status);
    }

    void* scratch(std::size_t bytes) {
        if (bytes > workspace_bytes) {
            if (workspace) { check(gf_stream_synchronize(stream)); gf_free(workspace); workspace = nullptr; }
            check(gf_malloc(&workspace, bytes));
            workspace_bytes = bytes;
        }
        return workspace;
    }

    // rows [first_row, first_row + row_count) of `input` times the weight, into rows 0.. of `output`.
    // Row counts above four go in groups of four: the library adds the same products in the same order
    // for every row count from one to four, so a row's value never depends on its neighbours.
    void project(const BackendBuffer& input, std::uint32_t first_row, const BackendBuffer& weight, const BackendBuffer& output,
                 std::uint32_t row_count) {
        if (committed) throw std::logic_error("the command has been committed: restart it first");
        const auto& w = device_storage(weight);
        const auto& x = device_storage(input);
        const auto& y = device_storage(output);
        const auto& wd = w.descriptor();
        if (wd.shape.rank() != 2U || x.descriptor().dtype != DType::f32 || y.descriptor().dtype != DType::f32)
            throw std::invalid_argument("projection needs F32 activations and a [K, N] weight matrix");
        if (wd.packing != TensorPacking::canonical)
            throw std::invalid_argument("this context takes weights in their native GGUF block order");
        const std::uint64_t k = wd.shape.dimension(0), n = wd.shape.dimension(1);
        if (row_count == 0U || (std::uint64_t(first_row) + row_count) * k > x.descriptor().element_count
            || std::uint64_t(row_count) * n > y.descriptor().element_count)
            throw std::invalid_argument("projection rows exceed the bound buffers");
        const int dtype = gguf_type(wd.dtype);
        const void* packed = w.packed_weight();
        void* scratch_dev = scratch(std::max<std::size_t>(gf_matmul_workspace_bytes(dtype, 4U, k, n), 256U));
        for (std::uint32_t done = 0U; done < row_count; done += 4U) {
            const std::uint32_t rows = std::min(4U, row_count - done);
            check(gf_matmul(dtype, packed, static_cast<const float*>(x.data()) + (std::uint64_t(first_row) + done) * k,
                            static_cast<float*>(y.data()) + std::uint64_t(done) * n, rows, k, n, scratch_dev, stream));
            ++stats.compute_dispatch_count;
            if (wd.dtype == DType::q4_k) ++(rows == 1U ? stats.q4_decode_projection_count : rows == 2U ? stats.q4_width_two_projection_count : stats.q4_small_batch_projection_count);
            if (wd.dtype == DType::q6_k) ++(rows == 1U ? stats.q6_decode_projection_count : rows == 2U ? stats.q6_width_two_projection_count : stats.q6_small_batch_projection_count);
            if (wd.dtype == DType::q8_0) ++(rows == 2U ? stats.q8_width_two_projection_count : stats.q8_decode_projection_count);
        }
    }
};

MetalCommandContext::MetalCommandContext(std::string_view label, bool, bool) : impl_(std::make_unique<Impl>()) {
    impl_->label = std::string(label);
    check(gf_stream_create(&impl_->stream));
    impl_->stats.command_buffer_count = 1U;
}

MetalCommandContext::~MetalCommandContext() {
    if (!impl_) return;
    if (impl_->stream) { gf_stream_synchronize(impl_->stream); gf_stream_destroy(impl_->stream); }
    if (impl_->workspace) gf_free(impl_->workspace);
    if (impl_->spare_status) gf_free(impl_->spare_status);
    for (auto& [key, selection] : impl_->selections) {
        if (selection.requests) gf_free(selection.requests);
        if (selection.results) gf_free(selection.results);
        if (selection.workspace) gf_free(selection.workspace);
    }
}

MetalCommandContext::MetalCommandContext(MetalCommandContext&&) noexcept = default;
MetalCommandContext& MetalCommandContext::operator=(MetalCommandContext&&) noexcept = default;

void MetalCommandContext::restart() {
    if (impl_->committed) check(gf_stream_synchronize(impl_->stream));
    impl_->committed = false;
    impl_->stats = MetalCommandStats();
    impl_->stats.command_buffer_count = 1U;
}

void MetalCommandContext::write_u32s(const BackendBuffer& destination, std::uint32_t element_offset, std::span<const std::uint32_t> values) {
    const auto& d = device_storage(destination);
    if ((std::uint64_t(element_offset) + values.size()) * sizeof(std::uint32_t) > d.descriptor().byte_count)
        throw std::invalid_argument("write_u32s exceeds its destination");
    // An immediate host write in the reference (shared memory); here a copy that completes before returning.
    check(gf_upload(static_cast<std::uint32_t*>(d.data()) + element_offset, values.data(), values.size_bytes(), impl_->stream));
    check(gf_stream_synchronize(impl_->stream));
}

void MetalCommandContext::write_u32(const BackendBuffer& destination, std::uint32_t value) { write_u32s(destination, 0U, std::span<const std::uint32_t>(&value, 1U)); }

void MetalCommandContext::encode_verifier_matmul(const BackendBuffer& input, const BackendBuffer& weight, const BackendBuffer& output,
    std::uint32_t row_count, bool, const BackendBuffer*) {
    impl_->project(input, 0U, weight, output, row_count);
}

void MetalCommandContext::encode_target_head_rows(const BackendBuffer& input, std::uint32_t input_row_start, const BackendBuffer& weight,
    const BackendBuffer& logits_tile, std::uint32_t row_count) {
    impl_->project(input, input_row_start, weight, logits_tile, row_count);
}

void MetalCommandContext::encode_target_head_q8_rows(const BackendBuffer& input, std::uint32_t input_row_start, const BackendBuffer& weight,
    const BackendBuffer& logits_tile, std::uint32_t row_count) {
    impl_->project(input, input_row_start, weight, logits_tile, row_count);
}

void MetalCommandContext::encode_gelu_tanh_multiply(const BackendBuffer& gate, const BackendBuffer& up, const BackendBuffer& output,
    std::uint64_t element_count, const BackendBuffer*) {
    const auto& g = device_storage(gate);
    const std::uint64_t count = element_count ? element_count : g.descriptor().element_count;
    check(gf_gelu_tanh_multiply(static_cast<const float*>(g.data()), static_cast<const float*>(device_storage(up).data()),
                                static_cast<float*>(device_storage(output).data()), count, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

namespace {

const float* floats(const BackendBuffer& buffer) {
    const auto& storage = device_storage(buffer);
    if (storage.descriptor().dtype != DType::f32) throw std::invalid_argument("an F32 buffer is required");
    return static_cast<const float*>(storage.data());
}
float* mutable_floats(const BackendBuffer& buffer) { return const_cast<float*>(floats(buffer)); }
// Words the reference keeps in F32-typed shared buffers (token ids, positions, status).
std::uint32_t* words_of(const BackendBuffer& buffer) { return static_cast<std::uint32_t*>(device_storage(buffer).data()); }

}  // namespace

void MetalCommandContext::encode_embedding(const BackendBuffer& token_ids, const BackendBuffer& weight, const BackendBuffer& output,
    float scale, std::uint32_t token_offset, std::uint32_t token_count) {
    impl_->encoding();
    const auto& w = device_storage(weight);
    const auto& wd = w.descriptor();
    if (wd.shape.rank() != 2U) throw std::invalid_argument("the embedding table is a [K, vocabulary] matrix");
    const auto k = static_cast<std::uint32_t>(wd.shape.dimension(0)), vocabulary = static_cast<std::uint32_t>(wd.shape.dimension(1));
    const auto available = static_cast<std::uint32_t>(device_storage(token_ids).descriptor().element_count);
    const std::uint32_t rows = token_count ? token_count : available - token_offset;
    if (token_offset > available || rows > available - token_offset || std::uint64_t(rows) * k > device_storage(output).descriptor().element_count)
        throw std::invalid_argument("embedding rows exceed the bound buffers");
    check(gf_embedding(gguf_type(wd.dtype), w.packed_weight(), k, vocabulary, words_of(token_ids) + token_offset, rows, scale,
                       mutable_floats(output), impl_->status_word(), impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

void MetalCommandContext::encode_rms_norm(const BackendBuffer& input, const BackendBuffer& weight, const BackendBuffer& output, float epsilon,
    std::uint32_t row_count, std::uint32_t input_row_start, const BackendBuffer*) {
    impl_->encoding();
    const auto hidden = static_cast<std::uint32_t>(device_storage(weight).descriptor().element_count);
    const std::uint32_t rows = row_count ? row_count : static_cast<std::uint32_t>(device_storage(input).descriptor().element_count / hidden);
    check(gf_rms_norm(floats(input) + std::uint64_t(input_row_start) * hidden, floats(weight), mutable_floats(output), rows, hidden, epsilon, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

void MetalCommandContext::encode_rms_norm_add(const BackendBuffer& input, const BackendBuffer& weight, const BackendBuffer& residual,
    const BackendBuffer& output, float epsilon, std::uint32_t row_count) {
    impl_->encoding();
    const auto hidden = static_cast<std::uint32_t>(device_storage(weight).descriptor().element_count);
    const std::uint32_t rows = row_count ? row_count : static_cast<std::uint32_t>(device_storage(input).descriptor().element_count / hidden);
    check(gf_rms_norm_add(floats(input), floats(weight), floats(residual), mutable_floats(output), rows, hidden, epsilon, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

// One RMS norm per (row, head): rows x heads vectors of `head_dimension` under one weight vector.
void MetalCommandContext::encode_head_rms_norm(const BackendBuffer& input, const BackendBuffer& weight, const BackendBuffer& output, float epsilon,
    std::uint32_t row_count, std::uint32_t head_count, std::uint32_t head_dimension) {
    impl_->encoding();
    if (device_storage(weight).descriptor().element_count != head_dimension) throw std::invalid_argument("one norm weight per head dimension");
    check(gf_rms_norm(floats(input), floats(weight), mutable_floats(output), row_count * head_count, head_dimension, epsilon, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

void MetalCommandContext::encode_verifier_rope(const BackendBuffer& input, const BackendBuffer& positions, const BackendBuffer& output,
    std::uint32_t row_count, std::uint32_t head_count, std::uint32_t head_dimension, std::uint32_t rope_dimension_count,
    float frequency_base, float frequency_scale) {
    impl_->encoding();
    check(gf_rope_store_rows(floats(input), nullptr, nullptr, nullptr, nullptr, mutable_floats(output), nullptr, nullptr, words_of(positions),
                             nullptr, row_count, head_count, 0U, head_dimension, rope_dimension_count, 1.0e-6F, frequency_base, frequency_scale,
                             0, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

void MetalCommandContext::encode_verifier_kv_store(const BackendBuffer& raw_key, const BackendBuffer& raw_value, const BackendBuffer& positions,
    const BackendBuffer& private_key, const BackendBuffer& private_value, std::uint32_t row_count, std::uint32_t head_count,
    std::uint32_t head_dimension, std::uint32_t rope_dimension_count, float frequency_base, float frequency_scale,
    const BackendBuffer* numerical_status) {
    impl_->encoding();
    const auto& key = device_storage(private_key);
    const auto& value = device_storage(private_value);
    const auto dtype = key.descriptor().dtype;
    if (value.descriptor().dtype != dtype || (dtype != DType::f32 && dtype != DType::f16))
        throw std::invalid_argument("the private cache rows are both F32 or both F16");
    if (numerical_status && (dtype != DType::f16 || device_storage(*numerical_status).descriptor().dtype != DType::f32))
        throw std::invalid_argument("a numerical status word belongs to a binary16 cache and is a 32-bit word");
    check(gf_rope_store_rows(nullptr, floats(raw_key), floats(raw_value), nullptr, nullptr, nullptr, key.data(), value.data(), words_of(positions),
                             numerical_status ? words_of(*numerical_status) : nullptr, row_count, 0U, head_count, head_dimension,
                             rope_dimension_count, 1.0e-6F, frequency_base, frequency_scale, dtype == DType::f16 ? 1 : 0, impl_->stream));
    ++impl_->stats.compute_dispatch_count;
}

std::uint32_t MetalCommandContext::read_verifier_status(const BackendBuffer& status) const {
    std::uint32_t word = 0U;
    check(gf_download(&word, device_storage(status).data(), sizeof word, impl_->stream));
    check(gf_stream_synchronize(impl_->stream));
    return word;
}

// The library's request row: { retain, history count, history[64] } (include/guffin_b200.h); `retain` is what the
// reference calls base_candidate_count (top-k plus the distinct history tokens).
std::uint32_t MetalCommandContext::encode_token_candidates(const BackendBuffer& logits, const engine::Gemma2MetalSelectionWorkspace& workspace,
    const engine::TokenSelectionRequest& request, float softcap) {
    impl_->encoding();
    if (request.history_token_count > 64U || request.base_candidate_count == 0U || request.base_candidate_count + request.history_token_count > engine::token_sampler_max_candidates)
        throw std::invalid_argument("selection request outside the compact candidate bounds");
    const auto vocabulary = static_cast<std::uint32_t>(device_storage(logits).descriptor().element_count);
    auto& selection = impl_->selections[&backend_buffer_storage(workspace.compact_result)];
    if (!selection.requests) check(gf_malloc(&selection.requests, gf_selection_request_bytes()));
    if (!selection.results) check(gf_malloc(&selection.results, gf_candidate_result_bytes()));
    const std::size_t need = gf_token_candidates_workspace_bytes(1U, vocabulary);
    if (need > selection.workspace_bytes) {
        if (selection.workspace) { check(gf_stream_synchronize(impl_->stream)); gf_free(selection.workspace); selection.workspace = nullptr; }
        check(gf_malloc(&selection.workspace, need));
        selection.workspace_bytes = need;
    }
    std::vector<std::uint32_t> row(gf_selection_request_bytes() / sizeof(std::uint32_t), 0U);
    row[0] = request.base_candidate_count;
    row[1] = request.history_token_count;
    std::copy_n(request.history_token_ids.begin(), request.history_token_count, row.begin() + 2);
    check(gf_upload(selection.requests, row.data(), row.size() * sizeof(std::uint32_t), impl_->stream));
    check(gf_stream_synchronize(impl_->stream));          // `row` leaves scope
    check(gf_token_candidates(floats(logits), 1U, vocabulary, softcap, selection.requests, selection.workspace, selection.results, impl_->stream));
    impl_->stats.compute_dispatch_count += 2U;
    return static_cast<std::uint32_t>(2U * sizeof(std::uint32_t) + (request.base_candidate_count + request.history_token_count) * sizeof(engine::TokenLogit));
}

engine::CompactTokenCandidates MetalCommandContext::read_token_candidates(const engine::Gemma2MetalSelectionWorkspace& workspace) const {
    const auto found = impl_->selections.find(&backend_buffer_storage(workspace.compact_result));
    if (found == impl_->selections.end()) throw std::logic_error("no selection was encoded for this workspace");
    std::vector<std::uint32_t> row(gf_candidate_result_bytes() / sizeof(std::uint32_t));
    check(gf_download(row.data(), found->second.results, row.size() * sizeof(std::uint32_t), impl_->stream));
    check(gf_stream_synchronize(impl_->stream));
    if (row[0] != 0U) throw std::invalid_argument("the device rejected the selection request");
    engine::CompactTokenCandidates result;
    result.count = row[1];
    for (std::uint32_t i = 0U; i < result.count; ++i) {
        result.values[i].token = row[2U + 2U * i];
        std::memcpy(&result.values[i].logit, &row[3U + 2U * i], sizeof(float));
    }
    result.readback_bytes = static_cast<std::uint32_t>(2U * sizeof(std::uint32_t) + result.count * sizeof(engine::TokenLogit));
    return result;
}

void MetalCommandContext::encode_memory_barrier() { ++impl_->stats.memory_barrier_count; }     // one in-order stream: nothing to do
void MetalCommandContext::push_debug_group(std::string_view) {}
void MetalCommandContext::pop_debug_group() {}

MetalCommandStats MetalCommandContext::commit() {
    if (impl_->committed) throw std::logic_error("the command has already been committed");
    impl_->committed = true;
    ++impl_->stats.commit_count;
    return impl_->stats;
}

MetalCommandStats MetalCommandContext::wait_until_completed() {
    if (!impl_->committed) throw std::logic_error("nothing has been committed");
    check(gf_matmul_check(impl_->stream));           // synchronises; a bounded wait that gave up becomes metal_execution_failed
    ++impl_->stats.synchronous_wait_count;
    return impl_->stats;
}

MetalCommandStats MetalCommandContext::completion_stats() const { return impl_->stats; }

MetalCommandStats MetalCommandContext::commit_and_wait() {
    static_cast<void>(commit());
    return wait_until_completed();
}

}  // namespace backends::metal

}  // namespace local_gguf_engine::tensor
