// Definitions for the few symbols the reference's CPU objects expect from behind its GPU seam
// (src/tensor/backend_buffer.mm).  The oracle build has no GPU backend, so these only carry
// CPU-backed handles.  TEST INFRASTRUCTURE ONLY.
#include "local_gguf_engine/tensor/backend_buffer.hpp"

#include <utility>

namespace local_gguf_engine::tensor::detail {
BackendBufferStorage::~BackendBufferStorage() = default;
BackendBuffer make_backend_buffer(std::shared_ptr<BackendBufferStorage> storage) {
    return BackendBuffer(std::move(storage));
}
}  // namespace local_gguf_engine::tensor::detail

namespace local_gguf_engine::tensor {
BackendBuffer::BackendBuffer(std::shared_ptr<detail::BackendBufferStorage> storage)
    : storage_(std::move(storage)) {}
runtime::BackendKind BackendBuffer::backend() const noexcept { return storage_->backend(); }
const TensorDescriptor& BackendBuffer::descriptor() const noexcept { return storage_->descriptor(); }
const detail::BackendBufferStorage& backend_buffer_storage(const BackendBuffer& buffer) noexcept {
    return *buffer.storage_;
}
}  // namespace local_gguf_engine::tensor
