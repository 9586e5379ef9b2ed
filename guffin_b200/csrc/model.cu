// Resident model plan and block schedule (see model.cuh).
#include "model.cuh"
#include "gemv.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace gf {

size_t candidates_workspace_bytes(uint32_t rows, uint32_t vocab);
int launch_candidates(const float* logits, uint32_t rows, uint32_t vocab, float softcap, const void* requests,
                      void* workspace, void* results, cudaStream_t stream, bool pdl);

static uint32_t next_pow2(uint32_t v) {
    uint32_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

Model::Model(const gf_model_config& config) : config_(config) {
    layers_.resize(config.layers);
    caches_.resize(config.layers);
}

Model::~Model() {
    release_stager();
    for (auto& per_rows : graphs_)
        for (auto& graph : per_rows)
            if (graph) cudaGraphExecDestroy(graph);
    invalidate_passes();
    for (void* p : allocations_) cudaFree(p);
    for (uint32_t s = 0; s < shard_.size; ++s)
        if (shard_.opened[s]) cudaIpcCloseMemHandle(shard_.mapped[s]);
    if (shard_.arena) cudaFree(shard_.arena);
    if (shard_.gathered_host) cudaFreeHost(shard_.gathered_host);
    if (tokens_copied_) cudaEventDestroy(tokens_copied_);
    if (requests_copied_) cudaEventDestroy(requests_copied_);
    if (tokens_pinned_) cudaFreeHost(tokens_pinned_);
    if (requests_pinned_) cudaFreeHost(requests_pinned_);
    if (stream_) cudaStreamDestroy(stream_);
}

bool Model::layer_is_local(uint32_t layer) const {
    if (config_.sliding_pattern == 6u) return (layer + 1u) % 6u != 0u;      // model.cpp:607-619 (Gemma 3)
    if (config_.sliding_pattern == 2u) return layer % 2u == 0u;              // Gemma 2: even layers slide
    return false;
}

#define GF_TRY(expr) do { const int gf_s_ = (expr); if (gf_s_ != GF_OK) return gf_s_; } while (0)

// Host views of the selection rows (candidates.cu: SelectionRequest, CandidateResult).
struct TokenLogit { uint32_t token; float logit; };
struct SelectionRequestRow { uint32_t retain, history_count, history[64]; };
struct CandidateRow { uint32_t status, count; TokenLogit candidates[384]; };

template <typename T>
static int device_alloc(std::vector<void*>& owner, T** out, size_t count) {
    void* p = nullptr;
    GF_CUDA(cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 16)));
    owner.push_back(p);
    *out = static_cast<T*>(p);
    return GF_OK;
}

// Copies `bytes` of native blocks into a device staging buffer without blocking on the device: the host
// fills one pinned chunk while the other is in flight; the staging buffer alternates between tensors, and is
// only overwritten once the repack that read it has finished.
int Model::stage_upload(const void* native_host, size_t bytes, uint8_t** out_staging, uint32_t* out_slot) {
    WeightStager& st = stager_;
    if (!st.ready) {
        GF_CUDA(cudaStreamCreateWithFlags(&st.copy_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&st.pinned[i]), WeightStager::kChunkBytes, cudaHostAllocDefault));
            GF_CUDA(cudaEventCreateWithFlags(&st.chunk_done[i], cudaEventDisableTiming));
            GF_CUDA(cudaEventCreateWithFlags(&st.uploaded[i], cudaEventDisableTiming));
            GF_CUDA(cudaEventCreateWithFlags(&st.packed[i], cudaEventDisableTiming));
        }
        st.ready = true;
    }
    const uint32_t slot = st.next;
    st.next ^= 1u;
    if (bytes > st.staging_bytes[slot]) {
        GF_CUDA(cudaEventSynchronize(st.packed[slot]));          // nothing reads the old buffer any more
        if (st.staging[slot]) GF_CUDA(cudaFree(st.staging[slot]));
        st.staging[slot] = nullptr;
        st.staging_bytes[slot] = 0;
        GF_CUDA(cudaMalloc(reinterpret_cast<void**>(&st.staging[slot]), bytes));
        st.staging_bytes[slot] = bytes;
    }
    GF_CUDA(cudaStreamWaitEvent(st.copy_stream, st.packed[slot], 0));
    const uint8_t* src = static_cast<const uint8_t*>(native_host);
    for (size_t done = 0; done < bytes; done += WeightStager::kChunkBytes) {
        const size_t part = std::min(WeightStager::kChunkBytes, bytes - done);
        const uint32_t c = st.chunk;
        st.chunk ^= 1u;
        GF_CUDA(cudaEventSynchronize(st.chunk_done[c]));
        std::memcpy(st.pinned[c], src + done, part);
        GF_CUDA(cudaMemcpyAsync(st.staging[slot] + done, st.pinned[c], part, cudaMemcpyHostToDevice, st.copy_stream));
        GF_CUDA(cudaEventRecord(st.chunk_done[c], st.copy_stream));
    }
    GF_CUDA(cudaEventRecord(st.uploaded[slot], st.copy_stream));
    GF_CUDA(cudaStreamWaitEvent(stream_, st.uploaded[slot], 0));
    *out_staging = st.staging[slot];
    *out_slot = slot;
    return GF_OK;
}

void Model::release_stager() {
    WeightStager& st = stager_;
    if (!st.ready) return;
    if (st.copy_stream) cudaStreamSynchronize(st.copy_stream);
    if (stream_) cudaStreamSynchronize(stream_);
    for (int i = 0; i < 2; ++i) {
        if (st.pinned[i]) cudaFreeHost(st.pinned[i]);
        if (st.staging[i]) cudaFree(st.staging[i]);
        if (st.chunk_done[i]) cudaEventDestroy(st.chunk_done[i]);
        if (st.uploaded[i]) cudaEventDestroy(st.uploaded[i]);
        if (st.packed[i]) cudaEventDestroy(st.packed[i]);
    }
    if (st.copy_stream) cudaStreamDestroy(st.copy_stream);
    st = WeightStager();
}

int launch_quantize_f16_q8_0(const void* f16_dev, uint64_t block_count, void* q8_dev, uint32_t* status_dev, cudaStream_t stream);
int launch_requantize_q6k_q4k(const void* q6_dev, uint64_t block_count, void* q4_dev, uint32_t* status_dev, cudaStream_t stream);

// Quantises a binary16 [K, vocab] table already on the device to Q8_0 and packs it as the output head.
int Model::bind_q8_head_from_f16(const void* f16_dev, uint64_t k, uint64_t n) {
    if (k % 128u) return fail(GF_ERR_INVALID, "a binary16 head needs K to be a multiple of 128");
    const uint64_t blocks = n * (k / 32u);
    const size_t native = (size_t)blocks * 34u, packed = gf_packed_weight_bytes(GF_Q8_0, k, n);
    if (packed == 0) return GF_ERR_INVALID;
    uint8_t* staging = nullptr;
    uint32_t* flag = nullptr;
    GF_CUDA(cudaMalloc(&staging, native + 16u));
    flag = reinterpret_cast<uint32_t*>(staging + ((native + 3u) & ~(size_t)3u));
    uint8_t* data = nullptr;
    int status = device_alloc(allocations_, &data, packed);
    uint32_t bad = 0;
    if (status == GF_OK) status = check_cuda(cudaMemsetAsync(flag, 0, 4, stream_), "clear");
    if (status == GF_OK) status = launch_quantize_f16_q8_0(f16_dev, blocks, staging, flag, stream_);
    if (status == GF_OK) status = gf_pack_weight(GF_Q8_0, staging, k, n, data, stream_);
    if (status == GF_OK) status = check_cuda(cudaMemcpyAsync(&bad, flag, 4, cudaMemcpyDeviceToHost, stream_), "status");
    if (status == GF_OK) status = check_cuda(cudaStreamSynchronize(stream_), "quantise");
    cudaFree(staging);
    if (status != GF_OK) return status;
    if (bad) return fail(GF_ERR_INVALID, "Q8_0 quantisation of a binary16 table needs finite values");
    head_ = PackedMatrix{GF_Q8_0, k, n, data, packed, native};
    weight_bytes_ += packed;
    native_weight_bytes_ += native;
    has_head_ = true;
    return GF_OK;
}

int Model::set_matrix(int kind, uint32_t layer, int dtype, const void* native_host, uint64_t k, uint64_t n, bool requantize) {
    if (finalized_) return fail(GF_ERR_STATE, "gf_model_set_matrix: the plan is already finalized");
    if (!native_host) return fail(GF_ERR_INVALID, "gf_model_set_matrix: null payload");
    const gf_model_config& c = config_;
    const uint64_t qw = (uint64_t)c.heads * c.head_dim, kvw = (uint64_t)c.kv_heads * c.head_dim;
    uint64_t want_k = 0, want_n = 0;
    PackedMatrix* dst = nullptr;
    if (kind >= GF_MAT_ATTN_Q && layer >= c.layers) return fail(GF_ERR_INVALID, "gf_model_set_matrix: layer %u out of range", layer);
    switch (kind) {
        case GF_MAT_TOKEN_EMBD: dst = &token_embd_; want_k = c.hidden; want_n = token_vocab(); break;
        case GF_MAT_OUTPUT: dst = &head_; want_k = c.hidden; want_n = c.vocab; break;
        case GF_MAT_ATTN_Q: dst = &layers_[layer].q; want_k = c.hidden; want_n = qw; break;
        case GF_MAT_ATTN_K: dst = &layers_[layer].k; want_k = c.hidden; want_n = kvw; break;
        case GF_MAT_ATTN_V: dst = &layers_[layer].v; want_k = c.hidden; want_n = kvw; break;
        case GF_MAT_ATTN_OUTPUT: dst = &layers_[layer].o; want_k = qw; want_n = c.hidden; break;
        case GF_MAT_FFN_GATE: dst = &layers_[layer].gate; want_k = c.hidden; want_n = c.ffn; break;
        case GF_MAT_FFN_UP: dst = &layers_[layer].up; want_k = c.hidden; want_n = c.ffn; break;
        case GF_MAT_FFN_DOWN: dst = &layers_[layer].down; want_k = c.ffn; want_n = c.hidden; break;
        default: return fail(GF_ERR_INVALID, "gf_model_set_matrix: unknown tensor kind %d", kind);
    }
    if (k != want_k || n != want_n)
        return fail(GF_ERR_INVALID, "gf_model_set_matrix: kind %d expects [%llu, %llu], got [%llu, %llu]", kind,
                    (unsigned long long)want_k, (unsigned long long)want_n, (unsigned long long)k, (unsigned long long)n);
    if (dst->data) return fail(GF_ERR_STATE, "gf_model_set_matrix: tensor kind %d layer %u bound twice", kind, layer);
    if (!stream_) GF_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    if (dtype == GF_F16) {
        // Binary16 tables: the embedding is gathered from the rows as stored; a head becomes Q8_0.
        if (requantize || (kind != GF_MAT_TOKEN_EMBD && kind != GF_MAT_OUTPUT))
            return fail(GF_ERR_INVALID, "gf_model_set_matrix: binary16 is accepted for the token embedding and the output head only");
        const size_t bytes = (size_t)n * k * 2u;
        if (kind == GF_MAT_TOKEN_EMBD) {
            uint8_t* data = nullptr;
            GF_TRY(device_alloc(allocations_, &data, bytes));
            GF_CUDA(cudaMemcpyAsync(data, native_host, bytes, cudaMemcpyHostToDevice, stream_));
            GF_CUDA(cudaStreamSynchronize(stream_));
            *dst = PackedMatrix{GF_F16, k, n, data, bytes, bytes};
            weight_bytes_ += bytes;
            native_weight_bytes_ += bytes;
            return GF_OK;
        }
        uint8_t* table = nullptr;
        GF_CUDA(cudaMalloc(&table, bytes));
        int status = check_cuda(cudaMemcpyAsync(table, native_host, bytes, cudaMemcpyHostToDevice, stream_), "upload");
        if (status == GF_OK) status = bind_q8_head_from_f16(table, k, n);
        cudaFree(table);
        return status;
    }
    if (requantize && dtype != GF_Q6_K) return fail(GF_ERR_INVALID, "gf_model_set_matrix_requantized: the source must be Q6_K");
    const int stored = requantize ? GF_Q4_K : dtype;
    const size_t packed = gf_packed_weight_bytes(stored, k, n);
    if (packed == 0) return GF_ERR_INVALID;
    const size_t source = (size_t)n * (k / block_elements(dtype)) * block_bytes(dtype);
    const size_t native = (size_t)n * (k / block_elements(stored)) * block_bytes(stored);
    if (!requantize) {
        // The common case: upload through the pinned pipeline, repack on the plan's stream, no wait here.
        uint8_t* data = nullptr;
        GF_TRY(device_alloc(allocations_, &data, packed));
        uint8_t* staged = nullptr;
        uint32_t slot = 0;
        GF_TRY(stage_upload(native_host, source, &staged, &slot));
        GF_TRY(gf_pack_weight(dtype, staged, k, n, data, stream_));
        GF_CUDA(cudaEventRecord(stager_.packed[slot], stream_));
        *dst = PackedMatrix{stored, k, n, data, packed, native};
        weight_bytes_ += packed;
        native_weight_bytes_ += native;
        if (kind == GF_MAT_OUTPUT) has_head_ = true;
        return GF_OK;
    }
    // Staging: the source blocks, then the converted blocks and a status word.
    const size_t converted_at = (source + 15u) & ~(size_t)15u, flag_at = converted_at + ((native + 15u) & ~(size_t)15u);
    uint8_t* staging = nullptr;
    GF_CUDA(cudaMalloc(&staging, flag_at + 16u));
    uint8_t* data = nullptr;
    int status = device_alloc(allocations_, &data, packed);
    if (status == GF_OK) status = check_cuda(cudaMemcpyAsync(staging, native_host, source, cudaMemcpyHostToDevice, stream_), "upload");
    uint32_t bad = 0;
    if (requantize) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(staging + flag_at);
        if (status == GF_OK) status = check_cuda(cudaMemsetAsync(flag, 0, 4, stream_), "clear");
        if (status == GF_OK) status = launch_requantize_q6k_q4k(staging, n * (k / 256u), staging + converted_at, flag, stream_);
        if (status == GF_OK) status = gf_pack_weight(stored, staging + converted_at, k, n, data, stream_);
        if (status == GF_OK) status = check_cuda(cudaMemcpyAsync(&bad, flag, 4, cudaMemcpyDeviceToHost, stream_), "status");
    } else if (status == GF_OK) {
        status = gf_pack_weight(dtype, staging, k, n, data, stream_);
    }
    if (status == GF_OK) status = check_cuda(cudaStreamSynchronize(stream_), "pack");
    cudaFree(staging);
    if (status != GF_OK) return status;
    if (bad) return fail(GF_ERR_INVALID, "Q6_K to Q4_K requantisation needs finite decoded values");
    *dst = PackedMatrix{stored, k, n, data, packed, native};
    weight_bytes_ += packed;
    native_weight_bytes_ += native;
    if (kind == GF_MAT_OUTPUT) has_head_ = true;
    return GF_OK;
}

int Model::set_vector(int kind, uint32_t layer, const float* host, uint32_t count) {
    if (finalized_) return fail(GF_ERR_STATE, "gf_model_set_vector: the plan is already finalized");
    if (!host) return fail(GF_ERR_INVALID, "gf_model_set_vector: null payload");
    if (kind != GF_VEC_OUTPUT_NORM && layer >= config_.layers) return fail(GF_ERR_INVALID, "gf_model_set_vector: layer out of range");
    float** dst = nullptr;
    uint32_t want = config_.hidden;
    switch (kind) {
        case GF_VEC_OUTPUT_NORM: dst = &output_norm_; break;
        case GF_VEC_ATTN_NORM: dst = &layers_[layer].attn_norm; break;
        case GF_VEC_POST_ATTENTION_NORM: dst = &layers_[layer].post_attention_norm; break;
        case GF_VEC_FFN_NORM: dst = &layers_[layer].ffn_norm; break;
        case GF_VEC_POST_FFW_NORM: dst = &layers_[layer].post_ffw_norm; break;
        case GF_VEC_ATTN_Q_NORM: dst = &layers_[layer].q_norm; want = config_.head_dim; break;
        case GF_VEC_ATTN_K_NORM: dst = &layers_[layer].k_norm; want = config_.head_dim; break;
        default: return fail(GF_ERR_INVALID, "gf_model_set_vector: unknown vector kind %d", kind);
    }
    if (count != want) return fail(GF_ERR_INVALID, "gf_model_set_vector: kind %d expects %u values, got %u", kind, want, count);
    if (*dst) return fail(GF_ERR_STATE, "gf_model_set_vector: vector bound twice");
    GF_TRY(device_alloc(allocations_, dst, count));
    GF_CUDA(cudaMemcpy(*dst, host, (size_t)count * 4, cudaMemcpyHostToDevice));
    native_weight_bytes_ += (size_t)count * 4;
    return GF_OK;
}

int Model::finalize() {
    if (finalized_) return fail(GF_ERR_STATE, "gf_model_finalize: already finalized");
    const gf_model_config& c = config_;
    if (c.row_capacity == 0 || c.row_capacity > GF_MAX_ROWS) return fail(GF_ERR_INVALID, "row_capacity must be 1..%d", GF_MAX_ROWS);
    if (c.head_dim != 256u) return fail(GF_ERR_INVALID, "head_dim must be 256 (the reference's kernels share this limit)");
    if (c.context == 0 || c.heads % c.kv_heads) return fail(GF_ERR_INVALID, "bad context or head geometry");
    if (!token_embd_.data || !output_norm_) return fail(GF_ERR_STATE, "token embedding or output norm missing");
    if (!stream_) GF_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    release_stager();          // waits for the last uploads and repacks, frees the staging buffers
    // A binary16 embedding cannot serve as the head: the tied head is its Q8_0 quantisation
    // (resolve_gemma_output_head_policy, gemma2_metal_plan.cpp:799-828).
    if (!has_head_ && token_vocab() != config_.vocab) return fail(GF_ERR_STATE, "a token table wider than the head needs its own output matrix");
    if (token_embd_.dtype == GF_F16 && !has_head_) GF_TRY(bind_q8_head_from_f16(token_embd_.data, token_embd_.k, token_embd_.n));
    for (uint32_t l = 0; l < c.layers; ++l) {
        const LayerWeights& w = layers_[l];
        if (!w.q.data || !w.k.data || !w.v.data || !w.o.data || !w.gate.data || !w.up.data || !w.down.data || !w.attn_norm
            || !w.post_attention_norm || !w.ffn_norm || !w.post_ffw_norm || (c.uses_qk_norm && (!w.q_norm || !w.k_norm)))
            return fail(GF_ERR_STATE, "layer %u has unbound tensors", l);
    }
    if (!stream_) GF_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    const uint32_t R = c.row_capacity, kvw = c.kv_heads * c.head_dim, qw = c.heads * c.head_dim;
    const size_t element = c.kv_f16 ? 2 : 4;
    for (uint32_t l = 0; l < c.layers; ++l) {
        LayerCache& cache = caches_[l];
        const bool local = layer_is_local(l);
        cache.window = local ? c.sliding_window : 0u;
        // A local ring keeps its window plus the rows a pass may publish, so the rows of an
        // unpublished pass never alias keys still inside a live window.
        cache.ring_rows = next_pow2(local ? std::min(c.context, c.sliding_window + R) : c.context);
        cache.rope_base = local ? c.rope_base_local : c.rope_base_global;
        cache.rope_scale = local ? c.rope_scale_local : c.rope_scale_global;
        uint8_t *rk, *rv, *pk, *pv;
        GF_TRY(device_alloc(allocations_, &rk, (size_t)cache.ring_rows * kvw * element));
        GF_TRY(device_alloc(allocations_, &rv, (size_t)cache.ring_rows * kvw * element));
        GF_TRY(device_alloc(allocations_, &pk, (size_t)R * kvw * element));
        GF_TRY(device_alloc(allocations_, &pv, (size_t)R * kvw * element));
        cache.ring_k = rk; cache.ring_v = rv; cache.private_k = pk; cache.private_v = pv;
        GF_CUDA(cudaMemsetAsync(rk, 0, (size_t)cache.ring_rows * kvw * element, stream_));
        GF_CUDA(cudaMemsetAsync(rv, 0, (size_t)cache.ring_rows * kvw * element, stream_));
    }
    {   // RoPE divisors, one table per distinct base (local and global layers).
        double* tables[2] = {nullptr, nullptr};
        const float bases[2] = {c.rope_base_local, c.rope_base_global};
        for (int kind = 0; kind < 2; ++kind) {
            if (kind == 1 && bases[1] == bases[0]) { tables[1] = tables[0]; break; }
            std::vector<double> host(c.head_dim / 2u);
            for (uint32_t i = 0; i < c.head_dim / 2u; ++i)
                host[i] = std::pow((double)bases[kind], (double)(2u * i) / (double)c.head_dim);
            GF_TRY(device_alloc(allocations_, &tables[kind], host.size()));
            GF_CUDA(cudaMemcpyAsync(tables[kind], host.data(), host.size() * sizeof(double), cudaMemcpyHostToDevice, stream_));
            GF_CUDA(cudaStreamSynchronize(stream_));
        }
        for (uint32_t l = 0; l < c.layers; ++l) caches_[l].rope_divisors = tables[layer_is_local(l) ? 0 : 1];
        // (cos, sin) of every position the plan can reach, formed on the host exactly as the
        // reference forms them: double angle = position * scale / base^(2i/d), then rounded to f32
        // (ops/rope.cpp:109-117).  256-wide heads only (the fused Q/K/V epilogue's layout).
        if (c.head_dim == 256u && c.context <= 65536u) {     // 1 KB per position and table; longer contexts rotate in rope_store_kernel
            float2* rotations[2] = {nullptr, nullptr};
            const float scales[2] = {c.rope_scale_local, c.rope_scale_global};
            const uint32_t table_rows = c.context + GF_MAX_ROWS;
            for (int kind = 0; kind < 2; ++kind) {
                if (kind == 1 && bases[1] == bases[0] && scales[1] == scales[0]) { rotations[1] = rotations[0]; break; }
                std::vector<float2> host((size_t)table_rows * 128u);
                for (uint32_t i = 0; i < 128u; ++i) {
                    const double divisor = std::pow((double)bases[kind], (double)(2u * i) / 256.0);
                    for (uint32_t position = 0; position < table_rows; ++position) {
                        const double angle = (double)position * (double)scales[kind] / divisor;
                        host[(size_t)position * 128u + i] = make_float2((float)std::cos(angle), (float)std::sin(angle));
                    }
                }
                GF_TRY(device_alloc(allocations_, &rotations[kind], host.size()));
                GF_CUDA(cudaMemcpyAsync(rotations[kind], host.data(), host.size() * sizeof(float2), cudaMemcpyHostToDevice, stream_));
                GF_CUDA(cudaStreamSynchronize(stream_));
            }
            for (uint32_t l = 0; l < c.layers; ++l) caches_[l].rope_rotation = rotations[layer_is_local(l) ? 0 : 1];
            // Twice: each half of a 5..8-row launch counts its own arrivals.
            GF_TRY(device_alloc(allocations_, &head_counters_, 2u * (c.heads + 2u * c.kv_heads)));
            GF_CUDA(cudaMemsetAsync(head_counters_, 0, 2u * (c.heads + 2u * c.kv_heads) * sizeof(uint32_t), stream_));
        }
    }
    {
        std::vector<KvPublishLayer> table(c.layers);
        for (uint32_t l = 0; l < c.layers; ++l)
            table[l] = KvPublishLayer{static_cast<uint8_t*>(caches_[l].ring_k), static_cast<uint8_t*>(caches_[l].ring_v),
                                      static_cast<const uint8_t*>(caches_[l].private_k), static_cast<const uint8_t*>(caches_[l].private_v),
                                      caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
        GF_TRY(device_alloc(allocations_, &publish_layers_, c.layers));
        GF_CUDA(cudaMemcpyAsync(publish_layers_, table.data(), sizeof(KvPublishLayer) * c.layers, cudaMemcpyHostToDevice, stream_));
        GF_CUDA(cudaStreamSynchronize(stream_));
    }
    GF_TRY(device_alloc(allocations_, &residual_, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &normalized_, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &raw_q_, (size_t)R * qw));
    GF_TRY(device_alloc(allocations_, &raw_k_, (size_t)R * kvw));
    GF_TRY(device_alloc(allocations_, &raw_v_, (size_t)R * kvw));
    GF_TRY(device_alloc(allocations_, &query_, (size_t)R * qw));
    GF_TRY(device_alloc(allocations_, &attention_out_, (size_t)R * qw));
    GF_TRY(device_alloc(allocations_, &projected_, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &post_attention_, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &gate_, (size_t)R * c.ffn));
    GF_TRY(device_alloc(allocations_, &up_, (size_t)R * c.ffn));
    GF_TRY(device_alloc(allocations_, &gated_, (size_t)R * c.ffn));
    GF_TRY(device_alloc(allocations_, &logits_, (size_t)R * c.vocab));
    // Split-K workspace: the largest any launch of the schedule needs, for every row count.
    size_t ws = 256, counters = 256;
    auto grow = [&](std::initializer_list<const PackedMatrix*> set, uint32_t prologue = kProloguePlain) {
        for (uint32_t rows = 1; rows <= R; ++rows) {
            GemvLaunch launch;
            launch.count = 0;
            launch.prologue = prologue;              // the merge prologue narrows the planner's choice of K chunks
            for (const PackedMatrix* m : set) {
                launch.matrices[launch.count++] = GemvMatrixDesc{m->dtype, m->data, logits_, m->n};
                launch.k = m->k;
            }
            launch.rows = rows;
            ws = std::max(ws, gemv_partial_bytes(launch));
            counters = std::max(counters, gemv_counter_bytes(launch));
        }
    };
    for (const LayerWeights& w : layers_) { grow({&w.q, &w.k, &w.v}); grow({&w.o}); grow({&w.o}, kPrologueMerge); grow({&w.gate, &w.up}); grow({&w.down}); }
    grow({has_head_ ? &head_ : &token_embd_});
    uint8_t* bytes = nullptr;
    GF_TRY(device_alloc(allocations_, &bytes, ws)); matmul_ws_ = bytes; matmul_ws_bytes_ = ws;
    GF_TRY(device_alloc(allocations_, &bytes, counters)); matmul_counters_ = reinterpret_cast<uint32_t*>(bytes);
    matmul_counters_bytes_ = counters;
    GF_CUDA(cudaMemsetAsync(matmul_counters_, 0, counters, stream_));   // arrival counters start (and stay) at zero
    GF_TRY(device_alloc(allocations_, &bytes, attention_workspace_bytes(R, c.heads))); attention_ws_ = bytes;
    GF_CUDA(cudaMemsetAsync(attention_counters(attention_ws_, R, c.heads), 0, (size_t)R * c.heads * sizeof(uint32_t), stream_));
    GF_TRY(device_alloc(allocations_, &bytes, candidates_workspace_bytes(R, c.vocab))); candidates_ws_ = bytes;
    GF_TRY(device_alloc(allocations_, &bytes, (size_t)R * gf_selection_request_bytes())); requests_dev_ = bytes;
    GF_TRY(device_alloc(allocations_, &bytes, (size_t)R * gf_candidate_result_bytes())); results_dev_ = bytes;
    GF_TRY(device_alloc(allocations_, &tokens_dev_, GF_MAX_ROWS));
    GF_TRY(device_alloc(allocations_, &state_dev_, 8));
    GF_TRY(device_alloc(allocations_, &status_dev_, 4));
    GF_TRY(device_alloc(allocations_, &error_flag_, 4));
    GF_TRY(device_alloc(allocations_, &pass_arrived_, 4));
    GF_CUDA(cudaMemsetAsync(pass_arrived_, 0, 16, stream_));
    GF_CUDA(cudaMemsetAsync(state_dev_, 0, 32, stream_));
    GF_CUDA(cudaMemsetAsync(status_dev_, 0, 16, stream_));
    GF_CUDA(cudaMemsetAsync(error_flag_, 0, 16, stream_));
    GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&tokens_pinned_), GF_MAX_ROWS * sizeof(uint32_t), cudaHostAllocDefault));
    GF_CUDA(cudaHostAlloc(&requests_pinned_, (size_t)R * gf_selection_request_bytes(), cudaHostAllocDefault));
    GF_CUDA(cudaEventCreateWithFlags(&tokens_copied_, cudaEventDisableTiming));
    GF_CUDA(cudaEventCreateWithFlags(&requests_copied_, cudaEventDisableTiming));
    GF_CUDA(cudaStreamSynchronize(stream_));
    finalized_ = true;
    position_ = 0;
    return GF_OK;
}

int Model::reset() {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    GF_CUDA(cudaMemsetAsync(state_dev_, 0, 32, stream_));
    GF_CUDA(cudaMemsetAsync(status_dev_, 0, 16, stream_));
    // A pass that was cut short (a bounded wait gave up) can leave arrival counters half way:
    // every kernel that counts arrivals expects zero.
    GF_CUDA(cudaMemsetAsync(error_flag_, 0, 16, stream_));
    GF_CUDA(cudaMemsetAsync(pass_arrived_, 0, 16, stream_));       // a pass kernel that gave up leaves its barrier count short
    pass_arrivals_ = 0;
    if (matmul_counters_bytes_) GF_CUDA(cudaMemsetAsync(matmul_counters_, 0, matmul_counters_bytes_, stream_));
    GF_CUDA(cudaMemsetAsync(attention_counters(attention_ws_, config_.row_capacity, config_.heads), 0,
                            (size_t)config_.row_capacity * config_.heads * sizeof(uint32_t), stream_));
    if (head_counters_) GF_CUDA(cudaMemsetAsync(head_counters_, 0, 2u * (config_.heads + 2u * config_.kv_heads) * sizeof(uint32_t), stream_));
    position_ = 0;
    poisoned_ = false;
    return GF_OK;
}

static GemvMatrixDesc desc(const PackedMatrix& w, float* out) { return GemvMatrixDesc{w.dtype, w.data, out, w.n}; }

int Model::run_gemv(GemvLaunch& launch, uint32_t rows) {
    launch.rows = rows;
    launch.eps = config_.rms_eps;
    if (recording_) {
        PassPhase phase {};
        GemvPlan plan;
        GF_TRY(gemv_prepare(launch, matmul_counters_, static_cast<float*>(matmul_ws_), matmul_ws_bytes_, error_flag_, phase.stream, plan));
        phase.kind = kPhaseStream;
        recording_->push_back(phase);
        recording_breaks_.push_back(pending_break_);
        pending_break_ = -1;
        return GF_OK;
    }
    ++launches_;
    return gemv_launch(launch, matmul_counters_, static_cast<float*>(matmul_ws_), matmul_ws_bytes_, error_flag_, stream_, true);
}

// Tensor-parallel shards (a plan built on 1 / G of the heads and of the FFN width) leave partial sums behind
// their O and down projections; the host's hook turns them into the full sums on the plan's stream.
int Model::reduce_partial(float* buffer, size_t count) {
    if (!reduce_hook_) return GF_OK;
    if (recording_) { recording_failed_ = true; return GF_OK; }          // the pass kernel has no phase for it
    const int status = reduce_hook_(reduce_user_, buffer, (uint64_t)count, stream_);
    return status == GF_OK ? GF_OK : fail(status, "the partial-sum reduction hook failed (%d)", status);
}

// ---- the exchange fused into the projection launches (see WeightStreamParams::Scatter / Gather)

int Model::shard_prepare(uint32_t rank, uint32_t size, void* ipc_handle_out) {
    if (size == 0 || size > (uint32_t)kGemvMaxShards || rank >= size) return fail(GF_ERR_INVALID, "shard %u of %u", rank, size);
    if (shard_.arena) return fail(GF_ERR_STATE, "this plan already has an exchange arena");
    ShardExchange& x = shard_;
    x.rank = rank; x.size = size;
    if (2u * config_.layers > 255u) return fail(GF_ERR_INVALID, "the exchange stamps name at most 127 layers");
    // A slot holds the rows of a pass, or of a whole prompt chunk on the tensor-core path.
    x.part_values = (((size_t)std::max<uint32_t>(config_.row_capacity, kPrefillRows) * config_.hidden) + 63u) & ~(size_t)63u;
    x.tick_offset = 2u * size * x.part_values * sizeof(uint2);
    x.rows_offset = x.tick_offset + 256u;
    x.rows_values = (size_t)config_.row_capacity * (gf_candidate_result_bytes() / sizeof(uint32_t));
    x.bytes = x.rows_offset + 2u * size * x.rows_values * sizeof(uint2);
    void* base = nullptr;
    GF_CUDA(cudaMalloc(&base, x.bytes));                 // an allocation of its own: peers map exactly this
    GF_CUDA(cudaMemset(base, 0, x.bytes));
    x.arena = static_cast<uint8_t*>(base);
    x.mapped[rank] = x.arena;
    if (ipc_handle_out) {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported handle travels as 64 bytes");
        cudaIpcMemHandle_t handle;
        GF_CUDA(cudaIpcGetMemHandle(&handle, base));
        std::memcpy(ipc_handle_out, &handle, sizeof handle);
    }
    return GF_OK;
}

int Model::shard_connect(void* const* arenas) {
    ShardExchange& x = shard_;
    if (!x.arena) return fail(GF_ERR_STATE, "prepare the exchange arena first");
    if (!arenas) return fail(GF_ERR_INVALID, "null arena list");
    int mine = 0;
    GF_CUDA(cudaGetDevice(&mine));
    for (uint32_t s = 0; s < x.size; ++s) {
        if (s == x.rank) continue;
        if (!arenas[s]) return fail(GF_ERR_INVALID, "shard %u has no arena", s);
        if (!x.opened[s]) {       // a pointer of this process: its device must be reachable from this one
            cudaPointerAttributes attributes;
            GF_CUDA(cudaPointerGetAttributes(&attributes, arenas[s]));
            if (attributes.device != mine) {
                int reachable = 0;
                GF_CUDA(cudaDeviceCanAccessPeer(&reachable, mine, attributes.device));
                if (!reachable) return fail(GF_ERR_STATE, "device %d cannot address device %d", mine, attributes.device);
                const cudaError_t enabled = cudaDeviceEnablePeerAccess(attributes.device, 0);
                if (enabled != cudaSuccess && enabled != cudaErrorPeerAccessAlreadyEnabled) GF_CUDA(enabled);
                cudaGetLastError();
            }
        }
        x.mapped[s] = static_cast<uint8_t*>(arenas[s]);
    }
    x.connected = true;
    drop_graphs();
    return GF_OK;
}

int Model::shard_connect_ipc(const void* handles) {
    ShardExchange& x = shard_;
    if (!x.arena) return fail(GF_ERR_STATE, "prepare the exchange arena first");
    if (!handles) return fail(GF_ERR_INVALID, "null handle list");
    void* arenas[8] = {};
    for (uint32_t s = 0; s < x.size; ++s) {
        if (s == x.rank) { arenas[s] = x.arena; continue; }
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, static_cast<const uint8_t*>(handles) + (size_t)s * sizeof handle, sizeof handle);
        GF_CUDA(cudaIpcOpenMemHandle(&arenas[s], handle, cudaIpcMemLazyEnablePeerAccess));
        x.opened[s] = true;
    }
    return shard_connect(arenas);
}

int Model::shard_global_selection(bool enable) {
    ShardExchange& x = shard_;
    if (enable && !x.connected) return fail(GF_ERR_STATE, "connect the shards first");
    if (enable && !x.gathered_dev) {
        const size_t bytes = (size_t)x.size * x.rows_values * sizeof(uint32_t);
        GF_TRY(device_alloc(allocations_, &x.gathered_dev, (size_t)x.size * x.rows_values));
        GF_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&x.gathered_host), bytes, cudaHostAllocDefault));
    }
    x.global_selection = enable;
    return GF_OK;
}

// The producing side: the launch keeps its part in `projected_` and mirrors it, stamped, into this shard's slot of
// every peer's arena.  `site` names the projection inside the pass.
void Model::shard_scatter(GemvLaunch& launch, uint32_t half, uint32_t site) {
    const ShardExchange& x = shard_;
    launch.scatter.count = 0;
    for (uint32_t s = 0; s < x.size; ++s) {
        if (s == x.rank) continue;
        launch.scatter.out[launch.scatter.count++] = x.part(x.mapped[s], half, x.rank);
    }
    launch.scatter.tick = x.tick();
    launch.scatter.site = site;
}

void Model::shard_gather(GemvLaunch& launch, uint32_t half, uint32_t site) {
    const ShardExchange& x = shard_;
    launch.gather.count = x.size;
    launch.gather.self = x.rank;
    launch.gather.own = launch.in;
    for (uint32_t s = 0; s < x.size; ++s) launch.gather.parts[s] = x.part(x.arena, half, s);
    launch.gather.tick = x.tick();
    launch.gather.site = site;
    launch.gather.wait_limit = x.wait_limit;
}

int Model::emit_embedding(uint32_t rows, float scale) {
    const gf_model_config& c = config_;
    if (recording_) {
        PassPhase phase {};
        phase.kind = kPhaseEmbedding;
        phase.embedding = EmbeddingPhase{token_embd_.data, tokens_dev_, residual_, status_dev_, token_embd_.dtype, c.hidden, token_vocab(), rows, scale};
        recording_->push_back(phase);
        recording_breaks_.push_back(pending_break_);
        pending_break_ = -1;
        return GF_OK;
    }
    ++launches_;
    return launch_embedding(token_embd_.dtype, token_embd_.data, c.hidden, token_vocab(), tokens_dev_, rows, scale, residual_, status_dev_, stream_, false);
}

int Model::emit_attention(const AttentionParams& params) {
    if (recording_) {
        AttentionParams ap = params;
        uint32_t group = 0, rows_per_block = 0, parts = 0;
        if (pass_mode_ == 1 && pending_break_ < 0 && pass_attention_supported(ap, ap.rows, group, rows_per_block, parts)) {
            PassPhase phase {};
            phase.kind = kPhaseAttention;
            phase.attention_group = group;
            phase.attention_rows = rows_per_block;
            ap.target_parts = parts;
            phase.attention = ap;
            recording_->push_back(phase);
            recording_breaks_.push_back(-1);
            return GF_OK;
        }
        if (pending_break_ >= 0) { recording_failed_ = true; return GF_OK; }      // two launches in a row: not a shape this schedule produces
        recording_pass_->attention_launches.push_back(ap);      // a launch of its own between two segments
        pending_break_ = (int)recording_pass_->attention_launches.size() - 1;
        return GF_OK;
    }
    ++launches_;
    return launch_attention(params, stream_, true);
}

void Model::invalidate_passes() {
    auto drop = [](RecordedPass& pass) {
        if (pass.table_dev) cudaFree(pass.table_dev);
        pass = RecordedPass();
    };
    for (auto& per_rows : passes_)
        for (auto& pass : per_rows) drop(pass);
    for (auto& pass : sweeps_) drop(pass);
}

// Records the launches of a pass (or of the weight sweep) as a phase table and cuts it into
// pass-kernel launches wherever an attention launch of its own has to run in between.
int Model::record_pass(uint32_t rows, uint32_t flags, bool sweep, RecordedPass& out) {
    std::vector<PassPhase> phases;
    out = RecordedPass();
    out.ready = true;
    recording_ = &phases;
    recording_pass_ = &out;
    recording_breaks_.clear();
    recording_failed_ = false;
    pending_break_ = -1;
    const uint32_t before = launches_;
    uint64_t bytes = 0;
    const int status = sweep ? encode_sweep(rows, nullptr, &bytes) : encode_blocks(rows, flags);
    launches_ = before;
    recording_ = nullptr;
    recording_pass_ = nullptr;
    if (status != GF_OK) return status;
    out.weight_bytes = bytes;
    if (recording_failed_ || pending_break_ >= 0 || phases.empty()) return GF_OK;       // not usable: the caller keeps the other schedule
    out.smem_bytes = pass_smem_bytes(phases.data(), (uint32_t)phases.size(), rows);
    if (out.smem_bytes == 0) return GF_OK;
    // Segments: a new one starts at every phase that an attention launch precedes.
    PassSegment segment{0, 0, ~0u, ~0u, -1};
    for (uint32_t i = 0; i < phases.size(); ++i) {
        if (recording_breaks_[i] >= 0) {
            if (segment.count == 0) return GF_OK;          // a pass does not begin with an attention launch
            segment.attention = recording_breaks_[i];
            out.segments.push_back(segment);
            segment = PassSegment{i, 0, ~0u, ~0u, -1};
        }
        if (phases[i].kind == kPhaseStream) {
            if (segment.first_stream == ~0u) segment.first_stream = segment.count;
            segment.last_stream = segment.count;
        }
        ++segment.count;
    }
    out.segments.push_back(segment);
    void* table = nullptr;
    GF_CUDA(cudaMalloc(&table, phases.size() * sizeof(PassPhase)));
    out.table_dev = static_cast<PassPhase*>(table);
    GF_CUDA(cudaMemcpyAsync(out.table_dev, phases.data(), phases.size() * sizeof(PassPhase), cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaStreamSynchronize(stream_));       // `phases` is pageable and goes out of scope
    out.phases = (uint32_t)phases.size();
    out.usable = true;
    return GF_OK;
}

int Model::run_recorded(const RecordedPass& pass, uint32_t rows) {
    for (const PassSegment& segment : pass.segments) {
        PassLaunch launch;
        launch.table_dev = pass.table_dev;
        launch.first = segment.first; launch.count = segment.count;
        launch.first_stream = segment.first_stream; launch.last_stream = segment.last_stream;
        launch.rows = rows;
        launch.smem_bytes = pass.smem_bytes;
        launch.arrived_dev = pass_arrived_;
        launch.base = pass_arrivals_;
        pass_arrivals_ += (segment.count - 1u) * (uint32_t)sm_count();      // one arrival per CTA and barrier
        launch.error_flag = error_flag_;
        launch.poll_limit = pass_poll_limit_;
        GF_TRY(launch_pass(launch, stream_));
        ++launches_;
        if (segment.attention >= 0) {
            GF_TRY(launch_attention(pass.attention_launches[(size_t)segment.attention], stream_, true));
            ++launches_;
        }
    }
    return GF_OK;
}

// One transformer pass: the operator order of encode_gemma_target_blocks
// (gemma_target_runtime.cpp:28-219), with the small operators folded into the GEMV launches:
//   QKV   <- prologue: [residual += norm(down; post_ffw)] ; norm(residual; attn_norm)
//   rope/norm/store, attention
//   O     <- prologue: merge of the attention partitions
//   gate,up <- prologue: residual2 = residual + norm(O; post_attention) ; norm(residual2; ffn_norm)
//   down  <- prologue: gelu_tanh(gate) * up
// The next layer's QKV (or the head) applies the post-FFW norm and residual of this layer.
int Model::encode_blocks(uint32_t rows, uint32_t flags) {
    const gf_model_config& c = config_;
    const float embedding_scale = sqrtf((float)c.hidden);     // f32, not bf16-rounded (model.cpp:599-605)
    const bool fused_exchange = shard_.connected;
    if (fused_exchange) {
        if (recording_) { recording_failed_ = true; return GF_OK; }      // the pass kernel has no phase for the exchange
        ++launches_;
        GF_TRY(launch_shard_tick(shard_.tick(), stream_));                // a new pass: new stamps
    }
    GF_TRY(emit_embedding(rows, embedding_scale));
    float* x = residual_;          // residual stream entering a layer
    float* x2 = post_attention_;   // residual stream after the attention branch
    // Weight sets of the launches.
    auto qkv_weights = [&](uint32_t l) {
        const LayerWeights& w = layers_[l];
        GemvLaunch g;
        g.k = c.hidden;
        g.matrices[0] = desc(w.q, raw_q_); g.matrices[1] = desc(w.k, raw_k_); g.matrices[2] = desc(w.v, raw_v_);
        g.count = unit_elements(w.q.dtype) == unit_elements(w.v.dtype) ? 3 : 2;
        return g;
    };
    auto o_weights = [&](uint32_t l) { GemvLaunch g; g.k = (uint64_t)c.heads * c.head_dim; g.matrices[0] = desc(layers_[l].o, projected_); return g; };
    auto gate_up_weights = [&](uint32_t l) {
        GemvLaunch g;
        g.k = c.hidden;
        g.matrices[0] = desc(layers_[l].gate, gate_); g.matrices[1] = desc(layers_[l].up, up_);
        g.count = 2;
        return g;
    };
    auto down_weights = [&](uint32_t l) { GemvLaunch g; g.k = c.ffn; g.matrices[0] = desc(layers_[l].down, projected_); return g; };
    auto head_weights = [&]() { GemvLaunch g; g.k = c.hidden; g.matrices[0] = desc(has_head_ ? head_ : token_embd_, logits_); return g; };
    for (uint32_t l = 0; l < c.layers; ++l) {
        const LayerWeights& w = layers_[l];
        const LayerCache& cache = caches_[l];
        GemvLaunch qkv = qkv_weights(l);
        if (qkv.count != 3) return fail(GF_ERR_INVALID, "attention projections of one layer must share a block family");
        if (l == 0) { qkv.prologue = kPrologueNorm; qkv.in = x; qkv.gamma1 = w.attn_norm; }
        else {
            qkv.prologue = kPrologueAddNorm; qkv.in = projected_; qkv.residual = x2; qkv.gamma0 = layers_[l - 1].post_ffw_norm;
            qkv.residual_out = x; qkv.gamma1 = w.attn_norm;
            if (fused_exchange) shard_gather(qkv, 1u, 2u * l);               // the down projection of the layer before
        }
        GemvLaunch o = o_weights(l);
        const bool fused_heads = cache.rope_rotation != nullptr;
        if (fused_heads) {      // per-head norm, RoPE and the private K/V store ride on the Q/K/V launch
            qkv.heads.q_norm = c.uses_qk_norm ? w.q_norm : nullptr; qkv.heads.k_norm = c.uses_qk_norm ? w.k_norm : nullptr;
            qkv.heads.q_out = query_; qkv.heads.private_k = cache.private_k; qkv.heads.private_v = cache.private_v;
            qkv.heads.rotation = cache.rope_rotation; qkv.heads.base_position = state_dev_; qkv.heads.status = status_dev_;
            qkv.heads.head_counters = head_counters_; qkv.heads.table_rows = c.context + GF_MAX_ROWS; qkv.heads.kv_f16 = c.kv_f16;
        }
        GF_TRY(run_gemv(qkv, rows));
        if (!fused_heads && recording_) { recording_failed_ = true; return GF_OK; }      // the separate rotation kernel has no phase
        if (!fused_heads) {
            RopeStoreParams rp{raw_q_, raw_k_, raw_v_, c.uses_qk_norm ? w.q_norm : nullptr, c.uses_qk_norm ? w.k_norm : nullptr,
                               query_, cache.private_k, cache.private_v, state_dev_, status_dev_, cache.rope_divisors, rows, c.heads, c.kv_heads,
                               c.head_dim, c.rms_eps, cache.rope_base, cache.rope_scale, c.kv_f16};
            GF_TRY(launch_rope_store(rp, stream_, true));
            launches_ += 1;
        }
        AttentionParams ap;
        ap.q = query_; ap.ring_k = cache.ring_k; ap.ring_v = cache.ring_v; ap.private_k = cache.private_k;
        ap.private_v = cache.private_v; ap.out = attention_out_;
        ap.partial_out = static_cast<float*>(attention_ws_);
        ap.partial_ml = ap.partial_out + (size_t)c.row_capacity * c.heads * kMaxAttentionPartitions * 256u;
        ap.counters = attention_counters(attention_ws_, c.row_capacity, c.heads);
        ap.base_position = state_dev_; ap.rows = rows; ap.heads = c.heads; ap.kv_heads = c.kv_heads; ap.head_dim = c.head_dim;
        ap.ring_mask = cache.ring_rows - 1u; ap.window = cache.window; ap.scale = c.attention_scale;
        ap.softcap = c.attn_softcap; ap.kv_f16 = c.kv_f16;
        ap.defer_merge = 1u;                 // the O projection's prologue merges the partitions
        GF_TRY(emit_attention(ap));
        o.prologue = kPrologueMerge; o.in = ap.partial_out; o.residual = ap.partial_ml;
        GemvLaunch gu = gate_up_weights(l);
        if (fused_exchange) shard_scatter(o, 0u, 2u * l + 1u);                    // a tensor-parallel shard holds a partial sum here:
        GF_TRY(run_gemv(o, rows));
        if (!fused_exchange) GF_TRY(reduce_partial(projected_, (size_t)rows * c.hidden));     // summed in the launches, or by the host's hook
        gu.prologue = kPrologueAddNorm; gu.in = projected_; gu.residual = x; gu.gamma0 = w.post_attention_norm;
        gu.residual_out = x2; gu.gamma1 = w.ffn_norm;
        if (fused_exchange) shard_gather(gu, 0u, 2u * l + 1u);
        GemvLaunch down = down_weights(l);
        GF_TRY(run_gemv(gu, rows));
        down.prologue = kPrologueGeglu; down.in = gate_; down.residual = up_;
        if (fused_exchange) shard_scatter(down, 1u, 2u * l + 2u);
        GF_TRY(run_gemv(down, rows));
        if (!fused_exchange) GF_TRY(reduce_partial(projected_, (size_t)rows * c.hidden));
    }
    if (flags & kForwardLogits) {
        GemvLaunch head = head_weights();
        head.prologue = kPrologueAddNorm; head.in = projected_; head.residual = x2;
        head.gamma0 = layers_[c.layers - 1].post_ffw_norm; head.residual_out = x; head.gamma1 = output_norm_;
        if (fused_exchange) shard_gather(head, 1u, 2u * c.layers);
        GF_TRY(run_gemv(head, rows));
    } else if (fused_exchange && shard_.size > 1u) {
        // Nobody reads the last down projection of a pass without logits.  Wait for the peers' parts of it all the
        // same: a peer then cannot start the next pass, whose first exchange reuses half 0, before this shard has
        // sent that part -- which it does only after it has finished reading half 0.
        ++launches_;
        ShardDrain drain {};
        drain.count = 0;
        for (uint32_t s = 0; s < shard_.size; ++s)
            if (s != shard_.rank) drain.parts[drain.count++] = shard_.part(shard_.arena, 1u, s);
        drain.tick = shard_.tick(); drain.site = 2u * c.layers; drain.values = rows * c.hidden;
        drain.wait_limit = shard_.wait_limit; drain.error_flag = error_flag_;
        GF_TRY(launch_shard_drain(drain, stream_, true));
    }
    return GF_OK;
}

int Model::run_graph_or_encode(uint32_t rows, uint32_t flags) {
    const int with_logits = (flags & kForwardLogits) ? 1 : 0;
    if (pass_mode_ != 0 && rows <= kPassMaxRows) {
        RecordedPass& pass = passes_[rows][with_logits];
        if (!pass.ready) GF_TRY(record_pass(rows, flags, false, pass));
        if (pass.usable) return run_recorded(pass, rows);
    }
    if (!use_graph_) return encode_blocks(rows, flags);
    cudaGraphExec_t& exec = graphs_[rows][with_logits];
    if (!exec) {
        // Record the pass once; every later token replays it (positions and ids live in device memory).
        const uint32_t before = launches_;
        cudaGraph_t graph = nullptr;
        GF_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
        const int status = encode_blocks(rows, flags);
        const cudaError_t end = cudaStreamEndCapture(stream_, &graph);
        graph_launches_[rows][with_logits] = launches_ - before;      // kernels recorded into this graph, counted as encoded
        launches_ = before;
        if (status != GF_OK) { if (graph) cudaGraphDestroy(graph); return status; }
        GF_CUDA(end);
        const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        GF_CUDA(inst);
    }
    GF_CUDA(cudaGraphLaunch(exec, stream_));
    launches_ += graph_launches_[rows][with_logits];
    return GF_OK;
}

int Model::forward(const uint32_t* tokens_host, uint32_t rows, uint32_t flags) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (poisoned_) return fail(GF_ERR_STATE, "plan is poisoned after an unknown GPU outcome; reset it");
    if (rows == 0 || rows > config_.row_capacity) return fail(GF_ERR_INVALID, "rows=%u outside [1, %u]", rows, config_.row_capacity);
    if (position_ > config_.context || rows > config_.context - position_)
        return fail(GF_ERR_INVALID, "pass exceeds the bound context (%u + %u > %u)", position_, rows, config_.context);
    if (!(flags & kForwardDeviceTokens)) {
        if (!tokens_host) return fail(GF_ERR_INVALID, "null token ids");
        for (uint32_t r = 0; r < rows; ++r)
            if (tokens_host[r] >= token_vocab()) return fail(GF_ERR_INVALID, "token id %u outside the vocabulary", tokens_host[r]);
        // The previous upload may still be reading the pinned staging words: wait for that copy only.
        GF_CUDA(cudaEventSynchronize(tokens_copied_));
        std::memcpy(tokens_pinned_, tokens_host, rows * sizeof(uint32_t));
        GF_CUDA(cudaMemcpyAsync(tokens_dev_, tokens_pinned_, rows * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
        GF_CUDA(cudaEventRecord(tokens_copied_, stream_));
    }
    return run_graph_or_encode(rows, flags);
}

int Model::publish(uint32_t rows) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (rows == 0 || rows > config_.row_capacity || rows > config_.context - position_)
        return fail(GF_ERR_INVALID, "cannot publish %u rows", rows);
    GF_TRY(launch_kv_publish(publish_layers_, config_.layers, state_dev_, rows, stream_));
    launches_ += 2u;
    position_ += rows;
    return GF_OK;
}

int Model::truncate(uint32_t position) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (position > position_) return fail(GF_ERR_INVALID, "cannot truncate forward");
    if (position_ - position > config_.row_capacity)
        return fail(GF_ERR_INVALID, "published sliding-window rows older than one pass cannot be restored");
    if (position != position_) {
        GF_CUDA(cudaMemcpyAsync(state_dev_, &position, sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
        GF_CUDA(cudaStreamSynchronize(stream_));
        position_ = position;
    }
    return GF_OK;
}

// Prompts with at least this many rows ahead of their last token take the tensor-core path.
constexpr uint32_t kTensorPrefillMinRows = 64;

int Model::prefill(const uint32_t* tokens_host, uint32_t count) {
    if (!tokens_host || count == 0) return fail(GF_ERR_INVALID, "empty prompt");
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    uint32_t done = 0;
    // A shard that sums through a host hook keeps to the row passes (the hook sits behind their launches).
    if (tensor_prefill_ && (!reduce_hook_ || shard_.connected) && count - 1u >= kTensorPrefillMinRows) {
        // All rows but the last as 128-row chunks through the tensor cores (K/V only: no chunk needs
        // logits, so the last layer stops after its K/V rows, gemma_target_runtime.cpp:59-61,125); the
        // last prompt token then runs as an ordinary one-row pass, which yields the logits.
        if (position_ > config_.context || count > config_.context - position_)
            return fail(GF_ERR_INVALID, "prompt exceeds the bound context (%u + %u > %u)", position_, count, config_.context);
        for (uint32_t i = 0; i < count; ++i)
            if (tokens_host[i] >= token_vocab()) return fail(GF_ERR_INVALID, "token id %u outside the vocabulary", tokens_host[i]);
        GF_TRY(ensure_prefill_arena());
        while (done < count - 1u) {
            const uint32_t rows = std::min(prefill_.chunk_rows, count - 1u - done);
            GF_TRY(prefill_chunk(tokens_host + done, rows));
            done += rows;
        }
        GF_TRY(forward(tokens_host + done, 1, kForwardLogits));
        GF_TRY(publish(1));
        prefill_logits_row_ = 0;
        return GF_OK;
    }
    while (done < count) {
        const uint32_t rows = std::min(config_.row_capacity, count - done);
        const bool last = done + rows == count;
        GF_TRY(forward(tokens_host + done, rows, last ? kForwardLogits : 0u));
        GF_TRY(publish(rows));
        prefill_logits_row_ = rows - 1u;
        done += rows;
    }
    return GF_OK;
}

int Model::ensure_prefill_arena() {
    if (prefill_.ready) return GF_OK;
    const gf_model_config& c = config_;
    const uint32_t qw = c.heads * c.head_dim, kvw = c.kv_heads * c.head_dim, R = kPrefillRows;
    if (qw % kPrefillTile || kvw % kPrefillTile || c.hidden % kPrefillTile || c.ffn % kPrefillTile)
        return fail(GF_ERR_INVALID, "tensor-core prefill needs projection widths that are multiples of %u", kPrefillTile);
    PrefillArena& a = prefill_;
    // A chunk must not publish two rows into one ring slot.
    a.chunk_rows = R;
    for (const LayerCache& cache : caches_) a.chunk_rows = std::min(a.chunk_rows, cache.ring_rows);
    uint8_t* bytes = nullptr;
    GF_TRY(device_alloc(allocations_, &bytes, tile_major_bytes(c.hidden))); a.a_hidden = bytes;
    GF_TRY(device_alloc(allocations_, &bytes, tile_major_bytes(qw))); a.a_q = bytes;
    GF_TRY(device_alloc(allocations_, &bytes, tile_major_bytes(c.ffn))); a.a_ffn = bytes;
    GF_TRY(device_alloc(allocations_, &a.residual, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &a.residual2, (size_t)R * c.hidden));
    GF_TRY(device_alloc(allocations_, &a.raw_q, (size_t)kPrefillMaxSplits * R * qw));           // K-split partial results
    GF_TRY(device_alloc(allocations_, &a.raw_k, (size_t)kPrefillMaxSplits * R * kvw));
    GF_TRY(device_alloc(allocations_, &a.raw_v, (size_t)kPrefillMaxSplits * R * kvw));
    GF_TRY(device_alloc(allocations_, &a.query, (size_t)R * qw));
    GF_TRY(device_alloc(allocations_, &a.attention_out, (size_t)R * qw));
    GF_TRY(device_alloc(allocations_, &a.projected, (size_t)kPrefillMaxSplits * R * c.hidden));      // K-split partial results
    GF_TRY(device_alloc(allocations_, &a.gate, (size_t)kPrefillMaxSplits * R * c.ffn));
    GF_TRY(device_alloc(allocations_, &a.up, (size_t)kPrefillMaxSplits * R * c.ffn));
    GF_TRY(device_alloc(allocations_, &a.tokens, R));
    const size_t element = c.kv_f16 ? 2 : 4;
    std::vector<KvPublishLayer> table(c.layers);
    a.private_k.resize(c.layers); a.private_v.resize(c.layers);
    for (uint32_t l = 0; l < c.layers; ++l) {
        uint8_t *pk, *pv;
        GF_TRY(device_alloc(allocations_, &pk, (size_t)R * kvw * element));
        GF_TRY(device_alloc(allocations_, &pv, (size_t)R * kvw * element));
        a.private_k[l] = pk; a.private_v[l] = pv;
        table[l] = KvPublishLayer{static_cast<uint8_t*>(caches_[l].ring_k), static_cast<uint8_t*>(caches_[l].ring_v), pk, pv,
                                  caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
    }
    GF_TRY(device_alloc(allocations_, &a.publish_layers, c.layers));
    GF_CUDA(cudaMemcpyAsync(a.publish_layers, table.data(), sizeof(KvPublishLayer) * c.layers, cudaMemcpyHostToDevice, stream_));
    GF_TRY(device_alloc(allocations_, &bytes, attention_workspace_bytes(R, c.heads))); a.attention_ws = bytes;
    GF_CUDA(cudaMemsetAsync(attention_counters(a.attention_ws, R, c.heads), 0, (size_t)R * c.heads * sizeof(uint32_t), stream_));
    GF_CUDA(cudaStreamSynchronize(stream_));       // `table` is pageable and goes out of scope
    a.ready = true;
    return GF_OK;
}

// One chunk of up to 128 prompt rows: every projection is one tensor-core GEMM over all rows of the
// chunk; norms, GeGLU and the attention output go through small kernels that write the next GEMM's bf16
// operand; RoPE / K/V store and attention reuse the row kernels.  The rows are published at the end.
int Model::prefill_chunk(const uint32_t* tokens_host, uint32_t rows) {
    const gf_model_config& c = config_;
    PrefillArena& a = prefill_;
    const uint32_t qw = c.heads * c.head_dim;
    GF_CUDA(cudaMemcpyAsync(a.tokens, tokens_host, rows * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
    GF_TRY(launch_embedding(token_embd_.dtype, token_embd_.data, c.hidden, token_vocab(), a.tokens, rows, sqrtf((float)c.hidden), a.residual,
                            status_dev_, stream_, false));
    launches_ += 1;
    const bool fused_exchange = shard_.connected;
    if (fused_exchange) { ++launches_; GF_TRY(launch_shard_tick(shard_.tick(), stream_)); }
    // A shard's O and down products are partial sums: the chunk's rows are summed over the shards in one launch.
    auto exchange = [&](uint32_t& splits, uint32_t half, uint32_t site) -> int {
        const ShardExchange& x = shard_;
        ShardBulk bulk {};
        bulk.x = a.projected; bulk.splits = splits; bulk.slab = kPrefillRows * c.hidden; bulk.values = rows * c.hidden;
        bulk.shards = x.size; bulk.self = x.rank; bulk.peers = 0;
        for (uint32_t s = 0; s < x.size; ++s) {
            bulk.parts[s] = x.part(x.arena, half, s);
            if (s != x.rank) bulk.out[bulk.peers++] = x.part(x.mapped[s], half, x.rank);
        }
        bulk.tick = x.tick(); bulk.site = site; bulk.wait_limit = x.wait_limit; bulk.error_flag = error_flag_;
        splits = 1;
        ++launches_;
        return launch_shard_bulk_exchange(bulk, stream_);
    };
    auto gemm = [&](std::initializer_list<std::pair<const PackedMatrix*, float*>> set, const void* operand, uint64_t k, uint32_t splits = 1) -> int {
        PrefillGemmLaunch launch;
        launch.count = 0;
        launch.splits = splits;
        for (const auto& entry : set) launch.matrices[launch.count++] = {entry.first->dtype, entry.first->data, entry.second, entry.first->n};
        launch.k = k;
        launch.a = operand;
        launch.rows = rows;
        ++launches_;
        return launch_prefill_gemm(launch, error_flag_, stream_);
    };
    uint32_t down_splits = 1;          // of the previous layer's down projection
    for (uint32_t l = 0; l < c.layers; ++l) {
        const LayerWeights& w = layers_[l];
        const LayerCache& cache = caches_[l];
        if (l == 0) GF_TRY(launch_prefill_norm(a.residual, 1, nullptr, nullptr, w.attn_norm, nullptr, a.a_hidden, rows, c.hidden, c.rms_eps, 0, stream_));
        else GF_TRY(launch_prefill_norm(a.projected, down_splits, a.residual2, layers_[l - 1].post_ffw_norm, w.attn_norm, a.residual, a.a_hidden, rows,
                                        c.hidden, c.rms_eps, 1, stream_));
        if (unit_elements(w.q.dtype) == unit_elements(w.v.dtype)) {
            const uint32_t splits = prefill_gemm_splits(w.q.n + w.k.n + w.v.n, c.hidden, w.q.dtype);
            GF_TRY(gemm({{&w.q, a.raw_q}, {&w.k, a.raw_k}, {&w.v, a.raw_v}}, a.a_hidden, c.hidden, splits));
            float* parts[3] = {a.raw_q, a.raw_k, a.raw_v};
            const uint64_t widths[3] = {w.q.n, w.k.n, w.v.n};
            GF_TRY(launch_prefill_reduce(parts, widths, 3, splits, rows, stream_));
        } else {
            GF_TRY(gemm({{&w.q, a.raw_q}, {&w.k, a.raw_k}}, a.a_hidden, c.hidden));
            GF_TRY(gemm({{&w.v, a.raw_v}}, a.a_hidden, c.hidden));
        }
        RopeStoreParams rp{a.raw_q, a.raw_k, a.raw_v, c.uses_qk_norm ? w.q_norm : nullptr, c.uses_qk_norm ? w.k_norm : nullptr, a.query,
                           a.private_k[l], a.private_v[l], state_dev_, status_dev_, cache.rope_divisors, rows, c.heads, c.kv_heads,
                           c.head_dim, c.rms_eps, cache.rope_base, cache.rope_scale, c.kv_f16};
        GF_TRY(launch_rope_store(rp, stream_, false));
        launches_ += 2;
        if (l + 1u == c.layers) break;          // nothing downstream of the last layer's K/V is needed
        AttentionParams ap;
        ap.q = a.query; ap.ring_k = cache.ring_k; ap.ring_v = cache.ring_v; ap.private_k = a.private_k[l]; ap.private_v = a.private_v[l];
        ap.out = a.attention_out;
        ap.partial_out = static_cast<float*>(a.attention_ws);
        ap.partial_ml = ap.partial_out + (size_t)kPrefillRows * c.heads * kMaxAttentionPartitions * 256u;
        ap.counters = attention_counters(a.attention_ws, kPrefillRows, c.heads);
        ap.base_position = state_dev_; ap.rows = rows; ap.heads = c.heads; ap.kv_heads = c.kv_heads; ap.head_dim = c.head_dim;
        ap.ring_mask = cache.ring_rows - 1u; ap.window = cache.window; ap.scale = c.attention_scale;
        ap.softcap = c.attn_softcap; ap.kv_f16 = c.kv_f16;
        ap.defer_merge = 0u;
        if (prefill_attention_supported(ap)) GF_TRY(launch_prefill_attention(ap, stream_));
        else GF_TRY(launch_attention(ap, stream_, false));
        GF_TRY(launch_prefill_pack(a.attention_out, a.a_q, rows, qw, stream_));
        uint32_t o_splits = prefill_gemm_splits(w.o.n, w.o.k, w.o.dtype);
        GF_TRY(gemm({{&w.o, a.projected}}, a.a_q, qw, o_splits));
        if (fused_exchange) GF_TRY(exchange(o_splits, 0u, 2u * l + 1u));
        GF_TRY(launch_prefill_norm(a.projected, o_splits, a.residual, w.post_attention_norm, w.ffn_norm, a.residual2, a.a_hidden, rows, c.hidden,
                                   c.rms_eps, 1, stream_));
        uint32_t ffn_splits = 1;
        if (unit_elements(w.gate.dtype) == unit_elements(w.up.dtype)) {
            ffn_splits = prefill_gemm_splits(w.gate.n + w.up.n, c.hidden, w.gate.dtype);
            GF_TRY(gemm({{&w.gate, a.gate}, {&w.up, a.up}}, a.a_hidden, c.hidden, ffn_splits));
        } else {
            GF_TRY(gemm({{&w.gate, a.gate}}, a.a_hidden, c.hidden));
            GF_TRY(gemm({{&w.up, a.up}}, a.a_hidden, c.hidden));
        }
        GF_TRY(launch_prefill_geglu(a.gate, a.up, ffn_splits, a.a_ffn, rows, c.ffn, stream_));
        down_splits = prefill_gemm_splits(w.down.n, w.down.k, w.down.dtype);
        GF_TRY(gemm({{&w.down, a.projected}}, a.a_ffn, c.ffn, down_splits));
        if (fused_exchange) GF_TRY(exchange(down_splits, 1u, 2u * l + 2u));
        launches_ += 5;
    }
    GF_TRY(launch_kv_publish(a.publish_layers, c.layers, state_dev_, rows, stream_));
    launches_ += 2;
    position_ += rows;
    return GF_OK;
}

int Model::weight_sweep(uint32_t rows, uint32_t* out_launches, uint64_t* out_bytes) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (rows == 0 || rows > config_.row_capacity) return fail(GF_ERR_INVALID, "bad row count");
    if (pass_mode_ != 0 && rows <= kPassMaxRows) {
        RecordedPass& pass = sweeps_[rows];
        if (!pass.ready) GF_TRY(record_pass(rows, 0, true, pass));
        if (pass.usable) {
            if (out_launches) *out_launches = (uint32_t)pass.segments.size();
            if (out_bytes) *out_bytes = pass.weight_bytes;
            return run_recorded(pass, rows);
        }
    }
    return encode_sweep(rows, out_launches, out_bytes);
}

int Model::encode_sweep(uint32_t rows, uint32_t* out_launches, uint64_t* out_bytes) {
    uint32_t launches = 0;
    uint64_t bytes = 0;
    std::vector<GemvLaunch> sequence;
    auto add = [&](std::initializer_list<std::pair<const PackedMatrix*, float*>> set, const float* x) {
        GemvLaunch launch;
        launch.count = 0;
        for (const auto& entry : set) {
            launch.matrices[launch.count++] = desc(*entry.first, entry.second);
            launch.k = entry.first->k;
            bytes += entry.first->native_bytes;
        }
        launch.in = x;
        sequence.push_back(launch);
    };
    for (const LayerWeights& w : layers_) {
        add({{&w.q, raw_q_}, {&w.k, raw_k_}, {&w.v, raw_v_}}, normalized_);
        add({{&w.o, projected_}}, attention_out_);
        add({{&w.gate, gate_}, {&w.up, up_}}, normalized_);
        add({{&w.down, projected_}}, gated_);
    }
    add({{has_head_ ? &head_ : &token_embd_, logits_}}, normalized_);
    for (size_t i = 0; i < sequence.size(); ++i) {
        ++launches;
        GF_TRY(run_gemv(sequence[i], rows));
    }
    if (out_launches) *out_launches = launches;
    if (out_bytes) *out_bytes = bytes;
    return GF_OK;
}

int Model::set_device_token(uint32_t row, uint32_t token) {
    if (row >= GF_MAX_ROWS || token >= token_vocab()) return fail(GF_ERR_INVALID, "bad device token slot or id");
    GF_CUDA(cudaEventSynchronize(tokens_copied_));
    tokens_pinned_[row] = token;
    GF_CUDA(cudaMemcpyAsync(tokens_dev_ + row, tokens_pinned_ + row, sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaEventRecord(tokens_copied_, stream_));
    return GF_OK;
}

int Model::select_device(uint32_t rows) {
    if (shard_.global_selection && !selecting_global_)
        return fail(GF_ERR_STATE, "selection requests written on the device are not offered on a shard with global selection (repetition penalty 1 only)");
    launches_ += 2;
    return launch_candidates(logits_, rows, config_.vocab, config_.final_softcap, requests_dev_, candidates_ws_, results_dev_,
                             stream_, false);
}

int Model::select(const void* requests_host, uint32_t rows) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (!requests_host || rows == 0 || rows > config_.row_capacity) return fail(GF_ERR_INVALID, "bad selection request");
    const size_t bytes = (size_t)rows * gf_selection_request_bytes();
    GF_CUDA(cudaEventSynchronize(requests_copied_));
    std::memcpy(requests_pinned_, requests_host, bytes);
    if (shard_.global_selection) {
        // Keep the caller's requests for the merge; this shard selects with the history tokens of its own slice.
        shard_.global_requests.assign(static_cast<const uint8_t*>(requests_host), static_cast<const uint8_t*>(requests_host) + bytes);
        const uint32_t first = shard_.rank * config_.vocab;
        SelectionRequestRow* local = static_cast<SelectionRequestRow*>(requests_pinned_);
        for (uint32_t r = 0; r < rows; ++r) {
            const SelectionRequestRow global = local[r];
            if (global.history_count > 64u) return fail(GF_ERR_INVALID, "selection request names more than 64 history tokens");
            local[r].history_count = 0;
            for (uint32_t i = 0; i < global.history_count; ++i) {
                const uint32_t token = global.history[i];
                if (token >= token_vocab()) return fail(GF_ERR_INVALID, "history token %u outside the vocabulary", token);
                if (token >= first && token - first < config_.vocab) local[r].history[local[r].history_count++] = token - first;
            }
        }
    }
    GF_CUDA(cudaMemcpyAsync(requests_dev_, requests_pinned_, bytes, cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaEventRecord(requests_copied_, stream_));
    selecting_global_ = true;
    const int status = select_device(rows);
    selecting_global_ = false;
    return status;
}

int Model::read_candidates(void* results_host, uint32_t rows) {
    if (!results_host || rows == 0 || rows > config_.row_capacity) return fail(GF_ERR_INVALID, "bad candidate readback");
    if (shard_.global_selection) return read_candidates_global(results_host, rows);
    GF_CUDA(cudaMemcpyAsync(results_host, results_dev_, (size_t)rows * gf_candidate_result_bytes(), cudaMemcpyDeviceToHost, stream_));
    return synchronize();
}

// Candidate rows of every shard, gathered over peer memory, merged into rows over the whole vocabulary: the best
// `retain` pairs of all slices by (logit descending, token ascending), then the history tokens' pairs in the
// request's order, each from the shard that owns the token.
int Model::read_candidates_global(void* results_host, uint32_t rows) {
    ShardExchange& x = shard_;
    if (x.global_requests.size() < (size_t)rows * sizeof(SelectionRequestRow)) return fail(GF_ERR_STATE, "no selection is in flight for these rows");
    const uint32_t row_words = (uint32_t)(gf_candidate_result_bytes() / sizeof(uint32_t)), words = rows * row_words;
    ShardGather g {};
    g.local = static_cast<const uint32_t*>(results_dev_); g.gathered = x.gathered_dev; g.words = words;
    g.shards = x.size; g.self = x.rank; g.peers = 0;
    const uint32_t parity = x.gathers & 1u;
    for (uint32_t s = 0; s < x.size; ++s) {
        g.parts[s] = x.rows_slot(x.arena, parity, s);
        if (s != x.rank) g.out[g.peers++] = x.rows_slot(x.mapped[s], parity, x.rank);
    }
    g.stamp = ++x.gathers;                  // never 0, the arena's initial content
    if (x.gathers == 0u) g.stamp = ++x.gathers;
    g.wait_limit = x.wait_limit; g.error_flag = error_flag_;
    ++launches_;
    GF_TRY(launch_shard_gather(g, stream_));
    for (uint32_t s = 0; s < x.size; ++s)
        GF_CUDA(cudaMemcpyAsync(x.gathered_host + (size_t)s * words, x.gathered_dev + (size_t)s * words,
                                (size_t)words * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_));
    GF_TRY(synchronize());
    const SelectionRequestRow* requests = reinterpret_cast<const SelectionRequestRow*>(x.global_requests.data());
    CandidateRow* out = static_cast<CandidateRow*>(results_host);
    std::vector<TokenLogit> pool;
    for (uint32_t r = 0; r < rows; ++r) {
        const SelectionRequestRow& request = requests[r];
        const uint32_t retain = request.retain;
        CandidateRow& merged = out[r];
        merged.status = 0;
        pool.clear();
        uint32_t history_seen[8] = {};       // history pairs consumed so far from each shard's row
        for (uint32_t s = 0; s < x.size; ++s) {
            const CandidateRow& theirs = *reinterpret_cast<const CandidateRow*>(x.gathered_host + (size_t)s * words + (size_t)r * row_words);
            merged.status |= theirs.status;
            for (uint32_t i = 0; i < retain && i < theirs.count; ++i)
                if (theirs.candidates[i].token != 0xffffffffu) pool.push_back(TokenLogit{theirs.candidates[i].token + s * config_.vocab, theirs.candidates[i].logit});
        }
        std::sort(pool.begin(), pool.end(), [](const TokenLogit& a, const TokenLogit& b) {
            return a.logit > b.logit || (a.logit == b.logit && a.token < b.token);      // +0 and -0 tie, as on the device
        });
        uint32_t count = 0;
        for (; count < retain && count < pool.size(); ++count) merged.candidates[count] = pool[count];
        for (; count < retain; ++count) merged.candidates[count] = TokenLogit{0xffffffffu, -INFINITY};
        for (uint32_t i = 0; i < request.history_count; ++i) {
            const uint32_t token = request.history[i], owner = token / config_.vocab;
            const CandidateRow& theirs = *reinterpret_cast<const CandidateRow*>(x.gathered_host + (size_t)owner * words + (size_t)r * row_words);
            const TokenLogit pair = theirs.candidates[retain + history_seen[owner]++];
            merged.candidates[count++] = TokenLogit{pair.token == 0xffffffffu ? pair.token : pair.token + owner * config_.vocab, pair.logit};
        }
        merged.count = count;
    }
    return GF_OK;
}

int Model::read_logits(uint32_t row, float* host) {
    if (!host || row >= config_.row_capacity) return fail(GF_ERR_INVALID, "bad logits readback");
    GF_CUDA(cudaMemcpyAsync(host, logits_ + (size_t)row * config_.vocab, (size_t)config_.vocab * 4, cudaMemcpyDeviceToHost, stream_));
    return synchronize();
}

int Model::read_kv(uint32_t layer, uint32_t first_position, uint32_t count, float* k_host, float* v_host) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (layer >= config_.layers || !k_host || !v_host || count == 0) return fail(GF_ERR_INVALID, "bad K/V readback");
    const LayerCache& cache = caches_[layer];
    if (first_position + count > position_ || position_ - first_position > cache.ring_rows)
        return fail(GF_ERR_INVALID, "K/V rows [%u, %u) are not all committed and still inside layer %u's ring", first_position,
                    first_position + count, layer);
    const size_t kvw = (size_t)config_.kv_heads * config_.head_dim, element = config_.kv_f16 ? 2 : 4;
    std::vector<uint8_t> raw[2];
    const void* rings[2] = {cache.ring_k, cache.ring_v};
    for (int which = 0; which < 2; ++which) {
        raw[which].resize((size_t)count * kvw * element);
        uint32_t done = 0;
        while (done < count) {                       // at most two contiguous runs of ring slots
            const uint32_t slot = (first_position + done) & (cache.ring_rows - 1u);
            const uint32_t run = std::min(count - done, cache.ring_rows - slot);
            GF_CUDA(cudaMemcpyAsync(raw[which].data() + (size_t)done * kvw * element,
                                    static_cast<const uint8_t*>(rings[which]) + (size_t)slot * kvw * element,
                                    (size_t)run * kvw * element, cudaMemcpyDeviceToHost, stream_));
            done += run;
        }
    }
    GF_TRY(synchronize());
    float* outs[2] = {k_host, v_host};
    for (int which = 0; which < 2; ++which) {
        if (!config_.kv_f16) { std::memcpy(outs[which], raw[which].data(), raw[which].size()); continue; }
        const __half* src = reinterpret_cast<const __half*>(raw[which].data());
        for (size_t i = 0; i < (size_t)count * kvw; ++i) outs[which][i] = __half2float(src[i]);
    }
    return GF_OK;
}

int Model::synchronize() {
    const cudaError_t error = cudaStreamSynchronize(stream_);
    if (error != cudaSuccess) { poisoned_ = true; return check_cuda(error, "stream synchronize"); }
    return GF_OK;
}

int Model::status_word(uint32_t* out) {
    uint32_t host[2] = {0, 0};
    GF_CUDA(cudaMemcpyAsync(&host[0], status_dev_, 4, cudaMemcpyDeviceToHost, stream_));
    GF_CUDA(cudaMemcpyAsync(&host[1], error_flag_, 4, cudaMemcpyDeviceToHost, stream_));
    GF_TRY(synchronize());
    if (out) *out = host[0];
    if (host[1] != 0) { poisoned_ = true; return fail(GF_ERR_TIMEOUT, "a bounded device wait gave up (a weight copy, or a peer shard's values)"); }
    if (host[0] & kStatusKvNonFinite) { poisoned_ = true; return fail(GF_ERR_NUMERIC, "non-finite F16 K/V (status %u)", host[0]); }
    if (host[0] & kStatusBadPosition) { poisoned_ = true; return fail(GF_ERR_STATE, "a pass ran beyond the tabulated positions (status %u)", host[0]); }
    return GF_OK;
}

size_t Model::kv_bytes_per_pass(uint32_t rows) const {
    // Cached rows one pass has to read: every committed row inside each layer's window, K and V,
    // once -- the rows of a pass look at the same cache (the reference counts it the same way,
    // docs/archive/DEVELOPMENT_HISTORY.md: 8 global x context + 40 local x window rows of 8 KB).
    if (rows == 0) return 0;
    const size_t row_bytes = (size_t)config_.kv_heads * config_.head_dim * (config_.kv_f16 ? 2 : 4) * 2;
    size_t total = 0;
    for (const LayerCache& cache : caches_) {
        const uint32_t seen = cache.window ? std::min(position_, cache.window) : position_;
        total += (size_t)seen * row_bytes;
    }
    return total;
}

}  // namespace gf

using namespace gf;

extern "C" {

int gf_model_create(const gf_model_config* config, gf_model** out_model) {
    if (!config || !out_model) return fail(GF_ERR_INVALID, "gf_model_create: null argument");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        return fail(GF_ERR_UNAVAILABLE, "no CUDA device is available; this backend has no CPU path");
    if (config->layers == 0 || config->hidden == 0 || config->vocab == 0 || config->hidden % 128u || config->ffn % 128u)
        return fail(GF_ERR_INVALID, "gf_model_create: bad geometry");
    *out_model = new gf_model(*config);
    return GF_OK;
}
int gf_model_destroy(gf_model* model) { delete model; return GF_OK; }
int gf_model_set_matrix(gf_model* m, int kind, uint32_t layer, int dtype, const void* native_host, uint64_t k, uint64_t n) {
    return m ? m->impl.set_matrix(kind, layer, dtype, native_host, k, n) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_set_matrix_requantized(gf_model* m, int kind, uint32_t layer, const void* native_q6_k_host, uint64_t k, uint64_t n) {
    return m ? m->impl.set_matrix(kind, layer, GF_Q6_K, native_q6_k_host, k, n, true) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_set_token_table_vocab(gf_model* m, uint32_t vocab) {
    return m ? m->impl.set_token_table_vocab(vocab) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_shard_prepare(gf_model* m, uint32_t rank, uint32_t size, void* ipc_handle_out) {
    return m ? m->impl.shard_prepare(rank, size, ipc_handle_out) : fail(GF_ERR_INVALID, "null model");
}
void* gf_model_shard_arena(gf_model* m) { return m ? m->impl.shard_arena() : nullptr; }
size_t gf_model_shard_arena_bytes(gf_model* m) { return m ? m->impl.shard_arena_bytes() : 0; }
int gf_model_shard_connect(gf_model* m, void* const* arenas) {
    return m ? m->impl.shard_connect(arenas) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_shard_connect_ipc(gf_model* m, const void* handles) {
    return m ? m->impl.shard_connect_ipc(handles) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_shard_global_selection(gf_model* m, int enable) {
    return m ? m->impl.shard_global_selection(enable != 0) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_shard_set_wait_limit(gf_model* m, uint32_t polls) {
    if (!m) return fail(GF_ERR_INVALID, "null model");
    m->impl.shard_set_wait_limit(polls);
    return GF_OK;
}
int gf_model_set_reduce_hook(gf_model* m, gf_reduce_fn hook, void* user) {
    return m ? m->impl.set_reduce_hook(hook, user) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_set_vector(gf_model* m, int kind, uint32_t layer, const float* values_host, uint32_t count) {
    return m ? m->impl.set_vector(kind, layer, values_host, count) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_finalize(gf_model* m) { return m ? m->impl.finalize() : fail(GF_ERR_INVALID, "null model"); }
int gf_model_reset(gf_model* m) { return m ? m->impl.reset() : fail(GF_ERR_INVALID, "null model"); }
int gf_model_position(const gf_model* m, uint32_t* out) {
    if (!m || !out) return fail(GF_ERR_INVALID, "null argument");
    *out = m->impl.position();
    return GF_OK;
}
int gf_model_forward(gf_model* m, const uint32_t* tokens_host, uint32_t rows, uint32_t flags) {
    return m ? m->impl.forward(tokens_host, rows, flags) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_publish(gf_model* m, uint32_t rows) { return m ? m->impl.publish(rows) : fail(GF_ERR_INVALID, "null model"); }
int gf_model_prefill(gf_model* m, const uint32_t* tokens_host, uint32_t count) {
    return m ? m->impl.prefill(tokens_host, count) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_truncate(gf_model* m, uint32_t position) { return m ? m->impl.truncate(position) : fail(GF_ERR_INVALID, "null model"); }
int gf_model_select(gf_model* m, const void* requests_host, uint32_t rows) {
    return m ? m->impl.select(requests_host, rows) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_read_candidates(gf_model* m, void* results_host, uint32_t rows) {
    return m ? m->impl.read_candidates(results_host, rows) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_read_logits(gf_model* m, uint32_t row, float* logits_host) {
    return m ? m->impl.read_logits(row, logits_host) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_read_kv(gf_model* m, uint32_t layer, uint32_t first_position, uint32_t count, float* k_host, float* v_host) {
    return m ? m->impl.read_kv(layer, first_position, count, k_host, v_host) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_synchronize(gf_model* m) { return m ? m->impl.synchronize() : fail(GF_ERR_INVALID, "null model"); }
int gf_model_status(gf_model* m, uint32_t* out_status) { return m ? m->impl.status_word(out_status) : fail(GF_ERR_INVALID, "null model"); }
void* gf_model_stream(gf_model* m) { return m ? m->impl.stream() : nullptr; }
uint32_t* gf_model_tokens_dev(gf_model* m) { return m ? m->impl.tokens_dev() : nullptr; }
float* gf_model_logits_dev(gf_model* m) { return m ? m->impl.logits_dev() : nullptr; }
size_t gf_model_weight_bytes(const gf_model* m, int native) {
    return m ? (native ? m->impl.native_weight_bytes() : m->impl.weight_bytes()) : 0;
}
size_t gf_model_kv_bytes_per_pass(const gf_model* m, uint32_t rows) { return m ? m->impl.kv_bytes_per_pass(rows) : 0; }
uint32_t gf_model_kernel_launches(const gf_model* m) { return m ? m->impl.kernel_launches() : 0; }
int gf_model_weight_sweep(gf_model* m, uint32_t rows, uint32_t* out_launches, uint64_t* out_weight_bytes) {
    return m ? m->impl.weight_sweep(rows, out_launches, out_weight_bytes) : fail(GF_ERR_INVALID, "null model");
}
int gf_model_use_graph(gf_model* m, int enable) {
    if (!m) return fail(GF_ERR_INVALID, "null model");
    m->impl.set_use_graph(enable != 0);
    return GF_OK;
}
int gf_model_use_tensor_prefill(gf_model* m, int enable) {
    if (!m) return fail(GF_ERR_INVALID, "null model");
    m->impl.set_tensor_prefill(enable != 0);
    return GF_OK;
}
uint32_t gf_model_prefill_logits_row(const gf_model* m) { return m ? m->impl.prefill_logits_row() : 0; }
int gf_model_use_pass_kernel(gf_model* m, int mode) {
    if (!m || mode < 0 || mode > 2) return fail(GF_ERR_INVALID, "gf_model_use_pass_kernel: mode must be 0, 1 or 2");
    m->impl.set_pass_mode(mode);
    return GF_OK;
}

}  // extern "C"
