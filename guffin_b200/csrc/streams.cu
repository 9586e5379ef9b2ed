// Independent conversation streams on one GPU: every stream has its own KV rings and position, all of
// them share one resident plan's weights, and a decode step streams the weights once per group of up to
// `row_capacity` streams instead of once per stream.  Streams never exchange anything: this is the
// data-parallel unit that is spread over the GPUs of a node, one process per GPU and no collective.
//
// A step for a group of streams is the block schedule of encode_gemma_target_blocks
// (src/engine/gemma_target_runtime.cpp:13-221) with the rows of the pass belonging to different
// conversations: row r is rotated at stream r's position, attends stream r's rings plus its own new
// key/value row, and that row is published into stream r's rings at the end of the pass.  The
// projections are the same row-count-invariant products as single-stream decoding, so a stream's logits
// do not depend on which other streams share its pass (rows 1-4; rows 5-8 likewise among themselves).
// Prompts are ingested per stream through the plan's own prefill path with the stream's rings bound.
// The reference decodes one conversation at a time; its Gemma 2 decode graph
// (run_gemma2_metal_resident_decode_step, src/engine/gemma2_runtime.cpp:250-418) is what each row computes.
#include "model.cuh"

#include <algorithm>
#include <cstring>

#define GF_TRY(expr) do { const int gf_s_ = (expr); if (gf_s_ != GF_OK) return gf_s_; } while (0)

namespace gf {

size_t candidates_workspace_bytes(uint32_t rows, uint32_t vocab);
int launch_candidates(const float* logits, uint32_t rows, uint32_t vocab, float softcap, const void* requests,
                      void* workspace, void* results, cudaStream_t stream, bool pdl);

StreamSet::~StreamSet() {
    for (cudaGraphExec_t exec : group_graphs) if (exec) cudaGraphExecDestroy(exec);
    if (wide_graph) cudaGraphExecDestroy(wide_graph);
    for (void* p : allocations) cudaFree(p);
    if (requests_pinned) cudaFreeHost(requests_pinned);
}

template <typename T>
static int stream_alloc(StreamSet& set, T** out, size_t count) {
    void* p = nullptr;
    GF_CUDA(cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 256)));
    set.allocations.push_back(p);
    *out = static_cast<T*>(p);
    return GF_OK;
}

int Model::streams_create(uint32_t count, StreamSet** out) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (sharded()) return fail(GF_ERR_STATE, "conversation streams are not offered on a tensor-parallel shard");
    if (!out || count == 0 || count > kMaxStreams) return fail(GF_ERR_INVALID, "between 1 and %u streams", kMaxStreams);
    const gf_model_config& c = config_;
    std::unique_ptr<StreamSet> set(new StreamSet());
    set->count = count;
    set->ring_k.assign(count, std::vector<void*>(c.layers));
    set->ring_v.assign(count, std::vector<void*>(c.layers));
    set->positions_host.assign(count, 0u);
    const size_t element = c.kv_f16 ? 2 : 4, kvw = (size_t)c.kv_heads * c.head_dim;
    std::vector<StreamRings> rings((size_t)c.layers * count);
    std::vector<StreamPublishLayer> layers(c.layers);
    for (uint32_t l = 0; l < c.layers; ++l) {
        const size_t bytes = (size_t)caches_[l].ring_rows * kvw * element;
        for (uint32_t s = 0; s < count; ++s) {
            uint8_t *k = nullptr, *v = nullptr;
            GF_TRY(stream_alloc(*set, &k, bytes));
            GF_TRY(stream_alloc(*set, &v, bytes));
            GF_CUDA(cudaMemsetAsync(k, 0, bytes, stream_));
            GF_CUDA(cudaMemsetAsync(v, 0, bytes, stream_));
            set->ring_k[s][l] = k;
            set->ring_v[s][l] = v;
            rings[(size_t)l * count + s] = StreamRings{k, v};
        }
        layers[l] = StreamPublishLayer{static_cast<const uint8_t*>(caches_[l].private_k), static_cast<const uint8_t*>(caches_[l].private_v),
                                       caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
    }
    GF_TRY(stream_alloc(*set, &set->rings_dev, rings.size()));
    GF_TRY(stream_alloc(*set, &set->publish_layers_dev, layers.size()));
    GF_TRY(stream_alloc(*set, &set->positions_dev, count));
    GF_TRY(stream_alloc(*set, &set->logits, (size_t)prefill_padded_rows(count) * c.vocab));      // a tensor-core step writes whole halves of 128 rows
    uint8_t* bytes = nullptr;
    GF_TRY(stream_alloc(*set, &bytes, candidates_workspace_bytes(count, c.vocab))); set->candidates_ws = bytes;
    GF_TRY(stream_alloc(*set, &bytes, (size_t)count * gf_selection_request_bytes())); set->requests_dev = bytes;
    GF_TRY(stream_alloc(*set, &bytes, (size_t)count * gf_candidate_result_bytes())); set->results_dev = bytes;
    GF_CUDA(cudaHostAlloc(&set->requests_pinned, (size_t)count * gf_selection_request_bytes(), cudaHostAllocDefault));
    GF_CUDA(cudaMemcpyAsync(set->rings_dev, rings.data(), rings.size() * sizeof(StreamRings), cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaMemcpyAsync(set->publish_layers_dev, layers.data(), layers.size() * sizeof(StreamPublishLayer), cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaMemsetAsync(set->positions_dev, 0, count * sizeof(uint32_t), stream_));
    GF_CUDA(cudaStreamSynchronize(stream_));
    *out = set.release();
    return GF_OK;
}

// Points the plan's cache at other rings (a stream's, or its own again): the publication tables name the
// rings, and recorded graphs and pass tables have the old pointers baked in.
int Model::bind_rings(const std::vector<void*>& ring_k, const std::vector<void*>& ring_v, uint32_t position) {
    const gf_model_config& c = config_;
    const size_t element = c.kv_f16 ? 2 : 4, kvw = (size_t)c.kv_heads * c.head_dim;
    std::vector<KvPublishLayer> table(c.layers), prefill_table(c.layers);
    for (uint32_t l = 0; l < c.layers; ++l) {
        caches_[l].ring_k = ring_k[l];
        caches_[l].ring_v = ring_v[l];
        table[l] = KvPublishLayer{static_cast<uint8_t*>(ring_k[l]), static_cast<uint8_t*>(ring_v[l]), static_cast<const uint8_t*>(caches_[l].private_k),
                                  static_cast<const uint8_t*>(caches_[l].private_v), caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
        if (prefill_.ready)
            prefill_table[l] = KvPublishLayer{static_cast<uint8_t*>(ring_k[l]), static_cast<uint8_t*>(ring_v[l]), static_cast<const uint8_t*>(prefill_.private_k[l]),
                                              static_cast<const uint8_t*>(prefill_.private_v[l]), caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
    }
    GF_CUDA(cudaMemcpyAsync(publish_layers_, table.data(), sizeof(KvPublishLayer) * c.layers, cudaMemcpyHostToDevice, stream_));
    if (prefill_.ready)
        GF_CUDA(cudaMemcpyAsync(prefill_.publish_layers, prefill_table.data(), sizeof(KvPublishLayer) * c.layers, cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaMemcpyAsync(state_dev_, &position, sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
    GF_CUDA(cudaStreamSynchronize(stream_));           // the tables above are pageable
    for (auto& per_rows : graphs_)
        for (cudaGraphExec_t& exec : per_rows)
            if (exec) { cudaGraphExecDestroy(exec); exec = nullptr; }
    invalidate_passes();
    position_ = position;
    return GF_OK;
}

int Model::streams_prefill(StreamSet& set, uint32_t stream, const uint32_t* tokens_host, uint32_t count) {
    if (stream >= set.count) return fail(GF_ERR_INVALID, "stream %u of %u", stream, set.count);
    std::vector<void*> home_k(config_.layers), home_v(config_.layers);
    for (uint32_t l = 0; l < config_.layers; ++l) { home_k[l] = caches_[l].ring_k; home_v[l] = caches_[l].ring_v; }
    const uint32_t home_position = position_;
    // The tensor-core prompt path allocates its arena on first use, before the rings are exchanged, so that
    // its publication table is rebuilt with the stream's rings like the plan's own.
    if (tensor_prefill_ && count > 64u) GF_TRY(ensure_prefill_arena());
    GF_TRY(bind_rings(set.ring_k[stream], set.ring_v[stream], set.positions_host[stream]));
    int status = prefill(tokens_host, count);
    if (status == GF_OK) {
        // The last prompt token's logits become the stream's row of the batch logits.
        status = check_cuda(cudaMemcpyAsync(set.logits + (size_t)stream * config_.vocab, logits_ + (size_t)prefill_logits_row_ * config_.vocab,
                                            (size_t)config_.vocab * sizeof(float), cudaMemcpyDeviceToDevice, stream_), "logits");
        set.positions_host[stream] = position_;
        if (status == GF_OK) status = check_cuda(cudaMemcpyAsync(set.positions_dev + stream, &set.positions_host[stream], sizeof(uint32_t),
                                                                 cudaMemcpyHostToDevice, stream_), "position");
        if (status == GF_OK) status = check_cuda(cudaStreamSynchronize(stream_), "prefill");
    }
    const int restored = bind_rings(home_k, home_v, home_position);
    return status != GF_OK ? status : restored;
}

// One pass over `rows` <= row_capacity streams starting at `first`: their token ids are in tokens_dev_.
int Model::encode_stream_group(StreamSet& set, uint32_t first, uint32_t rows) {
    const gf_model_config& c = config_;
    GF_TRY(emit_embedding(rows, sqrtf((float)c.hidden)));
    float* x = residual_;
    float* x2 = post_attention_;
    const uint32_t* positions = set.positions_dev + first;
    for (uint32_t l = 0; l < c.layers; ++l) {
        const LayerWeights& w = layers_[l];
        const LayerCache& cache = caches_[l];
        GemvLaunch qkv;
        qkv.k = c.hidden;
        qkv.matrices[0] = GemvMatrixDesc{w.q.dtype, w.q.data, raw_q_, w.q.n};
        qkv.matrices[1] = GemvMatrixDesc{w.k.dtype, w.k.data, raw_k_, w.k.n};
        qkv.matrices[2] = GemvMatrixDesc{w.v.dtype, w.v.data, raw_v_, w.v.n};
        qkv.count = 3;
        if (unit_elements(w.q.dtype) != unit_elements(w.v.dtype)) return fail(GF_ERR_INVALID, "attention projections of one layer must share a block family");
        if (l == 0) { qkv.prologue = kPrologueNorm; qkv.in = x; qkv.gamma1 = w.attn_norm; }
        else {
            qkv.prologue = kPrologueAddNorm; qkv.in = projected_; qkv.residual = x2; qkv.gamma0 = layers_[l - 1].post_ffw_norm;
            qkv.residual_out = x; qkv.gamma1 = w.attn_norm;
        }
        GF_TRY(run_gemv(qkv, rows));
        RopeStoreParams rp{raw_q_, raw_k_, raw_v_, c.uses_qk_norm ? w.q_norm : nullptr, c.uses_qk_norm ? w.k_norm : nullptr,
                           query_, cache.private_k, cache.private_v, state_dev_, status_dev_, cache.rope_divisors, rows, c.heads, c.kv_heads,
                           c.head_dim, c.rms_eps, cache.rope_base, cache.rope_scale, c.kv_f16};
        rp.row_positions = positions;
        GF_TRY(launch_rope_store(rp, stream_, true));
        AttentionParams ap;
        ap.q = query_; ap.ring_k = nullptr; ap.ring_v = nullptr; ap.private_k = cache.private_k; ap.private_v = cache.private_v;
        ap.out = attention_out_;
        ap.partial_out = static_cast<float*>(attention_ws_);
        ap.partial_ml = ap.partial_out + (size_t)c.row_capacity * c.heads * kMaxAttentionPartitions * 256u;
        ap.counters = attention_counters(attention_ws_, c.row_capacity, c.heads);
        ap.base_position = positions; ap.rows = rows; ap.heads = c.heads; ap.kv_heads = c.kv_heads; ap.head_dim = c.head_dim;
        ap.ring_mask = cache.ring_rows - 1u; ap.window = cache.window; ap.scale = c.attention_scale;
        ap.softcap = c.attn_softcap; ap.kv_f16 = c.kv_f16;
        GF_TRY(launch_stream_attention(ap, set.rings_dev + (size_t)l * set.count + first, positions, stream_));
        launches_ += 2;
        GemvLaunch o;
        o.k = (uint64_t)c.heads * c.head_dim;
        o.matrices[0] = GemvMatrixDesc{w.o.dtype, w.o.data, projected_, w.o.n};
        o.prologue = kProloguePlain; o.in = attention_out_;
        GF_TRY(run_gemv(o, rows));
        GemvLaunch gu;
        gu.k = c.hidden;
        gu.matrices[0] = GemvMatrixDesc{w.gate.dtype, w.gate.data, gate_, w.gate.n};
        gu.matrices[1] = GemvMatrixDesc{w.up.dtype, w.up.data, up_, w.up.n};
        gu.count = 2;
        gu.prologue = kPrologueAddNorm; gu.in = projected_; gu.residual = x; gu.gamma0 = w.post_attention_norm;
        gu.residual_out = x2; gu.gamma1 = w.ffn_norm;
        GF_TRY(run_gemv(gu, rows));
        GemvLaunch down;
        down.k = c.ffn;
        down.matrices[0] = GemvMatrixDesc{w.down.dtype, w.down.data, projected_, w.down.n};
        down.prologue = kPrologueGeglu; down.in = gate_; down.residual = up_;
        GF_TRY(run_gemv(down, rows));
    }
    GemvLaunch head;
    head.k = c.hidden;
    const PackedMatrix& table = has_head_ ? head_ : token_embd_;
    head.matrices[0] = GemvMatrixDesc{table.dtype, table.data, set.logits + (size_t)first * c.vocab, table.n};
    head.prologue = kPrologueAddNorm; head.in = projected_; head.residual = x2;
    head.gamma0 = layers_[c.layers - 1].post_ffw_norm; head.residual_out = x; head.gamma1 = output_norm_;
    GF_TRY(run_gemv(head, rows));
    GF_TRY(launch_stream_publish(set.publish_layers_dev, c.layers, set.rings_dev + first, set.count, set.positions_dev + first, rows, stream_));
    launches_ += 2;
    return GF_OK;
}

// A step's other form: every stream of the set (up to 128) in ONE pass whose projections are the prompt path's
// bf16 tensor-core GEMMs, so the weights are read and dequantised once per step however many streams there
// are.  Results differ from the exact row passes by the bf16 rounding of activations and weights (about 1e-2
// relative L2 on logits), which is why it is a mode the caller chooses.
int Model::streams_set_mode(StreamSet& set, int mode) {
    if (mode != 0 && mode != 1) return fail(GF_ERR_INVALID, "stream decode mode %d (0: exact row passes, 1: one tensor-core pass)", mode);
    if (mode == 1) {
        if (set.count > kPrefillRows) return fail(GF_ERR_INVALID, "a tensor-core step holds at most %u streams", kPrefillRows);
        const gf_model_config& c = config_;
        if ((has_head_ ? head_ : token_embd_).n % kPrefillTile) return fail(GF_ERR_INVALID, "the tensor-core head needs a vocabulary that is a multiple of %u", kPrefillTile);
        GF_TRY(ensure_prefill_arena());
        if (!set.wide_publish_layers_dev) {
            const size_t element = c.kv_f16 ? 2 : 4, kvw = (size_t)c.kv_heads * c.head_dim;
            std::vector<StreamPublishLayer> layers(c.layers);
            for (uint32_t l = 0; l < c.layers; ++l)
                layers[l] = StreamPublishLayer{static_cast<const uint8_t*>(prefill_.private_k[l]), static_cast<const uint8_t*>(prefill_.private_v[l]),
                                               caches_[l].ring_rows - 1u, (uint32_t)(kvw * element)};
            GF_TRY(stream_alloc(set, &set.wide_publish_layers_dev, layers.size()));
            GF_CUDA(cudaMemcpyAsync(set.wide_publish_layers_dev, layers.data(), layers.size() * sizeof(StreamPublishLayer), cudaMemcpyHostToDevice, stream_));
            GF_CUDA(cudaStreamSynchronize(stream_));
        }
    }
    set.mode = mode;
    return GF_OK;
}

int Model::encode_stream_batch(StreamSet& set) {
    const gf_model_config& c = config_;
    PrefillArena& a = prefill_;
    const uint32_t rows = set.count, qw = c.heads * c.head_dim;
    GF_TRY(launch_embedding(token_embd_.dtype, token_embd_.data, c.hidden, token_vocab(), a.tokens, rows, sqrtf((float)c.hidden), a.residual,
                            status_dev_, stream_, false));
    launches_ += 1;
    auto gemm = [&](std::initializer_list<std::pair<const PackedMatrix*, float*>> matrices, const void* operand, uint64_t k, uint32_t splits = 1) -> int {
        PrefillGemmLaunch launch;
        launch.count = 0;
        launch.splits = splits;
        for (const auto& entry : matrices) launch.matrices[launch.count++] = {entry.first->dtype, entry.first->data, entry.second, entry.first->n};
        launch.k = k;
        launch.a = operand;
        launch.rows = rows;
        ++launches_;
        return launch_prefill_gemm(launch, error_flag_, stream_);
    };
    uint32_t down_splits = 1;
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
        rp.row_positions = set.positions_dev;
        GF_TRY(launch_rope_store(rp, stream_, false));
        AttentionParams ap;
        ap.q = a.query; ap.ring_k = nullptr; ap.ring_v = nullptr; ap.private_k = a.private_k[l]; ap.private_v = a.private_v[l];
        ap.out = a.attention_out;
        ap.partial_out = static_cast<float*>(a.attention_ws);
        ap.partial_ml = ap.partial_out + (size_t)kPrefillRows * c.heads * kMaxAttentionPartitions * 256u;
        ap.counters = attention_counters(a.attention_ws, kPrefillRows, c.heads);
        ap.base_position = set.positions_dev; ap.rows = rows; ap.heads = c.heads; ap.kv_heads = c.kv_heads; ap.head_dim = c.head_dim;
        ap.ring_mask = cache.ring_rows - 1u; ap.window = cache.window; ap.scale = c.attention_scale;
        ap.softcap = c.attn_softcap; ap.kv_f16 = c.kv_f16;
        GF_TRY(launch_stream_attention(ap, set.rings_dev + (size_t)l * set.count, set.positions_dev, stream_));
        GF_TRY(launch_prefill_pack(a.attention_out, a.a_q, rows, qw, stream_));
        const uint32_t o_splits = prefill_gemm_splits(w.o.n, w.o.k, w.o.dtype);
        GF_TRY(gemm({{&w.o, a.projected}}, a.a_q, qw, o_splits));
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
        launches_ += 8;
    }
    // Final norm and the head: one GEMM over all rows into the set's logits.
    GF_TRY(launch_prefill_norm(a.projected, down_splits, a.residual2, layers_[c.layers - 1].post_ffw_norm, output_norm_, a.residual, a.a_hidden, rows,
                               c.hidden, c.rms_eps, 1, stream_));
    const PackedMatrix& table = has_head_ ? head_ : token_embd_;
    GF_TRY(gemm({{&table, set.logits}}, a.a_hidden, c.hidden));
    GF_TRY(launch_stream_publish(set.wide_publish_layers_dev, c.layers, set.rings_dev, set.count, set.positions_dev, rows, stream_));
    launches_ += 3;
    return GF_OK;
}

// One token per stream for every stream: groups of up to row_capacity streams share a pass over the weights.
int Model::streams_decode(StreamSet& set, const uint32_t* tokens_host) {
    if (!finalized_) return fail(GF_ERR_STATE, "plan is not finalized");
    if (poisoned_) return fail(GF_ERR_STATE, "plan is poisoned after an unknown GPU outcome; reset it");
    if (!tokens_host) return fail(GF_ERR_INVALID, "null token ids");
    for (uint32_t s = 0; s < set.count; ++s) {
        if (tokens_host[s] >= token_vocab()) return fail(GF_ERR_INVALID, "token id %u outside the vocabulary", tokens_host[s]);
        if (set.positions_host[s] >= config_.context) return fail(GF_ERR_INVALID, "stream %u has filled its context (%u)", s, config_.context);
    }
    if (set.mode == 1) {
        GF_CUDA(cudaMemcpyAsync(prefill_.tokens, tokens_host, set.count * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));      // pageable: staged by the driver
        if (!use_graph_) {
            GF_TRY(encode_stream_batch(set));
        } else {
            if (!set.wide_graph) {
                const uint32_t before = launches_;
                cudaGraph_t graph = nullptr;
                GF_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
                const int status = encode_stream_batch(set);
                const cudaError_t end = cudaStreamEndCapture(stream_, &graph);
                set.wide_launches = launches_ - before;
                launches_ = before;
                if (status != GF_OK) { if (graph) cudaGraphDestroy(graph); return status; }
                GF_CUDA(end);
                const cudaError_t inst = cudaGraphInstantiate(&set.wide_graph, graph, 0);
                cudaGraphDestroy(graph);
                GF_CUDA(inst);
            }
            GF_CUDA(cudaGraphLaunch(set.wide_graph, stream_));
            launches_ += set.wide_launches;
        }
        for (uint32_t s = 0; s < set.count; ++s) ++set.positions_host[s];
        return GF_OK;
    }
    for (uint32_t first = 0; first < set.count; first += config_.row_capacity) {
        const uint32_t rows = std::min(config_.row_capacity, set.count - first);
        GF_CUDA(cudaEventSynchronize(tokens_copied_));
        std::memcpy(tokens_pinned_, tokens_host + first, rows * sizeof(uint32_t));
        GF_CUDA(cudaMemcpyAsync(tokens_dev_, tokens_pinned_, rows * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
        GF_CUDA(cudaEventRecord(tokens_copied_, stream_));
        const uint32_t group = first / config_.row_capacity;
        if (!use_graph_) {
            GF_TRY(encode_stream_group(set, first, rows));
        } else {
            // The group's pass is recorded once and replayed: every pointer it uses is fixed, and positions
            // and token ids are read from device memory.
            if (set.group_graphs.size() <= group) { set.group_graphs.resize(group + 1u, nullptr); set.group_launches.resize(group + 1u, 0u); }
            cudaGraphExec_t& exec = set.group_graphs[group];
            if (!exec) {
                const uint32_t before = launches_;
                cudaGraph_t graph = nullptr;
                GF_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
                const int status = encode_stream_group(set, first, rows);
                const cudaError_t end = cudaStreamEndCapture(stream_, &graph);
                set.group_launches[group] = launches_ - before;
                launches_ = before;
                if (status != GF_OK) { if (graph) cudaGraphDestroy(graph); return status; }
                GF_CUDA(end);
                const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
                cudaGraphDestroy(graph);
                GF_CUDA(inst);
            }
            GF_CUDA(cudaGraphLaunch(exec, stream_));
            launches_ += set.group_launches[group];
        }
        for (uint32_t r = 0; r < rows; ++r) ++set.positions_host[first + r];
    }
    return GF_OK;
}

int Model::streams_select(StreamSet& set, const void* requests_host) {
    if (!requests_host) return fail(GF_ERR_INVALID, "null selection requests");
    const size_t bytes = (size_t)set.count * gf_selection_request_bytes();
    GF_CUDA(cudaStreamSynchronize(stream_));           // the previous upload may still be reading the pinned rows
    std::memcpy(set.requests_pinned, requests_host, bytes);
    GF_CUDA(cudaMemcpyAsync(set.requests_dev, set.requests_pinned, bytes, cudaMemcpyHostToDevice, stream_));
    launches_ += 2;
    return launch_candidates(set.logits, set.count, config_.vocab, config_.final_softcap, set.requests_dev, set.candidates_ws, set.results_dev, stream_, false);
}

int Model::streams_read_candidates(StreamSet& set, void* results_host) {
    if (!results_host) return fail(GF_ERR_INVALID, "null candidate buffer");
    GF_CUDA(cudaMemcpyAsync(results_host, set.results_dev, (size_t)set.count * gf_candidate_result_bytes(), cudaMemcpyDeviceToHost, stream_));
    return synchronize();
}

int Model::streams_read_logits(StreamSet& set, uint32_t stream, float* host) {
    if (!host || stream >= set.count) return fail(GF_ERR_INVALID, "bad logits readback");
    GF_CUDA(cudaMemcpyAsync(host, set.logits + (size_t)stream * config_.vocab, (size_t)config_.vocab * 4, cudaMemcpyDeviceToHost, stream_));
    return synchronize();
}

size_t Model::streams_kv_bytes(const StreamSet& set) const {
    // K and V bytes one decode step reads: every stream's committed rows inside every layer's window.
    const size_t element = config_.kv_f16 ? 2 : 4, row = (size_t)config_.kv_heads * config_.head_dim * element * 2u;
    size_t total = 0;
    for (uint32_t s = 0; s < set.count; ++s)
        for (uint32_t l = 0; l < config_.layers; ++l) {
            const uint32_t window = caches_[l].window, p = set.positions_host[s];
            total += (size_t)(window ? std::min(window, p) : p) * row;
        }
    return total;
}

}  // namespace gf

using namespace gf;

struct gf_streams {
    gf_model* model;
    StreamSet* set;
};

extern "C" {

int gf_streams_create(gf_model* model, uint32_t count, gf_streams** out_streams) {
    if (!model || !out_streams) return fail(GF_ERR_INVALID, "gf_streams_create: null argument");
    StreamSet* set = nullptr;
    const int status = model->impl.streams_create(count, &set);
    if (status != GF_OK) return status;
    *out_streams = new gf_streams{model, set};
    return GF_OK;
}
int gf_streams_destroy(gf_streams* s) {
    // The plan may already be gone (handles are destroyed in any order): wait for the device, not for its stream.
    if (s) { cudaDeviceSynchronize(); delete s->set; delete s; }
    return GF_OK;
}
int gf_streams_prefill(gf_streams* s, uint32_t stream, const uint32_t* tokens_host, uint32_t count) {
    return s ? s->model->impl.streams_prefill(*s->set, stream, tokens_host, count) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_decode(gf_streams* s, const uint32_t* tokens_host) {
    return s ? s->model->impl.streams_decode(*s->set, tokens_host) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_set_mode(gf_streams* s, int mode) {
    return s ? s->model->impl.streams_set_mode(*s->set, mode) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_select(gf_streams* s, const void* requests_host) {
    return s ? s->model->impl.streams_select(*s->set, requests_host) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_read_candidates(gf_streams* s, void* results_host) {
    return s ? s->model->impl.streams_read_candidates(*s->set, results_host) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_read_logits(gf_streams* s, uint32_t stream, float* logits_host) {
    return s ? s->model->impl.streams_read_logits(*s->set, stream, logits_host) : fail(GF_ERR_INVALID, "null streams");
}
int gf_streams_position(const gf_streams* s, uint32_t stream, uint32_t* out_position) {
    if (!s || !out_position || stream >= s->set->count) return fail(GF_ERR_INVALID, "bad stream");
    *out_position = s->set->positions_host[stream];
    return GF_OK;
}
uint32_t gf_streams_count(const gf_streams* s) { return s ? s->set->count : 0u; }
size_t gf_streams_kv_bytes_per_step(const gf_streams* s) { return s ? s->model->impl.streams_kv_bytes(*s->set) : 0u; }

}  // extern "C"
