// Embedding gather, RMSNorm (+residual), per-head norm + NEOX RoPE + private KV store, GeGLU,
// split-KV grouped-query attention over ring + private rows, and KV publication.
#include "ops.cuh"
#include "attention.cuh"

#include <algorithm>
#include "embedding.cuh"

#include <cmath>

namespace gf {

// ------------------------------------------------------------------ embedding (device code in embedding.cuh)

__global__ void __launch_bounds__(256) embedding_kernel(int dtype, const uint8_t* __restrict__ packed, uint32_t k,
                                                        uint32_t vocab, const uint32_t* __restrict__ tokens,
                                                        uint32_t rows, float scale, float* __restrict__ out,
                                                        uint32_t* status) {
    pdl_wait();
    pdl_launch_dependents();
    embedding_rows(dtype, packed, k, vocab, tokens, rows, scale, out, status, blockIdx.x * blockDim.x + threadIdx.x,
                   gridDim.x * blockDim.x);
}

// ------------------------------------------------------------------ RMSNorm (+ residual)

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < warps; ++w) total += scratch[w];   // same order in every thread
    __syncthreads();
    return total;
}

// out = x * rsqrt(mean(x^2) + eps) * gamma [+ residual]   (ops/normalization.cpp:70-101,
// metal_kernels.mm:2019-2158).  One block per row.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                       const float* __restrict__ residual, float* __restrict__ out,
                                                       uint32_t hidden, float eps) {
    __shared__ float scratch[8];
    pdl_wait();
    pdl_launch_dependents();
    const float* xr = x + (size_t)blockIdx.x * hidden;
    float sum = 0.0f;
    for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x) sum = fmaf(xr[c], xr[c], sum);
    const float total = block_sum(sum, scratch);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)hidden), eps)));
    for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = __fmul_rn(__fmul_rn(xr[c], inv), gamma[c]);
        if (residual) v = __fadd_rn(residual[(size_t)blockIdx.x * hidden + c], v);
        out[(size_t)blockIdx.x * hidden + c] = v;
    }
}

// ------------------------------------------------------------------ QK norm + RoPE + private KV store

// One block per (head, row); thread i owns the NEOX pair (i, i + head_dim/2).
// Query heads: optional per-head RMSNorm, rotate, write f32.  KV heads: K is normalised,
// rotated and rounded to the cache type, V is rounded and stored; non-finite F16 sets status
// bit 8 (metal_kernels.mm:1915-1930, 2406-2517; angle as ops/rope.cpp:109-117 in double).
__global__ void __launch_bounds__(256) rope_store_kernel(RopeStoreParams p) {
    __shared__ float scratch[8];
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t head = blockIdx.x, row = blockIdx.y, half = p.head_dim / 2u, i = threadIdx.x;
    const bool is_query = head < p.heads;
    const uint32_t kvh = head - p.heads;
    const float* src = is_query ? p.raw_q + ((size_t)row * p.heads + head) * p.head_dim
                                : p.raw_k + ((size_t)row * p.kv_heads + kvh) * p.head_dim;
    const float* gamma = is_query ? p.q_norm : p.k_norm;
    float first = src[i], second = src[i + half];
    if (gamma) {
        const float total = block_sum(fmaf(first, first, second * second), scratch);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)p.head_dim), p.eps)));
        first = __fmul_rn(__fmul_rn(first, inv), gamma[i]);
        second = __fmul_rn(__fmul_rn(second, inv), gamma[i + half]);
    }
    const uint32_t position = p.row_positions ? p.row_positions[row] : *p.base_position + row;
    // Angle in double as the reference forms it (ops/rope.cpp:109-117); the divisor
    // freq_base^(2i/d) comes from a table when the caller has one.  The angle is reduced to
    // [-pi, pi] in double (two-term 2*pi), after which single-precision sine and cosine are
    // within an ulp of the double ones rounded to f32.
    const double divisor = p.divisors ? p.divisors[i] : pow((double)p.freq_base, (double)(2u * i) / (double)p.head_dim);
    const double angle = (double)position * (double)p.freq_scale / divisor;
    const double turns = rint(angle * 0.15915494309189535);
    const double reduced = fma(-turns, 2.4492935982947064e-16, fma(-turns, 6.283185307179586, angle));
    float s, c;
    sincosf((float)reduced, &s, &c);
    const float r0 = p.rotate ? __fsub_rn(__fmul_rn(first, c), __fmul_rn(second, s)) : first;      // unrotated values keep their bits (-0 too)
    const float r1 = p.rotate ? __fadd_rn(__fmul_rn(first, s), __fmul_rn(second, c)) : second;
    if (is_query) {
        float* dst = p.q_out + ((size_t)row * p.heads + head) * p.head_dim;
        dst[i] = r0;
        dst[i + half] = r1;
        return;
    }
    const size_t o = ((size_t)row * p.kv_heads + kvh) * p.head_dim;
    const float* vsrc = p.raw_v + o;
    const float v0 = vsrc[i], v1 = vsrc[i + half];
    if (p.kv_f16) {
        __half* kd = static_cast<__half*>(p.private_k) + o;
        __half* vd = static_cast<__half*>(p.private_v) + o;
        const __half k0 = __float2half_rn(r0), k1 = __float2half_rn(r1), h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
        kd[i] = k0; kd[i + half] = k1; vd[i] = h0; vd[i + half] = h1;
        if (!isfinite(__half2float(k0)) || !isfinite(__half2float(k1)) || !isfinite(__half2float(h0)) || !isfinite(__half2float(h1)))
            if (p.status) atomicOr(p.status, kStatusKvNonFinite);
    } else {
        float* kd = static_cast<float*>(p.private_k) + o;
        float* vd = static_cast<float*>(p.private_v) + o;
        kd[i] = r0; kd[i + half] = r1; vd[i] = v0; vd[i + half] = v1;
    }
}

// ------------------------------------------------------------------ attention (bodies in attention.cuh)

// Online-softmax GQA, head_dim 256: grid (kv_head, partition, row group), kAttentionWarps warps per block.
template <typename KV, int G, int R>
__global__ void __launch_bounds__(kAttentionWarps * 32) attention_kernel(AttentionParams p) {
    __shared__ AttentionSmem<kAttentionWarps, G * R> sm;
    bool waited = false;
    attention_body<KV, G, R, true>(p, blockIdx.x, blockIdx.y, blockIdx.z, sm, LaunchBlock(), waited);
}

// The same for a binary16 cache, both contractions on the tensor cores.
template <int G, int R>
__global__ void __launch_bounds__(kAttentionMmaWarps * 32) attention_mma_kernel(AttentionParams p) {
    __shared__ AttentionMmaSmem<kAttentionMmaWarps, G * R> sm;
    bool waited = false;
    attention_mma_body<G, R, 1, true, true>(p, blockIdx.x, blockIdx.y, blockIdx.z, sm, LaunchBlock(), waited);
}

// One query row per conversation stream: block (kv head, partition, stream) runs the single-row body with
// the stream's rings and position substituted, and its own slice of the private rows and the workspace.
template <typename KV, int G>
__device__ __forceinline__ AttentionParams stream_view(AttentionParams p, const StreamRings* rings, const uint32_t* positions, uint32_t s) {
    const size_t qw = (size_t)p.heads * 256u, kvw = (size_t)p.kv_heads * 256u;
    p.q += s * qw;
    p.out += s * qw;
    p.ring_k = rings[s].ring_k;
    p.ring_v = rings[s].ring_v;
    p.private_k = static_cast<const KV*>(p.private_k) + s * kvw;
    p.private_v = static_cast<const KV*>(p.private_v) + s * kvw;
    p.partial_out += (size_t)s * p.heads * kMaxAttentionPartitions * 256u;
    p.partial_ml += (size_t)s * p.heads * kMaxAttentionPartitions * 2u;
    p.counters += s * p.heads;
    p.base_position = positions + s;
    p.rows = 1u;
    return p;
}

template <int G>
__global__ void __launch_bounds__(kAttentionMmaWarps * 32) stream_attention_mma_kernel(AttentionParams p, const StreamRings* rings,
                                                                                       const uint32_t* positions) {
    __shared__ AttentionMmaSmem<kAttentionMmaWarps, G> sm;
    bool waited = false;
    const AttentionParams view = stream_view<__half, G>(p, rings, positions, blockIdx.z);
    attention_mma_body<G, 1, 1, true, true>(view, blockIdx.x, blockIdx.y, 0u, sm, LaunchBlock(), waited);
}

template <int G>
__global__ void __launch_bounds__(kAttentionWarps * 32) stream_attention_kernel(AttentionParams p, const StreamRings* rings,
                                                                               const uint32_t* positions) {
    __shared__ AttentionSmem<kAttentionWarps, G> sm;
    bool waited = false;
    const AttentionParams view = stream_view<float, G>(p, rings, positions, blockIdx.z);
    attention_body<float, G, 1, true>(view, blockIdx.x, blockIdx.y, 0u, sm, LaunchBlock(), waited);
}

__global__ void __launch_bounds__(128) stream_publish_kernel(const StreamPublishLayer* __restrict__ layers, const StreamRings* __restrict__ rings,
                                                             uint32_t stride, const uint32_t* __restrict__ positions) {
    const uint32_t row = blockIdx.x, layer = blockIdx.y;
    const StreamPublishLayer L = layers[layer];
    const StreamRings R = rings[(size_t)layer * stride + row];
    const size_t dst = (size_t)(positions[row] & L.ring_mask) * L.row_bytes, src = (size_t)row * L.row_bytes;
    uint8_t* ring_k = static_cast<uint8_t*>(const_cast<void*>(R.ring_k));
    uint8_t* ring_v = static_cast<uint8_t*>(const_cast<void*>(R.ring_v));
    for (uint32_t b = threadIdx.x * 16u; b < L.row_bytes; b += blockDim.x * 16u) {
        *reinterpret_cast<uint4*>(ring_k + dst + b) = *reinterpret_cast<const uint4*>(L.private_k + src + b);
        *reinterpret_cast<uint4*>(ring_v + dst + b) = *reinterpret_cast<const uint4*>(L.private_v + src + b);
    }
}

__global__ void advance_positions_kernel(uint32_t* positions, uint32_t rows) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) positions[i] += 1u;
}

// ------------------------------------------------------------------ GeGLU, KV publication

// gelu_tanh(gate) * up   (ops/elementwise.cpp:79-94, metal_kernels.mm:1827-1843)
__global__ void __launch_bounds__(256) geglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                    float* __restrict__ out, uint64_t count) {
    pdl_wait();
    pdl_launch_dependents();
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = gate[i];
        const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
        out[i] = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner))), up[i]);
    }
}

// Publishes private rows 0..rows-1 into ring slots (base + r) & mask   (metal_kernels.mm:2519-2557).
__global__ void __launch_bounds__(256) kv_scatter_kernel(const uint8_t* __restrict__ private_k, const uint8_t* __restrict__ private_v,
                                                         uint8_t* __restrict__ ring_k, uint8_t* __restrict__ ring_v,
                                                         const uint32_t* base_position, uint32_t row_bytes, uint32_t ring_mask) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t row = blockIdx.x;
    const size_t dst = (size_t)((*base_position + row) & ring_mask) * row_bytes, src = (size_t)row * row_bytes;
    for (uint32_t b = threadIdx.x * 16u; b < row_bytes; b += blockDim.x * 16u) {
        *reinterpret_cast<uint4*>(ring_k + dst + b) = *reinterpret_cast<const uint4*>(private_k + src + b);
        *reinterpret_cast<uint4*>(ring_v + dst + b) = *reinterpret_cast<const uint4*>(private_v + src + b);
    }
}

// All layers at once: block (row, layer) copies that layer's private row into its ring; the last
// block advances the committed position after every copy of the launch has been issued (the
// position is only read by later launches).
__global__ void __launch_bounds__(128) kv_publish_kernel(const KvPublishLayer* __restrict__ layers, uint32_t* base_position,
                                                         uint32_t rows) {
    pdl_wait();
    const uint32_t row = blockIdx.x, layer = blockIdx.y;
    const KvPublishLayer L = layers[layer];
    const uint32_t base = *base_position;
    const size_t dst = (size_t)((base + row) & L.ring_mask) * L.row_bytes, src = (size_t)row * L.row_bytes;
    for (uint32_t b = threadIdx.x * 16u; b < L.row_bytes; b += blockDim.x * 16u) {
        *reinterpret_cast<uint4*>(L.ring_k + dst + b) = *reinterpret_cast<const uint4*>(L.private_k + src + b);
        *reinterpret_cast<uint4*>(L.ring_v + dst + b) = *reinterpret_cast<const uint4*>(L.private_v + src + b);
    }
}

__global__ void advance_position_kernel(uint32_t* state, uint32_t delta) {
    pdl_wait();
    if (threadIdx.x == 0) state[0] += delta;
}

int launch_kv_publish(const KvPublishLayer* layers_dev, uint32_t layer_count, uint32_t* base_position, uint32_t rows,
                      cudaStream_t stream) {
    const int status = launch_kernel(kv_publish_kernel, dim3(rows, layer_count), dim3(128), 0, stream, false, layers_dev,
                                     base_position, rows);
    if (status != GF_OK) return status;
    return launch_kernel(advance_position_kernel, dim3(1), dim3(32), 0, stream, false, base_position, rows);
}

__global__ void __launch_bounds__(256) add_kernel(const float* __restrict__ left, const float* __restrict__ right, float* __restrict__ out, uint64_t count) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = __fadd_rn(left[i], right[i]);
}

// Tensor-parallel shards: the pass counter behind the exchange stamps (gemv.cuh, WeightStreamParams::Scatter).
__global__ void shard_tick_kernel(uint32_t* tick) { *tick += 1u; }

// Waits (bounded, like the consuming launches' own polls) until every value of the peers' parts of the pass's last
// projection carries its stamp; nothing is read out.
__global__ void __launch_bounds__(256) shard_drain_kernel(const ShardDrain d) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t stamp = (__ldcg(d.tick) << 8) | d.site;
    for (uint32_t s = 0; s < d.count; ++s)
        for (uint32_t i = threadIdx.x; i < d.values; i += blockDim.x) {
            const volatile uint32_t* word = reinterpret_cast<const volatile uint32_t*>(d.parts[s] + i) + 1;
            for (uint32_t polls = 0; *word != stamp; ++polls) {
                if (polls > d.wait_limit || ((polls & 255u) == 255u && *reinterpret_cast<volatile int*>(d.error_flag) != 0)) { atomicExch(d.error_flag, 1); break; }
                if (polls > 32u) __nanosleep(100);
            }
        }
}

__global__ void __launch_bounds__(256) shard_bulk_exchange_kernel(const ShardBulk p) {
    const uint32_t stamp = (__ldcg(p.tick) << 8) | p.site;
    const uint32_t quads = p.values / 4u, stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    float4* own = reinterpret_cast<float4*>(p.x);
    // Every thread first sends all of its values, then waits for the peers' copies of the same values: no thread
    // waits for another thread of its own GPU, and every peer sends before it waits.
    for (uint32_t q = first; q < quads; q += stride) {
        float4 v = own[q];
        for (uint32_t s = 1; s < p.splits; ++s) {
            const float4 w = reinterpret_cast<const float4*>(p.x + (size_t)s * p.slab)[q];
            v.x = __fadd_rn(v.x, w.x); v.y = __fadd_rn(v.y, w.y); v.z = __fadd_rn(v.z, w.z); v.w = __fadd_rn(v.w, w.w);
        }
        own[q] = v;
        for (uint32_t g = 0; g < p.peers; ++g) {
            uint2* dst = p.out[g] + (size_t)q * 4u;      // 8-byte stores arrive whole
            dst[0] = make_uint2(__float_as_uint(v.x), stamp); dst[1] = make_uint2(__float_as_uint(v.y), stamp);
            dst[2] = make_uint2(__float_as_uint(v.z), stamp); dst[3] = make_uint2(__float_as_uint(v.w), stamp);
        }
    }
    for (uint32_t q = first; q < quads; q += stride) {
        const float4 mine = own[q];
        float4 total = mine;
        for (uint32_t s = 0; s < p.shards; ++s) {
            float4 w = mine;
            if (s != p.self) {
                const uint4* src = reinterpret_cast<const uint4*>(p.parts[s] + (size_t)q * 4u);
                uint4 a, b;
                for (uint32_t polls = 0;; ++polls) {
                    a = load_volatile16(src);
                    b = load_volatile16(src + 1);
                    if (a.y == stamp && a.w == stamp && b.y == stamp && b.w == stamp) break;
                    if (polls > p.wait_limit || ((polls & 255u) == 255u && *reinterpret_cast<volatile int*>(p.error_flag) != 0)) { atomicExch(p.error_flag, 1); break; }
                    if (polls > 32u) __nanosleep(100);
                }
                w = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
            }
            if (s == 0u) total = w;
            else { total.x = __fadd_rn(total.x, w.x); total.y = __fadd_rn(total.y, w.y); total.z = __fadd_rn(total.z, w.z); total.w = __fadd_rn(total.w, w.w); }
        }
        own[q] = total;
    }
}

__global__ void __launch_bounds__(256) shard_gather_kernel(const ShardGather p) {
    const uint32_t stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    for (uint32_t i = first; i < p.words; i += stride) {          // send everything first, then wait
        const uint32_t word = p.local[i];
        p.gathered[(size_t)p.self * p.words + i] = word;
        for (uint32_t g = 0; g < p.peers; ++g) p.out[g][i] = make_uint2(word, p.stamp);
    }
    for (uint32_t i = first; i < p.words; i += stride)
        for (uint32_t s = 0; s < p.shards; ++s) {
            if (s == p.self) continue;
            const volatile unsigned long long* src = reinterpret_cast<const volatile unsigned long long*>(p.parts[s] + i);
            unsigned long long pair = 0;
            for (uint32_t polls = 0;; ++polls) {
                pair = *src;                                       // one 8-byte load: value and stamp together
                if ((uint32_t)(pair >> 32) == p.stamp) break;
                if (polls > p.wait_limit || ((polls & 255u) == 255u && *reinterpret_cast<volatile int*>(p.error_flag) != 0)) { atomicExch(p.error_flag, 1); break; }
                if (polls > 32u) __nanosleep(100);
            }
            p.gathered[(size_t)s * p.words + i] = (uint32_t)pair;
        }
}

// ------------------------------------------------------------------ launchers

int launch_shard_gather(const ShardGather& gather, cudaStream_t stream) {
    if (!gather.local || !gather.gathered || gather.words == 0 || gather.shards == 0 || gather.shards > 8u || !gather.error_flag)
        return fail(GF_ERR_INVALID, "shard gather: bad arguments");
    const uint32_t blocks = std::min<uint32_t>((gather.words + 255u) / 256u, (uint32_t)sm_count());
    return launch_kernel(shard_gather_kernel, dim3(blocks), dim3(256), 0, stream, false, gather);
}
int launch_shard_bulk_exchange(const ShardBulk& bulk, cudaStream_t stream) {
    if (!bulk.x || bulk.splits == 0 || bulk.values == 0 || (bulk.values & 3u) || bulk.shards == 0 || bulk.shards > 8u || !bulk.tick || !bulk.error_flag)
        return fail(GF_ERR_INVALID, "shard bulk exchange: bad arguments");
    const uint32_t blocks = std::min<uint32_t>((bulk.values / 4u + 255u) / 256u, 2u * (uint32_t)sm_count());
    return launch_kernel(shard_bulk_exchange_kernel, dim3(blocks), dim3(256), 0, stream, false, bulk);
}
int launch_shard_tick(uint32_t* tick, cudaStream_t stream) {
    return launch_kernel(shard_tick_kernel, dim3(1), dim3(1), 0, stream, false, tick);
}
int launch_shard_drain(const ShardDrain& drain, cudaStream_t stream, bool pdl) {
    return launch_kernel(shard_drain_kernel, dim3(1), dim3(256), 0, stream, pdl, drain);
}

int launch_embedding(int dtype, const void* packed, uint32_t k, uint32_t vocab, const uint32_t* tokens, uint32_t rows,
                     float scale, float* out, uint32_t* status, cudaStream_t stream, bool pdl) {
    const uint32_t blocks = (rows * k + 255u) / 256u;
    return launch_kernel(embedding_kernel, dim3(blocks), dim3(256), 0, stream, pdl, dtype,
                         static_cast<const uint8_t*>(packed), k, vocab, tokens, rows, scale, out, status);
}

int launch_rms_norm(const float* x, const float* gamma, const float* residual, float* out, uint32_t rows,
                    uint32_t hidden, float eps, cudaStream_t stream, bool pdl) {
    return launch_kernel(rms_norm_kernel, dim3(rows), dim3(256), 0, stream, pdl, x, gamma, residual, out, hidden, eps);
}

int launch_rope_store(const RopeStoreParams& p, cudaStream_t stream, bool pdl) {
    if (p.head_dim < 64u || p.head_dim > 512u || (p.head_dim & 63u))
        return fail(GF_ERR_INVALID, "rope/store: head_dim=%u unsupported", p.head_dim);
    return launch_kernel(rope_store_kernel, dim3(p.heads + p.kv_heads, p.rows), dim3(p.head_dim / 2u), 0, stream, pdl, p);
}

static uint32_t attention_target_parts(const AttentionParams& p, uint32_t groups, uint32_t blocks_per_sm) {
    // About one wave of blocks: (kv head, row group) pairs times partitions.
    const uint32_t per_pair = (uint32_t)sm_count() * blocks_per_sm / (p.kv_heads * groups);
    return per_pair < 1u ? 1u : per_pair > (uint32_t)kMaxAttentionPartitions ? (uint32_t)kMaxAttentionPartitions : per_pair;
}

template <typename KV, int G, int R>
static int launch_attention_instance(const AttentionParams& params, cudaStream_t stream, bool pdl) {
    AttentionParams p = params;
    const uint32_t groups = (p.rows + R - 1u) / R;
    p.target_parts = attention_target_parts(p, groups, kAttentionBlocksPerSm);
    return launch_kernel(attention_kernel<KV, G, R>, dim3(p.kv_heads, p.target_parts, groups), dim3(kAttentionWarps * 32), 0,
                         stream, pdl, p);
}

template <int G, int R>
static int launch_attention_mma_instance(const AttentionParams& params, cudaStream_t stream, bool pdl) {
    AttentionParams p = params;
    const uint32_t groups = (p.rows + R - 1u) / R;
    p.target_parts = attention_target_parts(p, groups, 1u);
    return launch_kernel(attention_mma_kernel<G, R>, dim3(p.kv_heads, p.target_parts, groups), dim3(kAttentionMmaWarps * 32), 0,
                         stream, pdl, p);
}

// F32 cache.  Two query vectors per block where the head ratio allows it: measured on the 12B
// verify pass, four (both rows of a pair of heads in one block) halve the blocks but double each
// warp's serial work and came out 1 % slower per cycle.
static int launch_attention_f32(const AttentionParams& p, cudaStream_t stream, bool pdl) {
    const uint32_t group = p.heads / p.kv_heads;
    if (group == 1u) {
        if (p.rows >= 2u) return launch_attention_instance<float, 1, 2>(p, stream, pdl);
        return launch_attention_instance<float, 1, 1>(p, stream, pdl);
    }
    if (group == 2u) return launch_attention_instance<float, 2, 1>(p, stream, pdl);
    if (group == 4u) return launch_attention_instance<float, 4, 1>(p, stream, pdl);
    return fail(GF_ERR_INVALID, "attention: query/KV head ratio %u unsupported (1, 2, 4)", group);
}

// Binary16 cache: the tensor-core kernel, with as many rows per block as four query vectors allow.
static int launch_attention_f16(const AttentionParams& p, cudaStream_t stream, bool pdl) {
    const uint32_t group = p.heads / p.kv_heads;
    if (group == 1u) {
        if (p.rows >= 3u) return launch_attention_mma_instance<1, 4>(p, stream, pdl);
        if (p.rows == 2u) return launch_attention_mma_instance<1, 2>(p, stream, pdl);
        return launch_attention_mma_instance<1, 1>(p, stream, pdl);
    }
    if (group == 2u) {
        if (p.rows >= 2u) return launch_attention_mma_instance<2, 2>(p, stream, pdl);
        return launch_attention_mma_instance<2, 1>(p, stream, pdl);
    }
    if (group == 4u) return launch_attention_mma_instance<4, 1>(p, stream, pdl);
    return fail(GF_ERR_INVALID, "attention: query/KV head ratio %u unsupported (1, 2, 4)", group);
}

int launch_stream_attention(const AttentionParams& params, const StreamRings* rings_dev, const uint32_t* positions_dev, cudaStream_t stream) {
    AttentionParams p = params;
    if (p.head_dim != 256u || p.kv_heads == 0 || p.heads % p.kv_heads || p.rows == 0 || !rings_dev || !positions_dev)
        return fail(GF_ERR_INVALID, "stream attention: bad geometry");
    const uint32_t group = p.heads / p.kv_heads, streams = p.rows;
    // About one wave of blocks over (kv head, stream) pairs and partitions (measured at eight streams of 8192 rows:
    // 9.45 ms per step against 9.71 for two waves and 10.45 for eight; every partition costs a merge).
    const uint32_t per_pair = (uint32_t)sm_count() / (p.kv_heads * streams);
    p.target_parts = std::min<uint32_t>(std::max<uint32_t>(per_pair, 1u), (uint32_t)kMaxAttentionPartitions);
    p.defer_merge = 0u;
    const dim3 grid(p.kv_heads, p.target_parts, streams);
    if (p.kv_f16) {
        if (group == 1u) return launch_kernel(stream_attention_mma_kernel<1>, grid, dim3(kAttentionMmaWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
        if (group == 2u) return launch_kernel(stream_attention_mma_kernel<2>, grid, dim3(kAttentionMmaWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
        if (group == 4u) return launch_kernel(stream_attention_mma_kernel<4>, grid, dim3(kAttentionMmaWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
    } else {
        if (group == 1u) return launch_kernel(stream_attention_kernel<1>, grid, dim3(kAttentionWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
        if (group == 2u) return launch_kernel(stream_attention_kernel<2>, grid, dim3(kAttentionWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
        if (group == 4u) return launch_kernel(stream_attention_kernel<4>, grid, dim3(kAttentionWarps * 32), 0, stream, false, p, rings_dev, positions_dev);
    }
    return fail(GF_ERR_INVALID, "stream attention: query/KV head ratio %u unsupported (1, 2, 4)", group);
}

int launch_stream_publish(const StreamPublishLayer* layers_dev, uint32_t layer_count, const StreamRings* rings_dev, uint32_t stride,
                          uint32_t* positions_dev, uint32_t rows, cudaStream_t stream) {
    if (!layers_dev || !rings_dev || !positions_dev || rows == 0) return fail(GF_ERR_INVALID, "stream publish: bad arguments");
    const int status = launch_kernel(stream_publish_kernel, dim3(rows, layer_count), dim3(128), 0, stream, false, layers_dev, rings_dev,
                                     stride, (const uint32_t*)positions_dev);
    if (status != GF_OK) return status;
    return launch_kernel(advance_positions_kernel, dim3((rows + 127u) / 128u), dim3(128), 0, stream, false, positions_dev, rows);
}

int launch_attention(const AttentionParams& p, cudaStream_t stream, bool pdl) {
    if (p.head_dim != 256u) return fail(GF_ERR_INVALID, "attention: head_dim must be 256 (got %u)", p.head_dim);
    if (p.heads % p.kv_heads) return fail(GF_ERR_INVALID, "attention: heads %u not a multiple of kv heads %u", p.heads, p.kv_heads);
    return p.kv_f16 ? launch_attention_f16(p, stream, pdl) : launch_attention_f32(p, stream, pdl);
}

int launch_geglu(const float* gate, const float* up, float* out, uint64_t count, cudaStream_t stream, bool pdl) {
    const uint32_t blocks = (uint32_t)((count + 255u) / 256u);
    return launch_kernel(geglu_kernel, dim3(blocks), dim3(256), 0, stream, pdl, gate, up, out, count);
}

int launch_kv_scatter(const void* private_k, const void* private_v, void* ring_k, void* ring_v,
                      const uint32_t* base_position, uint32_t rows, uint32_t row_width, uint32_t ring_mask, int kv_f16,
                      cudaStream_t stream, bool pdl) {
    const uint32_t row_bytes = row_width * (kv_f16 ? 2u : 4u);
    return launch_kernel(kv_scatter_kernel, dim3(rows), dim3(128), 0, stream, pdl,
                         static_cast<const uint8_t*>(private_k), static_cast<const uint8_t*>(private_v),
                         static_cast<uint8_t*>(ring_k), static_cast<uint8_t*>(ring_v), base_position, row_bytes, ring_mask);
}

}  // namespace gf

using namespace gf;

// ------------------------------------------------------------------ C entry points (operator level)

extern "C" {

int gf_add(const float* left_dev, const float* right_dev, float* out_dev, uint64_t count, void* stream) {
    if (!left_dev || !right_dev || !out_dev) return fail(GF_ERR_INVALID, "gf_add: null buffer");
    if (count == 0) return GF_OK;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((count + 255u) / 256u, 4096u);
    return launch_kernel(add_kernel, dim3(blocks), dim3(256), 0, as_stream(stream), false, left_dev, right_dev, out_dev, count);
}

int gf_embedding(int dtype, const void* packed_dev, uint32_t k, uint32_t vocab, const uint32_t* tokens_dev,
                 uint32_t rows, float scale, float* out_dev, uint32_t* status_dev, void* stream) {
    if (!packed_dev || !tokens_dev || !out_dev || !status_dev || rows == 0 || k % unit_elements(dtype))
        return fail(GF_ERR_INVALID, "gf_embedding: bad arguments");
    return launch_embedding(dtype, packed_dev, k, vocab, tokens_dev, rows, scale, out_dev, status_dev, as_stream(stream), false);
}

int gf_rms_norm(const float* x_dev, const float* gamma_dev, float* out_dev, uint32_t rows, uint32_t hidden, float eps,
                void* stream) {
    if (!x_dev || !gamma_dev || !out_dev || rows == 0 || hidden == 0 || !(eps > 0.0f))
        return fail(GF_ERR_INVALID, "gf_rms_norm: bad arguments (epsilon must be positive)");
    return launch_rms_norm(x_dev, gamma_dev, nullptr, out_dev, rows, hidden, eps, as_stream(stream), false);
}

int gf_rms_norm_add(const float* x_dev, const float* gamma_dev, const float* residual_dev, float* out_dev, uint32_t rows,
                    uint32_t hidden, float eps, void* stream) {
    if (!x_dev || !gamma_dev || !residual_dev || !out_dev || rows == 0 || hidden == 0 || !(eps > 0.0f))
        return fail(GF_ERR_INVALID, "gf_rms_norm_add: bad arguments");
    return launch_rms_norm(x_dev, gamma_dev, residual_dev, out_dev, rows, hidden, eps, as_stream(stream), false);
}

int gf_qk_norm_rope_store(const float* raw_q_dev, const float* raw_k_dev, const float* raw_v_dev,
                          const float* q_norm_dev, const float* k_norm_dev, float* q_out_dev, void* private_k_dev,
                          void* private_v_dev, const uint32_t* base_position_dev, uint32_t* status_dev, uint32_t rows,
                          uint32_t heads, uint32_t kv_heads, uint32_t head_dim, float eps, float freq_base,
                          float freq_scale, int kv_f16, void* stream) {
    if (!raw_q_dev || !raw_k_dev || !raw_v_dev || !q_out_dev || !private_k_dev || !private_v_dev || !base_position_dev
        || !status_dev || rows == 0 || !(freq_base > 0.0f))
        return fail(GF_ERR_INVALID, "gf_qk_norm_rope_store: bad arguments");
    RopeStoreParams p{raw_q_dev, raw_k_dev, raw_v_dev, q_norm_dev, k_norm_dev, q_out_dev, private_k_dev, private_v_dev,
                      base_position_dev, status_dev, nullptr, rows, heads, kv_heads, head_dim, eps, freq_base, freq_scale, kv_f16};
    return launch_rope_store(p, as_stream(stream), false);
}

int gf_rope_store_rows(const float* raw_q_dev, const float* raw_k_dev, const float* raw_v_dev, const float* q_norm_dev,
                       const float* k_norm_dev, float* q_out_dev, void* private_k_dev, void* private_v_dev,
                       const uint32_t* row_positions_dev, uint32_t* status_dev, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                       uint32_t head_dim, uint32_t rotary_dim, float eps, float freq_base, float freq_scale, int kv_f16, void* stream) {
    if (!row_positions_dev || rows == 0 || heads + kv_heads == 0 || !(freq_base > 0.0f) || (rotary_dim != 0 && rotary_dim != head_dim)
        || (heads != 0 && (!raw_q_dev || !q_out_dev)) || (kv_heads != 0 && (!raw_k_dev || !raw_v_dev || !private_k_dev || !private_v_dev)))
        return fail(GF_ERR_INVALID, "gf_rope_store_rows: bad arguments (rotary_dim is 0 or head_dim)");
    RopeStoreParams p{raw_q_dev, raw_k_dev, raw_v_dev, q_norm_dev, k_norm_dev, q_out_dev, private_k_dev, private_v_dev,
                      nullptr, status_dev, nullptr, rows, heads, kv_heads, head_dim, eps, freq_base, freq_scale, kv_f16};
    p.row_positions = row_positions_dev;
    p.rotate = rotary_dim != 0 ? 1u : 0u;
    return launch_rope_store(p, as_stream(stream), false);
}

size_t gf_attention_workspace_bytes(uint32_t rows, uint32_t heads) {
    return attention_workspace_bytes(rows, heads);
}

int gf_attention(const float* q_dev, const void* ring_k_dev, const void* ring_v_dev, const void* private_k_dev,
                 const void* private_v_dev, float* out_dev, void* workspace_dev, const uint32_t* base_position_dev,
                 uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t ring_rows,
                 uint32_t window, float scale, float softcap, int kv_f16, void* stream) {
    if (!q_dev || !ring_k_dev || !ring_v_dev || !private_k_dev || !private_v_dev || !out_dev || !workspace_dev
        || !base_position_dev || rows == 0 || rows > GF_MAX_ROWS || ring_rows == 0 || (ring_rows & (ring_rows - 1u)))
        return fail(GF_ERR_INVALID, "gf_attention: bad arguments (ring rows must be a power of two)");
    // Queries, cache rows, outputs and partial results move as 16-byte vectors.
    const uintptr_t pointers = reinterpret_cast<uintptr_t>(q_dev) | reinterpret_cast<uintptr_t>(ring_k_dev) | reinterpret_cast<uintptr_t>(ring_v_dev)
        | reinterpret_cast<uintptr_t>(private_k_dev) | reinterpret_cast<uintptr_t>(private_v_dev) | reinterpret_cast<uintptr_t>(out_dev)
        | reinterpret_cast<uintptr_t>(workspace_dev);
    if (pointers & 15u) return fail(GF_ERR_INVALID, "gf_attention: device pointers must be 16-byte aligned");
    AttentionParams p;
    p.q = q_dev; p.ring_k = ring_k_dev; p.ring_v = ring_v_dev; p.private_k = private_k_dev; p.private_v = private_v_dev;
    p.out = out_dev;
    p.partial_out = static_cast<float*>(workspace_dev);
    p.partial_ml = p.partial_out + (size_t)rows * heads * kMaxAttentionPartitions * 256u;
    p.counters = attention_counters(workspace_dev, rows, heads);
    // The arrival counters must start at zero (a finished call leaves them zero again).
    GF_CUDA(cudaMemsetAsync(p.counters, 0, (size_t)rows * heads * sizeof(uint32_t), as_stream(stream)));
    p.base_position = base_position_dev;
    p.rows = rows; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.ring_mask = ring_rows - 1u; p.window = window; p.scale = scale; p.softcap = softcap; p.kv_f16 = kv_f16;
    return launch_attention(p, as_stream(stream), false);
}

int gf_gelu_tanh_multiply(const float* gate_dev, const float* up_dev, float* out_dev, uint64_t count, void* stream) {
    if (!gate_dev || !up_dev || !out_dev || count == 0) return fail(GF_ERR_INVALID, "gf_gelu_tanh_multiply: bad arguments");
    return launch_geglu(gate_dev, up_dev, out_dev, count, as_stream(stream), false);
}

int gf_kv_scatter(const void* private_k_dev, const void* private_v_dev, void* ring_k_dev, void* ring_v_dev,
                  const uint32_t* base_position_dev, uint32_t rows, uint32_t row_width, uint32_t ring_rows, int kv_f16,
                  void* stream) {
    if (!private_k_dev || !private_v_dev || !ring_k_dev || !ring_v_dev || !base_position_dev || rows == 0
        || (ring_rows & (ring_rows - 1u)) || (row_width * (kv_f16 ? 2u : 4u)) % 16u)
        return fail(GF_ERR_INVALID, "gf_kv_scatter: bad arguments");
    return launch_kv_scatter(private_k_dev, private_v_dev, ring_k_dev, ring_v_dev, base_position_dev, rows, row_width,
                             ring_rows - 1u, kv_f16, as_stream(stream), false);
}

}  // extern "C"
