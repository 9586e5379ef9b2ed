// Embedding gather, RMSNorm (+residual), per-head norm + NEOX RoPE + private KV store, GeGLU,
// split-KV grouped-query attention over ring + private rows, and KV publication.
#include "ops.cuh"

#include <cmath>

namespace gf {

// ------------------------------------------------------------------ embedding

// Decodes element e of output column `token` straight from the streaming layout, with the
// reference's rounding (quantization.cpp:457,517,590), then scales it (model.cpp:599-605).
__device__ __forceinline__ float packed_element(int dtype, const uint8_t* packed, uint32_t units, uint32_t token,
                                                uint32_t e) {
    const uint32_t unit = unit_elements(dtype), c16 = token & 15u;
    const uint8_t* base = packed + ((size_t)(token >> 4) * units + e / unit) * pair_row_bytes(dtype);
    // Byte `o` of the column's native unit (bytes keep their place inside a moved 16-bit word).
    auto byte_at = [&](uint32_t o) -> uint32_t { return base[packed_offset(dtype, c16, o & ~1u) + (o & 1u)]; };
    auto half_at = [&](uint32_t o) -> float {
        return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(base + packed_offset(dtype, c16, o))));
    };
    const uint32_t i = e % unit;
    if (dtype == GF_Q6_K) {
        const uint32_t half = i / 128u, w = i % 128u, lane = w % 32u, quarter = w / 32u;
        const uint32_t lowbyte = byte_at(half * 64u + (quarter % 2u) * 32u + lane);
        const uint32_t low = quarter < 2u ? (lowbyte & 15u) : (lowbyte >> 4);
        const uint32_t high = (byte_at(128u + half * 32u + lane) >> (quarter * 2u)) & 3u;
        const int q = (int)(low | (high << 4)) - 32;
        const float s = (float)(int)(signed char)byte_at(192u + i / 16u);
        return __fmul_rn(__fmul_rn(half_at(208u), s), (float)q);
    }
    if (dtype == GF_Q8_0) {
        const uint32_t block = i / 32u;
        return __fmul_rn(half_at(block * 34u), (float)(int)(signed char)byte_at(block * 34u + 2u + i % 32u));
    }
    const uint32_t group = i / 32u, in64 = i % 64u;
    const float d = half_at(0u), dmin = half_at(2u);
    uint32_t sc, mn;
    if (group < 4u) { sc = byte_at(4u + group) & 63u; mn = byte_at(8u + group) & 63u; }
    else {
        sc = (byte_at(8u + group) & 15u) | ((byte_at(group) >> 6) << 4);
        mn = (byte_at(8u + group) >> 4) | ((byte_at(4u + group) >> 6) << 4);
    }
    const uint32_t byte = byte_at(16u + (i / 64u) * 32u + in64 % 32u);
    const uint32_t q = in64 < 32u ? (byte & 15u) : (byte >> 4);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
}

__global__ void __launch_bounds__(256) embedding_kernel(int dtype, const uint8_t* __restrict__ packed, uint32_t k,
                                                        uint32_t vocab, const uint32_t* __restrict__ tokens,
                                                        uint32_t rows, float scale, float* __restrict__ out,
                                                        uint32_t* status) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t units = k / unit_elements(dtype);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * k; i += gridDim.x * blockDim.x) {
        const uint32_t row = i / k, e = i % k;
        const uint32_t token = tokens[row];
        if (token >= vocab) {          // out-of-range id: flag it and poison the row (metal_kernels.mm:461)
            if (e == 0) atomicOr(status, kStatusBadToken);
            out[i] = __int_as_float(0x7fc00000);
            continue;
        }
        out[i] = __fmul_rn(packed_element(dtype, packed, units, token, e), scale);
    }
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
    const uint32_t position = *p.base_position + row;
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
    const float r0 = __fsub_rn(__fmul_rn(first, c), __fmul_rn(second, s));
    const float r1 = __fadd_rn(__fmul_rn(first, s), __fmul_rn(second, c));
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
            atomicOr(p.status, kStatusKvNonFinite);
    } else {
        float* kd = static_cast<float*>(p.private_k) + o;
        float* vd = static_cast<float*>(p.private_v) + o;
        kd[i] = r0; kd[i + half] = r1; vd[i] = v0; vd[i + half] = v1;
    }
}

// ------------------------------------------------------------------ attention

// Eight consecutive cache elements of one lane: raw registers (so a load can be issued a whole
// iteration before its use) and their widening to f32.
template <typename KV> struct KvRaw;
template <> struct KvRaw<__half> { uint4 v; };
template <> struct KvRaw<float> { float4 a, b; };
__device__ __forceinline__ void load_raw(const __half* p, KvRaw<__half>& r) { r.v = *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void load_raw(const float* p, KvRaw<float>& r) {
    r.a = *reinterpret_cast<const float4*>(p); r.b = *reinterpret_cast<const float4*>(p + 4);
}
__device__ __forceinline__ void widen(const KvRaw<__half>& r, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void widen(const KvRaw<float>& r, float (&v)[8]) {
    v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// The cached positions a group of consecutive verify/decode rows reads: the union of the rows'
// key ranges.  Row r (position base + r) sees the positions from its window start (the sliding
// window includes the row itself) up to its own; positions below the committed base live in the
// ring, the rest are the private rows of the pass   (gemma_target_runtime.cpp:256-268,
// target_verifier.cpp:186-202).  Consecutive rows' ranges overlap in all but one position at
// each end, so one walk over the union serves the whole group with a per-row mask.
struct AttentionSpan { uint32_t base, first, count, parts; };

__device__ __forceinline__ uint32_t attention_window_start(uint32_t position, uint32_t window) {
    return (window != 0u && position + 1u > window) ? position + 1u - window : 0u;
}

__device__ __forceinline__ AttentionSpan attention_span(uint32_t base, uint32_t first_row, uint32_t row_count, uint32_t window,
                                                        uint32_t target_parts, uint32_t granule, uint32_t min_tokens) {
    AttentionSpan s;
    s.base = base;
    s.first = attention_window_start(base + first_row, window);
    s.count = base + first_row + row_count - s.first;
    // As many partitions as the launch has room for, none shorter than the minimum length, each a
    // whole number of block iterations (`granule` cached rows).
    uint32_t tokens = (s.count + target_parts - 1u) / target_parts;
    tokens = max(min_tokens, (tokens + granule - 1u) / granule * granule);
    s.parts = min((uint32_t)kMaxAttentionPartitions, (s.count + tokens - 1u) / tokens);
    return s;
}

// What follows the walk over the cache, for a block of W warps that has left each warp's running
// maximum, sum and unnormalised output of its Q = G * R query vectors in shared memory: the warps
// are combined in warp order; with one partition that is the result, otherwise it is parked and the
// block that arrives last for the (row group, kv head) merges the partitions.
template <int G, int R, int W>
__device__ __forceinline__ void attention_finish(const AttentionParams& p, const AttentionSpan& span, uint32_t kvh, uint32_t part,
                                                 uint32_t first_row, uint32_t live_rows, float (&warp_m)[W][G * R],
                                                 float (&warp_l)[W][G * R], float (&warp_acc)[W][G * R][256], uint32_t& arrival) {
    constexpr int Q = G * R;
    __shared__ float factor[W][Q], block_m[Q], block_l[Q];
    __syncthreads();
    // Each warp's weight in the block's result, once per (warp, query): warp 0, lane = query.
    if (threadIdx.x < live_rows * (uint32_t)G) {
        const uint32_t qi = threadIdx.x;
        float mm = -INFINITY;
        for (int w = 0; w < W; ++w) mm = fmaxf(mm, warp_m[w][qi]);
        float ll = 0.0f;
        for (int w = 0; w < W; ++w) {
            const float f = warp_l[w][qi] == 0.0f ? 0.0f : expf(warp_m[w][qi] - mm);
            factor[w][qi] = f;
            ll = fmaf(warp_l[w][qi], f, ll);
        }
        block_m[qi] = mm;
        block_l[qi] = ll;
    }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < live_rows * (uint32_t)G * 256u; idx += blockDim.x) {
        const uint32_t qi = idx / 256u, d = idx % 256u;
        float a = 0.0f;
#pragma unroll
        for (int w = 0; w < W; ++w) a = fmaf(warp_acc[w][qi][d], factor[w][qi], a);
        const uint32_t row = first_row + qi / G, head = kvh * G + qi % G;
        if (span.parts == 1u && !p.defer_merge) {
            p.out[((size_t)row * p.heads + head) * 256u + d] = a / block_l[qi];
        } else {
            const size_t slot = ((size_t)row * p.heads + head) * kMaxAttentionPartitions + part;
            p.partial_out[slot * 256u + d] = a;
            if (d == 0) { p.partial_ml[slot * 2u] = block_m[qi]; p.partial_ml[slot * 2u + 1u] = block_l[qi]; }
        }
    }
    if (p.defer_merge) {
        // The consumer merges; it looks at all slots, so partition 0 marks the unused ones empty.
        if (part == 0u)
            for (uint32_t idx = threadIdx.x; idx < live_rows * (uint32_t)G * 32u; idx += blockDim.x) {
                const uint32_t qi = idx >> 5, lane_part = idx & 31u;
                if (lane_part < span.parts) continue;
                const size_t slot = ((size_t)(first_row + qi / G) * p.heads + kvh * G + qi % G) * kMaxAttentionPartitions + lane_part;
                p.partial_ml[slot * 2u] = -INFINITY;
                p.partial_ml[slot * 2u + 1u] = 0.0f;
            }
        return;
    }
    if (span.parts == 1u) return;
    // The block that arrives last for this (row group, kv head) merges all partitions.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) arrival = atomicAdd(&p.counters[blockIdx.z * p.kv_heads + kvh], 1u);
    __syncthreads();
    if (arrival != span.parts - 1u) return;
    __threadfence();
    // A thread merges four consecutive dimensions of one query at a time (item = query * 64 +
    // dimension / 4): the partial outputs of all partitions of its first item are requested at
    // once, ahead of the partition weights (one warp per query), so the two round trips to L2
    // overlap.  A partition in which a row saw no position carries (-inf, 0) and weighs
    // nothing.
    constexpr uint32_t kChunk = kMaxAttentionPartitions;
    const uint32_t items = live_rows * (uint32_t)G * 64u;
    auto item_offset = [&](uint32_t item) -> size_t {      // of (row, head, dimension) in p.out; partials are 32 times as wide
        const uint32_t qi = item / 64u;
        return ((size_t)(first_row + qi / G) * p.heads + kvh * G + qi % G) * 256u + (item % 64u) * 4u;
    };
    float4 v[kChunk];
    auto load_chunk = [&](uint32_t item, uint32_t first_part) {
        const size_t o = item_offset(item);
        const float* src = p.partial_out + (o & ~(size_t)255u) * kMaxAttentionPartitions + (o & 255u);
#pragma unroll
        for (uint32_t j = 0; j < kChunk; ++j)
            v[j] = first_part + j < span.parts ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(first_part + j) * 256u))
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    };
    if (threadIdx.x < items) load_chunk(threadIdx.x, 0u);
    float* weight = &warp_acc[0][0][0];                 // [Q][kMaxAttentionPartitions] factor, then [Q] total
    for (uint32_t idx = threadIdx.x; idx < live_rows * (uint32_t)G * 32u; idx += blockDim.x) {
        const uint32_t qi = idx >> 5, lane_part = idx & 31u;
        const uint32_t row = first_row + qi / G, head = kvh * G + qi % G;
        const size_t slot = ((size_t)row * p.heads + head) * kMaxAttentionPartitions + lane_part;
        const bool live = lane_part < span.parts;
        const float pm = live ? __ldcg(&p.partial_ml[slot * 2u]) : -INFINITY;
        const float pl = live ? __ldcg(&p.partial_ml[slot * 2u + 1u]) : 0.0f;
        float mm = pm;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, offset));
        const float f = live && pl != 0.0f ? expf(pm - mm) : 0.0f;
        weight[qi * kMaxAttentionPartitions + lane_part] = f;
        // Sum of l_i * f_i over the partitions in a fixed butterfly order (the same on every lane).
        const float ll = warp_sum(pl * f);
        if (lane_part == 0u) weight[Q * kMaxAttentionPartitions + qi] = ll;
    }
    __syncthreads();
    for (uint32_t item = threadIdx.x; item < items; item += blockDim.x) {
        const uint32_t qi = item / 64u;
        const float* w = weight + qi * kMaxAttentionPartitions;
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t first_part = 0; first_part < span.parts; first_part += kChunk) {
            if (item != threadIdx.x || first_part != 0u) load_chunk(item, first_part);
#pragma unroll
            for (uint32_t j = 0; j < kChunk; ++j) {
                const float f = w[(first_part + j) & 31u];
                a.x = fmaf(v[j].x, f, a.x); a.y = fmaf(v[j].y, f, a.y);
                a.z = fmaf(v[j].z, f, a.z); a.w = fmaf(v[j].w, f, a.w);
            }
        }
        const float total = weight[Q * kMaxAttentionPartitions + qi];
        *reinterpret_cast<float4*>(p.out + item_offset(item)) = make_float4(a.x / total, a.y / total, a.z / total, a.w / total);
    }
    if (threadIdx.x == 0) p.counters[blockIdx.z * p.kv_heads + kvh] = 0u;
}

// Online-softmax GQA, head_dim 256: grid (kv_head, partition, row group), kAttentionWarps warps per
// block.  A block serves R consecutive rows and the G query heads of one KV head: Q = G * R query
// vectors against one walk over the cached rows.  A warp walks quads of cached rows, loading the
// next quad while it works on the current one; a lane owns eight of the 256 dimensions, so K and
// V rows are read as one coalesced 512-byte (F16) or 1-KiB (F32) line per row.  The block that
// finishes last for a (row group, kv head) merges the partitions in partition order.
template <typename KV, int G, int R>
__global__ void __launch_bounds__(kAttentionWarps * 32) attention_kernel(AttentionParams p) {
    constexpr int Q = G * R;
    static_assert(4 * Q <= 16, "scores hold sixteen (token, query) columns");
    __shared__ float scores[kAttentionWarps][16];
    __shared__ float warp_m[kAttentionWarps][Q], warp_l[kAttentionWarps][Q];
    __shared__ float warp_acc[kAttentionWarps][Q][256];
    __shared__ uint32_t arrival;
    // The committed position and the ring rows were written by launches that completed before
    // the launch ahead of this one began its work, so they are read ahead of the dependency wait:
    // the first ring rows are then in flight while that launch drains.  The queries and the private
    // rows come from it and are read after the wait.
    const uint32_t kvh = blockIdx.x, part = blockIdx.y, first_row = blockIdx.z * R;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t live_rows = min((uint32_t)R, p.rows - first_row);
    const AttentionSpan span = attention_span(*p.base_position, first_row, live_rows, p.window, p.target_parts,
                                               4u * kAttentionWarps, kAttentionTokensPerPartition);
    if (part >= span.parts) return;
    const uint32_t kv_width = p.kv_heads * 256u;
    const KV* ring_k = static_cast<const KV*>(p.ring_k);
    const KV* ring_v = static_cast<const KV*>(p.ring_v);
    const KV* priv_k = static_cast<const KV*>(p.private_k);
    const KV* priv_v = static_cast<const KV*>(p.private_v);

    // Row r of the group sees positions [low[r], high[r]]; rows past the launch see none.
    uint32_t low[R], high[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint32_t position = span.base + first_row + r;
        low[r] = (uint32_t)r < live_rows ? attention_window_start(position, p.window) : 1u;
        high[r] = (uint32_t)r < live_rows ? position : 0u;
    }
    float m[Q], l[Q], acc[Q][8];
#pragma unroll
    for (int qi = 0; qi < Q; ++qi) {
        m[qi] = -INFINITY; l[qi] = 0.0f;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[qi][d] = 0.0f;
    }
    const uint32_t quads = (span.count + 3u) / 4u, step = span.parts * kAttentionWarps;
    KvRaw<KV> kraw[4], vraw[4];
    // `which`: 0 = every row of the quad, 1 = only rows in the ring, 2 = only private rows.
    auto fetch = [&](uint32_t quad, int which) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t position = span.first + min(quad * 4u + t, span.count - 1u);
            const KV *kp, *vp;
            if (position < span.base) {
                if (which == 2) continue;
                const size_t slot = ((size_t)(position & p.ring_mask)) * kv_width + kvh * 256u + lane * 8u;
                kp = ring_k + slot; vp = ring_v + slot;
            } else {
                if (which == 1) continue;
                const size_t slot = (size_t)(position - span.base) * kv_width + kvh * 256u + lane * 8u;
                kp = priv_k + slot; vp = priv_v + slot;
            }
            load_raw(kp, kraw[t]);
            load_raw(vp, vraw[t]);
        }
    };
    uint32_t quad = part * kAttentionWarps + warp;
    if (quad < quads) fetch(quad, 1);
    pdl_wait();
    pdl_launch_dependents();
    float q[Q][8];
#pragma unroll
    for (int qi = 0; qi < Q; ++qi) {
        const uint32_t row = min(first_row + qi / G, p.rows - 1u);
        const float* qp = p.q + ((size_t)row * p.heads + kvh * G + qi % G) * 256u + lane * 8u;
        load8(qp, q[qi]);
    }
    if (quad < quads) fetch(quad, 2);
    for (; quad < quads; quad += step) {
        float kf[4][8], vf[4][8];
        uint32_t position[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            position[t] = span.first + quad * 4u + t;      // past the span: above every row's own position
            widen(kraw[t], kf[t]);
            widen(vraw[t], vf[t]);
        }
        if (quad + step < quads) fetch(quad + step, 0);
        // Partial dot products (token t, query qi) -> column t*Q+qi, reduced across the warp eight at a time.
#pragma unroll
        for (int half = 0; half < (4 * Q + 7) / 8; ++half) {
            float cols[8];
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx) {
                const int flat = half * 8 + cidx, t = flat / Q, qi = flat % Q;
                float dot = 0.0f;
                if (flat < 4 * Q) {
#pragma unroll
                    for (int d = 0; d < 8; ++d) dot = fmaf(q[qi][d], kf[t][d], dot);
                }
                cols[cidx] = dot;
            }
            const float total = reduce_columns8(cols, lane);
            if ((lane & 3u) == 0u) scores[warp][half * 8 + column_of_lane(lane)] = total;
        }
        __syncwarp();
        float s[4][Q];
        bool visible[4][R];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int qi = 0; qi < Q; ++qi) {
                float v = scores[warp][t * Q + qi] * p.scale;
                if (p.softcap > 0.0f) v = tanhf(v / p.softcap) * p.softcap;
                visible[t][qi / G] = position[t] >= low[qi / G] && position[t] <= high[qi / G];
                s[t][qi] = visible[t][qi / G] ? v : -INFINITY;
            }
        __syncwarp();
#pragma unroll
        for (int qi = 0; qi < Q; ++qi) {
            float m_new = m[qi];
#pragma unroll
            for (int t = 0; t < 4; ++t) m_new = fmaxf(m_new, s[t][qi]);
            const float corr = m[qi] == -INFINITY ? 0.0f : expf(m[qi] - m_new);
            float pr[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) pr[t] = visible[t][qi / G] ? expf(s[t][qi] - m_new) : 0.0f;
            l[qi] = l[qi] * corr + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
#pragma unroll
            for (int d = 0; d < 8; ++d) {
                float a = acc[qi][d] * corr;
#pragma unroll
                for (int t = 0; t < 4; ++t) a = fmaf(pr[t], vf[t][d], a);
                acc[qi][d] = a;
            }
            m[qi] = m_new;
        }
    }
    // Combine the warps in warp order.
#pragma unroll
    for (int qi = 0; qi < Q; ++qi) {
        if (lane == 0) { warp_m[warp][qi] = m[qi]; warp_l[warp][qi] = l[qi]; }
#pragma unroll
        for (int d = 0; d < 8; ++d) warp_acc[warp][qi][lane * 8 + d] = acc[qi][d];
    }
    attention_finish<G, R, kAttentionWarps>(p, span, kvh, part, first_row, live_rows, warp_m, warp_l, warp_acc, arrival);
}

// ---- attention over a binary16 cache on the tensor cores
//
// D (16 x 8, f32) += A (16 x 16, f16, row-major) * B (16 x 8, f16, column-major), one warp.  With
// g = lane / 4 and t = lane % 4, a lane holds A rows g (a[0], a[2]) and g + 8 (a[1], a[3]), columns
// 2t, 2t+1 (a[0], a[1]) and 2t+8, 2t+9 (a[2], a[3]); B rows 2t, 2t+1 (b0) and 2t+8, 2t+9 (b1) of
// column g; D rows g (d[0], d[1]) and g + 8 (d[2], d[3]), columns 2t and 2t+1.
__device__ __forceinline__ void mma_f16_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// An f32 value as the sum of two binary16 values (exact to about 2^-22 of its magnitude).
__device__ __forceinline__ void split_f16(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}
__device__ __forceinline__ uint32_t pack_halves(__half a, __half b) {
    const __half2 h = __halves2half2(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

constexpr int kAttentionMmaWarps = 8;

// The same online-softmax GQA as attention_kernel for a binary16 cache, with both contractions on
// the tensor cores.  A warp takes tiles of sixteen cached rows.  The Q <= 4 query vectors become
// eight B columns, column 2q the binary16 rounding of (scale * query q) and column 2q + 1 the
// rounding of what that left over, so the two columns' products add up to the f32 score; the
// softmax weights are split the same way for the second contraction.  The cache rows are the A
// operands as they lie in memory: the contraction index of a product may be permuted freely as long
// as both operands agree, so a lane reads whole 16-byte pieces -- for the scores, dimensions
// 32c + 8t .. +7 of rows g and g + 8 serve k-steps 2c and 2c + 1; for the outputs, dimensions
// 64J + 8g .. +7 of rows 2t, 2t+1, 2t+8, 2t+9 are paired across rows by byte permutes and serve the
// four output tiles of group J, whose rows g / g + 8 stand for dimensions 64J + 8g + j / + 4 + j.
// A lane ends up with dimensions 64J + 8g .. +7 (J = 0..3) of query t.
template <int G, int R>
__global__ void __launch_bounds__(kAttentionMmaWarps * 32) attention_mma_kernel(AttentionParams p) {
    constexpr int Q = G * R, W = kAttentionMmaWarps;
    static_assert(Q <= 4, "eight B columns hold four split query vectors");
    __shared__ float warp_m[W][Q], warp_l[W][Q];
    __shared__ float warp_acc[W][Q][256];
    __shared__ uint2 q_frag[16][32];            // B registers of k-step ks, per lane
    __shared__ uint32_t arrival;
    // As in attention_kernel: the committed position and ring rows are read ahead of the dependency
    // wait, the queries and the private rows after it.
    const uint32_t kvh = blockIdx.x, part = blockIdx.y, first_row = blockIdx.z * R;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t live_rows = min((uint32_t)R, p.rows - first_row), live_q = live_rows * G;
    const AttentionSpan span = attention_span(*p.base_position, first_row, live_rows, p.window, p.target_parts, 16u * W, 16u * W);
    if (part >= span.parts) return;
    const uint32_t kv_width = p.kv_heads * 256u;
    const __half* ring_k = static_cast<const __half*>(p.ring_k);
    const __half* ring_v = static_cast<const __half*>(p.ring_v);
    const __half* priv_k = static_cast<const __half*>(p.private_k);
    const __half* priv_v = static_cast<const __half*>(p.private_v);

    // This lane's query t belongs to row t / G of the group and sees positions [low, high].
    const bool my_live = t < live_q;
    const uint32_t my_position = span.base + first_row + t / G;
    const uint32_t low = my_live ? attention_window_start(my_position, p.window) : 1u, high = my_live ? my_position : 0u;

    // A cached row's address, or null when `which` (0 = every row, 1 = only rows in the ring, 2 =
    // only private rows) leaves it out.
    auto row_of = [&](uint32_t token, const __half* ring, const __half* priv, int which) -> const __half* {
        const uint32_t position = span.first + min(token, span.count - 1u);
        if (position < span.base) return which == 2 ? nullptr : ring + (size_t)(position & p.ring_mask) * kv_width + kvh * 256u;
        return which == 1 ? nullptr : priv + (size_t)(position - span.base) * kv_width + kvh * 256u;
    };
    uint4 kraw[2][8], vraw[4][4];
    auto fetch_k = [&](uint32_t tile, int which) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half* src = row_of(tile * 16u + g + 8u * h, ring_k, priv_k, which);
            if (!src) continue;
#pragma unroll
            for (int c = 0; c < 8; ++c) kraw[h][c] = *reinterpret_cast<const uint4*>(src + 8u * t + 32 * c);
        }
    };
    auto fetch_v = [&](uint32_t tile, int which) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const __half* src = row_of(tile * 16u + 2u * t + (u & 1) + 8u * (u >> 1), ring_v, priv_v, which);
            if (!src) continue;
#pragma unroll
            for (int J = 0; J < 4; ++J) vraw[u][J] = *reinterpret_cast<const uint4*>(src + 8u * g + 64 * J);
        }
    };
    const uint32_t tiles = (span.count + 15u) / 16u, step = span.parts * W;
    uint32_t tile = part * W + warp;
    if (tile < tiles) { fetch_k(tile, 1); fetch_v(tile, 1); }
    pdl_wait();
    pdl_launch_dependents();
    // B registers of the scores: lane (g, t) holds, of column g (query g / 2, rounding or left-over),
    // dimensions 32c + 8t + 4e .. +3 for k-step 2c + e.  Warp w prepares chunks c = w, w + W, ...
    {
        const uint32_t qv = g >> 1;
        for (uint32_t c = warp; c < 8u; c += W) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = 0.0f;
            if (qv < live_q) load8(p.q + ((size_t)(first_row + qv / G) * p.heads + kvh * G + qv % G) * 256u + 32u * c + 8u * t, x);
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __half h0, l0, h1, l1;
                split_f16(x[2 * k] * p.scale, h0, l0);
                split_f16(x[2 * k + 1] * p.scale, h1, l1);
                w[k] = (g & 1u) ? pack_halves(l0, l1) : pack_halves(h0, h1);
            }
            q_frag[2u * c][lane] = make_uint2(w[0], w[1]);
            q_frag[2u * c + 1u][lane] = make_uint2(w[2], w[3]);
        }
    }
    __syncthreads();
    if (tile < tiles) { fetch_k(tile, 2); fetch_v(tile, 2); }

    float m_run = -INFINITY, l_run = 0.0f;      // of query t, over this lane's rows g and g + 8 of every tile
    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
    for (; tile < tiles; tile += step) {
        // Two accumulators (even and odd k-steps) halve the chain of dependent products.
        float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s4odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint2 b = q_frag[2 * c + e][lane];
                mma_f16_k16(e ? s4odd : s4, word_of(kraw[0][c], 2 * e), word_of(kraw[1][c], 2 * e), word_of(kraw[0][c], 2 * e + 1),
                            word_of(kraw[1][c], 2 * e + 1), b.x, b.y);
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) s4[i] += s4odd[i];
        const bool more = tile + step < tiles;
        if (more) fetch_k(tile + step, 0);
        // Scores of rows g and g + 8 against query t: rounding column plus left-over column.
        float s0 = s4[0] + s4[1], s1 = s4[2] + s4[3];
        if (p.softcap > 0.0f) { s0 = tanhf(s0 / p.softcap) * p.softcap; s1 = tanhf(s1 / p.softcap) * p.softcap; }
        const uint32_t position0 = span.first + tile * 16u + g, position1 = position0 + 8u;
        const bool visible0 = position0 >= low && position0 <= high, visible1 = position1 >= low && position1 <= high;
        float m_new = fmaxf(visible0 ? s0 : -INFINITY, visible1 ? s1 : -INFINITY);
        m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 4));
        m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 8));
        m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 16));
        m_new = fmaxf(m_new, m_run);
        const float corr = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
        const float p0 = visible0 ? expf(s0 - m_new) : 0.0f, p1 = visible1 ? expf(s1 - m_new) : 0.0f;
        l_run = l_run * corr + (p0 + p1);
        m_run = m_new;
        if (!__all_sync(0xffffffffu, corr == 1.0f)) {
#pragma unroll
            for (int i = 0; i < 16; ++i) { acc[i][0] *= corr; acc[i][1] *= corr; acc[i][2] *= corr; acc[i][3] *= corr; }
        }
        // B registers of the outputs: lane (g, t) needs, of column g (query g / 2, rounding or
        // left-over of the weight), rows 2t, 2t+1, 2t+8, 2t+9; row r < 8 of query q is p0 of lane
        // 4r + q, row r + 8 its p1.
        __half h0, l0, h1, l1;
        split_f16(p0, h0, l0);
        split_f16(p1, h1, l1);
        const uint32_t rounded = pack_halves(h0, h1), left_over = pack_halves(l0, l1);
        const uint32_t source = 8u * t + (g >> 1);
        const uint32_t ra = __shfl_sync(0xffffffffu, rounded, source), la = __shfl_sync(0xffffffffu, left_over, source);
        const uint32_t rb = __shfl_sync(0xffffffffu, rounded, source + 4u), lb = __shfl_sync(0xffffffffu, left_over, source + 4u);
        const uint32_t xa = (g & 1u) ? la : ra, xb = (g & 1u) ? lb : rb;
        const uint32_t b0 = __byte_perm(xa, xb, 0x5410u), b1 = __byte_perm(xa, xb, 0x7632u);
#pragma unroll
        for (int J = 0; J < 4; ++J)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                const int wi = j >> 1;
                mma_f16_k16(acc[J * 4 + j],
                            __byte_perm(word_of(vraw[0][J], wi), word_of(vraw[1][J], wi), sel),
                            __byte_perm(word_of(vraw[0][J], 2 + wi), word_of(vraw[1][J], 2 + wi), sel),
                            __byte_perm(word_of(vraw[2][J], wi), word_of(vraw[3][J], wi), sel),
                            __byte_perm(word_of(vraw[2][J], 2 + wi), word_of(vraw[3][J], 2 + wi), sel), b0, b1);
            }
        if (more) fetch_v(tile + step, 0);
    }
    // Sum of the weights over the eight row pairs; then the warp's state goes to shared memory.
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
    if (my_live) {
        if (g == 0u) { warp_m[warp][t] = m_run; warp_l[warp][t] = l_run; }
#pragma unroll
        for (int J = 0; J < 4; ++J) {
            float* dst = &warp_acc[warp][t][64 * J + 8 * g];
            *reinterpret_cast<float4*>(dst) = make_float4(acc[J * 4][0] + acc[J * 4][1], acc[J * 4 + 1][0] + acc[J * 4 + 1][1],
                                                          acc[J * 4 + 2][0] + acc[J * 4 + 2][1], acc[J * 4 + 3][0] + acc[J * 4 + 3][1]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[J * 4][2] + acc[J * 4][3], acc[J * 4 + 1][2] + acc[J * 4 + 1][3],
                                                              acc[J * 4 + 2][2] + acc[J * 4 + 2][3], acc[J * 4 + 3][2] + acc[J * 4 + 3][3]);
        }
    }
    attention_finish<G, R, W>(p, span, kvh, part, first_row, live_rows, warp_m, warp_l, warp_acc, arrival);
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

// ------------------------------------------------------------------ launchers

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
