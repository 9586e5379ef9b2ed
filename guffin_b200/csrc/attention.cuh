// Split-KV grouped-query attention over ring + private rows, as device functions over a "block"
// context so that the same code runs as a kernel of its own (the CTA is the block) and as a phase
// of the decode pass kernel (some warps of a larger CTA are the block).
//
// Block concept:  tid() / threads()  thread index and count inside the block;  sync()  barrier of
// the block's threads;  dependency()  called once by every thread when the block first needs what
// the producer ahead of it wrote (queries, private K/V rows) and returns false if that wait gave up.
#pragma once

#include "ops.cuh"

namespace gf {

// The CTA of an attention launch.
struct LaunchBlock {
    __device__ __forceinline__ uint32_t tid() const { return threadIdx.x; }
    __device__ __forceinline__ uint32_t threads() const { return blockDim.x; }
    __device__ __forceinline__ void sync() const { __syncthreads(); }
    __device__ __forceinline__ bool dependency() const { pdl_wait(); pdl_launch_dependents(); return true; }
};

// Shared memory of one block: what the warps hand to the combine step, and the combine step's own.
template <int W, int Q>
struct AttentionCombine {
    float warp_m[W][Q], warp_l[W][Q];
    float warp_acc[W][Q][256];
    float factor[W][Q], block_m[Q], block_l[Q];
    uint32_t arrival;
};
template <int W, int Q>
struct AttentionSmem : AttentionCombine<W, Q> {
    float scores[W][16];
};
template <int W, int Q>
struct AttentionMmaSmem : AttentionCombine<W, Q> {
    uint2 q_frag[16][32];            // B registers of k-step ks, per lane
};

constexpr int kAttentionMmaWarps = 8;


// Eight consecutive cache elements of one lane: raw registers (so a load can be issued a whole
// iteration before its use) and their widening to f32.
template <typename KV> struct KvRaw;
template <> struct KvRaw<__half> { uint4 v; };
template <> struct KvRaw<float> { float4 a, b; };
// Cache rows and queries are read from L2: inside a pass kernel the private rows and the queries were
// written by other CTAs a phase earlier, and an older copy may still sit in this SM's L1.
__device__ __forceinline__ void load_raw(const __half* p, KvRaw<__half>& r) { r.v = __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void load_raw(const float* p, KvRaw<float>& r) {
    r.a = __ldcg(reinterpret_cast<const float4*>(p)); r.b = __ldcg(reinterpret_cast<const float4*>(p + 4));
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
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p + 4));
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
template <int G, int R, int W, bool MERGE, typename Block>
__device__ __forceinline__ void attention_finish(const AttentionParams& p, const AttentionSpan& span, uint32_t kvh, uint32_t part,
                                                 uint32_t group, uint32_t first_row, uint32_t live_rows,
                                                 AttentionCombine<W, G * R>& sm, const Block& block) {
    constexpr int Q = G * R;
    float (&warp_m)[W][Q] = sm.warp_m;
    float (&warp_l)[W][Q] = sm.warp_l;
    float (&warp_acc)[W][Q][256] = sm.warp_acc;
    float (&factor)[W][Q] = sm.factor;
    float (&block_m)[Q] = sm.block_m;
    float (&block_l)[Q] = sm.block_l;
    uint32_t& arrival = sm.arrival;
    const uint32_t tid = block.tid(), threads = block.threads();
    block.sync();
    // Each warp's weight in the block's result, once per (warp, query): warp 0, lane = query.
    if (tid < live_rows * (uint32_t)G) {
        const uint32_t qi = tid;
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
    block.sync();
    for (uint32_t idx = tid; idx < live_rows * (uint32_t)G * 256u; idx += threads) {
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
            for (uint32_t idx = tid; idx < live_rows * (uint32_t)G * 32u; idx += threads) {
                const uint32_t qi = idx >> 5, lane_part = idx & 31u;
                if (lane_part < span.parts) continue;
                const size_t slot = ((size_t)(first_row + qi / G) * p.heads + kvh * G + qi % G) * kMaxAttentionPartitions + lane_part;
                p.partial_ml[slot * 2u] = -INFINITY;
                p.partial_ml[slot * 2u + 1u] = 0.0f;
            }
        return;
    }
    if (!MERGE || span.parts == 1u) return;      // without MERGE the caller guarantees p.defer_merge
    // The block that arrives last for this (row group, kv head) merges all partitions.
    __threadfence();
    block.sync();
    if (tid == 0) arrival = atomicAdd(&p.counters[group * p.kv_heads + kvh], 1u);
    block.sync();
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
    if (tid < items) load_chunk(tid, 0u);
    float* weight = &warp_acc[0][0][0];                 // [Q][kMaxAttentionPartitions] factor, then [Q] total
    for (uint32_t idx = tid; idx < live_rows * (uint32_t)G * 32u; idx += threads) {
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
    block.sync();
    for (uint32_t item = tid; item < items; item += threads) {
        const uint32_t qi = item / 64u;
        const float* w = weight + qi * kMaxAttentionPartitions;
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t first_part = 0; first_part < span.parts; first_part += kChunk) {
            if (item != tid || first_part != 0u) load_chunk(item, first_part);
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
    if (tid == 0) p.counters[group * p.kv_heads + kvh] = 0u;
}

// Online-softmax GQA, head_dim 256: grid (kv_head, partition, row group), kAttentionWarps warps per
// block.  A block serves R consecutive rows and the G query heads of one KV head: Q = G * R query
// vectors against one walk over the cached rows.  A warp walks quads of cached rows, loading the
// next quad while it works on the current one; a lane owns eight of the 256 dimensions, so K and
// V rows are read as one coalesced 512-byte (F16) or 1-KiB (F32) line per row.  The block that
// finishes last for a (row group, kv head) merges the partitions in partition order.
template <typename KV, int G, int R, bool MERGE, typename Block>
__device__ __forceinline__ bool attention_body(const AttentionParams& p, uint32_t kvh, uint32_t part, uint32_t group,
                                               AttentionSmem<kAttentionWarps, G * R>& sm, const Block& block, bool& waited) {
    constexpr int Q = G * R;
    static_assert(4 * Q <= 16, "scores hold sixteen (token, query) columns");
    float (&scores)[kAttentionWarps][16] = sm.scores;
    // The committed position and the ring rows were written by launches that completed before
    // the launch ahead of this one began its work, so they are read ahead of the dependency wait:
    // the first ring rows are then in flight while that launch drains.  The queries and the private
    // rows come from it and are read after the wait.
    const uint32_t first_row = group * R;
    const uint32_t warp = block.tid() >> 5, lane = block.tid() & 31u;
    const uint32_t live_rows = min((uint32_t)R, p.rows - first_row);
    const AttentionSpan span = attention_span(*p.base_position, first_row, live_rows, p.window, p.target_parts,
                                               4u * kAttentionWarps, kAttentionTokensPerPartition);
    if (part >= span.parts) return true;
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
    waited = true;
    if (!block.dependency()) return false;
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
        if (lane == 0) { sm.warp_m[warp][qi] = m[qi]; sm.warp_l[warp][qi] = l[qi]; }
#pragma unroll
        for (int d = 0; d < 8; ++d) sm.warp_acc[warp][qi][lane * 8 + d] = acc[qi][d];
    }
    attention_finish<G, R, kAttentionWarps, MERGE>(p, span, kvh, part, group, first_row, live_rows, sm, block);
    return true;
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
//
// SPLIT warps share a tile (the block then has SPLIT * kAttentionMmaWarps warps): each computes the
// tile's scores and accumulates 256 / SPLIT of the output dimensions, which needs half the registers
// for the values and the accumulators.  PREFETCH requests the next tile's rows while the current one
// is worked on (more registers again); without it a tile's K rows are requested when its turn comes
// and its V rows once the scores are done.  Every variant performs the same arithmetic per output.
// MERGE = false leaves out the in-launch merge of the partitions (callers that always defer it).
template <int G, int R, int SPLIT, bool PREFETCH, bool MERGE, typename Block>
__device__ __forceinline__ bool attention_mma_body(const AttentionParams& p, uint32_t kvh, uint32_t part, uint32_t group,
                                                   AttentionMmaSmem<kAttentionMmaWarps, G * R>& sm, const Block& block, bool& waited) {
    constexpr int Q = G * R, W = kAttentionMmaWarps, JN = 4 / SPLIT;
    static_assert(Q <= 4, "eight B columns hold four split query vectors");
    static_assert(SPLIT == 1 || SPLIT == 2, "a tile is shared by one or two warps");
    uint2 (&q_frag)[16][32] = sm.q_frag;            // B registers of k-step ks, per lane
    // As in attention_kernel: the committed position and ring rows are read ahead of the dependency
    // wait, the queries and the private rows after it.
    const uint32_t first_row = group * R;
    const uint32_t warp = (block.tid() >> 5) % W, lane = block.tid() & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t j_base = ((block.tid() >> 5) / W) * JN;        // first group of 64 output dimensions this warp accumulates
    const uint32_t live_rows = min((uint32_t)R, p.rows - first_row), live_q = live_rows * G;
    const AttentionSpan span = attention_span(*p.base_position, first_row, live_rows, p.window, p.target_parts, 16u * W, 16u * W);
    if (part >= span.parts) return true;
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
    uint4 kraw[2][8], vraw[4][JN];
    auto fetch_k = [&](uint32_t tile, int which) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half* src = row_of(tile * 16u + g + 8u * h, ring_k, priv_k, which);
            if (!src) continue;
#pragma unroll
            for (int c = 0; c < 8; ++c) kraw[h][c] = __ldcg(reinterpret_cast<const uint4*>(src + 8u * t + 32 * c));
        }
    };
    auto fetch_v = [&](uint32_t tile, int which) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const __half* src = row_of(tile * 16u + 2u * t + (u & 1) + 8u * (u >> 1), ring_v, priv_v, which);
            if (!src) continue;
#pragma unroll
            for (int J = 0; J < JN; ++J) vraw[u][J] = __ldcg(reinterpret_cast<const uint4*>(src + 8u * g + 64u * (j_base + J)));
        }
    };
    const uint32_t tiles = (span.count + 15u) / 16u, step = span.parts * W;
    uint32_t tile = part * W + warp;
    if (tile < tiles) { fetch_k(tile, 1); if (PREFETCH) fetch_v(tile, 1); }
    waited = true;
    if (!block.dependency()) return false;
    // B registers of the scores: lane (g, t) holds, of column g (query g / 2, rounding or left-over),
    // dimensions 32c + 8t + 4e .. +3 for k-step 2c + e.  Warp w prepares chunks c = w, w + W, ...
    {
        const uint32_t qv = g >> 1;
        for (uint32_t c = block.tid() >> 5; c < 8u; c += W * SPLIT) {
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
    block.sync();
    if (tile < tiles) { fetch_k(tile, 2); if (PREFETCH) fetch_v(tile, 2); }

    float m_run = -INFINITY, l_run = 0.0f;      // of query t, over this lane's rows g and g + 8 of every tile
    float acc[4 * JN][4];
#pragma unroll
    for (int i = 0; i < 4 * JN; ++i) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
    bool first_tile = true;
    for (; tile < tiles; tile += step) {
        if (!PREFETCH && !first_tile) fetch_k(tile, 0);
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
        const bool more = PREFETCH && tile + step < tiles;
        if (more) fetch_k(tile + step, 0);
        if (!PREFETCH) fetch_v(tile, 0);
        first_tile = false;
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
            for (int i = 0; i < 4 * JN; ++i) { acc[i][0] *= corr; acc[i][1] *= corr; acc[i][2] *= corr; acc[i][3] *= corr; }
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
        for (int J = 0; J < JN; ++J)
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
        if (g == 0u && j_base == 0u) { sm.warp_m[warp][t] = m_run; sm.warp_l[warp][t] = l_run; }
#pragma unroll
        for (int J = 0; J < JN; ++J) {
            float* dst = &sm.warp_acc[warp][t][64u * (j_base + J) + 8u * g];
            *reinterpret_cast<float4*>(dst) = make_float4(acc[J * 4][0] + acc[J * 4][1], acc[J * 4 + 1][0] + acc[J * 4 + 1][1],
                                                          acc[J * 4 + 2][0] + acc[J * 4 + 2][1], acc[J * 4 + 3][0] + acc[J * 4 + 3][1]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[J * 4][2] + acc[J * 4][3], acc[J * 4 + 1][2] + acc[J * 4 + 1][3],
                                                              acc[J * 4 + 2][2] + acc[J * 4 + 2][3], acc[J * 4 + 3][2] + acc[J * 4 + 3][3]);
        }
    }
    attention_finish<G, R, W, MERGE>(p, span, kvh, part, group, first_row, live_rows, sm, block);
    return true;
}


}  // namespace gf
