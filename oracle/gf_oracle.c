/*
 * CPU oracle for the Gemma decode hot path -- TEST INFRASTRUCTURE, never shipped
 * and never linked into the CUDA library.  Plain C restatement of the reference
 * engine's scalar CPU algorithms; see gf_oracle.h for the file:line each function
 * follows.  Build with -ffp-contract=off so every f32 operation rounds separately,
 * as the reference's x86-64 / arm64 scalar code does.
 */
#include "gf_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ f16 */

static float bits_to_f32(uint32_t bits) { float f; memcpy(&f, &bits, 4); return f; }
static uint32_t f32_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

float gfo_f16_to_f32(uint16_t bits) {
    const uint32_t sign = (uint32_t)(bits & 0x8000u) << 16;
    uint32_t exponent = (bits >> 10) & 0x1Fu;
    uint32_t fraction = bits & 0x03FFu;
    if (exponent == 0) {
        if (fraction == 0) return bits_to_f32(sign);
        int e = -14;
        while ((fraction & 0x0400u) == 0) { fraction <<= 1; --e; }
        fraction &= 0x03FFu;
        return bits_to_f32(sign | ((uint32_t)(e + 127) << 23) | (fraction << 13));
    }
    if (exponent == 0x1Fu) return bits_to_f32(sign | (0xFFu << 23) | (fraction << 13));
    return bits_to_f32(sign | ((exponent + 112u) << 23) | (fraction << 13));
}

uint16_t gfo_f32_to_f16_half_up(float value) {
    const uint32_t bits = f32_to_bits(value);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int exponent = (int)((bits >> 23) & 0xFFu);
    uint32_t fraction = bits & 0x7FFFFFu;
    if (exponent == 0xFF) return (uint16_t)(sign | (fraction == 0 ? 0x7C00u : 0x7E00u));
    exponent = exponent - 127 + 15;
    if (exponent >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (exponent <= 0) {
        if (exponent < -10) return sign;
        fraction |= 0x800000u;
        const uint32_t shift = (uint32_t)(14 - exponent);
        return (uint16_t)(sign | (uint16_t)((fraction + (1u << (shift - 1u))) >> shift));
    }
    fraction += 0x00001000u;
    if (fraction & 0x00800000u) {
        fraction = 0;
        ++exponent;
        if (exponent >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    }
    return (uint16_t)(sign | ((uint16_t)exponent << 10) | (uint16_t)(fraction >> 13));
}

uint16_t gfo_f32_to_f16_rne(float value) {
    const uint32_t bits = f32_to_bits(value);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    const uint32_t magnitude = bits & 0x7FFFFFFFu;
    if (magnitude >= 0x7F800000u)
        return (uint16_t)(sign | (magnitude > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (magnitude >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 */
    if (magnitude < 0x33000001u) return sign;                         /* <= 2^-25 -> 0 */
    int exponent = (int)(magnitude >> 23) - 127;
    uint32_t mantissa = (magnitude & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (exponent < -14) { shift = (uint32_t)(13 + (-14 - exponent)); base = 0; }
    else { shift = 13; base = (uint32_t)(exponent + 15) << 10; mantissa &= 0x7FFFFFu; }
    uint32_t rounded = mantissa >> shift;
    const uint32_t remainder = mantissa & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1u);
    if (remainder > halfway || (remainder == halfway && (rounded & 1u))) ++rounded;
    return (uint16_t)(sign | (base + rounded)); /* a mantissa carry correctly bumps the exponent */
}

/* ------------------------------------------------------------------ blocks */

uint32_t gfo_block_elements(int dtype) {
    return dtype == GFO_Q8_0 ? 32u : (dtype == GFO_Q4_K || dtype == GFO_Q6_K) ? 256u : 0u;
}
uint32_t gfo_block_bytes(int dtype) {
    return dtype == GFO_Q8_0 ? 34u : dtype == GFO_Q4_K ? 144u : dtype == GFO_Q6_K ? 210u : 0u;
}

static uint16_t read_u16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

/* quantization.cpp:338-357 */
static uint8_t q4k_scale_min(const uint8_t* s, uint32_t group, int want_min) {
    if (group < 4u) return (uint8_t)(s[group + (want_min ? 4u : 0u)] & 0x3Fu);
    const uint8_t low_source = s[group + 4u];
    if (want_min) return (uint8_t)((low_source >> 4) | ((s[group] & 0xC0u) >> 2));
    return (uint8_t)((low_source & 0x0Fu) | ((s[group - 4u] & 0xC0u) >> 2));
}

static void dequant_q8_0_block(const uint8_t* b, float* out) {
    const float d = gfo_f16_to_f32(read_u16(b));
    for (uint32_t i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)b[2 + i];
}

static void dequant_q4_k_block(const uint8_t* b, float* out) {
    const float d = gfo_f16_to_f32(read_u16(b));
    const float dmin = gfo_f16_to_f32(read_u16(b + 2));
    const uint8_t* scales = b + 4;
    const uint8_t* qs = b + 16;
    for (uint32_t e = 0; e < 256; ++e) {
        const uint32_t group = e / 32u;
        const uint32_t in64 = e % 64u;
        const uint8_t byte = qs[(e / 64u) * 32u + (in64 % 32u)];
        const uint8_t nibble = (uint8_t)((byte >> (in64 < 32u ? 0u : 4u)) & 0x0Fu);
        const float sc = (float)q4k_scale_min(scales, group, 0);
        const float mn = (float)q4k_scale_min(scales, group, 1);
        out[e] = d * sc * (float)nibble - dmin * mn;
    }
}

static void dequant_q6_k_block(const uint8_t* b, float* out) {
    const uint8_t* ql = b;
    const uint8_t* qh = b + 128;
    const int8_t* sc = (const int8_t*)(b + 192);
    const float d = gfo_f16_to_f32(read_u16(b + 208));
    for (uint32_t e = 0; e < 256; ++e) {
        const uint32_t half = e / 128u, w = e % 128u, lane = w % 32u, quarter = w / 32u;
        const uint8_t lowbyte = ql[half * 64u + (quarter % 2u) * 32u + lane];
        const uint8_t low = (uint8_t)((lowbyte >> (w < 64u ? 0u : 4u)) & 0x0Fu);
        const uint8_t high = (uint8_t)((qh[half * 32u + lane] >> (quarter * 2u)) & 0x03u);
        const int8_t q = (int8_t)((int16_t)(uint8_t)(low | (high << 4)) - 32);
        out[e] = d * (float)sc[e / 16u] * (float)q;
    }
}

static void dequant_block(int dtype, const uint8_t* b, float* out) {
    if (dtype == GFO_Q8_0) dequant_q8_0_block(b, out);
    else if (dtype == GFO_Q4_K) dequant_q4_k_block(b, out);
    else dequant_q6_k_block(b, out);
}

void gfo_dequantize(int dtype, const uint8_t* blocks, uint64_t block_count, float* out) {
    const uint32_t be = gfo_block_elements(dtype), bb = gfo_block_bytes(dtype);
    for (uint64_t i = 0; i < block_count; ++i) dequant_block(dtype, blocks + i * bb, out + i * be);
}

/* ------------------------------------------------------------------ GEMV */

void gfo_matmul_quantized_columns(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                                  uint64_t k, uint64_t n, uint64_t n_begin, uint64_t n_end,
                                  float* out) {
    const uint32_t be = gfo_block_elements(dtype), bb = gfo_block_bytes(dtype);
    const uint64_t blocks_per_column = k / be;
    float decoded[256];
    /* Decoding a block once and then walking it in ascending order performs exactly the
     * additions of the reference's per-element loop, in the same order. */
    for (uint64_t column = n_begin; column < n_end; ++column) {
        const uint8_t* col = weight + column * blocks_per_column * bb;
        for (uint32_t row = 0; row < rows; ++row) {
            float sum = 0.0f;
            const float* xr = x + (uint64_t)row * k;
            for (uint64_t block = 0; block < blocks_per_column; ++block) {
                if (row == 0 || blocks_per_column > 1) dequant_block(dtype, col + block * bb, decoded);
                const float* xb = xr + block * be;
                for (uint32_t e = 0; e < be; ++e) sum += xb[e] * decoded[e];
            }
            out[(uint64_t)row * n + column] = sum;
        }
    }
}

void gfo_matmul_quantized(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                          uint64_t k, uint64_t n, float* out) {
    gfo_matmul_quantized_columns(dtype, x, weight, rows, k, n, 0, n, out);
}

void gfo_matmul_quantized_f64(int dtype, const float* x, const uint8_t* weight, uint32_t rows,
                              uint64_t k, uint64_t n, double* out, double* abs_out) {
    const uint32_t be = gfo_block_elements(dtype), bb = gfo_block_bytes(dtype);
    const uint64_t blocks_per_column = k / be;
    float decoded[256];
    for (uint64_t column = 0; column < n; ++column) {
        for (uint32_t row = 0; row < rows; ++row) {
            double sum = 0.0, abs_sum = 0.0;
            for (uint64_t block = 0; block < blocks_per_column; ++block) {
                dequant_block(dtype, weight + (column * blocks_per_column + block) * bb, decoded);
                const float* xb = x + (uint64_t)row * k + block * be;
                for (uint32_t e = 0; e < be; ++e) {
                    const double p = (double)xb[e] * (double)decoded[e];
                    sum += p;
                    abs_sum += fabs(p);
                }
            }
            out[(uint64_t)row * n + column] = sum;
            if (abs_out) abs_out[(uint64_t)row * n + column] = abs_sum;
        }
    }
}

/* ------------------------------------------------------------------ ops */

void gfo_rms_norm(const float* x, const float* gamma, uint32_t rows, uint32_t hidden, float eps,
                  float* out) {
    for (uint32_t r = 0; r < rows; ++r) {
        const float* xr = x + (uint64_t)r * hidden;
        float sum_squares = 0.0f;
        for (uint32_t c = 0; c < hidden; ++c) sum_squares += xr[c] * xr[c];
        const float mean_square = sum_squares / (float)hidden;
        const float inverse_rms = 1.0f / sqrtf(mean_square + eps);
        for (uint32_t c = 0; c < hidden; ++c) out[(uint64_t)r * hidden + c] = xr[c] * inverse_rms * gamma[c];
    }
}

static float gelu_tanh(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

void gfo_gelu_tanh_multiply(const float* gate, const float* up, uint64_t count, float* out) {
    for (uint64_t i = 0; i < count; ++i) out[i] = gelu_tanh(gate[i]) * up[i];
}

void gfo_softcap(const float* x, uint64_t count, float softcap, float* out) {
    for (uint64_t i = 0; i < count; ++i) out[i] = tanhf(x[i] / softcap) * softcap;
}

void gfo_softmax(const float* x, uint32_t rows, uint32_t columns, float* out) {
    for (uint32_t r = 0; r < rows; ++r) {
        const float* xr = x + (uint64_t)r * columns;
        float* o = out + (uint64_t)r * columns;
        float max_value = xr[0];
        for (uint32_t c = 1; c < columns; ++c) max_value = xr[c] > max_value ? xr[c] : max_value;
        double exp_sum = 0.0;
        for (uint32_t c = 0; c < columns; ++c) {
            const double e = exp((double)(xr[c] - max_value));
            exp_sum += e;
            o[c] = (float)e;
        }
        for (uint32_t c = 0; c < columns; ++c) o[c] = (float)((double)o[c] / exp_sum);
    }
}

void gfo_rope_neox(const float* x, const uint32_t* positions, uint32_t rows, uint32_t heads,
                   uint32_t head_dim, float base, float scale, float* out) {
    const uint32_t half = head_dim / 2u;
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t h = 0; h < heads; ++h) {
            const uint64_t o = ((uint64_t)r * heads + h) * head_dim;
            for (uint32_t pair = 0; pair < half; ++pair) {
                const double exponent = (double)(pair * 2u) / (double)head_dim;
                const double angle = (double)positions[r] * (double)scale / pow((double)base, exponent);
                const float c = (float)cos(angle), s = (float)sin(angle);
                const float first = x[o + pair], second = x[o + pair + half];
                out[o + pair] = first * c - second * s;
                out[o + pair + half] = first * s + second * c;
            }
        }
    }
}

void gfo_attention_row(const float* q, const float* keys, const float* values, uint32_t count,
                       uint32_t heads, uint32_t kv_heads, uint32_t head_dim, float scale,
                       float softcap, float* out) {
    const uint32_t group = heads / kv_heads;
    const uint32_t kv_width = kv_heads * head_dim;
    float* scores = (float*)malloc(sizeof(float) * (size_t)count);
    float* probs = (float*)malloc(sizeof(float) * (size_t)count);
    for (uint32_t h = 0; h < heads; ++h) {
        const uint32_t kvh = h / group;
        for (uint32_t t = 0; t < count; ++t) {
            float dot = 0.0f;
            const float* kr = keys + (uint64_t)t * kv_width + kvh * head_dim;
            for (uint32_t c = 0; c < head_dim; ++c) dot += q[h * head_dim + c] * kr[c];
            const float scaled = dot * scale;
            scores[t] = softcap > 0.0f ? tanhf(scaled / softcap) * softcap : scaled;
        }
        gfo_softmax(scores, 1, count, probs);
        for (uint32_t c = 0; c < head_dim; ++c) {
            float sum = 0.0f;
            for (uint32_t t = 0; t < count; ++t)
                sum += probs[t] * values[(uint64_t)t * kv_width + kvh * head_dim + c];
            out[h * head_dim + c] = sum;
        }
    }
    free(scores);
    free(probs);
}

/* ------------------------------------------------------------------ candidates */

static int better(gfo_token_logit a, gfo_token_logit b) {
    if (a.logit != b.logit) return a.logit > b.logit;
    return a.token < b.token;
}

static float transform_logit(float l, float softcap) {
    return softcap == 0.0f ? l : softcap * tanhf(l / softcap);
}

uint32_t gfo_select_candidates(const float* logits, uint32_t vocab, float softcap, uint32_t retain,
                               const uint32_t* history, uint32_t history_count,
                               gfo_token_logit* out) {
    /* Bounded insertion keeps the best `retain` pairs in (logit desc, token asc) order. */
    uint32_t kept = 0;
    for (uint32_t t = 0; t < vocab; ++t) {
        gfo_token_logit c = { t, transform_logit(logits[t], softcap) };
        if (!isfinite(c.logit)) continue;
        if (kept == retain && !better(c, out[kept - 1])) continue;
        uint32_t pos = kept < retain ? kept : retain - 1;
        while (pos > 0 && better(c, out[pos - 1])) { out[pos] = out[pos - 1]; --pos; }
        out[pos] = c;
        if (kept < retain) ++kept;
    }
    for (uint32_t i = kept; i < retain; ++i) { out[i].token = 0xFFFFFFFFu; out[i].logit = -INFINITY; }
    for (uint32_t i = 0; i < history_count; ++i) {
        out[retain + i].token = history[i];
        out[retain + i].logit = transform_logit(logits[history[i]], softcap);
    }
    return retain + history_count;
}

/* ------------------------------------------------------------------ sampling */

static int cmp_candidates(const void* a, const void* b) {
    const gfo_token_logit* l = (const gfo_token_logit*)a;
    const gfo_token_logit* r = (const gfo_token_logit*)b;
    if (better(*l, *r)) return -1;
    if (better(*r, *l)) return 1;
    return 0;
}

int gfo_prepare_distribution(const gfo_token_logit* compact, uint32_t count,
                             const gfo_sampler_options* options, uint32_t request_top_k,
                             const uint32_t* history, uint32_t history_count,
                             gfo_distribution* out) {
    if (count == 0 || count > 384) return -1;
    if (request_top_k == 0 || request_top_k > options->top_k || request_top_k > 256 || history_count > 64)
        return -2;
    gfo_token_logit candidates[384];
    uint32_t n = 0;
    for (uint32_t i = 0; i < count; ++i) {
        if (!isfinite(compact[i].logit)) return -3;
        uint32_t j = 0;
        while (j < n && candidates[j].token != compact[i].token) ++j;
        if (j == n) candidates[n++] = compact[i];
        else if (candidates[j].logit != compact[i].logit) return -4;
    }
    if (n < request_top_k) return -5;
    for (uint32_t i = 0; i < n; ++i) {
        for (uint32_t h = 0; h < history_count; ++h) {
            if (history[h] == candidates[i].token) {
                candidates[i].logit = candidates[i].logit < 0.0f
                    ? candidates[i].logit * options->repetition_penalty
                    : candidates[i].logit / options->repetition_penalty;
                break;
            }
        }
    }
    qsort(candidates, n, sizeof(candidates[0]), cmp_candidates); /* keys are unique: order is total */
    if (n > request_top_k) n = request_top_k;
    memset(out, 0, sizeof(*out));
    if (options->temperature == 0.0f) {
        out->values[0].token = candidates[0].token;
        out->values[0].probability = 1.0;
        out->values[0].weight = 1.0;
        out->count = 1;
        out->total_weight = 1.0;
        return 0;
    }
    double weights[256];
    const float max_logit = candidates[0].logit;
    for (uint32_t i = 0; i < n; ++i) weights[i] = exp((double)(candidates[i].logit - max_logit));
    double total = 0.0;
    for (uint32_t i = 0; i < n; ++i) total += weights[i];
    double retained = 0.0;
    uint32_t retained_count = 0;
    do { retained += weights[retained_count++]; }
    while (retained_count < n && retained / total < (double)options->top_p);
    n = retained_count;
    if (options->min_p > 0.0f) {
        uint32_t m = 1;
        while (m < n && weights[m] >= (double)options->min_p) ++m;
        n = m;
    }
    double normalization = 0.0;
    for (uint32_t i = 0; i < n; ++i) {
        weights[i] = exp((double)(candidates[i].logit - max_logit) / (double)options->temperature);
        normalization += weights[i];
    }
    if (!isfinite(normalization) || normalization <= 0.0) return -6;
    out->count = n;
    out->total_weight = normalization;
    for (uint32_t i = 0; i < n; ++i) {
        out->values[i].token = candidates[i].token;
        out->values[i].probability = weights[i] / normalization;
        out->values[i].weight = weights[i];
    }
    return 0;
}

/* sampling.cpp:117-158: Neumaier sum of the weights, the normaliser both laws divide by. */
static int validated_total(const gfo_distribution* d, double* total_out) {
    if (d->count == 0 || d->count > 256 || !isfinite(d->total_weight) || d->total_weight <= 0.0) return -1;
    double total = 0.0, correction = 0.0;
    for (uint32_t i = 0; i < d->count; ++i) {
        const double w = d->values[i].weight;
        const double sum = total + w;
        correction += total >= w ? (total - sum) + w : (w - sum) + total;
        total = sum;
    }
    total += correction;
    *total_out = total;
    return 0;
}

int gfo_prepare_speculative(uint32_t proposal, uint64_t proposal_mass, const uint64_t* q_mass,
                            const gfo_distribution* target, double* acceptance,
                            gfo_distribution* residual) {
    double normalization;
    if (validated_total(target, &normalization) != 0) return -1;
    if (proposal_mass == 0 || proposal_mass > (1ull << 32)) return -2;
    const double two32 = (double)(1ull << 32);
    const double proposed_probability = (double)proposal_mass / two32;
    memset(residual, 0, sizeof(*residual));
    *acceptance = 0.0;
    for (uint32_t i = 0; i < target->count; ++i) {
        const double probability = target->values[i].weight / normalization;
        if (target->values[i].token == proposal) {
            const double ratio = probability / proposed_probability;
            *acceptance = ratio < 1.0 ? ratio : 1.0;
        }
        const double q = (double)q_mass[i] / two32;
        const double difference = probability - q;
        if (difference <= 0.0) continue;
        residual->values[residual->count].token = target->values[i].token;
        residual->values[residual->count].weight = difference;
        residual->count++;
        residual->total_weight += difference;
    }
    if (residual->count != 0) {
        for (uint32_t i = 0; i < residual->count; ++i)
            residual->values[i].probability = residual->values[i].weight / residual->total_weight;
    } else if (*acceptance < 1.0) {
        return -3;
    }
    return 0;
}

uint32_t gfo_select_prepared(const gfo_distribution* d, double draw) {
    double cumulative = 0.0;
    for (uint32_t i = 0; i < d->count; ++i) {
        cumulative += d->values[i].weight;
        if (draw < cumulative) return d->values[i].token;
    }
    return d->values[d->count - 1].token;
}

int gfo_sample_speculative(uint32_t proposal, double acceptance, const gfo_distribution* residual,
                           double accept_draw, double residual_draw, uint32_t* token,
                           int* accepted) {
    if (!(accept_draw >= 0.0 && accept_draw < 1.0) || !(residual_draw >= 0.0 && residual_draw < 1.0)) return -1;
    if (!isfinite(acceptance) || acceptance < 0.0 || acceptance > 1.0) return -2;
    if (accept_draw < acceptance) { *token = proposal; *accepted = 1; return 0; }
    if (residual->count == 0) return -3;
    *token = gfo_select_prepared(residual, residual_draw * residual->total_weight);
    *accepted = 0;
    return 0;
}

/* ------------------------------------------------------------------ RNG */

void gfo_mt_seed(gfo_mt19937_64* rng, uint64_t seed) {
    rng->mt[0] = seed;
    for (uint32_t i = 1; i < 312; ++i)
        rng->mt[i] = 6364136223846793005ull * (rng->mt[i - 1] ^ (rng->mt[i - 1] >> 62)) + i;
    rng->index = 312;
}

/* std::seed_seq::generate followed by mersenne_twister_engine::seed(Sseq&) for w = 64. */
void gfo_mt_seed_seq(gfo_mt19937_64* rng, const uint32_t* v, uint32_t s) {
    enum { N = 624 };
    uint32_t b[N];
    for (uint32_t i = 0; i < N; ++i) b[i] = 0x8b8b8b8bu;
    const uint32_t n = N, t = 11, p = (n - t) / 2, q = p + t;
    const uint32_t m = s + 1 > n ? s + 1 : n;
    for (uint32_t k = 0; k < m; ++k) {
        const uint32_t arg = b[k % n] ^ b[(k + p) % n] ^ b[(k + n - 1) % n];
        const uint32_t r1 = 1664525u * (arg ^ (arg >> 27));
        uint32_t r2 = r1;
        if (k == 0) r2 += s;
        else if (k <= s) r2 += (k % n) + v[k - 1];
        else r2 += k % n;
        b[(k + p) % n] += r1;
        b[(k + q) % n] += r2;
        b[k % n] = r2;
    }
    for (uint32_t k = m; k < m + n; ++k) {
        const uint32_t arg = b[k % n] + b[(k + p) % n] + b[(k + n - 1) % n];
        const uint32_t r3 = 1566083941u * (arg ^ (arg >> 27));
        const uint32_t r4 = r3 - (k % n);
        b[(k + p) % n] ^= r3;
        b[(k + q) % n] ^= r4;
        b[k % n] = r4;
    }
    int zero = 1;
    for (uint32_t i = 0; i < 312; ++i) {
        rng->mt[i] = (uint64_t)b[2 * i] | ((uint64_t)b[2 * i + 1] << 32);
        if (zero) {
            if (i == 0) { if ((rng->mt[0] & 0xFFFFFFFF80000000ull) != 0) zero = 0; }
            else if (rng->mt[i] != 0) zero = 0;
        }
    }
    if (zero) rng->mt[0] = 1ull << 63;
    rng->index = 312;
}

uint64_t gfo_mt_next(gfo_mt19937_64* rng) {
    if (rng->index >= 312) {
        const uint64_t upper = 0xFFFFFFFF80000000ull, lower = 0x7FFFFFFFull, a = 0xB5026F5AA96619E9ull;
        for (uint32_t i = 0; i < 312; ++i) {
            const uint64_t y = (rng->mt[i] & upper) | (rng->mt[(i + 1) % 312] & lower);
            rng->mt[i] = rng->mt[(i + 156) % 312] ^ (y >> 1) ^ ((y & 1ull) ? a : 0ull);
        }
        rng->index = 0;
    }
    uint64_t z = rng->mt[rng->index++];
    z ^= (z >> 29) & 0x5555555555555555ull;
    z ^= (z << 17) & 0x71D67FFFEDA60000ull;
    z ^= (z << 37) & 0xFFF7EEE000000000ull;
    z ^= z >> 43;
    return z;
}

/* libstdc++ generate_canonical<double, 53> over a 64-bit engine takes one draw:
 * double(draw) / 2^64, clamped below 1; uniform_real maps it to (b - a) * u + a. */
double gfo_uniform_double(gfo_mt19937_64* rng, double a, double b) {
    double u = (double)gfo_mt_next(rng) / 18446744073709551616.0;
    if (u >= 1.0) u = nextafter(1.0, 0.0);
    return (b - a) * u + a;
}

void gfo_make_proposal_rng(const gfo_mt19937_64* target_rng, gfo_mt19937_64* out) {
    gfo_mt19937_64 copy = *target_rng;
    const uint64_t first = gfo_mt_next(&copy), second = gfo_mt_next(&copy);
    const uint32_t words[6] = { 0x4c475350u, 0x524f5031u, (uint32_t)first, (uint32_t)(first >> 32),
                                (uint32_t)second, (uint32_t)(second >> 32) };
    gfo_mt_seed_seq(out, words, 6);
}

uint32_t gfo_next_proposal_word(gfo_mt19937_64* rng) { return (uint32_t)(gfo_mt_next(rng) >> 32); }

/* ------------------------------------------------------------------ drafter law */

void gfo_draft_process_logits(const float* logits, uint32_t vocab, float temperature,
                              float repetition_penalty, const uint32_t* history,
                              uint32_t history_count, float* scores) {
    for (uint32_t i = 0; i < vocab; ++i) scores[i] = logits[i];
    if (repetition_penalty != 1.0f) {
        /* gd_history_mark builds a bitset: each distinct history token is penalised once. */
        uint8_t* seen = (uint8_t*)calloc(vocab, 1);
        for (uint32_t h = 0; h < history_count; ++h) {
            const uint32_t t = history[h];
            if (t < vocab && !seen[t]) {
                seen[t] = 1;
                scores[t] = scores[t] < 0.0f ? scores[t] * repetition_penalty : scores[t] / repetition_penalty;
            }
        }
        free(seen);
    }
    if (temperature > 0.0f)
        for (uint32_t i = 0; i < vocab; ++i) scores[i] = scores[i] / temperature;
}

typedef struct { uint32_t token; float score; } draft_pair;
static int draft_better(draft_pair a, draft_pair b) {
    return a.score > b.score || (a.score == b.score && a.token < b.token);
}
static int cmp_draft(const void* a, const void* b) {
    const draft_pair* l = (const draft_pair*)a; const draft_pair* r = (const draft_pair*)b;
    return draft_better(*l, *r) ? -1 : draft_better(*r, *l) ? 1 : 0;
}
static int cmp_draft_token(const void* a, const void* b) {
    const draft_pair* l = (const draft_pair*)a; const draft_pair* r = (const draft_pair*)b;
    return l->token < r->token ? -1 : l->token > r->token ? 1 : 0;
}

uint32_t gfo_draft_law_compact(const float* scores, uint32_t vocab, uint32_t top_k, float top_p,
                               float min_p, uint32_t* ids, uint64_t* cdf) {
    /* k-th best score under (score desc, token asc); every token tied with it survives. */
    draft_pair* best = (draft_pair*)malloc(sizeof(draft_pair) * top_k);
    uint32_t kept = 0;
    for (uint32_t t = 0; t < vocab; ++t) {
        draft_pair c = { t, scores[t] };
        if (kept == top_k && !draft_better(c, best[kept - 1])) continue;
        uint32_t pos = kept < top_k ? kept : top_k - 1;
        while (pos > 0 && draft_better(c, best[pos - 1])) { best[pos] = best[pos - 1]; --pos; }
        best[pos] = c;
        if (kept < top_k) ++kept;
    }
    const float cutoff = best[kept - 1].score;
    free(best);
    draft_pair values[256];
    uint32_t n = 0;
    for (uint32_t t = 0; t < vocab; ++t) {
        if (scores[t] < cutoff) continue;
        if (n == 256) return 0;
        values[n].token = t; values[n].score = scores[t]; ++n;
    }
    if (n == 0) return 0;
    qsort(values, n, sizeof(values[0]), cmp_draft);
    float weights[256];
    for (uint32_t i = 0; i < n; ++i) weights[i] = expf(values[i].score - values[0].score);
    float total = 0.0f, tail = 0.0f;
    for (uint32_t j = n; j > 0; --j) total += weights[j - 1];
    for (uint32_t j = n; j > 0; --j) {
        const uint32_t i = j - 1;
        tail += weights[i];
        const int keep = i == 0 || ((top_p >= 1.0f || tail / total > 1.0f - top_p)
                                    && (min_p <= 0.0f || weights[i] >= min_p));
        if (!keep) values[i].score = -INFINITY;
    }
    qsort(values, n, sizeof(values[0]), cmp_draft_token);
    float maximum = -INFINITY;
    for (uint32_t i = 0; i < n; ++i) maximum = values[i].score > maximum ? values[i].score : maximum;
    total = 0.0f;
    for (uint32_t i = 0; i < n; ++i) { weights[i] = expf(values[i].score - maximum); total += weights[i]; }
    if (!(total > 0.0f) || !isfinite(total)) return 0;
    float prefix = 0.0f;
    cdf[0] = 0;
    for (uint32_t i = 0; i < n; ++i) {
        ids[i] = values[i].token;
        prefix += weights[i];
        float scaled = (prefix / total) * 4294967296.0f;
        if (scaled < 0.0f) scaled = 0.0f;
        if (scaled > 4294967296.0f) scaled = 4294967296.0f;
        cdf[i + 1] = (uint64_t)scaled;
    }
    return n;
}

/* ---- load-time weight transforms of the Gemma 2 plan (src/engine/gemma2_metal_plan.cpp:301-316,495-512) ----
 * quantize_f16_gguf_weight_q8_0_into (src/tensor/quantization.cpp:634-673): per 32 consecutive F16
 * values d = max|v| / 127 stored as binary16 (the reference's own conversion, which rounds halves up),
 * codes round(v * (1 / d)) with halves away from zero.  Returns -1 on a non-finite value. */
int gfo_quantize_f16_q8_0(const uint16_t* f16, uint64_t block_count, uint8_t* out) {
    for (uint64_t b = 0; b < block_count; ++b) {
        float values[32];
        float amax = 0.0f;
        for (uint32_t e = 0; e < 32; ++e) {
            values[e] = gfo_f16_to_f32(f16[b * 32u + e]);
            if (!isfinite(values[e])) return -1;
            const float a = fabsf(values[e]);
            amax = a > amax ? a : amax;
        }
        const float scale = amax / 127.0f;
        const float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
        const uint16_t bits = gfo_f32_to_f16_half_up(scale);
        uint8_t* o = out + b * 34u;
        o[0] = (uint8_t)(bits & 0xFFu); o[1] = (uint8_t)(bits >> 8);
        for (uint32_t e = 0; e < 32; ++e) o[2 + e] = (uint8_t)(int8_t)roundf(values[e] * inverse);
    }
    return 0;
}

/* nearest_int (quantization.cpp:99-102): the GGML rounding primitive. */
static int q4k_nearest_int(float value) {
    float shifted = value + 12582912.0f;
    uint32_t bits;
    memcpy(&bits, &shifted, 4);
    return (int)(bits & 0x007FFFFFu) - 0x00400000;
}
static int clamp_int(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

/* make_q4_k_group (quantization.cpp:110-188): weighted least-squares scale and minimum of one
 * 32-element group over 21 candidate grids.  Returns the scale; *minimum_magnitude = -minimum. */
static float q4k_make_group(const float* values, const float* weights, float* minimum_magnitude) {
    float minimum = values[0], maximum = values[0], weight_sum = weights[0], weighted_value_sum = weights[0] * values[0];
    for (uint32_t i = 1; i < 32; ++i) {
        minimum = values[i] < minimum ? values[i] : minimum;
        maximum = values[i] > maximum ? values[i] : maximum;
        weight_sum += weights[i];
        weighted_value_sum += weights[i] * values[i];
    }
    minimum = minimum < 0.0f ? minimum : 0.0f;
    if (maximum == minimum) { *minimum_magnitude = -minimum; return 0.0f; }
    float inverse_scale = 15 / (maximum - minimum);
    float scale = 1.0f / inverse_scale;
    float best_error = 0.0f;
    for (uint32_t i = 0; i < 32; ++i) {
        const int level = clamp_int(q4k_nearest_int(inverse_scale * (values[i] - minimum)), 0, 15);
        const float difference = scale * (float)level + minimum - values[i];
        best_error += weights[i] * difference * difference;
    }
    for (int step = 0; step <= 20; ++step) {
        uint8_t candidate[32];
        inverse_scale = (-1.0f + 0.1f * (float)step + 15) / (maximum - minimum);
        float wl = 0.0f, wl2 = 0.0f, wlv = 0.0f;
        for (uint32_t i = 0; i < 32; ++i) {
            const int level = clamp_int(q4k_nearest_int(inverse_scale * (values[i] - minimum)), 0, 15);
            candidate[i] = (uint8_t)level;
            const float weighted_level = weights[i] * (float)level;
            wl += weighted_level;
            wl2 += weighted_level * (float)level;
            wlv += weighted_level * values[i];
        }
        const float determinant = weight_sum * wl2 - wl * wl;
        if (determinant <= 0.0f) continue;
        float candidate_scale = (weight_sum * wlv - weighted_value_sum * wl) / determinant;
        float candidate_minimum = (wl2 * weighted_value_sum - wl * wlv) / determinant;
        if (candidate_minimum > 0.0f) { candidate_minimum = 0.0f; candidate_scale = wlv / wl2; }
        float candidate_error = 0.0f;
        for (uint32_t i = 0; i < 32; ++i) {
            const float difference = candidate_scale * (float)candidate[i] + candidate_minimum - values[i];
            candidate_error += weights[i] * difference * difference;
        }
        if (candidate_error < best_error) { best_error = candidate_error; scale = candidate_scale; minimum = candidate_minimum; }
    }
    *minimum_magnitude = -minimum;
    return scale;
}

/* encode_q4_k_block (quantization.cpp:190-262). */
static void q4k_encode_block(const float* values, uint8_t* out) {
    float scales[8], minima[8], maximum_scale = 0.0f, maximum_minimum = 0.0f;
    for (uint32_t g = 0; g < 8; ++g) {
        const float* v = values + g * 32u;
        float sum_squares = 0.0f;
        for (uint32_t i = 0; i < 32; ++i) sum_squares += v[i] * v[i];
        const float average = sqrtf(sum_squares / 32.0f);
        float weights[32];
        for (uint32_t i = 0; i < 32; ++i) weights[i] = average + fabsf(v[i]);
        scales[g] = q4k_make_group(v, weights, &minima[g]);
        maximum_scale = scales[g] > maximum_scale ? scales[g] : maximum_scale;
        maximum_minimum = minima[g] > maximum_minimum ? minima[g] : maximum_minimum;
    }
    memset(out, 0, 144);
    const float inverse_scale = maximum_scale > 0.0f ? 63.0f / maximum_scale : 0.0f;
    const float inverse_minimum = maximum_minimum > 0.0f ? 63.0f / maximum_minimum : 0.0f;
    uint8_t* packed = out + 4;
    for (uint32_t g = 0; g < 8; ++g) {
        int si = q4k_nearest_int(inverse_scale * scales[g]); si = si < 63 ? si : 63;
        int mi = q4k_nearest_int(inverse_minimum * minima[g]); mi = mi < 63 ? mi : 63;
        const uint8_t sc = (uint8_t)si, mn = (uint8_t)mi;
        if (g < 4u) { packed[g] = sc; packed[g + 4u] = mn; }
        else {
            packed[g + 4u] = (uint8_t)((sc & 0x0Fu) | ((mn & 0x0Fu) << 4));
            packed[g - 4u] |= (uint8_t)((sc >> 4) << 6);
            packed[g] |= (uint8_t)((mn >> 4) << 6);
        }
    }
    const uint16_t scale_bits = gfo_f32_to_f16_half_up(maximum_scale / 63.0f);
    const uint16_t minimum_bits = gfo_f32_to_f16_half_up(maximum_minimum / 63.0f);
    out[0] = (uint8_t)(scale_bits & 0xFFu); out[1] = (uint8_t)(scale_bits >> 8);
    out[2] = (uint8_t)(minimum_bits & 0xFFu); out[3] = (uint8_t)(minimum_bits >> 8);
    const float stored_scale = gfo_f16_to_f32(scale_bits), stored_minimum = gfo_f16_to_f32(minimum_bits);
    uint8_t levels[256];
    memset(levels, 0, sizeof levels);
    for (uint32_t g = 0; g < 8; ++g) {
        const float group_scale = stored_scale * (float)q4k_scale_min(packed, g, 0);
        if (group_scale == 0.0f) continue;
        const float group_minimum = stored_minimum * (float)q4k_scale_min(packed, g, 1);
        for (uint32_t i = 0; i < 32; ++i)
            levels[g * 32u + i] = (uint8_t)clamp_int(q4k_nearest_int((values[g * 32u + i] + group_minimum) / group_scale), 0, 15);
    }
    uint8_t* quantized = out + 16;
    for (uint32_t g = 0; g < 4; ++g)
        for (uint32_t i = 0; i < 32; ++i)
            quantized[g * 32u + i] = (uint8_t)(levels[g * 64u + i] | (levels[g * 64u + i + 32u] << 4));
}

/* requantize_q6_k_gguf_weight_q4_k_into, canonical destination (quantization.cpp:752-800): every Q6_K
 * block decoded as (d * scale_g) * q and re-encoded as Q4_K in place of the same 256 elements.
 * Note the levels of a group whose stored scale is zero stay zero, and that the level search inside
 * make_q4_k_group never reaches the output: the codes are recomputed from the stored scales. */
int gfo_requantize_q6k_q4k(const uint8_t* q6, uint64_t block_count, uint8_t* out) {
    for (uint64_t b = 0; b < block_count; ++b) {
        const uint8_t* block = q6 + b * 210u;
        const uint8_t* ql = block;
        const uint8_t* qh = block + 128;
        const int8_t* sc = (const int8_t*)(block + 192);
        const float d = gfo_f16_to_f32(read_u16(block + 208));
        float values[256];
        for (uint32_t g = 0; g < 16; ++g) {
            const float group_scale = d * (float)sc[g];
            for (uint32_t lane = 0; lane < 16; ++lane) {
                const uint32_t e = g * 16u + lane;
                const uint32_t half = e / 128u, w = e % 128u, l = w % 32u, quarter = w / 32u;
                const uint8_t lowbyte = ql[half * 64u + (quarter % 2u) * 32u + l];
                const uint8_t low = (uint8_t)((lowbyte >> (w < 64u ? 0u : 4u)) & 0x0Fu);
                const uint8_t high = (uint8_t)((qh[half * 32u + l] >> (quarter * 2u)) & 0x03u);
                const int8_t q = (int8_t)((int16_t)(uint8_t)(low | (high << 4)) - 32);
                values[e] = group_scale * (float)q;
                if (!isfinite(values[e])) return -1;
            }
        }
        q4k_encode_block(values, out + b * 144u);
    }
    return 0;
}

/* The full-vocabulary proposal law (src/engine/gemma3_draft.mm:295-395, driven by Impl::sample
 * :995-1167): taken when the compact support would exceed 256 tokens, or when top_k is 0 or above 64,
 * or for a greedy drafter.  `scores` are the processed logits (penalty and temperature applied).
 *   filter (temperature > 0 and any of top_k / top_p / min_p active): all tokens sorted by (score desc,
 *   token asc); walking from the worst to the best in blocks of 256 (the vocabulary padded at the worst
 *   end to a multiple of 256), F32 weights exp(score - best) of the tokens at or above the top_k-th
 *   score are prefix-summed inside each block and the block totals in block order; a token is dropped
 *   when its tail share is <= 1 - top_p or its weight < min_p, the best token excepted.
 *   law: maximum over the survivors (lowest id wins ties), weights exp(score - maximum) prefix-summed in
 *   token-id order in blocks of 256, cdf[i] = u64(clamp(sum_before(i) / total * 2^32)), cdf[vocab] = 2^32.
 * Greedy (temperature == 0): cdf is a step at the argmax.
 * cdf has vocab + 1 entries.  Returns 0, or the reference's status code (6 no finite maximum, 7 bad total). */
typedef struct { uint32_t token; float score; } full_pair;
static int cmp_full(const void* a, const void* b) {
    const full_pair* x = (const full_pair*)a; const full_pair* y = (const full_pair*)b;
    if (x->score > y->score) return -1;
    if (x->score < y->score) return 1;
    return x->token < y->token ? -1 : x->token > y->token ? 1 : 0;
}
uint32_t gfo_draft_law_full(const float* scores_in, uint32_t vocab, float temperature, uint32_t top_k,
                            float top_p, float min_p, uint64_t* cdf) {
    const uint32_t groups = (vocab + 255u) / 256u, padded = groups * 256u;
    float* scores = (float*)malloc(sizeof(float) * vocab);
    float* prefix = (float*)malloc(sizeof(float) * padded);
    float* offsets = (float*)malloc(sizeof(float) * (groups + 1u));
    memcpy(scores, scores_in, sizeof(float) * vocab);
    uint32_t status = 0;
    if (temperature > 0.0f && (top_k != 0 || top_p < 1.0f || min_p > 0.0f)) {
        full_pair* sorted = (full_pair*)malloc(sizeof(full_pair) * vocab);
        for (uint32_t t = 0; t < vocab; ++t) { sorted[t].token = t; sorted[t].score = scores[t]; }
        qsort(sorted, vocab, sizeof(full_pair), cmp_full);
        const float cutoff = top_k ? sorted[(top_k < vocab ? top_k : vocab) - 1u].score : -INFINITY;
        const float best = sorted[0].score;
        /* position i counts from the worst end of the padded order: rank = padded - 1 - i */
        float sum = 0.0f;
        offsets[0] = 0.0f;
        for (uint32_t g = 0; g < groups; ++g) {
            float s = 0.0f;
            for (uint32_t j = 0; j < 256u; ++j) {
                const uint32_t i = g * 256u + j, rank = padded - 1u - i;
                float w = 0.0f;
                if (rank < vocab && sorted[rank].score >= cutoff) w = expf(sorted[rank].score - best);
                s += w;
                prefix[i] = s;
            }
            sum += s;
            offsets[g + 1u] = sum;
        }
        for (uint32_t i = 0; i < padded; ++i) {
            const uint32_t rank = padded - 1u - i;
            if (rank >= vocab) continue;
            int keep = sorted[rank].score >= cutoff;
            const float tail = (offsets[i / 256u] + prefix[i]) / offsets[groups];
            if (top_p < 1.0f && tail <= 1.0f - top_p && rank != 0u) keep = 0;
            if (min_p > 0.0f && expf(sorted[rank].score - best) < min_p && rank != 0u) keep = 0;
            scores[sorted[rank].token] = keep ? sorted[rank].score : -INFINITY;
        }
        free(sorted);
    }
    /* maximum of the survivors, lowest token id on ties */
    float maximum = -INFINITY;
    uint32_t argmax = 0;
    for (uint32_t t = 0; t < vocab; ++t)
        if (scores[t] > maximum) { maximum = scores[t]; argmax = t; }
    if (!isfinite(maximum)) status = 6;
    if (temperature == 0.0f) {
        for (uint32_t i = 0; i <= vocab; ++i) cdf[i] = i <= argmax ? 0ull : 4294967296ull;
    } else {
        float sum = 0.0f;
        offsets[0] = 0.0f;
        for (uint32_t g = 0; g < groups; ++g) {
            float s = 0.0f;
            for (uint32_t j = 0; j < 256u; ++j) {
                const uint32_t i = g * 256u + j;
                const float w = (i < vocab && scores[i] > -INFINITY) ? expf(scores[i] - maximum) : 0.0f;
                s += w;
                prefix[i] = s;
            }
            sum += s;
            offsets[g + 1u] = sum;
        }
        if (!(sum > 0.0f) || !isfinite(sum)) status = status ? status : 7;
        for (uint32_t i = 0; i <= vocab; ++i) {
            if (i == 0) { cdf[i] = 0; continue; }
            if (i == vocab) { cdf[i] = 4294967296ull; continue; }
            const uint32_t b = i / 256u;
            const float before = (i % 256u == 0u) ? offsets[b] : offsets[b] + prefix[i - 1u];
            float scaled = (before / offsets[groups]) * 4294967296.0f;
            if (scaled < 0.0f) scaled = 0.0f;
            if (scaled > 4294967296.0f) scaled = 4294967296.0f;
            cdf[i] = (uint64_t)scaled;
        }
    }
    free(scores); free(prefix); free(offsets);
    return status;
}

/* ------------------------------------------------------------------ whole model */

static int g_threads = 1;
void gfo_set_threads(int threads) { g_threads = threads < 1 ? 1 : threads; }

typedef struct {
    int dtype; const float* x; const uint8_t* w; uint32_t rows; uint64_t k, n, begin, end; float* out;
} gemv_job;
static void* gemv_worker(void* arg) {
    gemv_job* j = (gemv_job*)arg;
    gfo_matmul_quantized_columns(j->dtype, j->x, j->w, j->rows, j->k, j->n, j->begin, j->end, j->out);
    return NULL;
}
static void parallel_matmul(const gfo_tensor* t, const float* x, uint32_t rows, float* out) {
    int threads = g_threads;
    if ((uint64_t)threads > t->n) threads = (int)t->n;
    if (threads <= 1) { gfo_matmul_quantized(t->dtype, x, (const uint8_t*)t->data, rows, t->k, t->n, out); return; }
    pthread_t ids[64];
    gemv_job jobs[64];
    if (threads > 64) threads = 64;
    for (int i = 0; i < threads; ++i) {
        jobs[i] = (gemv_job){ t->dtype, x, (const uint8_t*)t->data, rows, t->k, t->n,
                              t->n * (uint64_t)i / threads, t->n * (uint64_t)(i + 1) / threads, out };
        pthread_create(&ids[i], NULL, gemv_worker, &jobs[i]);
    }
    for (int i = 0; i < threads; ++i) pthread_join(ids[i], NULL);
}

struct gfo_model {
    gfo_model_config c;
    gfo_tensor token_embd, head;
    const float* output_norm;
    gfo_layer* layers;
    uint32_t context, position;
    float** keys;   /* [layer][context * kv_width] */
    float** values;
    float *x, *u, *q, *k, *v, *att, *proj, *gate, *up, *act, *tmp;
};

gfo_model* gfo_model_create(const gfo_model_config* config, const gfo_tensor* token_embd,
                            const float* output_norm, const gfo_tensor* output_head,
                            const gfo_layer* layers, uint32_t context) {
    gfo_model* m = (gfo_model*)calloc(1, sizeof(gfo_model));
    m->c = *config;
    m->token_embd = *token_embd;
    m->head = output_head ? *output_head : *token_embd;
    m->output_norm = output_norm;
    m->layers = (gfo_layer*)malloc(sizeof(gfo_layer) * config->layers);
    memcpy(m->layers, layers, sizeof(gfo_layer) * config->layers);
    m->context = context;
    const size_t kvw = (size_t)config->kv_heads * config->head_dim;
    m->keys = (float**)malloc(sizeof(float*) * config->layers);
    m->values = (float**)malloc(sizeof(float*) * config->layers);
    for (uint32_t l = 0; l < config->layers; ++l) {
        m->keys[l] = (float*)calloc((size_t)context * kvw, sizeof(float));
        m->values[l] = (float*)calloc((size_t)context * kvw, sizeof(float));
    }
    const size_t qw = (size_t)config->heads * config->head_dim;
    m->x = (float*)malloc(4 * config->hidden); m->u = (float*)malloc(4 * config->hidden);
    m->q = (float*)malloc(4 * qw); m->k = (float*)malloc(4 * kvw); m->v = (float*)malloc(4 * kvw);
    m->att = (float*)malloc(4 * qw); m->proj = (float*)malloc(4 * config->hidden);
    m->gate = (float*)malloc(4 * (size_t)config->ffn); m->up = (float*)malloc(4 * (size_t)config->ffn);
    m->act = (float*)malloc(4 * (size_t)config->ffn);
    m->tmp = (float*)malloc(4 * (qw > config->hidden ? qw : config->hidden));
    return m;
}

void gfo_model_destroy(gfo_model* m) {
    if (!m) return;
    for (uint32_t l = 0; l < m->c.layers; ++l) { free(m->keys[l]); free(m->values[l]); }
    free(m->keys); free(m->values); free(m->layers);
    free(m->x); free(m->u); free(m->q); free(m->k); free(m->v); free(m->att); free(m->proj);
    free(m->gate); free(m->up); free(m->act); free(m->tmp);
    free(m);
}

void gfo_model_reset(gfo_model* m) { m->position = 0; }
uint32_t gfo_model_position(const gfo_model* m) { return m->position; }
void gfo_model_truncate(gfo_model* m, uint32_t position) { if (position < m->position) m->position = position; }
const float* gfo_model_key(const gfo_model* m, uint32_t layer, uint32_t position) {
    return m->keys[layer] + (size_t)position * m->c.kv_heads * m->c.head_dim;
}
const float* gfo_model_value(const gfo_model* m, uint32_t layer, uint32_t position) {
    return m->values[layer] + (size_t)position * m->c.kv_heads * m->c.head_dim;
}

/* Overwrites cached rows [first, first + count) of one layer and, with `position`, moves the
 * model's position: lets a test continue from a cache computed elsewhere (a long prefix the
 * scalar path would take hours to build) and check only the rows it appends itself. */
void gfo_model_set_kv(gfo_model* m, uint32_t layer, uint32_t first, uint32_t count, const float* keys, const float* values) {
    const size_t kvw = (size_t)m->c.kv_heads * m->c.head_dim;
    if (layer >= m->c.layers || first + count > m->context) return;
    memcpy(m->keys[layer] + (size_t)first * kvw, keys, (size_t)count * kvw * sizeof(float));
    memcpy(m->values[layer] + (size_t)first * kvw, values, (size_t)count * kvw * sizeof(float));
}
void gfo_model_seek(gfo_model* m, uint32_t position) { if (position <= m->context) m->position = position; }

static int layer_is_local(const gfo_model_config* c, uint32_t layer) {
    if (c->sliding_pattern == 6) return (layer + 1u) % 6u != 0u;
    if (c->sliding_pattern == 2) return layer % 2u == 0u;
    return 0;
}

static void cache_round(const gfo_model_config* c, const float* in, uint32_t n, float* out) {
    for (uint32_t i = 0; i < n; ++i)
        out[i] = c->kv_f16 ? gfo_f16_to_f32(gfo_f32_to_f16_rne(in[i])) : in[i];
}

void gfo_model_append(gfo_model* m, uint32_t token, float* logits, float* final_hidden) {
    const gfo_model_config* c = &m->c;
    const uint32_t H = c->hidden, kvw = c->kv_heads * c->head_dim, p = m->position;
    /* Embedding row times sqrt(hidden) in f32 (model.cpp:599-605). */
    {
        const uint32_t be = gfo_block_elements(m->token_embd.dtype), bb = gfo_block_bytes(m->token_embd.dtype);
        const uint8_t* row = (const uint8_t*)m->token_embd.data + (uint64_t)token * (H / be) * bb;
        gfo_dequantize(m->token_embd.dtype, row, H / be, m->x);
        const float scale = sqrtf((float)H);
        for (uint32_t i = 0; i < H; ++i) m->x[i] *= scale;
    }
    for (uint32_t l = 0; l < c->layers; ++l) {
        const gfo_layer* L = &m->layers[l];
        const int local = layer_is_local(c, l);
        const float base = local ? c->rope_base_local : c->rope_base_global;
        const float fscale = local ? c->rope_scale_local : c->rope_scale_global;
        gfo_rms_norm(m->x, L->attn_norm, 1, H, c->rms_eps, m->u);
        parallel_matmul(&L->attn_q, m->u, 1, m->q);
        parallel_matmul(&L->attn_k, m->u, 1, m->k);
        parallel_matmul(&L->attn_v, m->u, 1, m->v);
        if (c->uses_qk_norm) {
            gfo_rms_norm(m->q, L->q_norm, c->heads, c->head_dim, c->rms_eps, m->q);
            gfo_rms_norm(m->k, L->k_norm, c->kv_heads, c->head_dim, c->rms_eps, m->k);
        }
        gfo_rope_neox(m->q, &p, 1, c->heads, c->head_dim, base, fscale, m->tmp);
        memcpy(m->q, m->tmp, 4 * (size_t)c->heads * c->head_dim);
        gfo_rope_neox(m->k, &p, 1, c->kv_heads, c->head_dim, base, fscale, m->tmp);
        cache_round(c, m->tmp, kvw, m->keys[l] + (size_t)p * kvw);
        cache_round(c, m->v, kvw, m->values[l] + (size_t)p * kvw);
        const uint32_t first = local && p + 1u > c->sliding_window ? p + 1u - c->sliding_window : 0u;
        gfo_attention_row(m->q, m->keys[l] + (size_t)first * kvw, m->values[l] + (size_t)first * kvw,
                          p - first + 1u, c->heads, c->kv_heads, c->head_dim, c->attention_scale,
                          c->attn_softcap, m->att);
        parallel_matmul(&L->attn_output, m->att, 1, m->proj);
        gfo_rms_norm(m->proj, L->post_attention_norm, 1, H, c->rms_eps, m->proj);
        for (uint32_t i = 0; i < H; ++i) m->x[i] = m->x[i] + m->proj[i];
        gfo_rms_norm(m->x, L->ffn_norm, 1, H, c->rms_eps, m->u);
        parallel_matmul(&L->ffn_gate, m->u, 1, m->gate);
        parallel_matmul(&L->ffn_up, m->u, 1, m->up);
        gfo_gelu_tanh_multiply(m->gate, m->up, c->ffn, m->act);
        parallel_matmul(&L->ffn_down, m->act, 1, m->proj);
        gfo_rms_norm(m->proj, L->post_ffw_norm, 1, H, c->rms_eps, m->proj);
        for (uint32_t i = 0; i < H; ++i) m->x[i] = m->x[i] + m->proj[i];
    }
    m->position = p + 1u;
    if (!logits && !final_hidden) return;
    gfo_rms_norm(m->x, m->output_norm, 1, H, c->rms_eps, m->u);
    if (final_hidden) memcpy(final_hidden, m->u, 4 * (size_t)H);
    if (logits) parallel_matmul(&m->head, m->u, 1, logits);
}
