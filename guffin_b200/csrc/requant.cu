// Load-time weight transforms of the Gemma 2 plan (src/engine/gemma2_metal_plan.cpp:301-316,495-512):
//   F16 -> Q8_0   quantize_f16_gguf_weight_q8_0_into        (src/tensor/quantization.cpp:634-673)
//   Q6_K -> Q4_K  requantize_q6_k_gguf_weight_q4_k_into     (src/tensor/quantization.cpp:752-800,
//                 encode_q4_k_block :190-262, make_q4_k_group :110-188)
// on the device, block for block bit-identical to those functions built without floating-point
// contraction: every product, sum, quotient and square root below is a single correctly rounded F32
// operation in the reference's order (the intrinsics keep the compiler from fusing them), and the
// sums that the reference forms sequentially are formed sequentially by one thread.
#include "ops.cuh"

namespace gf {

namespace {

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float quo(float a, float b) { return __fdiv_rn(a, b); }

__device__ __forceinline__ float half_bits_to_float(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// f32_to_f16_bits of the reference (src/tensor/f16.cpp:39-82): halves round up in magnitude, subnormals
// are formed by a rounded shift, anything at or beyond the binary16 range becomes infinity.
__device__ __forceinline__ uint32_t float_to_half_bits_half_up(float value) {
    const uint32_t bits = __float_as_uint(value);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    int exponent = (int)((bits >> 23) & 0xFFu);
    uint32_t fraction = bits & 0x7FFFFFu;
    if (exponent == 0xFF) return sign | (fraction == 0u ? 0x7C00u : 0x7E00u);
    exponent = exponent - 127 + 15;
    if (exponent >= 0x1F) return sign | 0x7C00u;
    if (exponent <= 0) {
        if (exponent < -10) return sign;
        fraction |= 0x800000u;
        const uint32_t shift = (uint32_t)(14 - exponent);
        return sign | (((fraction + (1u << (shift - 1u))) >> shift) & 0xFFFFu);
    }
    fraction += 0x00001000u;
    if (fraction & 0x00800000u) {
        fraction = 0u;
        ++exponent;
        if (exponent >= 0x1F) return sign | 0x7C00u;
    }
    return sign | ((uint32_t)exponent << 10) | (fraction >> 13);
}

// nearest_int (quantization.cpp:99-102).
__device__ __forceinline__ int nearest_int(float value) {
    return (int)(__float_as_uint(add(value, 12582912.0f)) & 0x007FFFFFu) - 0x00400000;
}
__device__ __forceinline__ int clamp_level(int v) { return min(max(v, 0), 15); }

}  // namespace

// One warp per 32-element block: lane e owns element e.
__global__ void __launch_bounds__(256) quantize_f16_q8_0_kernel(const unsigned short* __restrict__ f16, uint64_t block_count,
                                                                uint8_t* __restrict__ out, uint32_t* status) {
    const uint64_t block = (uint64_t)blockIdx.x * 8u + threadIdx.x / 32u;
    if (block >= block_count) return;
    const uint32_t lane = threadIdx.x & 31u;
    const float value = half_bits_to_float(f16[block * 32u + lane]);
    if (!isfinite(value) && status) atomicOr(status, 1u);
    float amax = fabsf(value);
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    const float scale = quo(amax, 127.0f);
    const float inverse = scale == 0.0f ? 0.0f : quo(1.0f, scale);
    uint8_t* o = out + block * 34u;
    if (lane == 0) {
        const uint32_t bits = float_to_half_bits_half_up(scale);
        o[0] = (uint8_t)(bits & 0xFFu);
        o[1] = (uint8_t)(bits >> 8);
    }
    o[2u + lane] = (uint8_t)(int8_t)(int)roundf(mul(value, inverse));
}

// Eight threads per 256-element block, one per 32-element group; 32 blocks per CTA.
__global__ void __launch_bounds__(256) requantize_q6k_q4k_kernel(const uint8_t* __restrict__ q6, uint64_t block_count,
                                                                 uint8_t* __restrict__ out, uint32_t* status) {
    const uint64_t block = (uint64_t)blockIdx.x * 32u + threadIdx.x / 8u;
    const uint32_t group = threadIdx.x & 7u;
    const bool live = block < block_count;
    const uint8_t* src = q6 + (live ? block : 0) * 210u;
    // Elements 32g .. 32g+31 of the block: two Q6_K scale groups of sixteen.
    float values[32];
    {
        const float d = half_bits_to_float((uint32_t)src[208] | ((uint32_t)src[209] << 8));
#pragma unroll
        for (uint32_t half_group = 0; half_group < 2u; ++half_group) {
            const float group_scale = mul(d, (float)(int)(signed char)src[192u + group * 2u + half_group]);
#pragma unroll
            for (uint32_t lane = 0; lane < 16u; ++lane) {
                const uint32_t e = group * 32u + half_group * 16u + lane;
                const uint32_t half = e / 128u, w = e % 128u, l = w % 32u, quarter = w / 32u;
                const uint32_t lowbyte = src[half * 64u + (quarter % 2u) * 32u + l];
                const uint32_t low = w < 64u ? (lowbyte & 15u) : (lowbyte >> 4);
                const uint32_t high = ((uint32_t)src[128u + half * 32u + l] >> (quarter * 2u)) & 3u;
                const float value = mul(group_scale, (float)((int)(low | (high << 4)) - 32));
                if (!isfinite(value) && live && status) atomicOr(status, 1u);
                values[half_group * 16u + lane] = value;
            }
        }
    }
    // make_q4_k_group: the group's scale and minimum by weighted least squares over 21 grids.
    float scale = 0.0f, minimum_magnitude = 0.0f;
    {
        float sum_squares = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) sum_squares = add(sum_squares, mul(values[i], values[i]));
        const float average = __fsqrt_rn(quo(sum_squares, 32.0f));
        auto weight = [&](int i) { return add(average, fabsf(values[i])); };
        float minimum = values[0], maximum = values[0], weight_sum = weight(0), weighted_value_sum = mul(weight(0), values[0]);
#pragma unroll
        for (int i = 1; i < 32; ++i) {
            minimum = fminf(minimum, values[i]);
            maximum = fmaxf(maximum, values[i]);
            weight_sum = add(weight_sum, weight(i));
            weighted_value_sum = add(weighted_value_sum, mul(weight(i), values[i]));
        }
        minimum = fminf(minimum, 0.0f);
        if (maximum != minimum) {
            float inverse_scale = quo(15.0f, sub(maximum, minimum));
            scale = quo(1.0f, inverse_scale);
            float best_error = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int level = clamp_level(nearest_int(mul(inverse_scale, sub(values[i], minimum))));
                const float difference = sub(add(mul(scale, (float)level), minimum), values[i]);
                best_error = add(best_error, mul(mul(weight(i), difference), difference));
            }
            for (int step = 0; step <= 20; ++step) {
                // `minimum` is the running best: a grid is laid from the minimum the last improvement left.
                inverse_scale = quo(add(add(-1.0f, mul(0.1f, (float)step)), 15.0f), sub(maximum, minimum));
                float wl = 0.0f, wl2 = 0.0f, wlv = 0.0f;
                uint32_t packed_levels[4] = {0u, 0u, 0u, 0u};          // 32 candidate levels, four bits each
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int level = clamp_level(nearest_int(mul(inverse_scale, sub(values[i], minimum))));
                    packed_levels[i >> 3] |= (uint32_t)level << ((i & 7) * 4);
                    const float weighted_level = mul(weight(i), (float)level);
                    wl = add(wl, weighted_level);
                    wl2 = add(wl2, mul(weighted_level, (float)level));
                    wlv = add(wlv, mul(weighted_level, values[i]));
                }
                const float determinant = sub(mul(weight_sum, wl2), mul(wl, wl));
                if (determinant <= 0.0f) continue;
                float candidate_scale = quo(sub(mul(weight_sum, wlv), mul(weighted_value_sum, wl)), determinant);
                float candidate_minimum = quo(sub(mul(wl2, weighted_value_sum), mul(wl, wlv)), determinant);
                if (candidate_minimum > 0.0f) { candidate_minimum = 0.0f; candidate_scale = quo(wlv, wl2); }
                float candidate_error = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float level = (float)((packed_levels[i >> 3] >> ((i & 7) * 4)) & 15u);
                    const float difference = sub(add(mul(candidate_scale, level), candidate_minimum), values[i]);
                    candidate_error = add(candidate_error, mul(mul(weight(i), difference), difference));
                }
                if (candidate_error < best_error) { best_error = candidate_error; scale = candidate_scale; minimum = candidate_minimum; }
            }
        }
        minimum_magnitude = -minimum;
    }
    // encode_q4_k_block: six-bit scales and minima against the block's largest, then the codes from the
    // values the block will decode with.
    float maximum_scale = scale, maximum_minimum = minimum_magnitude;
#pragma unroll
    for (int offset = 4; offset; offset >>= 1) {
        maximum_scale = fmaxf(maximum_scale, __shfl_xor_sync(0xffffffffu, maximum_scale, offset));
        maximum_minimum = fmaxf(maximum_minimum, __shfl_xor_sync(0xffffffffu, maximum_minimum, offset));
    }
    maximum_scale = fmaxf(maximum_scale, 0.0f);             // the reference's running maxima start at zero
    maximum_minimum = fmaxf(maximum_minimum, 0.0f);
    const float inverse_scale = maximum_scale > 0.0f ? quo(63.0f, maximum_scale) : 0.0f;
    const float inverse_minimum = maximum_minimum > 0.0f ? quo(63.0f, maximum_minimum) : 0.0f;
    const uint32_t sc = (uint32_t)min(63, nearest_int(mul(inverse_scale, scale))) & 0xFFu;
    const uint32_t mn = (uint32_t)min(63, nearest_int(mul(inverse_minimum, minimum_magnitude))) & 0xFFu;
    const uint32_t scale_bits = float_to_half_bits_half_up(quo(maximum_scale, 63.0f));
    const uint32_t minimum_bits = float_to_half_bits_half_up(quo(maximum_minimum, 63.0f));
    uint8_t* dst = out + (live ? block : 0) * 144u;
    {   // the twelve scale / minimum bytes: thread g reads its neighbours' six-bit values
        const uint32_t lane_base = (threadIdx.x & 31u) & ~7u;
        uint32_t all_sc[8], all_mn[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            all_sc[g] = __shfl_sync(0xffffffffu, sc, lane_base + g);
            all_mn[g] = __shfl_sync(0xffffffffu, mn, lane_base + g);
        }
        if (group == 0 && live) {
            uint8_t packed[12];
#pragma unroll
            for (int g = 0; g < 4; ++g) { packed[g] = (uint8_t)all_sc[g]; packed[g + 4] = (uint8_t)all_mn[g]; }
#pragma unroll
            for (int g = 4; g < 8; ++g) {
                packed[g + 4] = (uint8_t)((all_sc[g] & 0x0Fu) | ((all_mn[g] & 0x0Fu) << 4));
                packed[g - 4] |= (uint8_t)((all_sc[g] >> 4) << 6);
                packed[g] |= (uint8_t)((all_mn[g] >> 4) << 6);
            }
            dst[0] = (uint8_t)(scale_bits & 0xFFu); dst[1] = (uint8_t)(scale_bits >> 8);
            dst[2] = (uint8_t)(minimum_bits & 0xFFu); dst[3] = (uint8_t)(minimum_bits >> 8);
#pragma unroll
            for (int i = 0; i < 12; ++i) dst[4 + i] = packed[i];
        }
    }
    const float group_scale = mul(half_bits_to_float(scale_bits), (float)(sc & 63u));
    const float group_minimum = mul(half_bits_to_float(minimum_bits), (float)(mn & 63u));
    // Code byte 32c + i holds group 2c's level i in its low nibble and group 2c+1's in its high nibble.
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        uint32_t level = 0u;
        if (group_scale != 0.0f) level = (uint32_t)clamp_level(nearest_int(quo(add(values[i], group_minimum), group_scale)));
        const uint32_t partner = __shfl_xor_sync(0xffffffffu, level, 1);
        if ((group & 1u) == 0u && live) dst[16u + (group >> 1) * 32u + i] = (uint8_t)(level | (partner << 4));
    }
}

int launch_quantize_f16_q8_0(const void* f16_dev, uint64_t block_count, void* q8_dev, uint32_t* status_dev, cudaStream_t stream) {
    if (!f16_dev || !q8_dev) return fail(GF_ERR_INVALID, "F16 -> Q8_0: null buffer");
    if (block_count == 0) return GF_OK;
    if (block_count > 0x7fffffffull * 8ull) return fail(GF_ERR_INVALID, "F16 -> Q8_0: too many blocks for one launch");
    return launch_kernel(quantize_f16_q8_0_kernel, dim3((unsigned)((block_count + 7u) / 8u)), dim3(256), 0, stream, false,
                         static_cast<const unsigned short*>(f16_dev), block_count, static_cast<uint8_t*>(q8_dev), status_dev);
}

int launch_requantize_q6k_q4k(const void* q6_dev, uint64_t block_count, void* q4_dev, uint32_t* status_dev, cudaStream_t stream) {
    if (!q6_dev || !q4_dev) return fail(GF_ERR_INVALID, "Q6_K -> Q4_K: null buffer");
    if (block_count == 0) return GF_OK;
    if (block_count > 0x7fffffffull * 32ull) return fail(GF_ERR_INVALID, "Q6_K -> Q4_K: too many blocks for one launch");
    return launch_kernel(requantize_q6k_q4k_kernel, dim3((unsigned)((block_count + 31u) / 32u)), dim3(256), 0, stream, false,
                         static_cast<const uint8_t*>(q6_dev), block_count, static_cast<uint8_t*>(q4_dev), status_dev);
}

}  // namespace gf

using namespace gf;

extern "C" {

int gf_quantize_f16_q8_0(const void* f16_dev, uint64_t block_count, void* q8_0_dev, uint32_t* status_dev, void* stream) {
    return launch_quantize_f16_q8_0(f16_dev, block_count, q8_0_dev, status_dev, as_stream(stream));
}

int gf_requantize_q6_k_q4_k(const void* q6_k_dev, uint64_t block_count, void* q4_k_dev, uint32_t* status_dev, void* stream) {
    return launch_requantize_q6k_q4k(q6_k_dev, block_count, q4_k_dev, status_dev, as_stream(stream));
}

}  // extern "C"
