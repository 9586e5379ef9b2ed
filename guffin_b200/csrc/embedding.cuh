// Embedding gather from the streaming layout, as device functions shared by the embedding kernel
// and the embedding phase of the decode pass kernel.
#pragma once

#include "ops.cuh"

namespace gf {

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

// Elements [first, rows * k) in steps of `stride` of the embedded rows: row = token's column of the
// packed [K, vocab] matrix, dequantised and scaled.  A token id >= vocab sets status bit 1 and yields
// NaN for that row (metal_kernels.mm:461).
__device__ __forceinline__ void embedding_rows(int dtype, const uint8_t* __restrict__ packed, uint32_t k, uint32_t vocab,
                                               const uint32_t* __restrict__ tokens, uint32_t rows, float scale,
                                               float* __restrict__ out, uint32_t* status, uint32_t first, uint32_t stride) {
    const uint32_t units = dtype == GF_F16 ? 0u : k / unit_elements(dtype);
    for (uint32_t i = first; i < rows * k; i += stride) {
        const uint32_t row = i / k, e = i % k;
        const uint32_t token = tokens[row];
        if (token >= vocab) {
            if (e == 0) atomicOr(status, kStatusBadToken);
            out[i] = __int_as_float(0x7fc00000);
            continue;
        }
        if (dtype == GF_F16) {      // a binary16 table as stored, [vocab][k] (the retained Gemma 2 9B embedding)
            const unsigned short bits = reinterpret_cast<const unsigned short*>(packed)[(size_t)token * k + e];
            out[i] = __fmul_rn(__half2float(__ushort_as_half(bits)), scale);
            continue;
        }
        out[i] = __fmul_rn(packed_element(dtype, packed, units, token, e), scale);
    }
}

}  // namespace gf
