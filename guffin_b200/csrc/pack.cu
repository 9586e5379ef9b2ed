// Weight preparation and bit-exact dequantisation.
//
// Streaming layout ("pair rows"): for column pair cp = n/16 and K unit u the group
// [(cp * units + u) * pair_row_bytes, +pair_row_bytes) holds the native bytes of the sixteen
// columns' blocks for that unit, permuted (16-bit words only) into the order the GEMV's lanes
// consume them; packed_offset() in common.cuh is the map.  Nothing is re-quantised:
// gf_unpack_weight restores the native payload byte for byte.  Columns beyond N inside the last
// group are zero bytes.
#include "common.cuh"

namespace gf {

struct PackGeometry {
    int dtype;
    uint64_t units;        // K units per column
    uint64_t columns;      // N
    uint64_t pairs;        // ceil(N / 16)
    uint32_t unit_native;  // native bytes of one column's unit
    uint32_t pair_row;     // packed bytes of sixteen columns' unit
};

// One thread per native 16-bit word of the (zero-extended) sixteen-column groups.
template <bool kPack>
__global__ void __launch_bounds__(256) repack_kernel(PackGeometry g, const uint16_t* __restrict__ src,
                                                     uint16_t* __restrict__ dst) {
    const uint64_t words_per_unit = g.unit_native / 2u;
    const uint64_t total = g.pairs * g.units * 16u * words_per_unit;
    for (uint64_t w = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; w < total;
         w += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t word = (uint32_t)(w % words_per_unit);
        const uint64_t rest = w / words_per_unit;
        const uint32_t c16 = (uint32_t)(rest % 16u);
        const uint64_t row = rest / 16u;                     // (cp, u)
        const uint64_t cp = row / g.units, u = row % g.units;
        const uint64_t column = cp * 16u + c16;
        const uint64_t packed_word = (row * g.pair_row + packed_offset(g.dtype, c16, word * 2u)) / 2u;
        const uint64_t native_word = (column * g.units + u) * words_per_unit + word;
        if (kPack) dst[packed_word] = column < g.columns ? src[native_word] : (uint16_t)0;
        else if (column < g.columns) dst[native_word] = src[packed_word];
    }
}

__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

// Bit-exact restatement of BlockView::dequantized_value: every product and the Q4_K
// subtraction round separately (no fused multiply-add).
__global__ void __launch_bounds__(256) dequantize_kernel(int dtype, const uint8_t* __restrict__ blocks,
                                                         uint64_t elements, float* __restrict__ out) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < elements;
         i += (uint64_t)gridDim.x * blockDim.x) {
        if (dtype == GF_Q8_0) {
            const uint8_t* b = blocks + (i / 32u) * 34u;
            const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
            out[i] = __fmul_rn(d, (float)(int8_t)b[2u + i % 32u]);
        } else if (dtype == GF_Q4_K) {
            const uint8_t* b = blocks + (i / 256u) * 144u;
            const uint32_t e = (uint32_t)(i % 256u), group = e / 32u, in64 = e % 64u;
            const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
            const float dmin = half_bits_to_float((uint16_t)(b[2] | (b[3] << 8)));
            const uint8_t* s = b + 4;
            uint32_t sc, mn;
            if (group < 4u) { sc = s[group] & 63u; mn = s[group + 4u] & 63u; }
            else {
                sc = (s[group + 4u] & 15u) | ((s[group - 4u] >> 6) << 4);
                mn = (s[group + 4u] >> 4) | ((s[group] >> 6) << 4);
            }
            const uint32_t byte = b[16u + (e / 64u) * 32u + in64 % 32u];
            const uint32_t q = in64 < 32u ? (byte & 15u) : (byte >> 4);
            out[i] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
        } else {
            const uint8_t* b = blocks + (i / 256u) * 210u;
            const uint32_t e = (uint32_t)(i % 256u), half = e / 128u, w = e % 128u, lane = w % 32u, quarter = w / 32u;
            const uint32_t lowbyte = b[half * 64u + (quarter % 2u) * 32u + lane];
            const uint32_t low = w < 64u ? (lowbyte & 15u) : (lowbyte >> 4);
            const uint32_t high = (b[128u + half * 32u + lane] >> (quarter * 2u)) & 3u;
            const int q = (int)(low | (high << 4)) - 32;
            const float d = half_bits_to_float((uint16_t)(b[208] | (b[209] << 8)));
            out[i] = __fmul_rn(__fmul_rn(d, (float)(int8_t)b[192u + e / 16u]), (float)q);
        }
    }
}

static int geometry(int dtype, uint64_t k, uint64_t n, PackGeometry& g) {
    if (dtype != GF_Q8_0 && dtype != GF_Q4_K && dtype != GF_Q6_K)
        return fail(GF_ERR_INVALID, "unsupported weight dtype %d", dtype);
    const uint32_t unit = unit_elements(dtype);
    if (k == 0 || n == 0 || k % unit != 0)
        return fail(GF_ERR_INVALID, "weight K=%llu must be a positive multiple of %u (N=%llu)",
                    (unsigned long long)k, unit, (unsigned long long)n);
    g.dtype = dtype;
    g.units = k / unit;
    g.columns = n;
    g.pairs = (n + 15u) / 16u;
    g.unit_native = unit_native_bytes(dtype);
    g.pair_row = pair_row_bytes(dtype);
    return GF_OK;
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_packed_weight_bytes(int dtype, uint64_t k, uint64_t n) {
    PackGeometry g;
    if (geometry(dtype, k, n, g) != GF_OK) return 0;
    return (size_t)(g.pairs * g.units * g.pair_row);
}

int gf_pack_weight(int dtype, const void* native_dev, uint64_t k, uint64_t n, void* packed_dev, void* stream) {
    PackGeometry g;
    const int status = geometry(dtype, k, n, g);
    if (status != GF_OK) return status;
    if (!native_dev || !packed_dev) return fail(GF_ERR_INVALID, "gf_pack_weight: null buffer");
    const int blocks = sm_count() * 8;
    repack_kernel<true><<<blocks, 256, 0, as_stream(stream)>>>(
        g, static_cast<const uint16_t*>(native_dev), static_cast<uint16_t*>(packed_dev));
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int gf_unpack_weight(int dtype, const void* packed_dev, uint64_t k, uint64_t n, void* native_dev, void* stream) {
    PackGeometry g;
    const int status = geometry(dtype, k, n, g);
    if (status != GF_OK) return status;
    if (!native_dev || !packed_dev) return fail(GF_ERR_INVALID, "gf_unpack_weight: null buffer");
    const int blocks = sm_count() * 8;
    repack_kernel<false><<<blocks, 256, 0, as_stream(stream)>>>(
        g, static_cast<const uint16_t*>(packed_dev), static_cast<uint16_t*>(native_dev));
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

int gf_dequantize(int dtype, const void* native_dev, uint64_t block_count, float* out_dev, void* stream) {
    if (dtype != GF_Q8_0 && dtype != GF_Q4_K && dtype != GF_Q6_K)
        return fail(GF_ERR_INVALID, "unsupported dtype %d", dtype);
    if (block_count == 0) return GF_OK;
    if (!native_dev || !out_dev) return fail(GF_ERR_INVALID, "gf_dequantize: null buffer");
    const uint64_t elements = block_count * block_elements(dtype);
    const int blocks = (int)((elements + 255u) / 256u < (uint64_t)sm_count() * 16u ? (elements + 255u) / 256u
                                                                                   : (uint64_t)sm_count() * 16u);
    dequantize_kernel<<<blocks, 256, 0, as_stream(stream)>>>(
        dtype, static_cast<const uint8_t*>(native_dev), elements, out_dev);
    GF_CUDA(cudaGetLastError());
    return GF_OK;
}

}  // extern "C"
