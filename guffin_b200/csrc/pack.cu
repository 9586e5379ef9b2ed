// Weight preparation and bit-exact dequantisation.
//
// Streaming layout ("columns8 units"): for column tile ct = n/8 and K unit u the group
// [(ct * units + u) * unit_row_bytes, +unit_row_bytes) holds the native bytes of the eight
// columns' blocks for that unit, split into planes so that a warp reads each plane with
// conflict-free aligned shared-memory loads after one contiguous bulk copy:
//   Q4_K (1152 B): qs[8][128] | header[8][16]  (header = d, dmin, 12 scale/min bytes)
//   Q6_K (1680 B): ql[8][128] | qh[8][64] | scales[8][16] | d[8][2]
//   Q8_0 (1088 B): q[8][4][32] | d[8][4][2]     (unit = four 32-element blocks)
// Nothing is re-quantised: gf_unpack_weight restores the native payload byte for byte.
#include "common.cuh"

namespace gf {

struct PackGeometry {
    int dtype;
    uint64_t units;        // K units per column
    uint64_t columns;      // N
    uint64_t tiles;        // ceil(N / 8)
    uint32_t unit_native;  // native bytes of one column's unit
    uint32_t unit_row;     // packed bytes of eight columns' unit
};

// Maps a byte offset inside a packed unit row to (column-in-tile, byte offset in that
// column's native unit).
__host__ __device__ inline void packed_offset_to_native(int dtype, uint32_t off, uint32_t& c, uint32_t& native) {
    if (dtype == GF_Q4_K) {
        if (off < 1024u) { c = off / 128u; native = 16u + off % 128u; }
        else { const uint32_t o = off - 1024u; c = o / 16u; native = o % 16u; }
    } else if (dtype == GF_Q6_K) {
        if (off < 1024u) { c = off / 128u; native = off % 128u; }
        else if (off < 1536u) { const uint32_t o = off - 1024u; c = o / 64u; native = 128u + o % 64u; }
        else if (off < 1664u) { const uint32_t o = off - 1536u; c = o / 16u; native = 192u + o % 16u; }
        else { const uint32_t o = off - 1664u; c = o / 2u; native = 208u + o % 2u; }
    } else {
        if (off < 1024u) { c = off / 128u; const uint32_t r = off % 128u; native = (r / 32u) * 34u + 2u + r % 32u; }
        else { const uint32_t o = off - 1024u; c = o / 8u; const uint32_t r = o % 8u; native = (r / 2u) * 34u + r % 2u; }
    }
}

// One thread per packed 16-bit word (every plane boundary and native field is 2-byte aligned).
template <bool kPack>
__global__ void __launch_bounds__(256) repack_kernel(PackGeometry g, const uint16_t* __restrict__ src,
                                                     uint16_t* __restrict__ dst) {
    const uint64_t words_per_row = g.unit_row / 2u;
    const uint64_t total = g.tiles * g.units * words_per_row;
    for (uint64_t w = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; w < total;
         w += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = w / words_per_row;             // (ct, u)
        const uint32_t off = (uint32_t)(w % words_per_row) * 2u;
        const uint64_t ct = row / g.units, u = row % g.units;
        uint32_t c, native;
        packed_offset_to_native(g.dtype, off, c, native);
        const uint64_t column = ct * 8u + c;
        const uint64_t native_word = ((column * g.units + u) * g.unit_native + native) / 2u;
        if (kPack) dst[w] = column < g.columns ? src[native_word] : (uint16_t)0;
        else if (column < g.columns) dst[native_word] = src[w];
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
    g.tiles = (n + 7u) / 8u;
    g.unit_native = unit / block_elements(dtype) * block_bytes(dtype);
    g.unit_row = unit_row_bytes(dtype);
    return GF_OK;
}

}  // namespace gf

using namespace gf;

extern "C" {

size_t gf_packed_weight_bytes(int dtype, uint64_t k, uint64_t n) {
    PackGeometry g;
    if (geometry(dtype, k, n, g) != GF_OK) return 0;
    return (size_t)(g.tiles * g.units * g.unit_row);
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
