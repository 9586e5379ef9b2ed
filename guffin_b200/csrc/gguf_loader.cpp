// GGUF v2/v3 tensor loader: binds the tensors of a checkpoint file to a resident plan.
//
// Takes the place of the reference's file-backed reader plus weight materialiser for this path
// (read_file_backed_gguf_model, include/local_gguf_engine/model_format/gguf_reader.hpp:85;
// WeightMaterializer, src/engine/gemma2_metal_plan.cpp:266-336): the file is mapped read-only,
// the metadata section is skipped value by value (only general.alignment is read), and every
// tensor whose name the Gemma block schedule knows is handed, as its native payload, to
// gf_model_set_matrix / gf_model_set_vector, which upload and repack on the device.  Tensor
// names are llama.cpp's: token_embd, output, output_norm, blk.<layer>.{attn_q, attn_k, attn_v,
// attn_output, ffn_gate, ffn_up, ffn_down, attn_norm, post_attention_norm, ffn_norm,
// post_ffw_norm, attn_q_norm, attn_k_norm}, each followed by ".weight".  Other tensors are
// ignored.  The model geometry comes from the caller's gf_model_config.
#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

namespace gf {
namespace {

struct Mapping {
    const uint8_t* data = nullptr;
    size_t size = 0;
    int fd = -1;
    ~Mapping() {
        if (data) munmap(const_cast<uint8_t*>(data), size);
        if (fd >= 0) close(fd);
    }
};

// Bounds-checked little-endian cursor over the mapped file.
struct Cursor {
    const uint8_t* data;
    size_t size, at = 0;
    bool ok = true;
    template <typename T> T read() {
        T value{};
        if (!ok || size - at < sizeof(T)) { ok = false; return value; }
        std::memcpy(&value, data + at, sizeof(T));
        at += sizeof(T);
        return value;
    }
    void skip(uint64_t bytes) {
        if (!ok || bytes > size - at) { ok = false; return; }
        at += (size_t)bytes;
    }
    std::string string() {
        const uint64_t length = read<uint64_t>();
        if (!ok || length > size - at) { ok = false; return std::string(); }
        std::string text(reinterpret_cast<const char*>(data + at), (size_t)length);
        at += (size_t)length;
        return text;
    }
};

// Byte size of a scalar metadata value type, 0 for strings / arrays / unknown.
size_t scalar_bytes(uint32_t type) {
    switch (type) {
        case 0: case 1: case 7: return 1;          // u8, i8, bool
        case 2: case 3: return 2;                  // u16, i16
        case 4: case 5: case 6: return 4;          // u32, i32, f32
        case 10: case 11: case 12: return 8;       // u64, i64, f64
        default: return 0;
    }
}

bool skip_value(Cursor& c, uint32_t type, int depth) {
    if (const size_t bytes = scalar_bytes(type)) { c.skip(bytes); return c.ok; }
    if (type == 8) { c.string(); return c.ok; }
    if (type == 9 && depth == 0) {
        const uint32_t element = c.read<uint32_t>();
        const uint64_t count = c.read<uint64_t>();
        if (!c.ok) return false;
        if (const size_t bytes = scalar_bytes(element)) {
            if (count > (c.size - c.at) / bytes) { c.ok = false; return false; }
            c.skip(count * bytes);
            return c.ok;
        }
        if (element != 8) return false;
        for (uint64_t i = 0; i < count && c.ok; ++i) c.string();
        return c.ok;
    }
    return false;
}

struct Known { const char* name; int kind; bool matrix; bool per_layer; };
const Known kKnown[] = {
    {"token_embd", GF_MAT_TOKEN_EMBD, true, false}, {"output", GF_MAT_OUTPUT, true, false},
    {"attn_q", GF_MAT_ATTN_Q, true, true}, {"attn_k", GF_MAT_ATTN_K, true, true}, {"attn_v", GF_MAT_ATTN_V, true, true},
    {"attn_output", GF_MAT_ATTN_OUTPUT, true, true}, {"ffn_gate", GF_MAT_FFN_GATE, true, true},
    {"ffn_up", GF_MAT_FFN_UP, true, true}, {"ffn_down", GF_MAT_FFN_DOWN, true, true},
    {"output_norm", GF_VEC_OUTPUT_NORM, false, false}, {"attn_norm", GF_VEC_ATTN_NORM, false, true},
    {"post_attention_norm", GF_VEC_POST_ATTENTION_NORM, false, true}, {"ffn_norm", GF_VEC_FFN_NORM, false, true},
    {"post_ffw_norm", GF_VEC_POST_FFW_NORM, false, true}, {"attn_q_norm", GF_VEC_ATTN_Q_NORM, false, true},
    {"attn_k_norm", GF_VEC_ATTN_K_NORM, false, true},
};

// "blk.<layer>.<short>.weight" or "<short>.weight" -> (layer, entry of kKnown) or null.
const Known* classify(const std::string& name, uint32_t& layer) {
    const std::string suffix = ".weight";
    if (name.size() <= suffix.size() || name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) return nullptr;
    std::string stem = name.substr(0, name.size() - suffix.size());
    layer = 0;
    const bool in_block = stem.compare(0, 4, "blk.") == 0;
    if (in_block) {
        const size_t dot = stem.find('.', 4);
        if (dot == std::string::npos || dot == 4 || dot - 4 > 6) return nullptr;
        uint32_t value = 0;
        for (size_t i = 4; i < dot; ++i) {
            if (stem[i] < '0' || stem[i] > '9') return nullptr;
            value = value * 10u + (uint32_t)(stem[i] - '0');
        }
        layer = value;
        stem = stem.substr(dot + 1);
    }
    for (const Known& known : kKnown)
        if (stem == known.name && in_block == known.per_layer) return &known;
    return nullptr;
}

uint64_t tensor_bytes(uint32_t type, uint64_t elements) {
    switch (type) {
        case 0: return elements * 4u;                                   // F32
        case 1: return elements * 2u;                                   // F16 (embedding / head tables of the retained Gemma 2 file)
        case GF_Q8_0: return elements % 32u ? 0 : elements / 32u * 34u;
        case GF_Q4_K: return elements % 256u ? 0 : elements / 256u * 144u;
        case GF_Q6_K: return elements % 256u ? 0 : elements / 256u * 210u;
        default: return 0;
    }
}

}  // namespace
}  // namespace gf

using namespace gf;

extern "C" int gf_model_load_gguf(gf_model* model, const char* path, uint32_t* out_bound_tensors) {
    if (!model || !path) return fail(GF_ERR_INVALID, "gf_model_load_gguf: null argument");
    Mapping file;
    file.fd = open(path, O_RDONLY);
    if (file.fd < 0) return fail(GF_ERR_INVALID, "gf_model_load_gguf: cannot open %s", path);
    struct stat info;
    if (fstat(file.fd, &info) != 0 || info.st_size < 24) return fail(GF_ERR_INVALID, "gf_model_load_gguf: %s is not a GGUF file", path);
    file.size = (size_t)info.st_size;
    void* mapped = mmap(nullptr, file.size, PROT_READ, MAP_PRIVATE, file.fd, 0);
    if (mapped == MAP_FAILED) return fail(GF_ERR_INVALID, "gf_model_load_gguf: cannot map %s", path);
    file.data = static_cast<const uint8_t*>(mapped);

    Cursor c{file.data, file.size};
    const uint32_t magic = c.read<uint32_t>(), version = c.read<uint32_t>();
    if (!c.ok || magic != 0x46554747u) return fail(GF_ERR_INVALID, "gf_model_load_gguf: %s has no GGUF magic", path);
    if (version != 2u && version != 3u) return fail(GF_ERR_INVALID, "gf_model_load_gguf: GGUF version %u is not supported (2, 3)", version);
    const uint64_t tensor_count = c.read<uint64_t>(), metadata_count = c.read<uint64_t>();
    if (!c.ok || tensor_count > (1u << 20) || metadata_count > (1u << 20)) return fail(GF_ERR_INVALID, "gf_model_load_gguf: implausible header counts");
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < metadata_count; ++i) {
        const std::string key = c.string();
        const uint32_t type = c.read<uint32_t>();
        if (!c.ok) break;
        if (key == "general.alignment" && type == 4u) {
            alignment = c.read<uint32_t>();
            continue;
        }
        if (!skip_value(c, type, 0)) return fail(GF_ERR_INVALID, "gf_model_load_gguf: cannot parse metadata value %llu (type %u)", (unsigned long long)i, type);
    }
    if (!c.ok || alignment == 0 || (alignment & (alignment - 1u))) return fail(GF_ERR_INVALID, "gf_model_load_gguf: truncated or malformed metadata");

    struct Entry { std::string name; uint64_t dims[4]; uint32_t rank, type; uint64_t offset; };
    std::vector<Entry> entries((size_t)tensor_count);
    for (Entry& e : entries) {
        e.name = c.string();
        e.rank = c.read<uint32_t>();
        if (!c.ok || e.rank == 0 || e.rank > 4) return fail(GF_ERR_INVALID, "gf_model_load_gguf: bad tensor directory entry");
        for (uint32_t d = 0; d < 4; ++d) e.dims[d] = d < e.rank ? c.read<uint64_t>() : 1u;
        e.type = c.read<uint32_t>();
        e.offset = c.read<uint64_t>();
    }
    if (!c.ok) return fail(GF_ERR_INVALID, "gf_model_load_gguf: truncated tensor directory");
    const uint64_t data_start = ((uint64_t)c.at + alignment - 1u) & ~(alignment - 1u);

    // Validate every tensor the path takes before binding any of them.
    struct Binding { const Entry* entry; const Known* known; uint32_t layer; uint64_t elements; };
    std::vector<Binding> bindings;
    for (const Entry& e : entries) {
        uint32_t layer = 0;
        const Known* known = classify(e.name, layer);
        if (!known) continue;
        uint64_t elements = 1;
        for (uint32_t d = 0; d < e.rank; ++d) {
            if (e.dims[d] == 0 || elements > (1ull << 40) / e.dims[d]) return fail(GF_ERR_INVALID, "gf_model_load_gguf: tensor %s has an implausible shape", e.name.c_str());
            elements *= e.dims[d];
        }
        const uint64_t bytes = tensor_bytes(e.type, elements);
        if (bytes == 0 || (known->matrix && (e.type == 0u || e.rank != 2u)) || (!known->matrix && e.type != 0u))
            return fail(GF_ERR_INVALID, "gf_model_load_gguf: tensor %s has type %u / rank %u, which this path does not take", e.name.c_str(), e.type, e.rank);
        if (e.offset % alignment || data_start > file.size || e.offset > file.size - data_start || bytes > file.size - data_start - e.offset)
            return fail(GF_ERR_INVALID, "gf_model_load_gguf: tensor %s lies outside the file", e.name.c_str());
        bindings.push_back(Binding{&e, known, layer, elements});
    }
    // Source I/O of the next tensor overlaps the upload and repack of the current one (the reference hints
    // the next block's byte range the same way, gemma2_metal_plan.cpp:427-461).
    auto read_ahead = [&](const Binding& binding) {
        const uint64_t begin = data_start + binding.entry->offset, bytes = tensor_bytes(binding.entry->type, binding.elements);
        const uint64_t page = 4096u, first = begin & ~(page - 1u);
        madvise(const_cast<uint8_t*>(file.data) + first, (size_t)(begin + bytes - first), MADV_WILLNEED);
    };
    uint32_t bound = 0;
    for (size_t index = 0; index < bindings.size(); ++index) {
        const Binding& binding = bindings[index];
        if (index == 0) read_ahead(binding);
        if (index + 1 < bindings.size()) read_ahead(bindings[index + 1]);
        const Entry& e = *binding.entry;
        const uint8_t* payload = file.data + data_start + e.offset;
        int status;
        if (binding.known->matrix) status = gf_model_set_matrix(model, binding.known->kind, binding.layer, (int)e.type, payload, e.dims[0], e.dims[1]);
        else status = gf_model_set_vector(model, binding.known->kind, binding.layer, reinterpret_cast<const float*>(payload), (uint32_t)binding.elements);
        if (status != GF_OK) return status;
        ++bound;
    }
    if (out_bound_tensors) *out_bound_tensors = bound;
    return GF_OK;
}
