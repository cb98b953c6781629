// GGUF v3 reader and staged upload of encoded tensors (host code; no kernels).
//
// Reference twins (crates/gguf/src/lib.rs of the reference project):
//   GgufFile::read_from      :191-280   header, metadata, tensor directory; bulk data is never read here
//   TensorInfo::byte_len     :139-163   block layout checks
//   tensor_data_range        :324-343   absolute byte range of one tensor
//   TensorDataReader         :400-505   bounded sequential reader; the file is opened when a read starts and closed when
//                                       the payload is exhausted, so holding many readers costs no descriptors
//   read_value / read_string :1085-1156 value grammar and parser bounds
// and CudaWeightStore::materialize_quantized (crates/nvidia/src/cuda.rs:321-387), which copies a tensor in 1 MiB pieces
// with a stream synchronisation after each.  Here the pieces go through two pinned buffers: the file read of one piece
// overlaps the host-to-device copy of the previous one, and only the buffer about to be refilled is waited for.
//
// Tensor-parallel loading: a shard is cut while it is uploaded.  Output-row shards are one contiguous byte range;
// input-column shards take the same range of whole blocks out of every row and pack them row after row.
#include <cuda_runtime.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/ribn_b200.h"
#include "internal.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u;   // "GGUF"
constexpr uint32_t kVersion = 3;
constexpr uint64_t kDefaultAlignment = 32;
constexpr uint64_t kMaxStringBytes = 16ull << 20;
constexpr uint64_t kMaxArrayItems = 1000000;
constexpr uint32_t kMaxDepth = 16;
constexpr uint32_t kMaxDims = RIBN_GGUF_MAX_DIMS;
constexpr uint64_t kMaxTensors = 10000000;

struct Value {
    uint32_t type = 0;   // GGUF value type 0..12
    uint64_t bits = 0;   // scalars: the raw little-endian bits, zero-extended
    std::string text;    // type 8
    uint32_t element_type = 0;
    std::vector<Value> items;   // type 9
};

struct Tensor {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t value_type = 0;
    uint64_t offset = 0;
};

struct Parse {
    int status = RIBN_OK;
    std::string message;
};

Parse bad(int status, std::string message) { return Parse{status, std::move(message)}; }

class Reader {
  public:
    explicit Reader(FILE* f) : f_(f) {}
    bool bytes(void* out, size_t n) { return n == 0 || fread(out, 1, n, f_) == n; }
    template <typename T>
    bool scalar(T* out) {
        unsigned char raw[sizeof(T)];
        if (!bytes(raw, sizeof raw)) return false;
        uint64_t v = 0;
        for (size_t i = 0; i < sizeof(T); ++i) v |= static_cast<uint64_t>(raw[i]) << (8 * i);
        *out = static_cast<T>(v);
        return true;
    }

  private:
    FILE* f_;
};

Parse eof() { return bad(RIBN_GGUF_E_UNEXPECTED_EOF, "truncated GGUF value"); }

bool valid_utf8(const std::string& s) {
    size_t i = 0, n = s.size();
    const auto* p = reinterpret_cast<const unsigned char*>(s.data());
    while (i < n) {
        const unsigned char c = p[i];
        size_t extra;
        uint32_t code;
        if (c < 0x80) { ++i; continue; }
        if ((c & 0xE0) == 0xC0) { extra = 1; code = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { extra = 2; code = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { extra = 3; code = c & 0x07; }
        else return false;
        if (i + extra >= n) return false;
        for (size_t j = 1; j <= extra; ++j) {
            if ((p[i + j] & 0xC0) != 0x80) return false;
            code = (code << 6) | (p[i + j] & 0x3F);
        }
        if ((extra == 1 && code < 0x80) || (extra == 2 && code < 0x800) || (extra == 3 && code < 0x10000)) return false;   // overlong
        if (code > 0x10FFFF || (code >= 0xD800 && code <= 0xDFFF)) return false;
        i += extra + 1;
    }
    return true;
}

Parse read_string(Reader& r, std::string* out) {
    uint64_t length = 0;
    if (!r.scalar(&length)) return eof();
    if (length > kMaxStringBytes) return bad(RIBN_GGUF_E_INVALID_LENGTH, "GGUF string length " + std::to_string(length) + " exceeds the parser bound");
    out->resize(static_cast<size_t>(length));
    if (!r.bytes(out->data(), out->size())) return eof();
    if (!valid_utf8(*out)) return bad(RIBN_GGUF_E_INVALID_UTF8, "GGUF string is not valid UTF-8");
    return {};
}

Parse read_count(Reader& r, const char* kind, uint64_t max, uint64_t* out) {
    if (!r.scalar(out)) return eof();
    if (*out > max) return bad(RIBN_GGUF_E_INVALID_LENGTH, std::string("GGUF ") + kind + " length " + std::to_string(*out) + " exceeds the parser bound");
    return {};
}

Parse read_value(Reader& r, uint32_t type, uint32_t depth, Value* out) {
    if (depth > kMaxDepth) return bad(RIBN_GGUF_E_ARRAY_NESTING_TOO_DEEP, "GGUF metadata array nesting is too deep");
    out->type = type;
    switch (type) {
        case 0: case 1: { uint8_t v; if (!r.scalar(&v)) return eof(); out->bits = v; return {}; }
        case 2: case 3: { uint16_t v; if (!r.scalar(&v)) return eof(); out->bits = v; return {}; }
        case 4: case 5: case 6: { uint32_t v; if (!r.scalar(&v)) return eof(); out->bits = v; return {}; }
        case 7: {
            uint8_t v;
            if (!r.scalar(&v)) return eof();
            if (v > 1) return bad(RIBN_GGUF_E_INVALID_BOOL, "invalid GGUF boolean value " + std::to_string(v));
            out->bits = v;
            return {};
        }
        case 8: return read_string(r, &out->text);
        case 9: {
            if (!r.scalar(&out->element_type)) return eof();
            uint64_t count = 0;
            Parse p = read_count(r, "array", kMaxArrayItems, &count);
            if (p.status != RIBN_OK) return p;
            out->items.resize(static_cast<size_t>(count));
            for (Value& item : out->items) {
                p = read_value(r, out->element_type, depth + 1, &item);
                if (p.status != RIBN_OK) return p;
            }
            return {};
        }
        case 10: case 11: case 12: { uint64_t v; if (!r.scalar(&v)) return eof(); out->bits = v; return {}; }
        default: return bad(RIBN_GGUF_E_INVALID_VALUE_TYPE, "invalid GGUF metadata value type " + std::to_string(type));
    }
}

bool as_u64(const Value& v, uint64_t* out) {   // MetadataValue::as_u64: the unsigned integer types only
    if (v.type == 0 || v.type == 2 || v.type == 4 || v.type == 10) { *out = v.bits; return true; }
    return false;
}

}  // namespace

struct ribn_gguf {
    std::string path;
    uint32_t version = 0;
    uint64_t tensor_count = 0;
    std::map<std::string, Value> metadata;
    std::vector<Tensor> tensors;
    uint64_t data_offset = 0;
    uint64_t file_len = 0;
    std::string message;   // last error of a call on this object
};

namespace {

int note(ribn_gguf* g, int status, std::string message) {
    if (g != nullptr) g->message = std::move(message);
    return status;
}

thread_local std::string g_open_error;

const Tensor* find_tensor(const ribn_gguf* g, const char* name) {
    for (const Tensor& t : g->tensors)
        if (t.name == name) return &t;
    return nullptr;
}

// TensorInfo::byte_len
int byte_len(ribn_gguf* g, const Tensor& t, uint64_t* out, uint64_t* block_elements_out = nullptr, uint64_t* block_bytes_out = nullptr) {
    uint64_t block_elements = 0, block_bytes = 0;
    if (ribn_tensor_layout(t.value_type, &block_elements, &block_bytes) != RIBN_OK)
        return note(g, RIBN_GGUF_E_UNSUPPORTED_TENSOR_TYPE, "unsupported GGML tensor type " + std::to_string(t.value_type));
    if (t.dims.empty()) return note(g, RIBN_GGUF_E_INVALID_DIMENSION_COUNT, "invalid GGUF tensor dimension count 0");
    if (t.dims[0] % block_elements != 0)
        return note(g, RIBN_GGUF_E_QUANTIZATION_DIMENSION_MISMATCH, "GGUF tensor \"" + t.name + "\" first dimension " + std::to_string(t.dims[0]) +
                                                                        " is not divisible by block size " + std::to_string(block_elements));
    uint64_t elements = 1;
    for (uint64_t d : t.dims) {
        if (d != 0 && elements > UINT64_MAX / d) return note(g, RIBN_GGUF_E_ELEMENT_COUNT_OVERFLOW, "GGUF tensor element count overflowed");
        elements *= d;
    }
    if (elements % block_elements != 0)
        return note(g, RIBN_GGUF_E_QUANTIZATION_BLOCK_MISMATCH, "GGUF tensor \"" + t.name + "\" has " + std::to_string(elements) +
                                                                    " elements, not divisible by block size " + std::to_string(block_elements));
    const uint64_t blocks = elements / block_elements;
    if (blocks != 0 && block_bytes > UINT64_MAX / blocks) return note(g, RIBN_GGUF_E_TENSOR_BYTE_LENGTH_OVERFLOW, "GGUF tensor byte length overflowed");
    *out = blocks * block_bytes;
    if (block_elements_out != nullptr) *block_elements_out = block_elements;
    if (block_bytes_out != nullptr) *block_bytes_out = block_bytes;
    return RIBN_OK;
}

int data_range(ribn_gguf* g, const Tensor& t, uint64_t* begin, uint64_t* end) {
    uint64_t length = 0;
    const int status = byte_len(g, t, &length);
    if (status != RIBN_OK) return status;
    if (t.offset > UINT64_MAX - g->data_offset || length > UINT64_MAX - (g->data_offset + t.offset))
        return note(g, RIBN_GGUF_E_TENSOR_BYTE_LENGTH_OVERFLOW, "GGUF tensor byte length overflowed");
    *begin = g->data_offset + t.offset;
    *end = *begin + length;
    if (*end > g->file_len)
        return note(g, RIBN_GGUF_E_TENSOR_OFFSET_OUT_OF_BOUNDS, "GGUF tensor \"" + t.name + "\" has out-of-bounds offset " + std::to_string(t.offset));
    return RIBN_OK;
}

Parse parse(FILE* f, ribn_gguf* g) {
    if (fseeko(f, 0, SEEK_END) != 0) return bad(RIBN_GGUF_E_IO, "could not read GGUF " + g->path + ": " + strerror(errno));
    g->file_len = static_cast<uint64_t>(ftello(f));
    if (fseeko(f, 0, SEEK_SET) != 0) return bad(RIBN_GGUF_E_IO, "could not read GGUF " + g->path + ": " + strerror(errno));
    Reader r(f);
    uint32_t magic = 0;
    if (!r.scalar(&magic)) return eof();
    if (magic != kMagic) {
        char text[64];
        snprintf(text, sizeof text, "invalid GGUF magic 0x%08x", magic);
        return bad(RIBN_GGUF_E_INVALID_MAGIC, text);
    }
    if (!r.scalar(&g->version)) return eof();
    if (g->version != kVersion) return bad(RIBN_GGUF_E_UNSUPPORTED_VERSION, "unsupported GGUF version " + std::to_string(g->version));
    Parse p = read_count(r, "tensor", kMaxTensors, &g->tensor_count);
    if (p.status != RIBN_OK) return p;
    uint64_t metadata_count = 0;
    p = read_count(r, "metadata", kMaxArrayItems, &metadata_count);
    if (p.status != RIBN_OK) return p;
    for (uint64_t i = 0; i < metadata_count; ++i) {
        std::string key;
        p = read_string(r, &key);
        if (p.status != RIBN_OK) return p;
        uint32_t type = 0;
        if (!r.scalar(&type)) return eof();
        Value value;
        p = read_value(r, type, 0, &value);
        if (p.status != RIBN_OK) return p;
        if (!g->metadata.emplace(key, std::move(value)).second) return bad(RIBN_GGUF_E_DUPLICATE_METADATA, "duplicate GGUF metadata key \"" + key + "\"");
    }
    g->tensors.reserve(static_cast<size_t>(std::min<uint64_t>(g->tensor_count, 1u << 20)));
    for (uint64_t i = 0; i < g->tensor_count; ++i) {
        Tensor t;
        p = read_string(r, &t.name);
        if (p.status != RIBN_OK) return p;
        uint32_t dims = 0;
        if (!r.scalar(&dims)) return eof();
        if (dims > kMaxDims) return bad(RIBN_GGUF_E_INVALID_DIMENSION_COUNT, "invalid GGUF tensor dimension count " + std::to_string(dims));
        t.dims.resize(dims);
        for (uint64_t& d : t.dims)
            if (!r.scalar(&d)) return eof();
        if (!r.scalar(&t.value_type) || !r.scalar(&t.offset)) return eof();
        g->tensors.push_back(std::move(t));
    }
    uint64_t alignment = kDefaultAlignment;
    const auto found = g->metadata.find("general.alignment");
    if (found != g->metadata.end()) {
        uint64_t v = 0;
        if (as_u64(found->second, &v)) alignment = v;
    }
    if (alignment == 0 || (alignment & (alignment - 1)) != 0) return bad(RIBN_GGUF_E_INVALID_ALIGNMENT, "invalid GGUF tensor-data alignment " + std::to_string(alignment));
    const uint64_t directory_end = static_cast<uint64_t>(ftello(f));
    const uint64_t remainder = directory_end % alignment;
    if (remainder != 0 && directory_end > UINT64_MAX - (alignment - remainder)) return bad(RIBN_GGUF_E_TRUNCATED, "GGUF tensor directory points past the file");
    g->data_offset = remainder == 0 ? directory_end : directory_end + (alignment - remainder);
    if (g->data_offset > g->file_len) return bad(RIBN_GGUF_E_TRUNCATED, "GGUF tensor directory points past the file");
    for (const Tensor& t : g->tensors)
        if (t.offset > g->file_len - g->data_offset)
            return bad(RIBN_GGUF_E_TENSOR_OFFSET_OUT_OF_BOUNDS, "GGUF tensor \"" + t.name + "\" has out-of-bounds offset " + std::to_string(t.offset));
    return {};
}

const Value* lookup(ribn_gguf* g, const char* key, uint64_t index, int* status) {
    const auto found = g->metadata.find(key);
    if (found == g->metadata.end()) {
        *status = note(g, RIBN_GGUF_E_MISSING_METADATA, std::string("missing GGUF metadata key \"") + key + "\"");
        return nullptr;
    }
    const Value* v = &found->second;
    if (index != RIBN_GGUF_SCALAR) {
        if (v->type != 9 || index >= v->items.size()) {
            *status = note(g, RIBN_GGUF_E_METADATA_TYPE_MISMATCH, std::string("GGUF metadata key \"") + key + "\" has an unexpected type");
            return nullptr;
        }
        v = &v->items[static_cast<size_t>(index)];
    }
    *status = RIBN_OK;
    return v;
}

int mismatch(ribn_gguf* g, const char* key) {
    return note(g, RIBN_GGUF_E_METADATA_TYPE_MISMATCH, std::string("GGUF metadata key \"") + key + "\" has an unexpected type");
}

// Two pinned buffers; piece i is read from the file into buffer i % 2 while piece i - 1 is still on its way to the device.
struct Stager {
    static constexpr size_t kPiece = 8u << 20;
    void* host[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};
    cudaError_t error = cudaSuccess;
    Stager() {
        for (int i = 0; i < 2 && error == cudaSuccess; ++i) {
            error = cudaHostAlloc(&host[i], kPiece, cudaHostAllocDefault);
            if (error == cudaSuccess) error = cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming);
        }
    }
    ~Stager() {
        for (int i = 0; i < 2; ++i) {
            if (done[i] != nullptr) cudaEventDestroy(done[i]);
            if (host[i] != nullptr) cudaFreeHost(host[i]);
        }
    }
};

}  // namespace

extern "C" {

int ribn_gguf_open(const char* path, ribn_gguf** out) {
    if (out == nullptr || path == nullptr) return RIBN_E_INVALID_ARGUMENT;
    *out = nullptr;
    std::unique_ptr<ribn_gguf> g(new ribn_gguf());
    g->path = path;
    FILE* f = fopen(path, "rb");
    if (f == nullptr) {
        g_open_error = std::string("could not read GGUF ") + path + ": " + strerror(errno);
        return RIBN_GGUF_E_IO;
    }
    const Parse p = parse(f, g.get());
    fclose(f);
    if (p.status != RIBN_OK) {
        g_open_error = p.message;
        return p.status;
    }
    g_open_error.clear();
    *out = g.release();
    return RIBN_OK;
}

void ribn_gguf_close(ribn_gguf* file) { delete file; }

const char* ribn_gguf_last_error(const ribn_gguf* file) { return file != nullptr ? file->message.c_str() : g_open_error.c_str(); }

uint32_t ribn_gguf_version(const ribn_gguf* file) { return file != nullptr ? file->version : 0; }
uint64_t ribn_gguf_tensor_count(const ribn_gguf* file) { return file != nullptr ? file->tensor_count : 0; }
uint64_t ribn_gguf_metadata_count(const ribn_gguf* file) { return file != nullptr ? file->metadata.size() : 0; }
uint64_t ribn_gguf_tensor_data_offset(const ribn_gguf* file) { return file != nullptr ? file->data_offset : 0; }

const char* ribn_gguf_metadata_key(const ribn_gguf* file, uint64_t index) {
    if (file == nullptr || index >= file->metadata.size()) return nullptr;
    auto it = file->metadata.begin();
    std::advance(it, static_cast<long>(index));
    return it->first.c_str();
}

int ribn_gguf_metadata_type(ribn_gguf* file, const char* key, uint32_t* type, uint32_t* element_type, uint64_t* count) {
    if (file == nullptr || key == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, RIBN_GGUF_SCALAR, &status);
    if (v == nullptr) return status;
    if (type != nullptr) *type = v->type;
    if (element_type != nullptr) *element_type = v->type == 9 ? v->element_type : 0;
    if (count != nullptr) *count = v->type == 9 ? v->items.size() : 0;
    return RIBN_OK;
}

int ribn_gguf_metadata_u64(ribn_gguf* file, const char* key, uint64_t index, uint64_t* out) {
    if (file == nullptr || key == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, index, &status);
    if (v == nullptr) return status;
    return as_u64(*v, out) ? RIBN_OK : mismatch(file, key);
}

int ribn_gguf_metadata_i64(ribn_gguf* file, const char* key, uint64_t index, int64_t* out) {
    if (file == nullptr || key == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, index, &status);
    if (v == nullptr) return status;
    switch (v->type) {   // the signed integer types, sign-extended (MetadataValue::as_i32 widened)
        case 1: *out = static_cast<int8_t>(v->bits); return RIBN_OK;
        case 3: *out = static_cast<int16_t>(v->bits); return RIBN_OK;
        case 5: *out = static_cast<int32_t>(v->bits); return RIBN_OK;
        case 11: *out = static_cast<int64_t>(v->bits); return RIBN_OK;
        default: return mismatch(file, key);
    }
}

int ribn_gguf_metadata_f64(ribn_gguf* file, const char* key, uint64_t index, double* out) {
    if (file == nullptr || key == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, index, &status);
    if (v == nullptr) return status;
    if (v->type == 6) {
        const uint32_t bits = static_cast<uint32_t>(v->bits);
        float f;
        memcpy(&f, &bits, sizeof f);
        *out = f;
        return RIBN_OK;
    }
    if (v->type == 12) {
        memcpy(out, &v->bits, sizeof *out);
        return RIBN_OK;
    }
    return mismatch(file, key);
}

int ribn_gguf_metadata_bool(ribn_gguf* file, const char* key, uint64_t index, int* out) {
    if (file == nullptr || key == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, index, &status);
    if (v == nullptr) return status;
    if (v->type != 7) return mismatch(file, key);
    *out = static_cast<int>(v->bits);
    return RIBN_OK;
}

int ribn_gguf_metadata_string(ribn_gguf* file, const char* key, uint64_t index, const char** data, uint64_t* length) {
    if (file == nullptr || key == nullptr || data == nullptr || length == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int status = RIBN_OK;
    const Value* v = lookup(file, key, index, &status);
    if (v == nullptr) return status;
    if (v->type != 8) return mismatch(file, key);
    *data = v->text.data();
    *length = v->text.size();
    return RIBN_OK;
}

int ribn_gguf_tensor_info(ribn_gguf* file, uint64_t index, ribn_gguf_tensor* out) {
    if (file == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (index >= file->tensors.size()) return note(file, RIBN_GGUF_E_MISSING_TENSOR, "GGUF tensor index " + std::to_string(index) + " was not found");
    const Tensor& t = file->tensors[static_cast<size_t>(index)];
    memset(out, 0, sizeof *out);
    out->name = t.name.c_str();
    out->value_type = t.value_type;
    out->n_dims = static_cast<uint32_t>(t.dims.size());
    for (size_t i = 0; i < t.dims.size(); ++i) out->dims[i] = t.dims[i];
    out->offset = t.offset;
    return RIBN_OK;
}

int ribn_gguf_find_tensor(ribn_gguf* file, const char* name, uint64_t* index) {
    if (file == nullptr || name == nullptr || index == nullptr) return RIBN_E_INVALID_ARGUMENT;
    for (size_t i = 0; i < file->tensors.size(); ++i)
        if (file->tensors[i].name == name) {
            *index = i;
            return RIBN_OK;
        }
    return note(file, RIBN_GGUF_E_MISSING_TENSOR, std::string("GGUF tensor \"") + name + "\" was not found");
}

int ribn_gguf_tensor_data_range(ribn_gguf* file, const char* name, uint64_t* begin, uint64_t* end) {
    if (file == nullptr || name == nullptr || begin == nullptr || end == nullptr) return RIBN_E_INVALID_ARGUMENT;
    const Tensor* t = find_tensor(file, name);
    if (t == nullptr) return note(file, RIBN_GGUF_E_MISSING_TENSOR, std::string("GGUF tensor \"") + name + "\" was not found");
    return data_range(file, *t, begin, end);
}

int ribn_gguf_read_tensor(ribn_gguf* file, const char* name, uint64_t offset, void* host_dst, uint64_t bytes, uint64_t* read_out) {
    if (file == nullptr || name == nullptr || (host_dst == nullptr && bytes != 0)) return RIBN_E_INVALID_ARGUMENT;
    uint64_t begin = 0, end = 0;
    const int status = ribn_gguf_tensor_data_range(file, name, &begin, &end);
    if (status != RIBN_OK) return status;
    const uint64_t length = end - begin;
    // TensorDataReader: a read never crosses the tensor's end; past it, nothing is returned
    const uint64_t count = offset >= length ? 0 : std::min(bytes, length - offset);
    if (read_out != nullptr) *read_out = count;
    if (count == 0) return RIBN_OK;
    FILE* f = fopen(file->path.c_str(), "rb");   // opened per call and closed before returning: no descriptor is held
    if (f == nullptr) return note(file, RIBN_GGUF_E_IO, "could not read GGUF " + file->path + ": " + strerror(errno));
    int result = RIBN_OK;
    if (fseeko(f, static_cast<off_t>(begin + offset), SEEK_SET) != 0 || fread(host_dst, 1, static_cast<size_t>(count), f) != count)
        result = note(file, RIBN_GGUF_E_UNEXPECTED_EOF, "truncated GGUF value");
    fclose(f);
    return result;
}

int ribn_gguf_shard_bytes(ribn_gguf* file, const char* name, int axis, uint64_t begin, uint64_t end, uint64_t* bytes, uint64_t* k_out,
                          uint64_t* n_out) {
    if (file == nullptr || name == nullptr || bytes == nullptr) return RIBN_E_INVALID_ARGUMENT;
    const Tensor* t = find_tensor(file, name);
    if (t == nullptr) return note(file, RIBN_GGUF_E_MISSING_TENSOR, std::string("GGUF tensor \"") + name + "\" was not found");
    uint64_t total = 0, block_elements = 0, block_bytes = 0;
    const int status = byte_len(file, *t, &total, &block_elements, &block_bytes);
    if (status != RIBN_OK) return status;
    if (t->dims.size() != 2) return note(file, RIBN_E_INVALID_WEIGHT, "invalid quantized weight: a shard needs a tensor of dimensions [input, output]");
    const uint64_t k = t->dims[0], n = t->dims[1];
    if (axis == RIBN_SHARD_ROWS) {
        if (begin > end || end > n) return note(file, RIBN_E_INVALID_ARGUMENT, "row shard outside the tensor");
        *bytes = (end - begin) * (k / block_elements) * block_bytes;
        if (k_out != nullptr) *k_out = k;
        if (n_out != nullptr) *n_out = end - begin;
        return RIBN_OK;
    }
    if (axis == RIBN_SHARD_INPUT) {
        // whole super-blocks of 256 inputs, whatever the block size of the format (eight Q8_0 blocks)
        if (k % 256 != 0 || begin > end || end > k / 256) return note(file, RIBN_E_INVALID_ARGUMENT, "input shard outside the tensor's super-blocks");
        *bytes = n * (end - begin) * (256 / block_elements) * block_bytes;
        if (k_out != nullptr) *k_out = (end - begin) * 256;
        if (n_out != nullptr) *n_out = n;
        return RIBN_OK;
    }
    return note(file, RIBN_E_INVALID_ARGUMENT, "unknown shard axis");
}

int ribn_materialize_quantized(ribn_ctx* ctx, ribn_gguf* file, const char* name, int axis, uint64_t begin, uint64_t end, void* device_dst,
                               uint64_t dst_bytes) {
    if (ctx == nullptr || file == nullptr || name == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t file_begin = 0, file_end = 0;
    int status = ribn_gguf_tensor_data_range(file, name, &file_begin, &file_end);
    if (status != RIBN_OK) return status;
    const Tensor* t = find_tensor(file, name);
    uint64_t total = 0, block_elements = 0, block_bytes = 0;
    status = byte_len(file, *t, &total, &block_elements, &block_bytes);
    if (status != RIBN_OK) return status;
    // the copy plan: `runs` runs of `run_bytes`, the first at `first`, consecutive ones `stride` apart in the file
    uint64_t first = file_begin, run_bytes = total, runs = 1, stride = 0, expected = total;
    if (axis != RIBN_SHARD_NONE) {
        status = ribn_gguf_shard_bytes(file, name, axis, begin, end, &expected, nullptr, nullptr);
        if (status != RIBN_OK) return status;
        const uint64_t row_bytes = t->dims[0] / block_elements * block_bytes;
        if (axis == RIBN_SHARD_ROWS) {
            first = file_begin + begin * row_bytes;
            run_bytes = expected;
        } else {
            const uint64_t super_bytes = 256 / block_elements * block_bytes;
            first = file_begin + begin * super_bytes;
            run_bytes = (end - begin) * super_bytes;
            runs = t->dims[1];
            stride = row_bytes;
        }
    }
    if (expected == 0) return note(file, RIBN_E_INVALID_WEIGHT, std::string("tensor \"") + name + "\" has an empty encoding");   // EmptyEncoding
    if (dst_bytes != expected)
        return note(file, RIBN_E_OUTPUT_LENGTH, "destination holds " + std::to_string(dst_bytes) + " bytes, the encoding has " + std::to_string(expected));
    int device = 0;
    void* stream_handle = nullptr;
    status = ribn_context_stream(ctx, &device, &stream_handle);
    if (status != RIBN_OK) return status;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(device);
    FILE* f = fopen(file->path.c_str(), "rb");
    if (f == nullptr) {
        cudaSetDevice(previous);
        return note(file, RIBN_GGUF_E_IO, "could not read GGUF " + file->path + ": " + strerror(errno));
    }
    Stager stager;
    int result = stager.error == cudaSuccess ? RIBN_OK : note(file, RIBN_E_DRIVER, std::string("pinned staging buffers: ") + cudaGetErrorString(stager.error));
    uint64_t written = 0;
    int slot = 0;
    size_t filled = 0;   // bytes gathered in the current buffer
    auto flush = [&]() {
        if (filled == 0 || result != RIBN_OK) return;
        cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(device_dst) + written, stager.host[slot], filled, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaEventRecord(stager.done[slot], stream);
        if (e != cudaSuccess) {
            result = note(file, RIBN_E_DRIVER, std::string("upload: ") + cudaGetErrorString(e));
            return;
        }
        stager.busy[slot] = true;
        written += filled;
        filled = 0;
        slot ^= 1;
        if (stager.busy[slot]) {   // the buffer about to be refilled: its copy must have left the host
            e = cudaEventSynchronize(stager.done[slot]);
            stager.busy[slot] = false;
            if (e != cudaSuccess) result = note(file, RIBN_E_DRIVER, std::string("upload: ") + cudaGetErrorString(e));
        }
    };
    for (uint64_t run = 0; run < runs && result == RIBN_OK; ++run) {
        if (fseeko(f, static_cast<off_t>(first + run * stride), SEEK_SET) != 0) {
            result = note(file, RIBN_GGUF_E_IO, "could not read GGUF " + file->path + ": " + strerror(errno));
            break;
        }
        uint64_t left = run_bytes;
        while (left != 0 && result == RIBN_OK) {
            const size_t want = static_cast<size_t>(std::min<uint64_t>(left, Stager::kPiece - filled));
            const size_t got = fread(static_cast<uint8_t*>(stager.host[slot]) + filled, 1, want, f);
            if (got != want)   // SourceIncomplete
                result = note(file, RIBN_GGUF_E_UNEXPECTED_EOF, std::string("tensor \"") + name + "\" ended after " + std::to_string(written + filled + got) +
                                                                    " of " + std::to_string(expected) + " bytes");
            filled += got;
            left -= got;
            if (filled == Stager::kPiece) flush();
        }
    }
    flush();
    fclose(f);
    // the pinned buffers go away with this call: wait for the copies that still read them
    for (int i = 0; i < 2; ++i)
        if (stager.busy[i]) {
            const cudaError_t e = cudaEventSynchronize(stager.done[i]);
            if (e != cudaSuccess && result == RIBN_OK) result = note(file, RIBN_E_DRIVER, std::string("upload: ") + cudaGetErrorString(e));
        }
    cudaSetDevice(previous);
    return result;
}

}  // extern "C"
