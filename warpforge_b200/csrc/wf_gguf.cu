// GGUF container reader on the native side of the boundary: the file is memory-mapped, its header,
// metadata and tensor directory are parsed once, and a quantized tensor goes from the mapping to a
// device-resident weight without passing through the host language.  Follows the reader at
// warpforge-data/src/main/java/io/surfworks/warpforge/data/format/GGUF.java:96-176 (open: magic,
// version 1..3, counts, key/values with general.alignment, tensor infos, aligned data offset),
// :221-225 (a tensor is the slice [dataOffset + offset, + size)), :294-351 (ggml type table and block
// sizes) and :357-470 (little-endian scalar / string / array decoding); same messages for the same
// failures.  Every read is bounds-checked against the mapping: a truncated or corrupt file is an
// error code, never a fault.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "wf_common.cuh"

namespace wf {

constexpr uint32_t GGUF_MAGIC = 0x46554747u;  // "GGUF" little-endian (GGUF.java:46)
constexpr int GGUF_DEFAULT_ALIGNMENT = 32;    // GGUF.java:49
constexpr uint32_t GGUF_HANDLE_MAGIC = 0x47475546u;

struct GgufTensor {
    std::string name;
    int ggml_type = 0;
    std::vector<int64_t> dims;  // file order: dims[0] varies fastest
    int64_t offset = 0;         // relative to the data section
    int64_t size = 0;           // bytes
};

struct GgufFile {
    uint32_t magic = GGUF_HANDLE_MAGIC;
    const uint8_t* map = nullptr;
    int64_t file_size = 0;
    int version = 0;
    int alignment = GGUF_DEFAULT_ALIGNMENT;
    int64_t data_offset = 0;
    std::vector<GgufTensor> tensors;
    std::map<std::string, size_t> by_name;
    std::vector<std::pair<std::string, std::string>> metadata;  // values rendered as text
};

static std::mutex g_gguf_mu;
static std::vector<GgufFile*> g_gguf_files;

static GgufFile* get_gguf(int64_t h) {
    std::lock_guard<std::mutex> lk(g_gguf_mu);
    for (GgufFile* f : g_gguf_files)
        if (reinterpret_cast<int64_t>(f) == h && f->magic == GGUF_HANDLE_MAGIC) return f;
    return nullptr;
}

// ggml type -> bytes for `elements` values (GGUF.java:294-351); -1 for a type the reader does not know
static int64_t ggml_tensor_bytes(int t, int64_t elements) {
    switch (t) {
        case 0: return elements * 4;                  // F32
        case 1: return elements * 2;                  // F16
        case 2: return (elements + 31) / 32 * 18;     // Q4_0
        case 3: return (elements + 31) / 32 * 20;     // Q4_1
        case 6: return (elements + 31) / 32 * 22;     // Q5_0
        case 7: return (elements + 31) / 32 * 24;     // Q5_1
        case 8: return (elements + 31) / 32 * 34;     // Q8_0
        case 9: return elements;                      // Q8_1 (the reference's "fallback": one byte per element)
        case 14: return (elements + 255) / 256 * 144; // Q4_K
        case 16: return (elements + 255) / 256 * 176; // Q5_K
        case 18: return elements * 2;                 // BF16
        case 26: case 27: case 28: return elements;   // F8_E5M2, F8_E4M3, I8
        case 29: return elements * 2;                 // I16
        case 30: return elements * 4;                 // I32
        case 31: case 32: return elements * 8;        // I64, F64
        default: return -1;
    }
}

struct Cursor {
    const uint8_t* p;
    int64_t size, pos = 0;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (!ok || pos + (int64_t)sizeof(T) > size) {
            ok = false;
            return v;
        }
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str(int version) {  // length is 64-bit from version 2 on (GGUF.java:399-408)
        const uint64_t n = version >= 2 ? get<uint64_t>() : get<uint32_t>();
        if (!ok || n > (uint64_t)(size - pos)) {
            ok = false;
            return std::string();
        }
        std::string s(reinterpret_cast<const char*>(p + pos), (size_t)n);
        pos += (int64_t)n;
        return s;
    }
};

// one metadata value as text; *number receives integer values (for general.alignment)
static bool read_value(Cursor& c, int version, uint32_t type, bool in_array, std::string& text, int64_t* number, std::string& err) {
    char buf[64];
    switch (type) {
        case 0: { uint8_t v = c.get<uint8_t>(); snprintf(buf, sizeof buf, "%u", v); text = buf; if (number) *number = v; break; }
        case 1: { int8_t v = c.get<int8_t>(); snprintf(buf, sizeof buf, "%d", v); text = buf; if (number) *number = v; break; }
        case 2: { uint16_t v = c.get<uint16_t>(); snprintf(buf, sizeof buf, "%u", v); text = buf; if (number) *number = v; break; }
        case 3: { int16_t v = c.get<int16_t>(); snprintf(buf, sizeof buf, "%d", v); text = buf; if (number) *number = v; break; }
        case 4: { uint32_t v = c.get<uint32_t>(); snprintf(buf, sizeof buf, "%u", v); text = buf; if (number) *number = v; break; }
        case 5: { int32_t v = c.get<int32_t>(); snprintf(buf, sizeof buf, "%d", v); text = buf; if (number) *number = v; break; }
        case 6: { float v = c.get<float>(); snprintf(buf, sizeof buf, "%.9g", v); text = buf; break; }
        case 7: { uint8_t v = c.get<uint8_t>(); text = v ? "true" : "false"; break; }
        case 8: text = c.str(version); break;
        case 9: {
            if (in_array) {  // the reference's element decoder has no case for nested arrays
                err = "Unknown GGUF value type: 9";
                return false;
            }
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = version >= 2 ? c.get<uint64_t>() : c.get<uint32_t>();
            if (!c.ok || n > (uint64_t)INT32_MAX) {
                err = "Array too long";
                return false;
            }
            text = "[";
            for (uint64_t i = 0; i < n; i++) {
                std::string e;
                if (!read_value(c, version, et, true, e, nullptr, err)) return false;
                if (!c.ok) break;
                if (i < 8) text += (i ? ", " : "") + e;
            }
            if (n > 8) text += ", ...";
            text += "]";
            break;
        }
        case 10: { uint64_t v = c.get<uint64_t>(); snprintf(buf, sizeof buf, "%llu", (unsigned long long)v); text = buf; if (number) *number = (int64_t)v; break; }
        case 11: { int64_t v = c.get<int64_t>(); snprintf(buf, sizeof buf, "%lld", (long long)v); text = buf; if (number) *number = v; break; }
        case 12: { double v = c.get<double>(); snprintf(buf, sizeof buf, "%.17g", v); text = buf; break; }
        default:
            snprintf(buf, sizeof buf, "Unknown GGUF value type: %u", type);
            err = buf;
            return false;
    }
    return true;
}

static void put_err(char* err, int64_t n, const std::string& msg) {
    if (err && n > 0) snprintf(err, (size_t)n, "%s", msg.c_str());
}

}  // namespace wf

using namespace wf;

extern "C" {

int wf_gguf_open(const char* path, int64_t* gguf, char* err, int64_t err_len) {
    if (!path || !gguf) return WF_ERR_INVALID_ARGUMENT;
    *gguf = 0;
    char msg[256];
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        snprintf(msg, sizeof msg, "cannot open %s", path);
        put_err(err, err_len, msg);
        return WF_ERR_GGUF;
    }
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        put_err(err, err_len, "cannot stat the file");
        return WF_ERR_GGUF;
    }
    if (st.st_size < 24) {
        close(fd);
        snprintf(msg, sizeof msg, "File too small to be a GGUF file: %lld bytes", (long long)st.st_size);
        put_err(err, err_len, msg);
        return WF_ERR_GGUF;
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) {
        put_err(err, err_len, "mmap failed");
        return WF_ERR_GGUF;
    }
    GgufFile* f = new GgufFile();
    f->map = static_cast<const uint8_t*>(map);
    f->file_size = st.st_size;
    auto fail = [&](const std::string& m) {
        put_err(err, err_len, m);
        munmap(map, (size_t)st.st_size);
        delete f;
        return WF_ERR_GGUF;
    };
    Cursor c{f->map, f->file_size};
    const uint32_t magic = c.get<uint32_t>();
    if (magic != GGUF_MAGIC) {
        snprintf(msg, sizeof msg, "Invalid GGUF magic: expected 0x%08X, got 0x%08X", GGUF_MAGIC, magic);
        return fail(msg);
    }
    f->version = (int)c.get<uint32_t>();
    if (f->version < 1 || f->version > 3) {
        snprintf(msg, sizeof msg, "Unsupported GGUF version: %d", f->version);
        return fail(msg);
    }
    const int64_t n_tensors = c.get<int64_t>(), n_kv = c.get<int64_t>();
    if (!c.ok || n_tensors < 0 || n_kv < 0 || n_tensors > f->file_size || n_kv > f->file_size) return fail("corrupt counts in the GGUF header");
    for (int64_t i = 0; i < n_kv; i++) {
        const std::string key = c.str(f->version);
        const uint32_t type = c.get<uint32_t>();
        std::string text, verr;
        int64_t number = INT64_MIN;
        if (!read_value(c, f->version, type, false, text, &number, verr)) return fail(verr);
        if (!c.ok) return fail("truncated GGUF metadata");
        if (key == "general.alignment" && number != INT64_MIN) f->alignment = (int)number;
        f->metadata.emplace_back(key, text);
    }
    if (f->alignment <= 0) return fail("general.alignment must be positive");
    for (int64_t i = 0; i < n_tensors; i++) {
        GgufTensor t;
        t.name = c.str(f->version);
        const int32_t nd = c.get<int32_t>();
        if (!c.ok || nd < 0 || nd > 8) return fail("corrupt tensor info in the GGUF header");
        int64_t elements = 1;
        for (int d = 0; d < nd; d++) {
            const int64_t v = c.get<int64_t>();
            if (v < 0 || (v > 0 && elements > INT64_MAX / v)) return fail("tensor dimensions overflow");
            t.dims.push_back(v);
            elements *= v;
        }
        t.ggml_type = c.get<int32_t>();
        t.offset = c.get<int64_t>();
        if (!c.ok) return fail("truncated GGUF tensor directory");
        t.size = ggml_tensor_bytes(t.ggml_type, elements);
        if (t.size < 0) {
            snprintf(msg, sizeof msg, "Unknown GGML type: %d", t.ggml_type);
            return fail(msg);
        }
        f->by_name[t.name] = f->tensors.size();
        f->tensors.push_back(std::move(t));
    }
    f->data_offset = (c.pos + f->alignment - 1) / f->alignment * f->alignment;
    {
        std::lock_guard<std::mutex> lk(g_gguf_mu);
        g_gguf_files.push_back(f);
    }
    *gguf = reinterpret_cast<int64_t>(f);
    return WF_OK;
}

int wf_gguf_close(int64_t gguf) {
    GgufFile* f = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_gguf_mu);
        for (size_t i = 0; i < g_gguf_files.size(); i++)
            if (reinterpret_cast<int64_t>(g_gguf_files[i]) == gguf) {
                f = g_gguf_files[i];
                g_gguf_files.erase(g_gguf_files.begin() + i);
                break;
            }
    }
    if (!f) return WF_ERR_INVALID_HANDLE;
    munmap(const_cast<uint8_t*>(f->map), (size_t)f->file_size);
    f->magic = 0;
    delete f;
    return WF_OK;
}

int wf_gguf_info(int64_t gguf, int* version, int64_t* tensor_count, int64_t* metadata_count, int64_t* data_offset,
                 int* alignment, int64_t* file_size) {
    GgufFile* f = get_gguf(gguf);
    if (!f) return WF_ERR_INVALID_HANDLE;
    if (version) *version = f->version;
    if (tensor_count) *tensor_count = (int64_t)f->tensors.size();
    if (metadata_count) *metadata_count = (int64_t)f->metadata.size();
    if (data_offset) *data_offset = f->data_offset;
    if (alignment) *alignment = f->alignment;
    if (file_size) *file_size = f->file_size;
    return WF_OK;
}

int wf_gguf_tensor_name(int64_t gguf, int64_t index, char* buf, int64_t n) {
    GgufFile* f = get_gguf(gguf);
    if (!f) return WF_ERR_INVALID_HANDLE;
    if (!buf || n <= 0 || index < 0 || index >= (int64_t)f->tensors.size()) return WF_ERR_INVALID_ARGUMENT;
    snprintf(buf, (size_t)n, "%s", f->tensors[(size_t)index].name.c_str());
    return WF_OK;
}

int wf_gguf_tensor_info(int64_t gguf, const char* name, int* ggml_type, int* n_dims, int64_t* dims8, int64_t* offset, int64_t* size) {
    GgufFile* f = get_gguf(gguf);
    if (!f) return WF_ERR_INVALID_HANDLE;
    if (!name) return WF_ERR_INVALID_ARGUMENT;
    auto it = f->by_name.find(name);
    if (it == f->by_name.end()) return WF_ERR_INVALID_ARGUMENT;  // "No tensor named: ..." (GGUF.java:206-212)
    const GgufTensor& t = f->tensors[it->second];
    if (ggml_type) *ggml_type = t.ggml_type;
    if (n_dims) *n_dims = (int)t.dims.size();
    if (dims8)
        for (size_t d = 0; d < 8; d++) dims8[d] = d < t.dims.size() ? t.dims[d] : 1;
    if (offset) *offset = t.offset;
    if (size) *size = t.size;
    return WF_OK;
}

int wf_gguf_tensor_data(int64_t gguf, const char* name, const void** data, int64_t* size) {
    GgufFile* f = get_gguf(gguf);
    if (!f) return WF_ERR_INVALID_HANDLE;
    if (!name || !data) return WF_ERR_INVALID_ARGUMENT;
    auto it = f->by_name.find(name);
    if (it == f->by_name.end()) return WF_ERR_INVALID_ARGUMENT;
    const GgufTensor& t = f->tensors[it->second];
    if (t.offset < 0 || f->data_offset + t.offset > f->file_size || t.size > f->file_size - f->data_offset - t.offset)
        return WF_ERR_GGUF;  // the directory points outside the file
    *data = f->map + f->data_offset + t.offset;
    if (size) *size = t.size;
    return WF_OK;
}

int wf_gguf_metadata(int64_t gguf, int64_t index, char* key, int64_t key_len, char* value, int64_t value_len) {
    GgufFile* f = get_gguf(gguf);
    if (!f) return WF_ERR_INVALID_HANDLE;
    if (index < 0 || index >= (int64_t)f->metadata.size()) return WF_ERR_INVALID_ARGUMENT;
    if (key && key_len > 0) snprintf(key, (size_t)key_len, "%s", f->metadata[(size_t)index].first.c_str());
    if (value && value_len > 0) snprintf(value, (size_t)value_len, "%s", f->metadata[(size_t)index].second.c_str());
    return WF_OK;
}

int wf_gguf_upload(int64_t ctx, int64_t gguf, const char* name, int shard_rank, int shard_world, int q4_0_order, int64_t* weight) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    GgufFile* f = get_gguf(gguf);
    if (!f) return set_error(c, WF_ERR_INVALID_HANDLE, "bad GGUF handle");
    if (!name || !weight) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer");
    *weight = 0;
    auto it = f->by_name.find(name);
    if (it == f->by_name.end()) return set_error(c, WF_ERR_INVALID_ARGUMENT, "No tensor named: %s", name);
    const GgufTensor& t = f->tensors[it->second];
    // a linear weight is stored with dims {K, N}: dims[0] = K varies fastest, blocks run along K
    if (t.dims.size() != 2) return set_error(c, WF_ERR_SHAPE, "tensor %s has %d dims; a linear weight has 2", name, (int)t.dims.size());
    const void* data = nullptr;
    int64_t size = 0;
    int rc = wf_gguf_tensor_data(gguf, name, &data, &size);
    if (rc != WF_OK) return set_error(c, rc, "tensor %s lies outside the file", name);
    if (q4_0_order != WF_Q4_0_ORDER_REFERENCE && q4_0_order != WF_Q4_0_ORDER_GGML)
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "q4_0_order %d is neither REFERENCE nor GGML", q4_0_order);
    return weight_upload(c, t.ggml_type, data, t.dims[1], t.dims[0], shard_rank, shard_world, q4_0_order, weight);
}

}  // extern "C"
