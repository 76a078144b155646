// gguf.cc - weight-format table and a bounds-checked GGUF v2/v3 reader.
//
// Follows the reference parser's rules (crates/paddock-models/src/gguf.rs): little
// endian only, every count capped, every read checked against the buffer, a
// specific error for each way a file can be wrong, and a final pass that makes
// sure every tensor whose size is computable lies inside the file.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/paddock_host.h"

#define PDKH_EXPORT extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// weight formats
// ---------------------------------------------------------------------------
PDKH_EXPORT int pdk_ggml_block_layout(uint32_t raw, uint32_t* elems, uint32_t* bytes) {
    uint32_t e = 0, b = 0;
    switch (raw) {
        case 0: e = 1; b = 4; break;       // F32
        case 1: case 30: e = 1; b = 2; break;  // F16, BF16
        case 28: case 27: e = 1; b = 8; break; // F64, I64
        case 26: e = 1; b = 4; break;      // I32
        case 25: e = 1; b = 2; break;      // I16
        case 24: e = 1; b = 1; break;      // I8
        case 2: e = 32; b = 18; break;     // Q4_0
        case 3: e = 32; b = 20; break;     // Q4_1
        case 6: e = 32; b = 22; break;     // Q5_0
        case 7: e = 32; b = 24; break;     // Q5_1
        case 8: e = 32; b = 34; break;     // Q8_0
        case 9: e = 32; b = 36; break;     // Q8_1
        case 10: e = 256; b = 84; break;   // Q2_K
        case 11: e = 256; b = 110; break;  // Q3_K
        case 12: e = 256; b = 144; break;  // Q4_K
        case 13: e = 256; b = 176; break;  // Q5_K
        case 14: e = 256; b = 210; break;  // Q6_K
        case 15: e = 256; b = 292; break;  // Q8_K
        case 20: e = 32; b = 18; break;    // IQ4_NL
        case 23: e = 256; b = 136; break;  // IQ4_XS
        case 16: e = 256; b = 66; break;   // IQ2_XXS
        case 17: e = 256; b = 74; break;   // IQ2_XS
        case 22: e = 256; b = 82; break;   // IQ2_S
        case 18: e = 256; b = 98; break;   // IQ3_XXS
        case 21: e = 256; b = 110; break;  // IQ3_S
        case 19: e = 256; b = 50; break;   // IQ1_S
        case 29: e = 256; b = 56; break;   // IQ1_M
        case 39: e = 32; b = 17; break;    // MXFP4: E8M0 scale + 16 nibble bytes
        case 40: e = 64; b = 36; break;    // NVFP4: 4 UE4M3 scales + 32 nibble bytes
        case 142: e = 128; b = 34; break;  // PQ2_0
        case 143: e = 128; b = 28; break;  // PTQ1_0
        default: return 0;
    }
    if (elems) *elems = e;
    if (bytes) *bytes = b;
    return 1;
}

PDKH_EXPORT int pdk_ggml_byte_size(uint32_t raw, uint64_t n_elements, uint64_t* bytes) {
    uint32_t e, b;
    if (!pdk_ggml_block_layout(raw, &e, &b)) return 0;
    if (n_elements % e != 0) return 0;
    const uint64_t blocks = n_elements / e;
    if (blocks > UINT64_MAX / b) return 0;
    if (bytes) *bytes = blocks * b;
    return 1;
}

// ---------------------------------------------------------------------------
// GGUF
// ---------------------------------------------------------------------------
namespace {

constexpr uint64_t kMaxTensors = 262144, kMaxKv = 65536, kMaxString = 64ull << 20, kMaxArray = 16777216;
constexpr uint32_t kMaxArrayDepth = 4, kMaxDims = 8;

struct Tensor {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t raw_type = 0;
    uint64_t offset = 0;
    bool sized = false;
    uint64_t n_bytes = 0;
};

struct Meta {
    enum Kind { None, U64, I64, F64, Bool, Str, Array } kind = None;
    uint64_t u = 0;
    std::string s;
};

void set_err(char* err, size_t n, const char* fmt, ...) {
    if (!err || n == 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, n, fmt, ap);
    va_end(ap);
}

bool valid_utf8(const uint8_t* p, size_t n) {
    size_t i = 0;
    while (i < n) {
        const uint8_t c = p[i];
        size_t len;
        uint32_t cp;
        if (c < 0x80) { ++i; continue; }
        else if ((c & 0xE0) == 0xC0) { len = 2; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { len = 3; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { len = 4; cp = c & 0x07; }
        else return false;
        if (i + len > n) return false;
        for (size_t k = 1; k < len; ++k) {
            if ((p[i + k] & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (p[i + k] & 0x3F);
        }
        if ((len == 2 && cp < 0x80) || (len == 3 && cp < 0x800) || (len == 4 && cp < 0x10000)) return false;
        if (cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) return false;
        i += len;
    }
    return true;
}

struct Cursor {
    const uint8_t* bytes;
    size_t len;
    size_t pos = 0;
    int err = 0;
    char* msg;
    size_t msg_len;

    const uint8_t* take(uint64_t n) {
        if (err) return nullptr;
        if (n > len - pos) {
            err = PDK_GGUF_TRUNCATED;
            set_err(msg, msg_len, "file truncated: needed %llu bytes at offset %zu", (unsigned long long)n, pos);
            return nullptr;
        }
        const uint8_t* p = bytes + pos;
        pos += (size_t)n;
        return p;
    }
    template <typename T>
    T rd() {
        const uint8_t* p = take(sizeof(T));
        T v{};
        if (p) memcpy(&v, p, sizeof(T));
        return v;
    }
    bool str(std::string& out) {
        const size_t at = pos;
        const uint64_t n = rd<uint64_t>();
        if (err) return false;
        if (n > kMaxString) {
            err = PDK_GGUF_COUNT_TOO_LARGE;
            set_err(msg, msg_len, "string length count %llu exceeds cap %llu", (unsigned long long)n,
                    (unsigned long long)kMaxString);
            return false;
        }
        const uint8_t* p = take(n);
        if (!p) return false;
        if (!valid_utf8(p, (size_t)n)) {
            err = PDK_GGUF_BAD_UTF8;
            set_err(msg, msg_len, "string at offset %zu is not valid UTF-8", at);
            return false;
        }
        out.assign((const char*)p, (size_t)n);
        return true;
    }
    // GGUF value types: 0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32, 7 bool, 8 string, 9 array,
    // 10 u64, 11 i64, 12 f64
    bool value(uint32_t type, uint32_t depth, Meta* out) {
        switch (type) {
            case 0: { uint8_t v = rd<uint8_t>(); if (out) { out->kind = Meta::U64; out->u = v; } break; }
            case 1: { int8_t v = rd<int8_t>(); if (out) { out->kind = Meta::I64; out->u = (uint64_t)(int64_t)v; } break; }
            case 2: { uint16_t v = rd<uint16_t>(); if (out) { out->kind = Meta::U64; out->u = v; } break; }
            case 3: { int16_t v = rd<int16_t>(); if (out) { out->kind = Meta::I64; out->u = (uint64_t)(int64_t)v; } break; }
            case 4: { uint32_t v = rd<uint32_t>(); if (out) { out->kind = Meta::U64; out->u = v; } break; }
            case 5: { int32_t v = rd<int32_t>(); if (out) { out->kind = Meta::I64; out->u = (uint64_t)(int64_t)v; } break; }
            case 6: { (void)rd<uint32_t>(); if (out) out->kind = Meta::F64; break; }
            case 7: { uint8_t v = rd<uint8_t>(); if (out) { out->kind = Meta::Bool; out->u = v != 0; } break; }
            case 8: { std::string s; if (!str(s)) return false; if (out) { out->kind = Meta::Str; out->s = std::move(s); } break; }
            case 9: {
                if (depth >= kMaxArrayDepth) {
                    err = PDK_GGUF_ARRAY_TOO_DEEP;
                    set_err(msg, msg_len, "array nesting deeper than %u", kMaxArrayDepth);
                    return false;
                }
                const uint32_t et = rd<uint32_t>();
                const uint64_t n = rd<uint64_t>();
                if (err) return false;
                if (n > kMaxArray) {
                    err = PDK_GGUF_COUNT_TOO_LARGE;
                    set_err(msg, msg_len, "array count %llu exceeds cap %llu", (unsigned long long)n,
                            (unsigned long long)kMaxArray);
                    return false;
                }
                for (uint64_t i = 0; i < n; ++i)
                    if (!value(et, depth + 1, nullptr)) return false;
                if (out) { out->kind = Meta::Array; out->u = n; }
                break;
            }
            case 10: { uint64_t v = rd<uint64_t>(); if (out) { out->kind = Meta::U64; out->u = v; } break; }
            case 11: { int64_t v = rd<int64_t>(); if (out) { out->kind = Meta::I64; out->u = (uint64_t)v; } break; }
            case 12: { (void)rd<uint64_t>(); if (out) out->kind = Meta::F64; break; }
            default:
                err = PDK_GGUF_UNKNOWN_VALUE_TYPE;
                set_err(msg, msg_len, "unknown metadata value type %u", type);
                return false;
        }
        return err == 0;
    }
};

}  // namespace

struct PdkGguf {
    const uint8_t* bytes = nullptr;
    size_t len = 0;
    bool mapped = false;
    std::vector<uint8_t> owned;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
    std::unordered_map<std::string, Meta> meta;
};

static int parse_into(PdkGguf* g, char* err, size_t err_len) {
    Cursor c{g->bytes, g->len, 0, 0, err, err_len};
    if (c.rd<uint32_t>() != 0x46554747u || c.err) {
        set_err(err, err_len, "not a GGUF file (bad magic)");
        return PDK_GGUF_BAD_MAGIC;
    }
    g->version = c.rd<uint32_t>();
    if (c.err) return c.err;
    if (g->version < 2 || g->version > 3) {
        set_err(err, err_len, "GGUF version %u not supported (this parser reads v2/v3)", g->version);
        return PDK_GGUF_UNSUPPORTED_VERSION;
    }
    const uint64_t n_tensors = c.rd<uint64_t>();
    if (c.err) return c.err;
    if (n_tensors > kMaxTensors) {
        set_err(err, err_len, "tensor count %llu exceeds cap %llu", (unsigned long long)n_tensors,
                (unsigned long long)kMaxTensors);
        return PDK_GGUF_COUNT_TOO_LARGE;
    }
    const uint64_t n_kv = c.rd<uint64_t>();
    if (c.err) return c.err;
    if (n_kv > kMaxKv) {
        set_err(err, err_len, "metadata kv count %llu exceeds cap %llu", (unsigned long long)n_kv,
                (unsigned long long)kMaxKv);
        return PDK_GGUF_COUNT_TOO_LARGE;
    }
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key;
        if (!c.str(key)) return c.err;
        const uint32_t type = c.rd<uint32_t>();
        if (c.err) return c.err;
        Meta m;
        if (!c.value(type, 0, &m)) return c.err;
        g->meta[key] = std::move(m);
    }
    auto it = g->meta.find("general.alignment");
    if (it != g->meta.end() && (it->second.kind == Meta::U64 || it->second.kind == Meta::I64)) {
        const uint64_t a = it->second.u;
        if (a > 0xffffffffull || a == 0 || (a & (a - 1)) != 0) {
            set_err(err, err_len, "alignment %llu is not a power of two", (unsigned long long)a);
            return PDK_GGUF_BAD_ALIGNMENT;
        }
        g->alignment = a;
    }
    std::unordered_set<std::string> seen;
    g->tensors.reserve((size_t)(n_tensors < 4096 ? n_tensors : 4096));
    for (uint64_t i = 0; i < n_tensors; ++i) {
        Tensor t;
        if (!c.str(t.name)) return c.err;
        if (!seen.insert(t.name).second) {
            set_err(err, err_len, "duplicate tensor name %s", t.name.c_str());
            return PDK_GGUF_DUPLICATE_TENSOR;
        }
        const uint32_t n_dims = c.rd<uint32_t>();
        if (c.err) return c.err;
        if (n_dims > kMaxDims) {
            set_err(err, err_len, "tensor %s: %u dimensions (max %u)", t.name.c_str(), n_dims, kMaxDims);
            return PDK_GGUF_BAD_TENSOR;
        }
        for (uint32_t d = 0; d < n_dims; ++d) t.dims.push_back(c.rd<uint64_t>());
        t.raw_type = c.rd<uint32_t>();
        t.offset = c.rd<uint64_t>();
        if (c.err) return c.err;
        if (t.offset % g->alignment != 0) {
            set_err(err, err_len, "tensor %s: data offset %llu not aligned to %llu", t.name.c_str(),
                    (unsigned long long)t.offset, (unsigned long long)g->alignment);
            return PDK_GGUF_BAD_TENSOR;
        }
        // element count with overflow check, then the byte size if the layout is known
        uint64_t n = 1;
        bool overflow = false;
        for (uint64_t d : t.dims) {
            if (d != 0 && n > UINT64_MAX / d) { overflow = true; break; }
            n *= d;
        }
        t.sized = !overflow && pdk_ggml_byte_size(t.raw_type, n, &t.n_bytes) != 0;
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    g->data_offset = ((uint64_t)c.pos + g->alignment - 1) / g->alignment * g->alignment;
    const uint64_t data_len = g->len > g->data_offset ? g->len - g->data_offset : 0;
    for (const Tensor& t : g->tensors) {
        if (t.sized) {
            if (t.n_bytes > UINT64_MAX - t.offset || t.offset + t.n_bytes > data_len) {
                set_err(err, err_len, "tensor %s: extends past end of file (offset %llu + %llu bytes > data section %llu)",
                        t.name.c_str(), (unsigned long long)t.offset, (unsigned long long)t.n_bytes,
                        (unsigned long long)data_len);
                return PDK_GGUF_BAD_TENSOR;
            }
        } else if (t.offset >= data_len && !(t.offset == 0 && data_len == 0)) {
            set_err(err, err_len, "tensor %s: offset %llu outside data section %llu", t.name.c_str(),
                    (unsigned long long)t.offset, (unsigned long long)data_len);
            return PDK_GGUF_BAD_TENSOR;
        }
    }
    return PDK_GGUF_OK;
}

PDKH_EXPORT int pdk_gguf_parse(const void* bytes, size_t len, PdkGguf** out, char* err, size_t err_len) {
    if (!out) return PDK_GGUF_IO;
    *out = nullptr;
    PdkGguf* g = new PdkGguf();
    g->owned.assign((const uint8_t*)bytes, (const uint8_t*)bytes + len);
    g->bytes = g->owned.data();
    g->len = len;
    const int rc = parse_into(g, err, err_len);
    if (rc != PDK_GGUF_OK) { delete g; return rc; }
    *out = g;
    return rc;
}

PDKH_EXPORT int pdk_gguf_open(const char* path, PdkGguf** out, char* err, size_t err_len) {
    if (!out) return PDK_GGUF_IO;
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { set_err(err, err_len, "cannot open %s", path); return PDK_GGUF_IO; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        set_err(err, err_len, "cannot stat %s (or empty file)", path);
        return st.st_size == 0 ? PDK_GGUF_TRUNCATED : PDK_GGUF_IO;
    }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { set_err(err, err_len, "cannot map %s", path); return PDK_GGUF_IO; }
    PdkGguf* g = new PdkGguf();
    g->bytes = (const uint8_t*)p;
    g->len = (size_t)st.st_size;
    g->mapped = true;
    const int rc = parse_into(g, err, err_len);
    if (rc != PDK_GGUF_OK) { pdk_gguf_close(g); return rc; }
    *out = g;
    return rc;
}

PDKH_EXPORT void pdk_gguf_close(PdkGguf* g) {
    if (!g) return;
    if (g->mapped && g->bytes) munmap((void*)g->bytes, g->len);
    delete g;
}

PDKH_EXPORT uint32_t pdk_gguf_version(const PdkGguf* g) { return g->version; }
PDKH_EXPORT uint64_t pdk_gguf_alignment(const PdkGguf* g) { return g->alignment; }
PDKH_EXPORT uint64_t pdk_gguf_data_offset(const PdkGguf* g) { return g->data_offset; }
PDKH_EXPORT uint64_t pdk_gguf_tensor_count(const PdkGguf* g) { return g->tensors.size(); }

static void fill_info(const Tensor& t, const char** name, uint32_t* n_dims, uint64_t dims[8], uint32_t* raw_type,
                      uint64_t* offset, uint64_t* n_bytes) {
    if (name) *name = t.name.c_str();
    if (n_dims) *n_dims = (uint32_t)t.dims.size();
    if (dims)
        for (size_t d = 0; d < 8; ++d) dims[d] = d < t.dims.size() ? t.dims[d] : 1;
    if (raw_type) *raw_type = t.raw_type;
    if (offset) *offset = t.offset;
    if (n_bytes) *n_bytes = t.sized ? t.n_bytes : 0;
}

PDKH_EXPORT int pdk_gguf_tensor_at(const PdkGguf* g, uint64_t i, const char** name, uint32_t* n_dims,
                                   uint64_t dims[8], uint32_t* raw_type, uint64_t* offset, uint64_t* n_bytes) {
    if (i >= g->tensors.size()) return PDK_GGUF_NOT_FOUND;
    fill_info(g->tensors[(size_t)i], name, n_dims, dims, raw_type, offset, n_bytes);
    return PDK_GGUF_OK;
}

PDKH_EXPORT int pdk_gguf_tensor_bytes(const PdkGguf* g, const char* name, const void** data, uint64_t* n_bytes,
                                      uint32_t* raw_type, uint32_t* n_dims, uint64_t dims[8]) {
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return PDK_GGUF_NOT_FOUND;
    const Tensor& t = g->tensors[it->second];
    if (!t.sized) return PDK_GGUF_BAD_TENSOR;
    // re-check against the mapping actually held (mapped.rs:343 does the same)
    if (g->data_offset > g->len || t.offset > g->len - g->data_offset ||
        t.n_bytes > g->len - g->data_offset - t.offset)
        return PDK_GGUF_BAD_TENSOR;
    fill_info(t, nullptr, n_dims, dims, raw_type, nullptr, n_bytes);
    if (data) *data = g->bytes + g->data_offset + t.offset;
    return PDK_GGUF_OK;
}

PDKH_EXPORT int pdk_gguf_meta_u64(const PdkGguf* g, const char* key, uint64_t* value) {
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return PDK_GGUF_NOT_FOUND;
    const Meta& m = it->second;
    if (m.kind == Meta::U64 || m.kind == Meta::Bool || (m.kind == Meta::I64 && (int64_t)m.u >= 0)) {
        if (value) *value = m.u;
        return PDK_GGUF_OK;
    }
    return PDK_GGUF_NOT_FOUND;
}

PDKH_EXPORT int pdk_gguf_meta_str(const PdkGguf* g, const char* key, const char** value) {
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.kind != Meta::Str) return PDK_GGUF_NOT_FOUND;
    if (value) *value = it->second.s.c_str();
    return PDK_GGUF_OK;
}

// ---- split families (crates/paddock-models/src/split.rs, mapped.rs:176-290) --------------------
// A model shipped as N whole GGUF files `<prefix>-%05d-of-%05d.gguf` (numbers 1-based in the
// name).  Every shard carries split.no (0-based) and split.count; the first one also carries
// split.tensors.count, the size of the union.  A family opens through its first shard only; a
// shard that is absent, out of place or short of tensors is an error, never a smaller model.

namespace {
constexpr uint64_t kMaxSplits = 2048;   // the field is a u16 and real families are single digits

struct SplitName {
    std::string prefix;
    uint32_t no = 0, count = 0;   // no is 1-based
    std::string sibling(uint32_t no_1based) const {
        char tail[40];
        snprintf(tail, sizeof tail, "-%05u-of-%05u.gguf", no_1based, count);
        return prefix + tail;
    }
};

// exactly "<prefix>-DDDDD-of-DDDDD.gguf", prefix not empty, 1 <= no <= count
bool parse_split_name(const std::string& path, SplitName* out) {
    static const char kExt[] = ".gguf";
    const size_t tail = 1 + 5 + 4 + 5 + 5;   // "-" no "-of-" count ".gguf"
    if (path.size() <= tail || path.compare(path.size() - 5, 5, kExt) != 0) return false;
    const size_t at = path.size() - tail;
    if (path[at] != '-' || path.compare(at + 6, 4, "-of-") != 0) return false;
    uint32_t field[2] = {0, 0};
    const size_t start[2] = {at + 1, at + 10};
    for (int f = 0; f < 2; ++f)
        for (size_t i = 0; i < 5; ++i) {
            const char ch = path[start[f] + i];
            if (ch < '0' || ch > '9') return false;
            field[f] = field[f] * 10u + (uint32_t)(ch - '0');
        }
    if (field[0] == 0 || field[1] == 0 || field[0] > field[1]) return false;
    out->prefix = path.substr(0, at);
    out->no = field[0];
    out->count = field[1];
    return true;
}
}  // namespace

struct PdkGgufFamily {
    std::vector<PdkGguf*> shards;
    std::vector<std::string> paths;
    std::vector<std::pair<uint32_t, uint32_t>> order;                       // (shard, index in shard), family order
    std::unordered_map<std::string, std::pair<uint32_t, uint32_t>> by_name;
    ~PdkGgufFamily() {
        for (PdkGguf* g : shards) pdk_gguf_close(g);
    }
};

PDKH_EXPORT int pdk_split_name_parse(const char* path, char* prefix, size_t prefix_len, uint32_t* no_1based,
                                     uint32_t* count) {
    SplitName n;
    if (!path || !parse_split_name(path, &n)) return 1;
    if (prefix && prefix_len) snprintf(prefix, prefix_len, "%s", n.prefix.c_str());
    if (no_1based) *no_1based = n.no;
    if (count) *count = n.count;
    return 0;
}

static int family_fail(PdkGgufFamily* f, int code) {
    delete f;
    return code;
}

PDKH_EXPORT int pdk_gguf_family_open(const char* path, PdkGgufFamily** out, char* err, size_t err_len) {
    if (!out || !path) return PDK_MAP_IO;
    *out = nullptr;
    PdkGgufFamily* f = new PdkGgufFamily();
    PdkGguf* first = nullptr;
    int rc = pdk_gguf_open(path, &first, err, err_len);
    if (rc != PDK_GGUF_OK) return family_fail(f, rc == PDK_GGUF_IO ? PDK_MAP_IO : PDK_MAP_PARSE);
    f->shards.push_back(first);
    f->paths.push_back(path);

    uint64_t split_count = 0;
    if (pdk_gguf_meta_u64(first, "split.count", &split_count) != PDK_GGUF_OK) split_count = 0;
    if (split_count > 1) {
        if (split_count > kMaxSplits) {
            set_err(err, err_len, "split.count %llu exceeds the cap of %llu", (unsigned long long)split_count,
                    (unsigned long long)kMaxSplits);
            return family_fail(f, PDK_MAP_TOO_MANY_SPLITS);
        }
        uint64_t no = 0;
        if (pdk_gguf_meta_u64(first, "split.no", &no) != PDK_GGUF_OK) {
            set_err(err, err_len, "%s: split model without split.no", path);
            return family_fail(f, PDK_MAP_MISSING_SPLIT_KEY);
        }
        // the file name is the only locator of the siblings, so it has to agree with the metadata first
        SplitName name;
        if (!parse_split_name(path, &name) || name.count != split_count) {
            set_err(err, err_len, "%s: split.count = %llu but the name is not ...-00001-of-%05llu.gguf", path,
                    (unsigned long long)split_count, (unsigned long long)split_count);
            return family_fail(f, PDK_MAP_SPLIT_NAME_MISMATCH);
        }
        if (no != 0) {
            set_err(err, err_len, "%s is shard %u of %u: load the model through %s", path, name.no, name.count,
                    name.sibling(1).c_str());
            return family_fail(f, PDK_MAP_NOT_FIRST_SPLIT);
        }
        for (uint64_t idx = 1; idx < split_count; ++idx) {
            const std::string sib = name.sibling((uint32_t)idx + 1u);
            PdkGguf* g = nullptr;
            rc = pdk_gguf_open(sib.c_str(), &g, err, err_len);
            if (rc != PDK_GGUF_OK) return family_fail(f, rc == PDK_GGUF_IO ? PDK_MAP_IO : PDK_MAP_PARSE);
            f->shards.push_back(g);
            f->paths.push_back(sib);
            const char* keys[2] = {"split.no", "split.count"};
            const uint64_t want[2] = {idx, split_count};
            for (int k = 0; k < 2; ++k) {
                uint64_t got = 0;
                if (pdk_gguf_meta_u64(g, keys[k], &got) != PDK_GGUF_OK) {
                    set_err(err, err_len, "%s: split model without %s", sib.c_str(), keys[k]);
                    return family_fail(f, PDK_MAP_MISSING_SPLIT_KEY);
                }
                if (got != want[k]) {
                    set_err(err, err_len, "%s: %s = %llu, expected %llu", sib.c_str(), keys[k], (unsigned long long)got,
                            (unsigned long long)want[k]);
                    return family_fail(f, PDK_MAP_SHARD_MISMATCH);
                }
            }
        }
    }

    for (uint32_t s = 0; s < f->shards.size(); ++s) {
        const std::vector<Tensor>& ts = f->shards[s]->tensors;
        for (uint32_t i = 0; i < ts.size(); ++i) {
            auto ins = f->by_name.emplace(ts[i].name, std::make_pair(s, i));
            if (!ins.second) {
                set_err(err, err_len, "tensor %s appears in shard %u and in shard %u", ts[i].name.c_str(),
                        ins.first->second.first, s);
                return family_fail(f, PDK_MAP_DUPLICATE_ACROSS_SHARDS);
            }
            f->order.emplace_back(s, i);
        }
    }
    if (split_count > 1) {
        uint64_t expected = 0;
        if (pdk_gguf_meta_u64(first, "split.tensors.count", &expected) != PDK_GGUF_OK) {
            set_err(err, err_len, "%s: split model without split.tensors.count", path);
            return family_fail(f, PDK_MAP_MISSING_SPLIT_KEY);
        }
        if (expected != f->by_name.size()) {
            set_err(err, err_len, "split.tensors.count says %llu tensors but the %zu shards hold %zu",
                    (unsigned long long)expected, f->shards.size(), f->by_name.size());
            return family_fail(f, PDK_MAP_TENSOR_COUNT_MISMATCH);
        }
    }
    *out = f;
    return PDK_MAP_OK;
}

PDKH_EXPORT void pdk_gguf_family_close(PdkGgufFamily* f) { delete f; }
PDKH_EXPORT uint64_t pdk_gguf_family_shard_count(const PdkGgufFamily* f) { return f->shards.size(); }
PDKH_EXPORT uint64_t pdk_gguf_family_tensor_count(const PdkGgufFamily* f) { return f->order.size(); }
PDKH_EXPORT uint64_t pdk_gguf_family_total_len(const PdkGgufFamily* f) {
    uint64_t n = 0;
    for (const PdkGguf* g : f->shards) n += g->len;
    return n;
}
PDKH_EXPORT const PdkGguf* pdk_gguf_family_shard(const PdkGgufFamily* f, uint64_t shard) {
    return shard < f->shards.size() ? f->shards[(size_t)shard] : nullptr;
}
PDKH_EXPORT const char* pdk_gguf_family_shard_path(const PdkGgufFamily* f, uint64_t shard) {
    return shard < f->paths.size() ? f->paths[(size_t)shard].c_str() : nullptr;
}

PDKH_EXPORT int pdk_gguf_family_tensor_at(const PdkGgufFamily* f, uint64_t i, const char** name, uint32_t* n_dims,
                                          uint64_t dims[8], uint32_t* raw_type, uint64_t* n_bytes, uint32_t* shard) {
    if (i >= f->order.size()) return PDK_MAP_NO_SUCH_TENSOR;
    const auto at = f->order[(size_t)i];
    fill_info(f->shards[at.first]->tensors[at.second], name, n_dims, dims, raw_type, nullptr, n_bytes);
    if (shard) *shard = at.first;
    return PDK_MAP_OK;
}

PDKH_EXPORT int pdk_gguf_family_tensor_bytes(const PdkGgufFamily* f, const char* name, const void** data,
                                             uint64_t* n_bytes, uint32_t* raw_type, uint32_t* n_dims, uint64_t dims[8],
                                             uint32_t* shard) {
    auto it = f->by_name.find(name);
    if (it == f->by_name.end()) return PDK_MAP_NO_SUCH_TENSOR;
    const PdkGguf* g = f->shards[it->second.first];
    const Tensor& t = g->tensors[it->second.second];
    if (!t.sized) return PDK_MAP_UNSIZABLE;
    if (g->data_offset > g->len || t.offset > g->len - g->data_offset || t.n_bytes > g->len - g->data_offset - t.offset)
        return PDK_MAP_OUT_OF_RANGE;
    fill_info(t, nullptr, n_dims, dims, raw_type, nullptr, n_bytes);
    if (data) *data = g->bytes + g->data_offset + t.offset;
    if (shard) *shard = it->second.first;
    return PDK_MAP_OK;
}
