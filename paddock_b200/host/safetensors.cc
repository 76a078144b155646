// safetensors.cc - safetensors reader (single file or sharded directory), the
// ModelOpt / llm-compressor quantized views over it, and the GGUF-NVFP4 row repack.
//
// File layout: u64 little-endian header length, a JSON object
// {name: {dtype, shape, data_offsets:[begin,end]}, "__metadata__": {...}}, then the
// data section.  Every offset pair is validated against the mapping and against
// shape x dtype size before any pointer is handed out
// (crates/paddock-models/src/safetensors.rs:102-190).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/paddock_host.h"
#include "json_min.h"

#define PDKH_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

void set_err(char* err, size_t n, const char* fmt, ...) {
    if (!err || n == 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, n, fmt, ap);
    va_end(ap);
}

struct Mapping {
    const uint8_t* p = nullptr;
    size_t len = 0;
    ~Mapping() {
        if (p) munmap((void*)p, len);
    }
};

struct StTensor {
    uint32_t dtype = PDK_ST_OTHER;
    std::vector<uint64_t> shape;
    const uint8_t* data = nullptr;
    uint64_t n_bytes = 0;
};

uint32_t parse_dtype(const std::string& s) {
    if (s == "F8_E4M3") return PDK_ST_F8_E4M3;
    if (s == "BF16") return PDK_ST_BF16;
    if (s == "F16") return PDK_ST_F16;
    if (s == "F32") return PDK_ST_F32;
    if (s == "U8") return PDK_ST_U8;
    if (s == "U32") return PDK_ST_U32;
    if (s == "I64") return PDK_ST_I64;
    return PDK_ST_OTHER;
}

uint64_t dtype_bytes(uint32_t d) {
    switch (d) {
        case PDK_ST_F8_E4M3: case PDK_ST_U8: return 1;
        case PDK_ST_BF16: case PDK_ST_F16: return 2;
        case PDK_ST_F32: case PDK_ST_U32: return 4;
        case PDK_ST_I64: return 8;
        default: return 0;  // Other: callers must reject, not guess
    }
}

bool map_file(const std::string& path, std::unique_ptr<Mapping>& out, char* err, size_t err_len) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) { set_err(err, err_len, "cannot open %s", path.c_str()); return false; }
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); set_err(err, err_len, "cannot stat %s", path.c_str()); return false; }
    out.reset(new Mapping());
    if (st.st_size > 0) {
        void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (p == MAP_FAILED) { close(fd); set_err(err, err_len, "cannot map %s", path.c_str()); return false; }
        out->p = (const uint8_t*)p;
        out->len = (size_t)st.st_size;
    }
    close(fd);
    return true;
}

}  // namespace

struct PdkSafetensors {
    std::vector<std::unique_ptr<Mapping>> maps;
    std::unordered_map<std::string, StTensor> tensors;
    std::vector<std::unique_ptr<std::vector<float>>> owned_scales;
};

static int load_file(PdkSafetensors* s, const std::string& path, char* err, size_t err_len) {
    std::unique_ptr<Mapping> m;
    if (!map_file(path, m, err, err_len)) return PDK_ST_IO;
    if (m->len < 8) { set_err(err, err_len, "%s: file shorter than the length prefix", path.c_str()); return PDK_ST_HEADER; }
    uint64_t hlen;
    memcpy(&hlen, m->p, 8);
    if (hlen > m->len - 8) { set_err(err, err_len, "%s: header length %llu exceeds file", path.c_str(), (unsigned long long)hlen); return PDK_ST_HEADER; }
    const uint64_t data_off = 8 + hlen, data_len = m->len - data_off;
    pdkjson::Value root;
    pdkjson::Parser parser((const char*)m->p + 8, (size_t)hlen);
    if (!parser.parse(root)) { set_err(err, err_len, "%s: header is not valid JSON", path.c_str()); return PDK_ST_HEADER; }
    if (root.kind != pdkjson::Value::Object) { set_err(err, err_len, "%s: header is not a JSON object", path.c_str()); return PDK_ST_HEADER; }
    for (const auto& kv : root.obj) {
        const std::string& name = kv.first;
        if (name == "__metadata__") continue;
        const pdkjson::Value& v = kv.second;
        const pdkjson::Value* dt = v.get("dtype");
        if (!dt || dt->kind != pdkjson::Value::String) { set_err(err, err_len, "%s: missing dtype", name.c_str()); return PDK_ST_HEADER; }
        const pdkjson::Value* sh = v.get("shape");
        if (!sh || sh->kind != pdkjson::Value::Array || sh->arr.size() > 8) { set_err(err, err_len, "%s: missing shape", name.c_str()); return PDK_ST_HEADER; }
        StTensor t;
        t.dtype = parse_dtype(dt->str);
        uint64_t n = 1;
        for (const auto& d : sh->arr) {
            if (d.kind != pdkjson::Value::Number || !d.is_uint) { set_err(err, err_len, "%s: missing shape", name.c_str()); return PDK_ST_HEADER; }
            if (d.u != 0 && n > UINT64_MAX / d.u) { set_err(err, err_len, "%s: element count overflow", name.c_str()); return PDK_ST_HEADER; }
            n *= d.u;
            t.shape.push_back(d.u);
        }
        const pdkjson::Value* off = v.get("data_offsets");
        if (!off || off->kind != pdkjson::Value::Array || off->arr.size() != 2) { set_err(err, err_len, "%s: missing data_offsets", name.c_str()); return PDK_ST_HEADER; }
        const uint64_t begin = off->arr[0].is_uint ? off->arr[0].u : UINT64_MAX;
        const uint64_t end = off->arr[1].is_uint ? off->arr[1].u : UINT64_MAX;
        if (begin > end || end > data_len) {
            set_err(err, err_len, "%s: offsets [%llu, %llu) exceed data section (%llu)", name.c_str(),
                    (unsigned long long)begin, (unsigned long long)end, (unsigned long long)data_len);
            return PDK_ST_HEADER;
        }
        const uint64_t eb = dtype_bytes(t.dtype);
        if (eb != 0 && (n > UINT64_MAX / eb || n * eb != end - begin)) {
            set_err(err, err_len, "%s: shape x dtype != %llu bytes", name.c_str(), (unsigned long long)(end - begin));
            return PDK_ST_HEADER;
        }
        t.data = m->p + data_off + begin;
        t.n_bytes = end - begin;
        s->tensors[name] = std::move(t);
    }
    s->maps.push_back(std::move(m));
    return PDK_ST_OK;
}

PDKH_EXPORT int pdk_st_open(const char* path, PdkSafetensors** out, char* err, size_t err_len) {
    if (!out) return PDK_ST_IO;
    *out = nullptr;
    std::unique_ptr<PdkSafetensors> s(new PdkSafetensors());
    struct stat st;
    if (stat(path, &st) != 0) { set_err(err, err_len, "cannot stat %s", path); return PDK_ST_IO; }
    int rc = PDK_ST_OK;
    if (!S_ISDIR(st.st_mode)) {
        rc = load_file(s.get(), path, err, err_len);
    } else {
        const std::string dir(path);
        const std::string index = dir + "/model.safetensors.index.json";
        if (stat(index.c_str(), &st) != 0) {
            rc = load_file(s.get(), dir + "/model.safetensors", err, err_len);
        } else {
            std::unique_ptr<Mapping> m;
            if (!map_file(index, m, err, err_len)) return PDK_ST_IO;
            pdkjson::Value root;
            pdkjson::Parser parser((const char*)m->p, m->len);
            const pdkjson::Value* wm = parser.parse(root) ? root.get("weight_map") : nullptr;
            if (!wm || wm->kind != pdkjson::Value::Object) { set_err(err, err_len, "%s: no weight_map", index.c_str()); return PDK_ST_HEADER; }
            std::vector<std::string> shards;
            for (const auto& kv : wm->obj) {
                if (kv.second.kind != pdkjson::Value::String) { set_err(err, err_len, "%s: weight_map value is not a string", index.c_str()); return PDK_ST_HEADER; }
                const std::string& f = kv.second.str;
                if (f.find('/') != std::string::npos || f.find("..") != std::string::npos) {
                    set_err(err, err_len, "%s: shard name %s leaves the directory", index.c_str(), f.c_str());
                    return PDK_ST_HEADER;
                }
                bool have = false;
                for (const auto& x : shards) have = have || x == f;
                if (!have) shards.push_back(f);
            }
            for (const auto& f : shards) {
                rc = load_file(s.get(), dir + "/" + f, err, err_len);
                if (rc != PDK_ST_OK) break;
            }
        }
    }
    if (rc != PDK_ST_OK) return rc;
    *out = s.release();
    return PDK_ST_OK;
}

PDKH_EXPORT void pdk_st_close(PdkSafetensors* s) { delete s; }
PDKH_EXPORT uint64_t pdk_st_tensor_count(const PdkSafetensors* s) { return s->tensors.size(); }

PDKH_EXPORT int pdk_st_tensor(const PdkSafetensors* s, const char* name, uint32_t* dtype, uint32_t* n_dims,
                              uint64_t shape[8], const void** data, uint64_t* n_bytes) {
    auto it = s->tensors.find(name);
    if (it == s->tensors.end()) return PDK_ST_NOT_FOUND;
    const StTensor& t = it->second;
    if (dtype) *dtype = t.dtype;
    if (n_dims) *n_dims = (uint32_t)t.shape.size();
    if (shape)
        for (size_t d = 0; d < 8; ++d) shape[d] = d < t.shape.size() ? t.shape[d] : 1;
    if (data) *data = t.data;
    if (n_bytes) *n_bytes = t.n_bytes;
    return PDK_ST_OK;
}

static const StTensor* find(const PdkSafetensors* s, const std::string& name) {
    auto it = s->tensors.find(name);
    return it == s->tensors.end() ? nullptr : &it->second;
}

// crates/paddock-models/src/modelopt.rs:168-238
PDKH_EXPORT int pdk_st_nvfp4_view(const PdkSafetensors* s, const char* prefix, const void** packed,
                                  const void** scales, float* scale2, uint64_t* n, uint64_t* k, char* err,
                                  size_t err_len) {
    const std::string p(prefix);
    bool compressed = true;
    const StTensor* w = find(s, p + ".weight_packed");
    if (!w) { compressed = false; w = find(s, p + ".weight"); }
    if (!w) { set_err(err, err_len, "%s.weight[_packed]: missing", prefix); return PDK_ST_HEADER; }
    if (w->dtype != PDK_ST_U8 || w->shape.size() != 2) { set_err(err, err_len, "%s.weight%s: want U8 2-D", prefix, compressed ? "_packed" : ""); return PDK_ST_HEADER; }
    const uint64_t rows = w->shape[0], kh = w->shape[1];
    const StTensor* sc = find(s, p + ".weight_scale");
    if (!sc) { set_err(err, err_len, "%s.weight_scale: missing", prefix); return PDK_ST_HEADER; }
    if (sc->dtype != PDK_ST_F8_E4M3 || sc->shape.size() != 2 || sc->shape[0] != rows || sc->shape[1] != kh / 8) {
        set_err(err, err_len, "%s.weight_scale: want F8_E4M3 [%llu, %llu]", prefix, (unsigned long long)rows, (unsigned long long)(kh / 8));
        return PDK_ST_HEADER;
    }
    const char* s2name = compressed ? ".weight_global_scale" : ".weight_scale_2";
    const StTensor* s2 = find(s, p + s2name);
    if (!s2) { set_err(err, err_len, "%s%s: missing", prefix, s2name); return PDK_ST_HEADER; }
    if (s2->dtype != PDK_ST_F32 || s2->n_bytes != 4) { set_err(err, err_len, "%s%s: want scalar F32", prefix, s2name); return PDK_ST_HEADER; }
    float raw;
    memcpy(&raw, s2->data, 4);
    if (compressed && !(std::isfinite(raw) && raw > 0.0f)) { set_err(err, err_len, "%s%s: not a positive finite scale", prefix, s2name); return PDK_ST_HEADER; }
    if (packed) *packed = w->data;
    if (scales) *scales = sc->data;
    if (scale2) *scale2 = compressed ? 1.0f / raw : raw;
    if (n) *n = rows;
    if (k) *k = kh * 2;
    return PDK_ST_OK;
}

// crates/paddock-models/src/modelopt.rs:291-342 and 361-383
PDKH_EXPORT int pdk_st_fp8_channel_view(PdkSafetensors* s, const char* prefix, const void** weight,
                                        const float** row_scales, uint64_t* n, uint64_t* k, char* err,
                                        size_t err_len) {
    const std::string p(prefix);
    const StTensor* w = find(s, p + ".weight");
    if (!w) { set_err(err, err_len, "%s.weight: missing", prefix); return PDK_ST_HEADER; }
    if (w->dtype != PDK_ST_F8_E4M3 || w->shape.size() != 2) { set_err(err, err_len, "%s.weight: want F8_E4M3 2-D", prefix); return PDK_ST_HEADER; }
    const uint64_t rows = w->shape[0];
    const StTensor* sc = find(s, p + ".weight_scale");
    if (!sc) { set_err(err, err_len, "%s.weight_scale: missing", prefix); return PDK_ST_HEADER; }
    uint64_t count = 1;
    for (uint64_t d : sc->shape) count *= d;
    std::unique_ptr<std::vector<float>> out(new std::vector<float>());
    if (sc->dtype == PDK_ST_BF16 && count == rows && sc->n_bytes == rows * 2) {
        out->resize((size_t)rows);
        for (uint64_t i = 0; i < rows; ++i) {
            uint16_t h;
            memcpy(&h, sc->data + 2 * i, 2);
            const uint32_t bits = (uint32_t)h << 16;
            memcpy(&(*out)[(size_t)i], &bits, 4);
        }
    } else if (sc->dtype == PDK_ST_F32 && count == 1 && sc->n_bytes == 4) {
        float v;
        memcpy(&v, sc->data, 4);
        out->assign((size_t)rows, v);
    } else if (sc->dtype == PDK_ST_F32 && count == rows && sc->n_bytes == rows * 4) {
        out->resize((size_t)rows);
        memcpy(out->data(), sc->data, (size_t)rows * 4);
    } else {
        set_err(err, err_len, "%s.weight_scale: want %llu channel scales (BF16 / F32) or one F32", prefix, (unsigned long long)rows);
        return PDK_ST_HEADER;
    }
    if (weight) *weight = w->data;
    if (row_scales) *row_scales = out->data();
    if (n) *n = rows;
    if (k) *k = w->shape[1];
    s->owned_scales.push_back(std::move(out));
    return PDK_ST_OK;
}

// crates/paddock-models/src/gguf_nvfp4.rs:34-83: inside sub-block s of a 64-element block,
// byte j holds element j (low nibble) and j + 8 (high nibble); the row layout packs elements
// 2i / 2i+1 into byte i.  Scale bytes carry over; 0x7F (NaN) reads as 0; a sign bit is refused.
PDKH_EXPORT int pdk_nvfp4_gguf_repack_rows(const void* src_v, uint64_t src_len, uint64_t rows, uint64_t in_dim,
                                           void* codes_v, void* scales_v, uint64_t* nan_scales, char* err,
                                           size_t err_len) {
    const uint8_t* src = (const uint8_t*)src_v;
    uint8_t* codes = (uint8_t*)codes_v;
    uint8_t* scales = (uint8_t*)scales_v;
    if (in_dim % 64 != 0) {
        set_err(err, err_len, "nvfp4 row of %llu elements is not a whole number of 64-element blocks", (unsigned long long)in_dim);
        return 1;
    }
    const uint64_t blocks = rows * (in_dim / 64);
    if (src_len != blocks * 36) {
        set_err(err, err_len, "nvfp4 tensor holds %llu bytes, [%llu, %llu] needs %llu", (unsigned long long)src_len,
                (unsigned long long)rows, (unsigned long long)in_dim, (unsigned long long)(blocks * 36));
        return 1;
    }
    uint64_t nans = 0;
    for (uint64_t b = 0; b < blocks; ++b) {
        const uint8_t* blk = src + b * 36;
        for (uint32_t s = 0; s < 4; ++s) {
            const uint8_t byte = blk[s];
            if (byte & 0x80) {
                set_err(err, err_len, "nvfp4 block %llu: scale byte 0x%02x has its sign bit set", (unsigned long long)b, byte);
                return 1;
            }
            if (byte == 0x7f) { scales[b * 4 + s] = 0; ++nans; }
            else scales[b * 4 + s] = byte;
            const uint8_t* sub = blk + 4 + s * 8;
            uint8_t* out = codes + b * 32 + s * 8;
            for (uint32_t i = 0; i < 8; ++i) {
                const uint32_t m0 = 2 * i, m1 = 2 * i + 1;
                const uint8_t lo = m0 < 8 ? (sub[m0] & 0x0f) : (uint8_t)(sub[m0 - 8] >> 4);
                const uint8_t hi = m1 < 8 ? (sub[m1] & 0x0f) : (uint8_t)(sub[m1 - 8] >> 4);
                out[i] = (uint8_t)(lo | (hi << 4));
            }
        }
    }
    if (nan_scales) *nan_scales = nans;
    return 0;
}
