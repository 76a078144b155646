// executor.cc - libpaddock_exec.so: the operator layer above the kernel-pack table
// (include/paddock_exec.h).  Owns a loaded pack, a stream, a staging buffer and the resident
// weight planes; every launch is a call through a slot of the table it copied at load time.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/paddock_exec.h"
#include "../../include/paddock_pack.h"

#define PDX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// (raw ggml id, raw bytes, repacked data bytes) per 256 weights and the scale record size, as
// the pack's k-quant slots lay planes out (gpu/types.rs:285-381; this pack serves five types)
struct KqLayout {
    uint32_t raw_id, raw_b, data_b, scale_b;
};
bool kq_layout(uint32_t ty, KqLayout* out) {
    switch (ty) {
        case PDK_GGML_Q4_0: *out = {2u, 144u, 128u, 24u}; return true;
        case PDK_GGML_Q4_K: *out = {12u, 144u, 128u, 24u}; return true;
        case PDK_GGML_Q5_K: *out = {13u, 176u, 160u, 24u}; return true;
        case PDK_GGML_Q6_K: *out = {14u, 210u, 192u, 24u}; return true;
        case PDK_GGML_IQ4_XS: *out = {23u, 136u, 128u, 24u}; return true;
        default: return false;
    }
}

struct DevBuf {
    void* p = nullptr;
    size_t n = 0;
};

}  // namespace

struct PdxPlane {
    uint32_t kind = 0, ggml_type = 0, layout = PDX_NVF4_ROW;
    uint64_t in_dim = 0, out_dim = 0;
    DevBuf data, scale, scale_tc5;
    float scale2 = 1.0f;
};

struct PdxExecutor {
    void* lib = nullptr;
    int device = 0;
    cudaStream_t stream = nullptr;
    void* slot[PDK_TABLE_SLOTS] = {};
    // named exports outside the table
    decltype(&pdk_kquant_gemm_f32) kquant_gemm_f32 = nullptr;
    DevBuf staging;
    size_t staging_cap = 128u << 20;
    std::mutex mu;
    std::string last_error;

    int fail(int code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        last_error = buf;
        return code;
    }
    int drv(cudaError_t e, const char* what) {
        if (e == cudaSuccess) return PDX_OK;
        return fail(PDX_DRIVER, "%s: %s", what, cudaGetErrorString(e));
    }
    int launched(int rc, const char* what) {
        if (rc == 0) return PDX_OK;
        return fail(PDX_LAUNCH, "%s: launcher returned %d", what, rc);
    }
    template <typename Fn>
    Fn op(int idx) const {
        return reinterpret_cast<Fn>(slot[idx]);
    }
    int alloc(size_t n, DevBuf* out, const char* what) {
        out->p = nullptr;
        out->n = n;
        if (n == 0) return PDX_OK;
        return drv(cudaMalloc(&out->p, n), what);
    }
    void release(DevBuf* b) {
        if (b->p) cudaFree(b->p);
        b->p = nullptr;
        b->n = 0;
    }
    // with_staged_raw (gpu/upload.rs:203-304): host bytes -> a device buffer that lives until
    // the work queued on the stream behind it has run.  Tensors up to the cap share one buffer
    // that grows to the largest of them; a larger one gets a buffer of its own, freed after
    // the stream has drained.
    template <typename Work>
    int with_staged_raw(const void* bytes, size_t n, Work work) {
        std::lock_guard<std::mutex> lock(mu);
        if (n <= staging_cap) {
            if (staging.n < n) {
                // the previous tensor's repack may still be reading the old buffer
                if (int rc = drv(cudaStreamSynchronize(stream), "staging grow")) return rc;
                release(&staging);
                if (int rc = alloc(n, &staging, "staging buffer")) return rc;
            } else {
                // the buffer is reused: wait for the launch that read its previous contents
                if (int rc = drv(cudaStreamSynchronize(stream), "staging reuse")) return rc;
            }
            if (int rc = drv(cudaMemcpyAsync(staging.p, bytes, n, cudaMemcpyHostToDevice, stream), "staging copy")) return rc;
            return work(staging.p);
        }
        DevBuf own;
        if (int rc = alloc(n, &own, "transient staging")) return rc;
        int rc = drv(cudaMemcpyAsync(own.p, bytes, n, cudaMemcpyHostToDevice, stream), "staging copy");
        if (rc == PDX_OK) rc = work(own.p);
        cudaStreamSynchronize(stream);
        release(&own);
        return rc;
    }
    int clone_htod(const void* bytes, size_t n, DevBuf* out, const char* what) {
        if (int rc = alloc(n, out, what)) return rc;
        if (n == 0) return PDX_OK;
        // pageable host memory: the copy has left the host buffer when the call returns
        return drv(cudaMemcpyAsync(out->p, bytes, n, cudaMemcpyHostToDevice, stream), what);
    }
};

namespace {

int tensor_of(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, const void** data, uint64_t* n_bytes,
              uint32_t* ty, uint64_t dims[8], uint32_t* n_dims) {
    if (!map || !name) return ex->fail(PDX_FORMAT, "no weight file / tensor name");
    const int rc = pdk_gguf_family_tensor_bytes(map, name, data, n_bytes, ty, n_dims, dims, nullptr);
    if (rc != PDK_MAP_OK) return ex->fail(PDX_FORMAT, "tensor %s: weight file error %d", name, rc);
    return PDX_OK;
}

// q40_to_q8_blocks (gpu/kquant.rs:15-33): 18-byte Q4_0 blocks {f16 d, 16 nibble bytes} -> 34-byte
// Q8_0 blocks {f16 d, int8 q[32]} with q = nibble - 8; element j of the low nibbles, j + 16 of the
// high ones.  The dequantized values are bit-identical.
std::vector<uint8_t> q40_to_q8_blocks(const uint8_t* src, size_t len) {
    const size_t n = len / 18u;
    std::vector<uint8_t> out(n * 34u);
    for (size_t b = 0; b < n; ++b) {
        const uint8_t* s = src + b * 18u;
        uint8_t* d = out.data() + b * 34u;
        d[0] = s[0];
        d[1] = s[1];
        for (int j = 0; j < 16; ++j) {
            d[2 + j] = (uint8_t)(int8_t)((int)(s[2 + j] & 15u) - 8);
            d[2 + 16 + j] = (uint8_t)(int8_t)((int)(s[2 + j] >> 4) - 8);
        }
    }
    return out;
}

int make_q8(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t out_dim, PdxPlane** out) {
    auto f = ex->op<decltype(&pd_q8_0_repack)>(PDK_SLOT_q8_0_repack);
    if (!f) return ex->fail(PDX_MISSING_OP, "q8_0_repack");
    if (in_dim == 0 || in_dim % 32u != 0) return ex->fail(PDX_UNSUPPORTED, "Q8_0 rows of %llu elements", (unsigned long long)in_dim);
    const uint64_t n_blocks = in_dim / 32u * out_dim;
    if (len != n_blocks * 34u)
        return ex->fail(PDX_DRIVER, "q8 repack: %llu raw bytes for %llu blocks (want %llu)", (unsigned long long)len,
                        (unsigned long long)n_blocks, (unsigned long long)(n_blocks * 34u));
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_Q8;
    p->ggml_type = PDK_GGML_Q8_0;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    int rc = ex->alloc(n_blocks * 32u, &p->data, "q8 data plane");
    if (rc == PDX_OK) rc = ex->alloc(n_blocks * 2u, &p->scale, "q8 scale plane");
    if (rc == PDX_OK)
        rc = ex->with_staged_raw(bytes, len, [&](void* sp) {
            return ex->launched(f(sp, p->data.p, p->scale.p, n_blocks, ex->stream), "q8_0_repack");
        });
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

// One repack launch of n_super super-blocks of `raw` into a plane's streams at a super-block offset.
int kq_repack_into(PdxExecutor* ex, const KqLayout& lay, const void* raw, uint64_t n_super, PdxPlane* p, uint64_t at) {
    auto f = ex->op<decltype(&pd_kquant_repack)>(PDK_SLOT_kquant_repack);
    if (!f) return ex->fail(PDX_MISSING_OP, "kquant_repack");
    return ex->with_staged_raw(raw, n_super * lay.raw_b, [&](void* sp) {
        return ex->launched(f(sp, (uint8_t*)p->data.p + at * lay.data_b, (uint8_t*)p->scale.p + at * lay.scale_b, n_super,
                              lay.raw_id, ex->stream),
                            "kquant_repack");
    });
}

int make_kq(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t out_dim, uint32_t ty,
            const char* what, PdxPlane** out) {
    KqLayout lay;
    if (!kq_layout(ty, &lay)) return ex->fail(PDX_NO_KERNEL, "%s: no k-quant kernel class for ggml type %u", what, ty);
    if (in_dim == 0 || in_dim % 256u != 0)
        return ex->fail(PDX_DRIVER, "kquant repack %s: in_dim %llu is not superblock-aligned", what, (unsigned long long)in_dim);
    const uint64_t n_super = in_dim / 256u * out_dim;
    if (len != n_super * lay.raw_b)
        return ex->fail(PDX_DRIVER, "kquant repack %s: %llu raw bytes for %llu superblocks (want %llu)", what,
                        (unsigned long long)len, (unsigned long long)n_super, (unsigned long long)(n_super * lay.raw_b));
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_KQ;
    p->ggml_type = ty;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    int rc = ex->alloc(n_super * lay.data_b, &p->data, "kquant data plane");
    if (rc == PDX_OK) rc = ex->alloc(n_super * lay.scale_b, &p->scale, "kquant scale plane");
    if (rc == PDX_OK) rc = kq_repack_into(ex, lay, bytes, n_super, p, 0);
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

const char* const kSlotNames[] = {
    "mxfp4_dequant_f32", "q8_0_dequant_f32", "add_inplace_f32", "mxfp4_repack", "q8_0_repack", "q8_0_gemv_repacked",
    "q8_0_gemm_repacked", "kquant_dequant", "kquant_repack", "kquant_gemv", "quantize_e4m3_row", "f8row_gemm",
    "bf16_to_f8row", "f8row_gemm_tc5x", "quantize_nvf4", "nvf4_dequant", "nvf4_gemv", "nvf4_gemm_tc5w",
    "nvf4_tc5_tile_scales", "swiglu_quant_e4m3_row", "rmsnorm_quant_e4m3_row", "add_rmsnorm_scaled_quant_e4m3_row"};
const int kSlotIndex[] = {
    PDK_SLOT_mxfp4_dequant_f32, PDK_SLOT_q8_0_dequant_f32, PDK_SLOT_add_inplace_f32, PDK_SLOT_mxfp4_repack,
    PDK_SLOT_q8_0_repack, PDK_SLOT_q8_0_gemv_repacked, PDK_SLOT_q8_0_gemm_repacked, PDK_SLOT_kquant_dequant,
    PDK_SLOT_kquant_repack, PDK_SLOT_kquant_gemv, PDK_SLOT_quantize_e4m3_row, PDK_SLOT_f8row_gemm,
    PDK_SLOT_bf16_to_f8row, PDK_SLOT_f8row_gemm_tc5x, PDK_SLOT_quantize_nvf4, PDK_SLOT_nvf4_dequant,
    PDK_SLOT_nvf4_gemv, PDK_SLOT_nvf4_gemm_tc5w, PDK_SLOT_nvf4_tc5_tile_scales, PDK_SLOT_swiglu_quant_e4m3_row,
    PDK_SLOT_rmsnorm_quant_e4m3_row, PDK_SLOT_add_rmsnorm_scaled_quant_e4m3_row};

void set_msg(char* err, size_t n, const char* fmt, ...) {
    if (!err || n == 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, n, fmt, ap);
    va_end(ap);
}

std::string default_pack_path() {
    Dl_info info;
    if (dladdr((void*)&default_pack_path, &info) == 0 || info.dli_fname == nullptr) return "libpaddock_b200.so";
    std::string here = info.dli_fname;
    const size_t cut = here.find_last_of('/');
    return (cut == std::string::npos ? std::string() : here.substr(0, cut + 1)) + "libpaddock_b200.so";
}

}  // namespace

// ---- executor ---------------------------------------------------------------------------------

PDX_EXPORT int pdx_open(const char* pack_path, int device, PdxExecutor** out, char* err, size_t err_len) {
    if (!out) return PDX_PACK;
    *out = nullptr;
    const std::string path = pack_path ? pack_path : default_pack_path();
    // the engine binds its device before it loads a pack: the pack resolves its table against it
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        set_msg(err, err_len, "cannot bind device %d: %s", device, cudaGetErrorString(e));
        return PDX_DRIVER;
    }
    void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        set_msg(err, err_len, "cannot load %s: %s", path.c_str(), dlerror());
        return PDX_PACK;
    }
    // loader.rs:140-194: both symbols, the magic, the ABI version
    auto info_fn = (const PdkPackInfo* (*)(void))dlsym(lib, "paddock_pack_info");
    auto table_fn = (const PdkKernelTableV1* (*)(void))dlsym(lib, "paddock_pack_kernels_v1");
    if (!info_fn || !table_fn) {
        set_msg(err, err_len, "%s is not a kernel pack (symbols missing)", path.c_str());
        dlclose(lib);
        return PDX_PACK;
    }
    const PdkPackInfo* info = info_fn();
    if (!info || info->magic != PDK_PACK_MAGIC || info->abi_version != PDK_PACK_ABI_VERSION) {
        set_msg(err, err_len, "%s: bad magic or ABI version", path.c_str());
        dlclose(lib);
        return PDX_PACK;
    }
    const PdkKernelTableV1* table = table_fn();
    if (!table || table->size < 8u) {
        set_msg(err, err_len, "%s: no kernel table", path.c_str());
        dlclose(lib);
        return PDX_PACK;
    }
    PdxExecutor* ex = new PdxExecutor();
    ex->lib = lib;
    ex->device = device;
    // loader.rs:253-283: copy min(pack's size, ours); members past a shorter table read NULL
    const size_t n = ((size_t)table->size < (size_t)PDK_TABLE_BYTES ? (size_t)table->size : (size_t)PDK_TABLE_BYTES) - 8u;
    memcpy(ex->slot, table->slot, n);
    ex->kquant_gemm_f32 = (decltype(&pdk_kquant_gemm_f32))dlsym(lib, "pdk_kquant_gemm_f32");
    if (const char* cap = getenv("PADDOCK_STAGING_MAX")) {
        const long long v = atoll(cap);
        if (v > 0) ex->staging_cap = (size_t)v;
    }
    e = cudaStreamCreateWithFlags(&ex->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        set_msg(err, err_len, "cannot create a stream: %s", cudaGetErrorString(e));
        dlclose(lib);
        delete ex;
        return PDX_DRIVER;
    }
    *out = ex;
    return PDX_OK;
}

PDX_EXPORT void pdx_close(PdxExecutor* ex) {
    if (!ex) return;
    if (ex->stream) {
        cudaStreamSynchronize(ex->stream);
        if (auto rel = (void (*)(void*))dlsym(ex->lib, "pdk_stream_release")) rel(ex->stream);
        cudaStreamDestroy(ex->stream);
    }
    ex->release(&ex->staging);
    // the pack stays loaded: its static tables may be referenced by other executors
    delete ex;
}

PDX_EXPORT void* pdx_stream(const PdxExecutor* ex) { return ex->stream; }
PDX_EXPORT int pdx_synchronize(PdxExecutor* ex) { return ex->drv(cudaStreamSynchronize(ex->stream), "synchronize"); }
PDX_EXPORT const char* pdx_last_error(const PdxExecutor* ex) { return ex->last_error.c_str(); }
PDX_EXPORT uint64_t pdx_staging_bytes(const PdxExecutor* ex) { return ex->staging.n; }
PDX_EXPORT void pdx_release_staging(PdxExecutor* ex) {
    std::lock_guard<std::mutex> lock(ex->mu);
    cudaStreamSynchronize(ex->stream);
    ex->release(&ex->staging);
}

PDX_EXPORT int pdx_has(const PdxExecutor* ex, const char* slot_name) {
    if (!slot_name) return 0;
    for (size_t i = 0; i < sizeof(kSlotNames) / sizeof(kSlotNames[0]); ++i)
        if (strcmp(slot_name, kSlotNames[i]) == 0) return ex->slot[kSlotIndex[i]] != nullptr;
    if (strcmp(slot_name, "pdk_kquant_gemm_f32") == 0) return ex->kquant_gemm_f32 != nullptr;
    return 0;
}

// ---- planes -----------------------------------------------------------------------------------

PDX_EXPORT int pdx_plane_info(const PdxPlane* p, PdxPlaneInfo* out) {
    if (!p || !out) return PDX_UNSUPPORTED;
    out->kind = p->kind;
    out->ggml_type = p->ggml_type;
    out->in_dim = p->in_dim;
    out->out_dim = p->out_dim;
    out->bytes = p->data.n + p->scale.n + p->scale_tc5.n;
    out->data = p->data.p;
    out->scale = p->scale.p;
    out->scale_tc5 = p->scale_tc5.p;
    out->scale2 = p->scale2;
    out->layout = p->layout;
    return PDX_OK;
}

PDX_EXPORT void pdx_plane_free(PdxExecutor* ex, PdxPlane* p) {
    if (!p) return;
    cudaStreamSynchronize(ex->stream);
    ex->release(&p->data);
    ex->release(&p->scale);
    ex->release(&p->scale_tc5);
    delete p;
}

PDX_EXPORT int pdx_upload_raw(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, PdxPlane** out) {
    if (!out) return PDX_UNSUPPORTED;
    *out = nullptr;
    const void* data = nullptr;
    uint64_t n_bytes = 0, dims[8];
    uint32_t ty = 0, n_dims = 0;
    if (int rc = tensor_of(ex, map, name, &data, &n_bytes, &ty, dims, &n_dims)) return rc;
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_RAW;
    p->in_dim = dims[0];
    p->out_dim = 1;
    for (uint32_t d = 1; d < n_dims; ++d) p->out_dim *= dims[d];
    int rc;
    if (ty == PDK_GGML_Q4_0) {
        const std::vector<uint8_t> q8 = q40_to_q8_blocks((const uint8_t*)data, (size_t)n_bytes);
        p->ggml_type = PDK_GGML_Q8_0;
        rc = ex->clone_htod(q8.data(), q8.size(), &p->data, "raw upload");
        if (rc == PDX_OK) rc = ex->drv(cudaStreamSynchronize(ex->stream), "raw upload");   // q8 dies with this frame
    } else {
        p->ggml_type = ty;
        rc = ex->clone_htod(data, (size_t)n_bytes, &p->data, "raw upload");
    }
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

PDX_EXPORT int pdx_repack_q8_blocks(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t out_dim,
                                    PdxPlane** out) {
    if (!out || !bytes) return PDX_UNSUPPORTED;
    *out = nullptr;
    return make_q8(ex, bytes, len, in_dim, out_dim, out);
}

PDX_EXPORT int pdx_repack_kquant_raw(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim,
                                     uint64_t out_dim, uint32_t ggml_type, PdxPlane** out) {
    if (!out || !bytes) return PDX_UNSUPPORTED;
    *out = nullptr;
    return make_kq(ex, bytes, len, in_dim, out_dim, ggml_type, "host bytes", out);
}

PDX_EXPORT int pdx_load_quantw(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, PdxPlane** out) {
    if (!out) return PDX_UNSUPPORTED;
    *out = nullptr;
    const void* data = nullptr;
    uint64_t n_bytes = 0, dims[8];
    uint32_t ty = 0, n_dims = 0;
    if (int rc = tensor_of(ex, map, name, &data, &n_bytes, &ty, dims, &n_dims)) return rc;
    uint64_t out_dim = 1;
    for (uint32_t d = 1; d < n_dims; ++d) out_dim *= dims[d];
    KqLayout lay;
    switch (ty) {
        case PDK_GGML_Q8_0: return make_q8(ex, data, n_bytes, dims[0], out_dim, out);
        case PDK_GGML_Q4_0:
            // k-quant resident at 4.5 bits per weight when the row is whole super-blocks and the pack
            // has the repack; else the exact Q8_0 transcode (twice the bytes, the same values)
            if (dims[0] % 256u == 0 && ex->slot[PDK_SLOT_kquant_repack] && ex->slot[PDK_SLOT_kquant_gemv])
                return make_kq(ex, data, n_bytes, dims[0], out_dim, ty, name, out);
            {
                const std::vector<uint8_t> q8 = q40_to_q8_blocks((const uint8_t*)data, (size_t)n_bytes);
                int rc = make_q8(ex, q8.data(), q8.size(), dims[0], out_dim, out);
                if (rc == PDX_OK) rc = ex->drv(cudaStreamSynchronize(ex->stream), "q4_0 transcode");
                return rc;
            }
        default:
            if (!kq_layout(ty, &lay)) return ex->fail(PDX_NO_KERNEL, "%s: no kernel class for ggml type %u", name, ty);
            if (!ex->slot[PDK_SLOT_kquant_repack] || !ex->slot[PDK_SLOT_kquant_gemv])
                return ex->fail(PDX_NO_KERNEL, "%s: the pack has no k-quant lanes", name);
            return make_kq(ex, data, n_bytes, dims[0], out_dim, ty, name, out);
    }
}

PDX_EXPORT int pdx_repack_kquant_bands(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, uint32_t n_bands,
                                       PdxPlane** out) {
    if (!out) return PDX_UNSUPPORTED;
    const void* data = nullptr;
    uint64_t n_bytes = 0, dims[8];
    uint32_t ty = 0, n_dims = 0;
    if (int rc = tensor_of(ex, map, name, &data, &n_bytes, &ty, dims, &n_dims)) return rc;
    KqLayout lay;
    if (!kq_layout(ty, &lay)) return ex->fail(PDX_NO_KERNEL, "%s: no k-quant kernel class for ggml type %u", name, ty);
    const uint64_t in_dim = dims[0], out_dim = n_dims > 1 ? dims[1] : 1;
    if (n_bands == 0 || in_dim % n_bands != 0 || (in_dim / n_bands) % 256u != 0)
        return ex->fail(PDX_DRIVER, "kquant bands %s: in_dim %llu does not split into %u superblock-aligned strips", name,
                        (unsigned long long)in_dim, n_bands);
    const uint64_t band_in = in_dim / n_bands, row_sb = in_dim / 256u, band_sb = band_in / 256u;
    std::vector<uint8_t> raw((size_t)(out_dim * band_sb * lay.raw_b));
    for (uint32_t b = 0; b < n_bands; ++b) out[b] = nullptr;
    for (uint32_t b = 0; b < n_bands; ++b) {
        for (uint64_t o = 0; o < out_dim; ++o)
            memcpy(raw.data() + o * band_sb * lay.raw_b, (const uint8_t*)data + (o * row_sb + b * band_sb) * lay.raw_b,
                   (size_t)(band_sb * lay.raw_b));
        int rc = make_kq(ex, raw.data(), raw.size(), band_in, out_dim, ty, name, &out[b]);
        // `raw` is refilled for the next band: the copy out of it has to be done first
        if (rc == PDX_OK) rc = ex->drv(cudaStreamSynchronize(ex->stream), "kquant bands");
        if (rc != PDX_OK) {
            for (uint32_t j = 0; j < n_bands; ++j) {
                pdx_plane_free(ex, out[j]);
                out[j] = nullptr;
            }
            return rc;
        }
    }
    return PDX_OK;
}

PDX_EXPORT int pdx_repack_kquant_concat(PdxExecutor* ex, const PdkGgufFamily* map, const char* const* names,
                                        uint32_t n_names, PdxPlane** out) {
    if (!out || !names || n_names == 0) return PDX_UNSUPPORTED;
    *out = nullptr;
    struct Part {
        const void* data;
        uint64_t n_super;
    };
    std::vector<Part> parts;
    uint32_t ty0 = 0;
    uint64_t in_dim = 0, out_dim = 0, total = 0;
    for (uint32_t i = 0; i < n_names; ++i) {
        const void* data = nullptr;
        uint64_t n_bytes = 0, dims[8];
        uint32_t ty = 0, n_dims = 0;
        if (int rc = tensor_of(ex, map, names[i], &data, &n_bytes, &ty, dims, &n_dims)) return rc;
        if (i == 0) {
            ty0 = ty;
            in_dim = dims[0];
        } else if (ty != ty0 || dims[0] != in_dim) {
            return ex->fail(PDX_DRIVER, "kquant concat: %s breaks type/in_dim agreement", names[i]);
        }
        uint64_t rows = 1;
        for (uint32_t d = 1; d < n_dims; ++d) rows *= dims[d];
        out_dim += rows;
        parts.push_back({data, dims[0] / 256u * rows});
        total += parts.back().n_super;
    }
    KqLayout lay;
    if (!kq_layout(ty0, &lay)) return ex->fail(PDX_NO_KERNEL, "%s: no k-quant kernel class for ggml type %u", names[0], ty0);
    if (in_dim % 256u != 0) return ex->fail(PDX_DRIVER, "kquant concat: in_dim %llu not superblock-aligned", (unsigned long long)in_dim);
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_KQ;
    p->ggml_type = ty0;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    int rc = ex->alloc(total * lay.data_b, &p->data, "kquant data plane");
    if (rc == PDX_OK) rc = ex->alloc(total * lay.scale_b, &p->scale, "kquant scale plane");
    uint64_t done = 0;
    for (size_t i = 0; rc == PDX_OK && i < parts.size(); ++i) {
        rc = kq_repack_into(ex, lay, parts[i].data, parts[i].n_super, p, done);
        done += parts[i].n_super;
    }
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

PDX_EXPORT int pdx_repack_mxfp4(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t rows,
                                PdxPlane** out) {
    if (!out || !bytes) return PDX_UNSUPPORTED;
    *out = nullptr;
    auto f = ex->op<decltype(&pd_mxfp4_repack)>(PDK_SLOT_mxfp4_repack);
    if (!f) return ex->fail(PDX_MISSING_OP, "mxfp4_repack");
    if (in_dim == 0 || in_dim % 32u != 0) return ex->fail(PDX_UNSUPPORTED, "MXFP4 rows of %llu elements", (unsigned long long)in_dim);
    const uint64_t n_blocks = in_dim / 32u * rows;
    if (len != n_blocks * 17u) return ex->fail(PDX_DRIVER, "mxfp4 repack: %llu raw bytes for %llu blocks", (unsigned long long)len, (unsigned long long)n_blocks);
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_MXFP4;
    p->ggml_type = PDK_GGML_MXFP4;
    p->in_dim = in_dim;
    p->out_dim = rows;
    int rc = ex->alloc(n_blocks * 16u, &p->data, "mxfp4 data plane");
    if (rc == PDX_OK) rc = ex->alloc(n_blocks, &p->scale, "mxfp4 scale plane");
    if (rc == PDX_OK)
        rc = ex->with_staged_raw(bytes, len, [&](void* sp) {
            return ex->launched(f(sp, p->data.p, p->scale.p, n_blocks, ex->stream), "mxfp4_repack");
        });
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

PDX_EXPORT int pdx_bf16_to_f8row(PdxExecutor* ex, const void* bf16, uint64_t in_dim, uint64_t out_dim, PdxPlane** out) {
    if (!out || !bf16) return PDX_UNSUPPORTED;
    *out = nullptr;
    auto f = ex->op<decltype(&pd_bf16_to_f8row)>(PDK_SLOT_bf16_to_f8row);
    if (!f) return ex->fail(PDX_MISSING_OP, "bf16_to_f8row");
    if (in_dim == 0 || out_dim == 0 || in_dim > 0xffffffffull || out_dim > 0xffffffffull)
        return ex->fail(PDX_UNSUPPORTED, "bf16_to_f8row [%llu, %llu]", (unsigned long long)out_dim, (unsigned long long)in_dim);
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_F8ROW;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    int rc = ex->alloc(in_dim * out_dim, &p->data, "f8row data plane");
    if (rc == PDX_OK) rc = ex->alloc(out_dim * 4u, &p->scale, "f8row scale plane");
    if (rc == PDX_OK)
        rc = ex->with_staged_raw(bf16, in_dim * out_dim * 2u, [&](void* sp) {
            return ex->launched(f(sp, p->data.p, p->scale.p, (uint32_t)in_dim, (uint32_t)out_dim, ex->stream), "bf16_to_f8row");
        });
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

PDX_EXPORT int pdx_f8row_upload(PdxExecutor* ex, const void* e4m3, const float* row_scales, uint64_t in_dim,
                                uint64_t out_dim, PdxPlane** out) {
    if (!out || !e4m3 || !row_scales) return PDX_UNSUPPORTED;
    *out = nullptr;
    if (in_dim == 0 || out_dim == 0 || in_dim % 16u != 0)
        return ex->fail(PDX_UNSUPPORTED, "f8row plane [%llu, %llu]: in_dim must be a multiple of 16", (unsigned long long)out_dim,
                        (unsigned long long)in_dim);
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_F8ROW;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    int rc = ex->clone_htod(e4m3, in_dim * out_dim, &p->data, "f8row data plane");
    if (rc == PDX_OK) rc = ex->clone_htod(row_scales, out_dim * 4u, &p->scale, "f8row scale plane");
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

PDX_EXPORT int pdx_nvf4_upload(PdxExecutor* ex, const void* packed, uint64_t packed_len, const void* scales,
                               uint64_t scales_len, float scale2, uint64_t out_dim, uint64_t in_dim, PdxPlane** out) {
    if (!out || !packed || !scales) return PDX_UNSUPPORTED;
    *out = nullptr;
    if (in_dim % 32u != 0 || packed_len != out_dim * (in_dim / 2u) || scales_len != out_dim * (in_dim / 16u))
        return ex->fail(PDX_UNSUPPORTED, "nvf4 triple geometry mismatch: packed %llu scales %llu bytes for [%llu, %llu]",
                        (unsigned long long)packed_len, (unsigned long long)scales_len, (unsigned long long)out_dim,
                        (unsigned long long)in_dim);
    PdxPlane* p = new PdxPlane();
    p->kind = PDX_PLANE_NVF4;
    p->ggml_type = PDK_GGML_NVFP4;
    p->in_dim = in_dim;
    p->out_dim = out_dim;
    p->scale2 = scale2;
    p->layout = PDX_NVF4_ROW;
    // both copies are ordered on the executor's stream, the tiling launch behind them
    int rc = ex->clone_htod(packed, packed_len, &p->data, "nvf4 data plane");
    if (rc == PDX_OK) rc = ex->clone_htod(scales, scales_len, &p->scale, "nvf4 scale plane");
    // nvf4_tc5_tile: only where the tensor-core arm exists and K is whole slabs; else the plane serves as before
    auto tile = ex->op<decltype(&pd_nvf4_tc5_tile_scales)>(PDK_SLOT_nvf4_tc5_tile_scales);
    if (rc == PDX_OK && tile && ex->slot[PDK_SLOT_nvf4_gemm_tc5w] && in_dim % 256u == 0 && out_dim != 0) {
        rc = ex->alloc((out_dim + 127u) / 128u * (in_dim / 256u) * 2048u, &p->scale_tc5, "nvf4 tiled scales");
        if (rc == PDX_OK)
            rc = ex->launched(tile(p->scale.p, p->scale_tc5.p, (uint32_t)in_dim, (uint32_t)out_dim, ex->stream),
                              "nvf4_tc5_tile_scales");
    }
    if (rc != PDX_OK) {
        pdx_plane_free(ex, p);
        return rc;
    }
    *out = p;
    return PDX_OK;
}

// ---- launches ---------------------------------------------------------------------------------

PDX_EXPORT int pdx_dequant_rows(PdxExecutor* ex, const PdxPlane* p, uint64_t row0, uint64_t rows, void* out_f32) {
    if (!p || !out_f32) return PDX_UNSUPPORTED;
    if (p->kind != PDX_PLANE_RAW) return ex->fail(PDX_UNSUPPORTED, "dequant_rows reads a raw plane");
    if (row0 + rows > p->out_dim) return ex->fail(PDX_UNSUPPORTED, "rows %llu..%llu of %llu", (unsigned long long)row0,
                                                  (unsigned long long)(row0 + rows), (unsigned long long)p->out_dim);
    uint32_t elems = 0, bytes = 0;
    if (!pdk_ggml_block_layout(p->ggml_type, &elems, &bytes) || p->in_dim % elems != 0)
        return ex->fail(PDX_NO_KERNEL, "no dequant for ggml type %u", p->ggml_type);
    const uint64_t row_bytes = p->in_dim / elems * bytes;   // QuantTensor::row_bytes, types.rs:96-103
    const uint8_t* src = (const uint8_t*)p->data.p + row0 * row_bytes;
    const uint64_t n_blocks = p->in_dim / elems * rows;
    KqLayout lay;
    if (p->ggml_type == PDK_GGML_Q8_0) {
        auto f = ex->op<decltype(&pd_q8_0_dequant_f32)>(PDK_SLOT_q8_0_dequant_f32);
        if (!f) return ex->fail(PDX_MISSING_OP, "q8_0_dequant_f32");
        return ex->launched(f(src, out_f32, n_blocks, ex->stream), "q8_0_dequant_f32");
    }
    if (p->ggml_type == PDK_GGML_MXFP4) {
        auto f = ex->op<decltype(&pd_mxfp4_dequant_f32)>(PDK_SLOT_mxfp4_dequant_f32);
        if (!f) return ex->fail(PDX_MISSING_OP, "mxfp4_dequant_f32");
        return ex->launched(f(src, out_f32, n_blocks, ex->stream), "mxfp4_dequant_f32");
    }
    if (kq_layout(p->ggml_type, &lay) && p->ggml_type != PDK_GGML_Q4_0) {
        auto f = ex->op<decltype(&pd_kquant_dequant)>(PDK_SLOT_kquant_dequant);
        if (!f) return ex->fail(PDX_MISSING_OP, "kquant_dequant");
        return ex->launched(f(src, out_f32, n_blocks, lay.raw_id, ex->stream), "kquant_dequant");
    }
    return ex->fail(PDX_NO_KERNEL, "no dequant for ggml type %u", p->ggml_type);
}

PDX_EXPORT int pdx_quantw_gemv(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y) {
    if (!w || !x || !y) return PDX_UNSUPPORTED;
    if (w->kind == PDX_PLANE_Q8) {
        auto f = ex->op<decltype(&pd_q8_0_gemv_repacked)>(PDK_SLOT_q8_0_gemv_repacked);
        if (!f) return ex->fail(PDX_MISSING_OP, "q8_0_gemv_repacked");
        return ex->launched(f(w->data.p, w->scale.p, bias, x, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, ex->stream),
                            "q8_0_gemv_repacked");
    }
    if (w->kind == PDX_PLANE_KQ) {
        if (bias) return ex->fail(PDX_UNSUPPORTED, "kquant_gemv takes no bias");
        auto f = ex->op<decltype(&pd_kquant_gemv)>(PDK_SLOT_kquant_gemv);
        if (!f) return ex->fail(PDX_MISSING_OP, "kquant_gemv");
        KqLayout lay;
        kq_layout(w->ggml_type, &lay);
        return ex->launched(f(w->data.p, w->scale.p, x, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, lay.raw_id, ex->stream),
                            "kquant_gemv");
    }
    return ex->fail(PDX_UNSUPPORTED, "quantw_gemv needs a Q8 or k-quant plane");
}

PDX_EXPORT int pdx_quantw_gemm(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y, uint32_t batch) {
    if (!w || !x || !y) return PDX_UNSUPPORTED;
    if (w->kind == PDX_PLANE_Q8) {
        auto f = ex->op<decltype(&pd_q8_0_gemm_repacked)>(PDK_SLOT_q8_0_gemm_repacked);
        if (!f) return ex->fail(PDX_MISSING_OP, "q8_0_gemm_repacked");
        return ex->launched(
            f(w->data.p, w->scale.p, bias, x, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, batch, ex->stream),
            "q8_0_gemm_repacked");
    }
    if (w->kind == PDX_PLANE_KQ) {
        if (bias) return ex->fail(PDX_UNSUPPORTED, "the k-quant small-batch GEMM takes no bias");
        if (!ex->kquant_gemm_f32) return ex->fail(PDX_MISSING_OP, "pdk_kquant_gemm_f32");
        KqLayout lay;
        kq_layout(w->ggml_type, &lay);
        return ex->launched(ex->kquant_gemm_f32(w->data.p, w->scale.p, x, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, batch,
                                                lay.raw_id, ex->stream),
                            "pdk_kquant_gemm_f32");
    }
    return ex->fail(PDX_UNSUPPORTED, "quantw_gemm needs a Q8 or k-quant plane");
}

PDX_EXPORT int pdx_quantize_e4m3_row(PdxExecutor* ex, const void* x, void* q, void* rscale, uint32_t n_dim, uint32_t batch) {
    auto f = ex->op<decltype(&pd_quantize_e4m3_row)>(PDK_SLOT_quantize_e4m3_row);
    if (!f) return ex->fail(PDX_MISSING_OP, "quantize_e4m3_row");
    return ex->launched(f(x, q, rscale, n_dim, batch, ex->stream), "quantize_e4m3_row");
}

// The fused producers in front of f8row_gemm (gpu/fp8.rs:469-590).  *fused receives 1 when the pack
// ran the fused kernel and 0 when the slot is absent or declined (status 100): the caller then runs
// the unfused chain, as the engine does on Ok(false).
PDX_EXPORT int pdx_swiglu_quant_e4m3_row(PdxExecutor* ex, const void* gate, const void* up, void* q, void* rs, uint32_t n_ff,
                                         uint32_t batch, int* fused) {
    if (fused) *fused = 0;
    auto f = ex->op<decltype(&pd_swiglu_quant_e4m3_row)>(PDK_SLOT_swiglu_quant_e4m3_row);
    if (!f) return PDX_OK;
    if (int rc = ex->launched(f(gate, up, q, rs, n_ff, batch, ex->stream), "swiglu_quant_e4m3_row")) return rc;
    if (fused) *fused = 1;
    return PDX_OK;
}

PDX_EXPORT int pdx_rmsnorm_quant_e4m3_row(PdxExecutor* ex, const void* x, const void* w, void* xn, void* q, void* rs,
                                          uint32_t n, float eps, uint32_t batch, int* fused) {
    if (fused) *fused = 0;
    auto f = ex->op<decltype(&pd_rmsnorm_quant_e4m3_row)>(PDK_SLOT_rmsnorm_quant_e4m3_row);
    if (!f) return PDX_OK;
    const int rc = f(x, w, xn, q, rs, n, eps, batch, ex->stream);
    if (rc == 100) return PDX_OK;
    if (int e = ex->launched(rc, "rmsnorm_quant_e4m3_row")) return e;
    if (fused) *fused = 1;
    return PDX_OK;
}

PDX_EXPORT int pdx_add_rmsnorm_scaled_quant_e4m3_row(PdxExecutor* ex, void* x, const void* proj, const void* w, void* xn,
                                                     void* q, void* rs, uint32_t n, float eps, float pscale, uint32_t batch,
                                                     int* fused) {
    if (fused) *fused = 0;
    auto f = ex->op<decltype(&pd_add_rmsnorm_scaled_quant_e4m3_row)>(PDK_SLOT_add_rmsnorm_scaled_quant_e4m3_row);
    if (!f) return PDX_OK;
    const int rc = f(x, proj, w, xn, q, rs, n, eps, pscale, batch, ex->stream);
    if (rc == 100) return PDX_OK;
    if (int e = ex->launched(rc, "add_rmsnorm_scaled_quant_e4m3_row")) return e;
    if (fused) *fused = 1;
    return PDX_OK;
}

PDX_EXPORT int pdx_f8row_gemm(PdxExecutor* ex, const PdxPlane* w, const void* xq, const void* xrs, void* y, uint32_t batch) {
    if (!w || w->kind != PDX_PLANE_F8ROW) return ex->fail(PDX_UNSUPPORTED, "f8row_gemm needs an F8RowPlane");
    // fp8.rs:606-636: the warp-specialized tcgen05 slot first, PADDOCK_NO_F8ROW_TC5X keeps the older arm
    static const bool no_tc5x = getenv("PADDOCK_NO_F8ROW_TC5X") != nullptr;
    auto fx = ex->op<decltype(&pd_f8row_gemm_tc5x)>(PDK_SLOT_f8row_gemm_tc5x);
    if (fx && !no_tc5x && w->in_dim % 128u == 0)
        return ex->launched(fx(w->data.p, w->scale.p, xq, xrs, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, batch, ex->stream),
                            "f8row_gemm_tc5x");
    auto f = ex->op<decltype(&pd_f8row_gemm)>(PDK_SLOT_f8row_gemm);
    if (!f) return ex->fail(PDX_MISSING_OP, "f8row_gemm");
    return ex->launched(f(w->data.p, w->scale.p, xq, xrs, y, (uint32_t)w->in_dim, (uint32_t)w->out_dim, batch, ex->stream),
                        "f8row_gemm");
}

PDX_EXPORT int pdx_quantize_nvf4(PdxExecutor* ex, const void* x, void* q, void* scale, uint32_t n) {
    auto f = ex->op<decltype(&pd_quantize_nvf4)>(PDK_SLOT_quantize_nvf4);
    if (!f) return ex->fail(PDX_MISSING_OP, "quantize_nvf4");
    return ex->launched(f(x, q, scale, n, ex->stream), "quantize_nvf4");
}

PDX_EXPORT int pdx_nvf4_gemm_f4(PdxExecutor* ex, const PdxPlane* w, const void* xq, const void* xs, void* y,
                                const void* bias, uint32_t batch) {
    if (!w || w->kind != PDX_PLANE_NVF4) return ex->fail(PDX_UNSUPPORTED, "nvf4_gemm_f4 needs an Nvf4Plane");
    if (w->layout != PDX_NVF4_ROW)
        return ex->fail(PDX_UNSUPPORTED, "nvf4_gemm_f4 reads the row-major layout; tiled/frag plane refused");
    auto f = ex->op<decltype(&pd_nvf4_gemm_tc5w)>(PDK_SLOT_nvf4_gemm_tc5w);
    if (!f || !w->scale_tc5.p)
        return ex->fail(PDX_MISSING_OP, "nvf4_gemm_f4: the plane has no tensor-core scale cells (in_dim %% 256) or the pack no tcgen05 arm");
    return ex->launched(f(w->data.p, w->scale_tc5.p, bias, xq, xs, y, w->scale2, (uint32_t)w->in_dim, (uint32_t)w->out_dim,
                          batch, nullptr, 0, ex->stream),
                        "nvf4_gemm_tc5w");
}

PDX_EXPORT int pdx_nvf4_gemv(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y) {
    if (!w || w->kind != PDX_PLANE_NVF4 || w->layout != PDX_NVF4_ROW)
        return ex->fail(PDX_UNSUPPORTED, "nvf4_gemv needs a row-major Nvf4Plane");
    auto f = ex->op<decltype(&pd_nvf4_gemv)>(PDK_SLOT_nvf4_gemv);
    if (!f) return ex->fail(PDX_MISSING_OP, "nvf4_gemv");
    return ex->launched(f(w->data.p, w->scale.p, bias, x, y, w->scale2, (uint32_t)w->in_dim, (uint32_t)w->out_dim, ex->stream),
                        "nvf4_gemv");
}
