/*
 * paddock_host.h - C ABI of libpaddock_host.so: the host-side file formats that
 * feed the kernel pack (weight-format table, GGUF and safetensors readers,
 * ModelOpt / llm-compressor quantized views, GGUF-NVFP4 row repack).
 *
 * Host-only C++ (no CUDA).  Everything that reads a file treats it as untrusted:
 * every read is bounds checked, every count capped, and a malformed file yields
 * an error code plus a message, never a crash.  Pointers handed out point into a
 * read-only mapping that stays valid until the handle is closed.
 */
#ifndef PADDOCK_HOST_H
#define PADDOCK_HOST_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- weight formats (crates/paddock-models/src/ggml_type.rs:16-54,146-200) ---------------- */

enum PdkGgmlType {
    PDK_GGML_F32 = 0, PDK_GGML_F16 = 1, PDK_GGML_Q4_0 = 2, PDK_GGML_Q8_0 = 8, PDK_GGML_Q4_K = 12,
    PDK_GGML_Q5_K = 13, PDK_GGML_Q6_K = 14, PDK_GGML_IQ4_XS = 23, PDK_GGML_BF16 = 30,
    PDK_GGML_MXFP4 = 39, PDK_GGML_NVFP4 = 40
};
/* (elements, bytes) of one block of raw type id `raw`; returns 0 when the layout is unknown */
int pdk_ggml_block_layout(uint32_t raw, uint32_t* elems, uint32_t* bytes);
/* bytes of n_elements in that type; returns 0 when unknown or n is not a whole number of blocks */
int pdk_ggml_byte_size(uint32_t raw, uint64_t n_elements, uint64_t* bytes);

/* ---- GGUF (crates/paddock-models/src/gguf.rs:176-322, mapped.rs:176,343) -------------------- */

enum PdkGgufError {
    PDK_GGUF_OK = 0, PDK_GGUF_BAD_MAGIC = 1, PDK_GGUF_UNSUPPORTED_VERSION = 2, PDK_GGUF_TRUNCATED = 3,
    PDK_GGUF_COUNT_TOO_LARGE = 4, PDK_GGUF_BAD_UTF8 = 5, PDK_GGUF_UNKNOWN_VALUE_TYPE = 6,
    PDK_GGUF_ARRAY_TOO_DEEP = 7, PDK_GGUF_BAD_ALIGNMENT = 8, PDK_GGUF_BAD_TENSOR = 9,
    PDK_GGUF_DUPLICATE_TENSOR = 10, PDK_GGUF_IO = 11, PDK_GGUF_NOT_FOUND = 12
};
typedef struct PdkGguf PdkGguf;
/* mmap + parse; err (may be NULL) receives a message */
int pdk_gguf_open(const char* path, PdkGguf** out, char* err, size_t err_len);
/* parse an in-memory image (the handle keeps a copy) */
int pdk_gguf_parse(const void* bytes, size_t len, PdkGguf** out, char* err, size_t err_len);
void pdk_gguf_close(PdkGguf* g);
uint32_t pdk_gguf_version(const PdkGguf* g);
uint64_t pdk_gguf_alignment(const PdkGguf* g);
uint64_t pdk_gguf_data_offset(const PdkGguf* g);
uint64_t pdk_gguf_tensor_count(const PdkGguf* g);
/* i-th tensor: name (valid until close), dims (dims[0] fastest), raw ggml type, byte size or 0 */
int pdk_gguf_tensor_at(const PdkGguf* g, uint64_t i, const char** name, uint32_t* n_dims, uint64_t dims[8],
                       uint32_t* raw_type, uint64_t* offset, uint64_t* n_bytes);
/* zero-copy bytes of a named tensor, bounds re-checked against the mapping */
int pdk_gguf_tensor_bytes(const PdkGguf* g, const char* name, const void** data, uint64_t* n_bytes,
                          uint32_t* raw_type, uint32_t* n_dims, uint64_t dims[8]);
/* scalar / string metadata; return PDK_GGUF_NOT_FOUND when absent or of another kind */
int pdk_gguf_meta_u64(const PdkGguf* g, const char* key, uint64_t* value);
int pdk_gguf_meta_str(const PdkGguf* g, const char* key, const char** value);

/* ---- split GGUF families (crates/paddock-models/src/split.rs:13-62, mapped.rs:176-345) -------- */

enum PdkMapError {
    PDK_MAP_OK = 0, PDK_MAP_IO = 1, PDK_MAP_PARSE = 2, PDK_MAP_NO_SUCH_TENSOR = 3, PDK_MAP_OUT_OF_RANGE = 4,
    PDK_MAP_UNSIZABLE = 5, PDK_MAP_NOT_FIRST_SPLIT = 6, PDK_MAP_SPLIT_NAME_MISMATCH = 7, PDK_MAP_SHARD_MISMATCH = 8,
    PDK_MAP_MISSING_SPLIT_KEY = 9, PDK_MAP_TENSOR_COUNT_MISMATCH = 10, PDK_MAP_DUPLICATE_ACROSS_SHARDS = 11,
    PDK_MAP_TOO_MANY_SPLITS = 12
};
/* "<prefix>-%05d-of-%05d.gguf" (1-based shard number): 0 and the fields, or 1 for any other name */
int pdk_split_name_parse(const char* path, char* prefix, size_t prefix_len, uint32_t* no_1based, uint32_t* count);
typedef struct PdkGgufFamily PdkGgufFamily;
/* One file, or - when its split.count exceeds 1 - the whole family, one mapping per shard, opened
 * through the FIRST shard: every sibling's split.no / split.count is checked against its place,
 * a tensor name may appear in one shard only, and split.tensors.count of the first shard must
 * equal the union.  Any failure is an error; a family never loads as a smaller model. */
int pdk_gguf_family_open(const char* path, PdkGgufFamily** out, char* err, size_t err_len);
void pdk_gguf_family_close(PdkGgufFamily* f);
uint64_t pdk_gguf_family_shard_count(const PdkGgufFamily* f);
uint64_t pdk_gguf_family_tensor_count(const PdkGgufFamily* f);
uint64_t pdk_gguf_family_total_len(const PdkGgufFamily* f);
/* shard 0 carries the model's metadata; the handle stays owned by the family */
const PdkGguf* pdk_gguf_family_shard(const PdkGgufFamily* f, uint64_t shard);
const char* pdk_gguf_family_shard_path(const PdkGgufFamily* f, uint64_t shard);
/* i-th tensor of the union: shards in family order, file order inside a shard */
int pdk_gguf_family_tensor_at(const PdkGgufFamily* f, uint64_t i, const char** name, uint32_t* n_dims,
                              uint64_t dims[8], uint32_t* raw_type, uint64_t* n_bytes, uint32_t* shard);
/* zero-copy bytes of a named tensor out of the shard that holds it */
int pdk_gguf_family_tensor_bytes(const PdkGgufFamily* f, const char* name, const void** data, uint64_t* n_bytes,
                                 uint32_t* raw_type, uint32_t* n_dims, uint64_t dims[8], uint32_t* shard);

/* ---- safetensors (crates/paddock-models/src/safetensors.rs:102-190, 336-420) ------------------ */

enum PdkStDtype {
    PDK_ST_F8_E4M3 = 0, PDK_ST_BF16 = 1, PDK_ST_F16 = 2, PDK_ST_F32 = 3, PDK_ST_I64 = 4, PDK_ST_U8 = 5,
    PDK_ST_U32 = 6, PDK_ST_OTHER = 7
};
enum PdkStError { PDK_ST_OK = 0, PDK_ST_IO = 1, PDK_ST_HEADER = 2, PDK_ST_NOT_FOUND = 3 };
typedef struct PdkSafetensors PdkSafetensors;
/* a single .safetensors file, or a directory holding model.safetensors.index.json / model.safetensors */
int pdk_st_open(const char* path, PdkSafetensors** out, char* err, size_t err_len);
void pdk_st_close(PdkSafetensors* s);
uint64_t pdk_st_tensor_count(const PdkSafetensors* s);
int pdk_st_tensor(const PdkSafetensors* s, const char* name, uint32_t* dtype, uint32_t* n_dims, uint64_t shape[8],
                  const void** data, uint64_t* n_bytes);

/* ---- quantized checkpoint views (crates/paddock-models/src/modelopt.rs:168-352) ---------------- */

/* NVFP4 triple of `<prefix>`: ModelOpt (weight / weight_scale / weight_scale_2) or llm-compressor
 * (weight_packed / weight_scale / weight_global_scale, scale2 = 1 / global). */
int pdk_st_nvfp4_view(const PdkSafetensors* s, const char* prefix, const void** packed, const void** scales,
                      float* scale2, uint64_t* n, uint64_t* k, char* err, size_t err_len);
/* FP8 per-channel: weight F8_E4M3 [n][k] + weight_scale (BF16 [n] / [n,1], or one F32 broadcast);
 * row_scales points at n f32 owned by the handle. */
int pdk_st_fp8_channel_view(PdkSafetensors* s, const char* prefix, const void** weight, const float** row_scales,
                            uint64_t* n, uint64_t* k, char* err, size_t err_len);

/* ---- GGUF NVFP4 blocks -> row layout (crates/paddock-models/src/gguf_nvfp4.rs:34-83) ----------- */
/* src: rows * in_dim/64 blocks of 36 bytes; codes [rows][in_dim/2], scales [rows][in_dim/16].
 * Returns 0, or 1 with a message (bad sizes, signed scale byte).  0x7F scale bytes become 0. */
int pdk_nvfp4_gguf_repack_rows(const void* src, uint64_t src_len, uint64_t rows, uint64_t in_dim, void* codes,
                               void* scales, uint64_t* nan_scales, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif
