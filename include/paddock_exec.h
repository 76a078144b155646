/*
 * paddock_exec.h - C ABI of libpaddock_exec.so: the operator layer above the kernel-pack table.
 *
 * It is the C++ counterpart of the part of crates/paddock-engine/src/gpu that drives the
 * quantized linear layer: the executor that owns a loaded pack, a stream and a staging buffer
 * (gpu/mod.rs:143-252), the resident weight planes (gpu/types.rs:83-258, 425-520) and the
 * wrappers that upload, repack and launch (gpu/upload.rs:183-353, gpu/kquant.rs:180-528,
 * gpu/q8_gemm.rs:11-47, gpu/fp8.rs:228-659, gpu/fp4.rs:181-215, 1125-1168, 1712-1975).  Names
 * and argument meaning follow those wrappers; errors come back as the GpuError kinds of
 * gpu/error.rs.  Every launch goes through a slot of the pack's table: nothing here computes,
 * and nothing falls back to the host.
 *
 * Weight bytes come from host memory (normally a mapping handed out by paddock_host.h);
 * activations and outputs are device pointers owned by the caller.
 */
#ifndef PADDOCK_EXEC_H
#define PADDOCK_EXEC_H
#include <stddef.h>
#include <stdint.h>

#include "paddock_host.h"

#ifdef __cplusplus
extern "C" {
#endif

/* gpu/error.rs:8-60 */
enum PdxError {
    PDX_OK = 0,
    PDX_MISSING_OP = 1,   /* the pack's table has NULL in the slot this call needs */
    PDX_NO_KERNEL = 2,    /* no kernel class for this tensor's type */
    PDX_UNSUPPORTED = 3,  /* geometry or layout the wrapper refuses */
    PDX_DRIVER = 4,       /* a CUDA runtime call failed */
    PDX_LAUNCH = 5,       /* the launcher returned a status other than 0 */
    PDX_PACK = 6,         /* the pack could not be loaded or failed validation (loader.rs:140-283) */
    PDX_FORMAT = 7        /* the weight file refused the request (paddock_host.h error) */
};

/* which resident form a plane has (gpu/types.rs) */
enum PdxPlaneKind {
    PDX_PLANE_RAW = 0,    /* QuantTensor: the file's bytes, dequantized per use */
    PDX_PLANE_Q8 = 1,     /* RepackedQ8: int8 [out][in] + f16 [out][in/32] */
    PDX_PLANE_KQ = 2,     /* RepackedKQ: k-quant data + 24-byte records */
    PDX_PLANE_F8ROW = 3,  /* F8RowPlane: e4m3 [out][in] + one f32 scale per row */
    PDX_PLANE_NVF4 = 4,   /* Nvf4Plane: e2m1 pairs [out][in/2] + e4m3 [out][in/16] + scale2 */
    PDX_PLANE_MXFP4 = 5   /* RepackedMxfp4: 16 data bytes + 1 e8m0 byte per block, split */
};
/* gpu/types.rs:146-160; this pack reads the Row order only */
enum PdxNvf4Layout { PDX_NVF4_ROW = 0, PDX_NVF4_TILED = 1, PDX_NVF4_FRAG = 2 };

typedef struct PdxExecutor PdxExecutor;
typedef struct PdxPlane PdxPlane;

typedef struct PdxPlaneInfo {
    uint32_t kind;        /* PdxPlaneKind */
    uint32_t ggml_type;   /* raw ggml id of the resident form (a Q4_0 tensor uploaded raw reads 8) */
    uint64_t in_dim, out_dim;
    uint64_t bytes;       /* exact resident bytes, all streams (QuantW::bytes, types.rs:437-442) */
    void* data;           /* device pointers; NULL where the kind has no such stream */
    void* scale;
    void* scale_tc5;      /* Nvf4Plane: scale cells in the tensor core's order, or NULL */
    float scale2;         /* Nvf4Plane: per-tensor factor */
    uint32_t layout;      /* PdxNvf4Layout */
} PdxPlaneInfo;

/* ---- executor (gpu/mod.rs:143-252, loader.rs:140-283) ------------------------------------- */

/* Binds `device`, loads and validates the pack (NULL: the library beside this one), copies its
 * table and creates a non-blocking stream.  err (may be NULL) receives a message. */
int pdx_open(const char* pack_path, int device, PdxExecutor** out, char* err, size_t err_len);
void pdx_close(PdxExecutor* ex);
void* pdx_stream(const PdxExecutor* ex);
int pdx_synchronize(PdxExecutor* ex);
/* has_*() probes: 1 when the named table member (abi.rs field name) is filled */
int pdx_has(const PdxExecutor* ex, const char* slot_name);
/* message of the last failed call on this executor (valid until the next call) */
const char* pdx_last_error(const PdxExecutor* ex);
/* bytes the staging buffer holds now; it grows to the largest tensor at or below the cap
 * (128 MiB, PADDOCK_STAGING_MAX overrides) and larger tensors take a transient buffer
 * (gpu/upload.rs:203-304) */
uint64_t pdx_staging_bytes(const PdxExecutor* ex);
void pdx_release_staging(PdxExecutor* ex);

/* ---- planes -------------------------------------------------------------------------------- */

int pdx_plane_info(const PdxPlane* p, PdxPlaneInfo* out);
void pdx_plane_free(PdxExecutor* ex, PdxPlane* p);

/* upload_raw (gpu/upload.rs:183-203): the tensor's bytes as they are; Q4_0 lands as its exact
 * Q8_0 transcode */
int pdx_upload_raw(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, PdxPlane** out);
/* load_quantw (gpu/kquant.rs:180-240): per-tensor dispatch.  Q8_0 -> RepackedQ8; Q4_K / Q5_K /
 * Q6_K / IQ4_XS -> RepackedKQ; Q4_0 -> RepackedKQ when the row is whole super-blocks, else the Q8_0
 * transcode; anything else PDX_NO_KERNEL. */
int pdx_load_quantw(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, PdxPlane** out);
/* repack_q8_blocks (gpu/upload.rs:305-353) and repack_kquant_raw (gpu/kquant.rs:284-374) on host bytes */
int pdx_repack_q8_blocks(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t out_dim,
                         PdxPlane** out);
int pdx_repack_kquant_raw(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t out_dim,
                          uint32_t ggml_type, PdxPlane** out);
/* repack_kquant_bands (gpu/kquant.rs:381-414): the in dimension cut into n_bands equal strips of
 * whole super-blocks, each repacked as a weight of its own; out receives n_bands planes */
int pdx_repack_kquant_bands(PdxExecutor* ex, const PdkGgufFamily* map, const char* name, uint32_t n_bands,
                            PdxPlane** out);
/* repack_kquant_concat (gpu/kquant.rs:422-496): same-type tensors of one in_dim stacked along the
 * out dimension into one plane, each repacked at its running super-block offset */
int pdx_repack_kquant_concat(PdxExecutor* ex, const PdkGgufFamily* map, const char* const* names, uint32_t n_names,
                             PdxPlane** out);
/* repack_mxfp4 (gpu/moe_mxfp4.rs:908-936) on host bytes of 17-byte blocks */
int pdx_repack_mxfp4(PdxExecutor* ex, const void* bytes, uint64_t len, uint64_t in_dim, uint64_t rows, PdxPlane** out);
/* bf16_to_f8row (gpu/fp8.rs:247-289): host bf16 [out][in] -> F8RowPlane, quantized on the device */
int pdx_bf16_to_f8row(PdxExecutor* ex, const void* bf16, uint64_t in_dim, uint64_t out_dim, PdxPlane** out);
/* an FP8 per-channel checkpoint (pdk_st_fp8_channel_view) uploaded as it is */
int pdx_f8row_upload(PdxExecutor* ex, const void* e4m3, const float* row_scales, uint64_t in_dim, uint64_t out_dim,
                     PdxPlane** out);
/* nvf4_upload (gpu/fp4.rs:1125-1168): the checkpoint triple byte for byte, sizes checked against
 * the dims, plus nvf4_tc5_tile (fp4.rs:1712-1746) when in_dim is whole 256-element slabs */
int pdx_nvf4_upload(PdxExecutor* ex, const void* packed, uint64_t packed_len, const void* scales, uint64_t scales_len,
                    float scale2, uint64_t out_dim, uint64_t in_dim, PdxPlane** out);

/* ---- launches (device pointers; on the executor's stream) ---------------------------------- */

/* dequantize rows [row0, row0 + rows) of a RAW / Q8-transcoded / k-quant raw plane into f32 */
int pdx_dequant_rows(PdxExecutor* ex, const PdxPlane* p, uint64_t row0, uint64_t rows, void* out_f32);
/* QuantW decode GEMV: Q8 -> q8_0_gemv_repacked (bias may be NULL), Kq -> kquant_gemv (bias must be NULL) */
int pdx_quantw_gemv(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y);
/* small batch: Q8 -> q8_0_gemm_repacked, Kq -> the pack's f32 small-batch export (batch <= 64) */
int pdx_quantw_gemm(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y, uint32_t batch);
/* quantize_e4m3_row (gpu/fp8.rs:388-418) and f8row_gemm (fp8.rs:593-659: the tc5x slot when
 * in_dim % 128 == 0 and the pack has it, else slot f8row_gemm) */
int pdx_quantize_e4m3_row(PdxExecutor* ex, const void* x, void* q, void* rscale, uint32_t n_dim, uint32_t batch);
int pdx_f8row_gemm(PdxExecutor* ex, const PdxPlane* w, const void* xq, const void* xrs, void* y, uint32_t batch);
/* the fused producers in front of f8row_gemm (gpu/fp8.rs:469-590): *fused = 1 when the pack ran the
 * fused kernel, 0 when the slot is absent or declined (the engine's Ok(false)): run the unfused chain */
int pdx_swiglu_quant_e4m3_row(PdxExecutor* ex, const void* gate, const void* up, void* q, void* rs, uint32_t n_ff,
                              uint32_t batch, int* fused);
int pdx_rmsnorm_quant_e4m3_row(PdxExecutor* ex, const void* x, const void* w, void* xn, void* q, void* rs, uint32_t n,
                               float eps, uint32_t batch, int* fused);
int pdx_add_rmsnorm_scaled_quant_e4m3_row(PdxExecutor* ex, void* x, const void* proj, const void* w, void* xn, void* q,
                                          void* rs, uint32_t n, float eps, float pscale, uint32_t batch, int* fused);
/* quantize_nvf4 (gpu/fp4.rs:181-205), nvf4_gemm_f4 (fp4.rs:1902-1975: Row layout only; the tcgen05
 * slot when the plane carries tiled scales) and the W4A16 decode GEMV (slot nvf4_gemv) */
int pdx_quantize_nvf4(PdxExecutor* ex, const void* x, void* q, void* scale, uint32_t n);
int pdx_nvf4_gemm_f4(PdxExecutor* ex, const PdxPlane* w, const void* xq, const void* xs, void* y, const void* bias,
                     uint32_t batch);
int pdx_nvf4_gemv(PdxExecutor* ex, const PdxPlane* w, const void* bias, const void* x, void* y);

#ifdef __cplusplus
}
#endif
#endif
