/*
 * paddock_pack.h - C ABI of libpaddock_b200.so, a B200 (sm_100a) kernel pack
 * for Paddock's quantized linear-layer path.
 *
 * The library is a drop-in "kernel pack": it exports the two symbols the
 * reference's loader resolves (crates/paddock-kernels/src/abi.rs:42-46,
 * loader.rs:140-288) and fills the slots of KernelTableV1 that belong to this
 * path; every other slot is NULL, which the engine reports as a missing op at
 * the point of use (crates/paddock-engine/src/gpu/error.rs:36-40).
 *
 * Conventions shared by every launcher (abi.rs:48-54, packs/cuda/src/abi.cuh:11-16):
 *   - all pointers are raw device pointers owned by the caller;
 *   - the last argument is the caller's CUstream; launches are asynchronous;
 *   - the return value is 0 or a raw cudaError_t; shapes the kernel cannot
 *     take are refused up front with cudaErrorInvalidValue (1) or
 *     cudaErrorNotSupported (801), never assumed;
 *   - the pack never allocates, synchronizes or creates streams.
 *
 * The launchers are also exported by name (pd_*), with the signatures the
 * reference gives the same names in packs/cuda/src/abi.cuh, so a host that
 * links instead of walking the table binds the same entry points.
 */
#ifndef PADDOCK_PACK_H
#define PADDOCK_PACK_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PDK_PACK_MAGIC 0x504b4450u      /* "PDKP", abi.rs:13 */
#define PDK_PACK_ABI_VERSION 2u         /* abi.rs:10 */
#define PDK_TABLE_SLOTS 953u            /* abi.rs:1186-12800 */
#define PDK_TABLE_BYTES (8u + 8u * PDK_TABLE_SLOTS) /* 7632, abi.rs:12805-12812 */

/* ggml type ids used as the k-quant `dtype` tag (packs/cuda/src/quant/kquant.cuh:64-68) */
#define PDK_KQ_Q4_0 2u
#define PDK_KQ_Q4K 12u
#define PDK_KQ_Q5K 13u
#define PDK_KQ_Q6K 14u
#define PDK_KQ_IQ4XS 23u

#define PDK_MOE_PAD 0xFFFFFFFFu         /* packs/cuda/src/attn/decode.cuh: PD_MOE_PAD */

/* abi.rs:20-28, packs/cuda/src/abi.cuh:361-366 */
typedef struct PdkPackInfo {
    uint32_t magic;
    uint32_t abi_version;
    uint8_t arch[16];
    uint32_t pack_version[3];
} PdkPackInfo;

/* abi.rs:1186-1189: {u32 size; u32 reserved; 953 nullable fn pointers} */
typedef struct PdkKernelTableV1 {
    uint32_t size;
    uint32_t reserved;
    void* slot[PDK_TABLE_SLOTS];
} PdkKernelTableV1;

/* 0-based member index of each implemented slot inside KernelTableV1 (byte
 * offset 8 + 8*idx), in the member order of packs/cuda/src/abi.cuh:368-... */
enum PdkSlot {
    PDK_SLOT_mxfp4_dequant_f32 = 0,
    PDK_SLOT_q8_0_dequant_f32 = 1,
    PDK_SLOT_add_inplace_f32 = 6,
    PDK_SLOT_mxfp4_repack = 37,
    PDK_SLOT_q8_0_repack = 51,
    PDK_SLOT_q8_0_gemv_repacked = 52,
    PDK_SLOT_q8_0_gemm_repacked = 57,
    PDK_SLOT_kquant_dequant = 202,
    PDK_SLOT_kquant_repack = 203,
    PDK_SLOT_kquant_gemv = 204,
    PDK_SLOT_quantize_e4m3_row = 183,
    PDK_SLOT_f8row_gemm = 184,
    PDK_SLOT_bf16_to_f8row = 375,
    PDK_SLOT_f8row_gemm_tc5x = 855,
    PDK_SLOT_quantize_nvf4 = 119,
    PDK_SLOT_add_rmsnorm_quant_nvf4_batch = 436,
    PDK_SLOT_nvf4_dequant = 393,
    PDK_SLOT_nvf4_gemv = 394,
    PDK_SLOT_nvf4_gemm_tc5w = 852,
    PDK_SLOT_nvf4_tc5_tile_scales = 853,
    PDK_SLOT_moe_topk_batch = 29,
    PDK_SLOT_moe_align = 34,
    PDK_SLOT_moe_slot_combine = 91,
    PDK_SLOT_moe_align_bm = 146,
    PDK_SLOT_quantize_q8 = 18,
    PDK_SLOT_quantize_q8_sums = 218,
    PDK_SLOT_kquant_gemv_w4a8 = 217,
    PDK_SLOT_kquant_gemm_mma_ks = 212,
    PDK_SLOT_kquant_gemm_w4a8_sb = 837,
    PDK_SLOT_mxfp4_moe_gate_up_mmq = 88,
    PDK_SLOT_mxfp4_moe_down_mmq = 89,
    PDK_SLOT_mxfp4_moe_gate_up_dp4a_b = 92,
    PDK_SLOT_mxfp4_moe_down_dp4a_b = 93,
    PDK_SLOT_mxfp4_gu_interleave = 155,
    PDK_SLOT_swiglu_quant_e4m3_row = 511,
    PDK_SLOT_rmsnorm_quant_e4m3_row = 512,
    PDK_SLOT_add_rmsnorm_scaled_quant_e4m3_row = 513,
    PDK_SLOT_quantize_nvf4_swiglu = 120,
    PDK_SLOT_swiglu_fused_nvf4 = 516,
    PDK_SLOT_add_rmsnorm_nvf4_batch = 861
};

/* ---- the drop-in boundary ------------------------------------------------ */

/* abi.rs:42, packs/cuda/src/exports.cuh:757.  Static storage. */
const PdkPackInfo* paddock_pack_info(void);
/* abi.rs:46, packs/cuda/src/exports.cuh:2114-2400.  Static storage; slots this pack does not
 * implement are NULL, and so is every slot when the device that is current at the first call is
 * not of compute capability 10.0 (the only one sm_100a code loads on). */
const PdkKernelTableV1* paddock_pack_kernels_v1(void);
/* Diagnostics, no counterpart in the reference: the table as paddock_pack_kernels_v1 resolves it
 * for a device of the given compute capability, written to caller storage (PDK_TABLE_BYTES). */
int pdk_kernels_for_cc(int cc_major, int cc_minor, PdkKernelTableV1* out);

/* ---- Q8_0 (packs/cuda/src/deltanet/core.cuh:2552-3090) -------------------- */

/* slot 1, packs/cuda/src/gemm/f32_qkv.cuh:138-147 + elementwise.cuh:65-79:
 * n_blocks 34-byte blocks {f16 d, int8 q[32]} -> f32[n_blocks*32], y = q*d. */
int pd_q8_0_dequant_f32(const void* in, void* out, uint64_t n_blocks, void* stream);
/* slot 51, core.cuh:2567-2576: 34-byte blocks -> int8 plane [n_blocks*32] +
 * f16 scale plane [n_blocks]. */
int pd_q8_0_repack(const void* src, void* dst_data, void* dst_scale, uint64_t n_blocks, void* stream);
/* slot 52, core.cuh:2698-2730: y[o] = bias[o] + sum_b d[o,b] * sum_i q*x over
 * repacked planes; x f32[in_dim], y f32[out_dim], bias f32 or NULL, f32 math. */
int pd_q8_0_gemv_repacked(const void* data, const void* scale, const void* bias, const void* x,
                          void* y, uint32_t in_dim, uint32_t out_dim, void* stream);
/* slot 57, core.cuh:3076-3090: x f32[batch][in_dim], y f32[batch][out_dim]. */
int pd_q8_0_gemm_repacked(const void* data, const void* scale, const void* bias, const void* x,
                          void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);

/* ---- k-quants (packs/cuda/src/quant/kquant.cuh) --------------------------- */

/* slot 202, kquant.cuh:144-250: n_super raw GGUF super-blocks -> f32[n_super*256].
 * Q4_K: y = (d*sc_j)*q - (dmin*m_j).  dtype = PDK_KQ_*. */
int pd_kquant_dequant(const void* src, void* dst, uint64_t n_super, uint32_t dtype, void* stream);
/* slot 203, kquant.cuh:255-345 (layout kquant.cuh:37-54): Q4_K -> data 128 B/sb
 * (nibbles verbatim) + 24 B/sb record {f16 d, f16 dmin, u8 sc[8], u8 m[8], pad4}. */
int pd_kquant_repack(const void* src, void* dst_data, void* dst_scales, uint64_t n_super,
                     uint32_t dtype, void* stream);
/* slot 204, kquant.cuh:372-653: exact-f32 decode GEMV over repacked planes. */
int pd_kquant_gemv(const void* data, const void* scales, const void* x, void* y, uint32_t in_dim,
                   uint32_t out_dim, uint32_t dtype, void* stream);
/* slot 18, packs/cuda/src/gemm/f32_qkv.cuh:283-292 (kernel attn/decode.cuh:2981-3004): per-32
 * int8 activation quantization, scale = amax / 127 (f32 [n/32]), q = RN(x / scale) in +-127. */
int pd_quantize_q8(const void* x, void* q, void* scale, uint32_t n, void* stream);
/* slot 218, f32_qkv.cuh:304-311 (kernel attn/decode.cuh:3041-3068): slot 18 plus the per-16
 * sums of q as f32 [n/16]. */
int pd_quantize_q8_sums(const void* x, void* q, void* scale, void* sums, uint32_t n, void* stream);
/* slot 217, packs/cuda/src/quant/kquant_w4a8.cuh:1266-1330: decode GEMV on the int8 activations of
 * slot 18 / 218.  The activations are widened (q * scale) inside the kernel; xsums is not needed.
 * 801 for shapes outside the GEMV kernel's plan. */
int pd_kquant_gemv_w4a8(const void* data, const void* scales, const void* xq, const void* xs, const void* xsums,
                        void* y, uint32_t in_dim, uint32_t out_dim, uint32_t dtype, void* stream);
/* slots 212 and 837, kquant_w4a8.cuh:2364-2430 and kquant_w4a8_sb.cuh:300-353: batch <= 64 on the
 * same operands, y f32[batch][out_dim]; `part` (>= 8 * out_dim * batch floats by the slots'
 * contract) holds the widened activations.  in_dim <= 8 * out_dim. */
int pd_kquant_gemm_mma_ks(const void* data, const void* scales, const void* xq, const void* xs, const void* xsums,
                          void* part, void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t dtype,
                          void* stream);
int pd_kquant_gemm_w4a8_sb(const void* data, const void* scales, const void* xq, const void* xs, const void* xsums,
                           void* part, void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t dtype,
                           void* stream);
/* No slot: small-batch sibling of pd_kquant_gemv with f32 activations,
 * x f32[batch][in_dim], y f32[batch][out_dim], batch <= 64.  The reference's
 * small-batch route quantizes activations to int8 first (kquant_w4a8_sb.cuh);
 * this keeps them f32, the numeric class of slot 204. */
int pdk_kquant_gemm_f32(const void* data, const void* scales, const void* x, void* y,
                        uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t dtype,
                        void* stream);

/* ---- FP8 E4M3, one f32 scale per row ----------------------------------------- */

/* slot 375, packs/cuda/src/gemm/dense_fp4_w8.cuh:627-677: bf16 weights [out][in] ->
 * e4m3 [out][in] + f32 row scale 2^e, e = ex - 9 + (fr > 0.875) for amax = fr*2^ex. */
int pd_bf16_to_f8row(const void* bf16, void* f8_data, void* row_scale, uint32_t in_dim, uint32_t out_dim,
                     void* stream);
/* slot 183, packs/cuda/src/gemm/dense_f8_decode.cuh:3179-3235: f32 activations
 * [batch][n_dim] -> e4m3 + f32 scale per token row, same power-of-two rule. */
int pd_quantize_e4m3_row(const void* x, void* q, void* rscale, uint32_t n_dim, uint32_t batch, void* stream);
/* slot 184, packs/cuda/src/gemm/dense_f8_decode.cuh:4638-4722 (kernel gemm/dense_tc5.cuh:46-215):
 * y f32 [batch][out] = (sum_k W[o][k] Xq[t][k]) * w_rowscale[o] * x_rowscale[t], tcgen05 + TMA.
 * in_dim must be a multiple of 16; data and xq 16-byte aligned. */
int pd_f8row_gemm(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale, void* y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);
/* slot 855, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:1480-1515: same contract as slot 184. */
int pd_f8row_gemm_tc5x(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale, void* y,
                       uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);
/* slots 511, 512, 513 (packs/cuda/src/exports.cuh:380-500, gemm/dense_f8_decode.cuh:4357-4575; callers
 * gpu/fp8.rs:469-590): the fused producers in front of the e4m3 GEMM.  All end in slot 183's row
 * quantizer (q e4m3 [batch][n] + one power-of-two f32 scale per row); n % 32 == 0, 16-byte
 * aligned rows.
 *   swiglu_quant:  h = silu(gate) * up in f32
 *   rmsnorm_quant: xn f32 [batch][n] = x * (1 / sqrtf(mean(x^2) + eps)) * w, quantized
 *   add_rmsnorm_scaled_quant: x += pscale * proj first (written back), then as rmsnorm_quant
 * Status 100 = declined (rows beyond 65536 elements): the engine then runs the unfused chain. */
int pd_swiglu_quant_e4m3_row(const void* gate, const void* up, void* q, void* rscale, uint32_t n, uint32_t batch,
                             void* stream);
int pd_rmsnorm_quant_e4m3_row(const void* x, const void* w, void* xn, void* q, void* rscale, uint32_t n, float eps,
                              uint32_t batch, void* stream);
int pd_add_rmsnorm_scaled_quant_e4m3_row(void* x, const void* proj, const void* w, void* xn, void* q, void* rscale,
                                         uint32_t n, float eps, float pscale, uint32_t batch, void* stream);
/* No slot: slot 184 with bf16 output (the reference writes f32). */
int pdk_f8row_gemm_bf16(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale, void* y,
                        uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);
/* No slot: reads and clears the device error word the tcgen05 kernels report a
 * timed-out wait in (0 = none; code << 8 | detail otherwise).  Synchronizes the
 * device, so it is a test / diagnostics call, never part of a launch path. */
unsigned int pdk_device_error(void);

/* ---- NVFP4: e2m1 nibbles (low nibble = even k), e4m3 scale per 16, f32 scale2 per tensor --- */

/* slot 119, packs/cuda/src/quant/nvf4.cuh:405-421 (rules quant/e2m1.cuh:12-41): f32 x[n] ->
 * q u8[n/2] + scale u8[n/16]; scale = RN_e4m3(amax/6), at least the smallest subnormal when
 * amax > 0; element = RN-even e2m1 of v/scale.  n % 32 == 0. */
int pd_quantize_nvf4(const void* x, void* q, void* scale, uint32_t n, void* stream);
/* Slot 436 (packs/cuda/src/quant/nvf4.cuh:545-571; caller gpu_model/nemotron MoE prologue): the
 * producer in front of an NVFP4 GEMM.  x f32 [batch][n] += proj (null: no residual), written back;
 * out f32 [batch][n] = x * inv * w with inv = 1 / sqrtf(mean(x^2) + eps); q u8 [batch][n/2] and
 * scale e4m3 [batch][n/16] = pd_quantize_nvf4 of each row of out.  n % 32 == 0, n <= 51200. */
int pd_add_rmsnorm_quant_nvf4_batch(void* x, const void* proj, const void* w, void* out, void* q, void* scale,
                                    uint32_t n, float eps, uint32_t batch, void* stream);
/* slots 120 and 516 (packs/cuda/src/quant/nvf4.cuh:714-775; gpu/fp4.rs:206-260): SwiGLU in front of
 * the NVFP4 quantizer, h = (g / (1 + expf(-g))) * u in f32.  120: gate and up are planes of n
 * elements; 516: the two halves of fused rows [n_rows][2 * ff].  n, ff multiples of 32. */
int pd_quantize_nvf4_swiglu(const void* gate, const void* up, void* q, void* scale, uint32_t n, void* stream);
int pd_swiglu_fused_nvf4(const void* fused, void* q, void* scale, uint32_t ff, uint32_t n_rows, void* stream);
/* slot 861 (packs/cuda/src/exports.cuh:505-520): slot 436's contract with proj required */
int pd_add_rmsnorm_nvf4_batch(void* x, const void* proj, const void* w, void* out, void* q, void* qs, uint32_t n, float eps,
                              uint32_t batch, void* stream);
/* slot 393, packs/cuda/src/quant/nvf4.cuh:4365-4403: y f32[out][in] = (e2m1 * e4m3) * scale2. */
int pd_nvf4_dequant(const void* data, const void* scale, float scale2, void* y, uint32_t in_dim,
                    uint32_t out_dim, void* stream);
/* slot 394, packs/cuda/src/quant/nvf4.cuh:4436-4779: W4A16 decode GEMV, f32 x,
 * y[o] = scale2 * sum + bias[o] (bias may be NULL). */
int pd_nvf4_gemv(const void* data, const void* scale, const void* bias, const void* x, void* y, float scale2,
                 uint32_t in_dim, uint32_t out_dim, void* stream);
/* slot 853, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:845-861,981-994: weight scales [out][in/16]
 * -> ceil(out/128) * (in/256) records of 2048 bytes in the tensor core's scale-cell order.
 * in_dim % 256 == 0. */
int pd_nvf4_tc5_tile_scales(const void* scale, void* tiled, uint32_t in_dim, uint32_t out_dim, void* stream);
/* slot 852, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:1216-1263: W4A4 GEMM, tcgen05 kind::mxf4nvf4 with
 * hardware block scaling.  xq u8[batch][in/2] + xs e4m3[batch][in/16] as pd_quantize_nvf4 writes
 * them; y f32[batch][out] = scale2 * acc + bias.  part / part_floats are accepted and unused. */
int pd_nvf4_gemm_tc5w(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs,
                      void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* part,
                      uint64_t part_floats, void* stream);
/* No slot: slot 852 with bf16 output and without the unused scratch arguments. */
int pdk_nvf4_gemm_bf16(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs,
                       void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream);

/* ---- MXFP4 ----------------------------------------------------------------- */

/* slot 0, packs/cuda/src/elementwise.cuh:47-62: 17-byte blocks {e8m0, 16 nibble
 * bytes} -> f32[n_blocks*32]; element j = low nibble of byte j, j+16 = high. */
int pd_mxfp4_dequant_f32(const void* in, void* out, uint64_t n_blocks, void* stream);
/* slot 37, packs/cuda/src/attn/decode.cuh:2294-2304 (launcher gemm/f32_qkv.cuh:1465). */
int pd_mxfp4_repack(const void* src, void* dst_data, void* dst_scale, uint64_t n_blocks, void* stream);

/* ---- MoE routing and MXFP4 expert GEMMs (caller: crates/paddock-engine/src/gpu_model/gpt_oss.rs:2279-2521) --- */

/* slot 29, packs/cuda/src/attn/decode.cuh:1392-1500: per token, k rounds of argmax over
 * logits + bias (ties to the lowest index); out_w = softmax over the k selected logits.
 * logits f32[batch][n_expert], out_idx u32[batch][k], out_w f32[batch][k]; n_expert <= 512, k <= 16. */
int pd_moe_topk_batch(const void* logits, const void* bias, uint32_t n_expert, uint32_t k, void* out_idx,
                      void* out_w, uint32_t batch, void* stream);
/* slot 34, packs/cuda/src/attn/decode.cuh:2316-2396: group the (token, slot) pairs by expert into
 * blocks of 32, padding each expert's tail.  sorted_row / sorted_slot u32[max_blocks*32]
 * (PDK_MOE_PAD = padding), block_expert u32[max_blocks] (PDK_MOE_PAD = unused block).
 * Entries of an expert are in ascending pair order (the reference's order is unspecified). */
int pd_moe_align(const void* idx, void* sorted_row, void* sorted_slot, void* block_expert, uint32_t rows,
                 uint32_t n_active, uint32_t n_expert, uint32_t max_blocks, void* stream);
/* slot 146, packs/cuda/src/gemm/f32_qkv.cuh:1269-1279: same with block size bm (a power of two). */
int pd_moe_align_bm(const void* idx, void* sorted_row, void* sorted_slot, void* block_expert, uint32_t rows,
                    uint32_t n_active, uint32_t n_expert, uint32_t bm, uint32_t max_blocks, void* stream);
/* slot 91, packs/cuda/src/moe/mmq.cuh:447-483: residual[t] += sum over slots (ascending) of
 * part[t*n_active + slot]; f32, embd % 4 == 0. */
int pd_moe_slot_combine(const void* part, void* residual, uint32_t embd, uint32_t n_active, uint32_t rows,
                        void* stream);
/* slot 155, packs/cuda/src/gemm/f32_qkv.cuh:1474-1505 (caller gpt_oss.rs:715-735): fuse the
 * repacked gate and up planes (n_kb 16-byte blocks per row) into one plane of `rows` rows with row
 * pitch ceil(n_kb / 4) * 128 bytes.  The fused plane is only ever read by slots of the same pack,
 * so its contents are the pack's own: here a row is [gate row | up row | padding]. */
int pd_mxfp4_gu_interleave(const void* gate, const void* up, void* dst, uint32_t n_kb, uint64_t rows, void* stream);
/* slot 88, packs/cuda/src/moe/mmq.cuh:550-571: gate + up + SwiGLU (xg * sigmoid(alpha xg) * (yu + up_add))
 * over the 32-row blocks of pd_moe_align.  gate_data = the fused plane of slot 155 (up_data, the
 * engine's dummy, is not read); xq int8[tokens][in_dim], xs f32[tokens][in_dim/32]; the result
 * leaves as fq int8[max_blocks*32][ff] with fs f32[..][ff/32] (amax / 127 per 32, round to nearest). */
int pd_mxfp4_moe_gate_up_mmq(const void* gate_data, const void* gate_scale, const void* gate_bias, const void* up_data,
                             const void* up_scale, const void* up_bias, const void* sorted_row,
                             const void* block_expert, const void* xq, const void* xs, void* fq, void* fs,
                             uint32_t in_dim, uint32_t ff, uint32_t max_blocks, float alpha, float limit, float up_add,
                             void* stream);
/* slot 89, packs/cuda/src/moe/mmq.cuh:592-626: part f32[rows*n_active][embd] = topk_w * (W_down h + bias)
 * per (token, slot), h = the fq / fs of slot 88. */
int pd_mxfp4_moe_down_mmq(const void* down_data, const void* down_scale, const void* down_bias, const void* sorted_row,
                          const void* sorted_slot, const void* block_expert, const void* topk_w, const void* fq,
                          const void* fs, void* part, uint32_t ff, uint32_t embd, uint32_t n_active,
                          uint32_t max_blocks, void* stream);
/* slots 92 / 93, packs/cuda/src/gemm/f32_qkv.cuh:370-398: the unsorted decode pair (the engine's
 * route up to 8 tokens on this GPU, gpt_oss.rs:104-135): pair (token, slot) reads expert idx[pair].
 * gate_up: out f32[batch][n_active][ff], SwiGLU with up + 1.  down: residual f32[batch][embd] +=
 * the token's slots in order; at most 262,144 f32 of per-pair rows (batch*n_active*embd). */
int pd_mxfp4_moe_gate_up_dp4a_b(const void* gate_data, const void* gate_scale, const void* gate_bias,
                                const void* up_data, const void* up_scale, const void* up_bias, const void* idx,
                                const void* xq, const void* xs, void* out, uint32_t in_dim, uint32_t ff,
                                uint32_t n_active, uint32_t batch, float alpha, float limit, void* stream);
int pd_mxfp4_moe_down_dp4a_b(const void* down_data, const void* down_scale, const void* down_bias, const void* idx,
                             const void* topk_w, const void* fused_q, const void* fused_s, void* residual, uint32_t ff,
                             uint32_t embd, uint32_t n_active, uint32_t batch, void* stream);
/* No slot.  Activation step in front of the expert GEMMs; the reference quantizes to int8 at this
 * point (pd_quantize_q8, packs/cuda/src/attn/decode.cuh:2981-3004).  x f32[rows][dim] ->
 * xq f16[rows][dim] (2*dim bytes per row, mma fragment order) + xscale f32[rows] (power-of-two
 * step per row): bf16 activations exactly, f32 ones to 11 significant bits.  dim % 32 == 0. */
int pdk_moe_prep_act(const void* x, void* xq, void* xscale, uint32_t dim, uint32_t rows, void* stream);
/* No slot; counterpart of slot 88 (pd_mxfp4_moe_gate_up_mmq, packs/cuda/src/moe/mmq.cuh:550-590)
 * with the activation operands of pdk_moe_prep_act.  gate/up planes as pd_mxfp4_repack writes
 * them: data [expert][ff][in/32*16], scale [expert][ff][in/32]; bias f32[expert][ff] or NULL.
 * h f32[max_blocks*bm][ff] = swiglu_oai(gate, up) in block order; bm = 8 or 32 as given to
 * pd_moe_align_bm. */
int pdk_mxfp4_moe_gate_up(const void* gate_data, const void* gate_scale, const void* gate_bias, const void* up_data,
                          const void* up_scale, const void* up_bias, const void* sorted_row, const void* block_expert,
                          const void* xq, const void* xscale, void* h, uint32_t in_dim, uint32_t ff, uint32_t bm,
                          uint32_t max_blocks, float alpha, float limit, void* stream);
/* No slot; counterpart of slot 89 (pd_mxfp4_moe_down_mmq, packs/cuda/src/moe/mmq.cuh:592-626).
 * hq / hscale = pdk_moe_prep_act of h.  part f32[rows*n_active][embd] = topk_w * (W_down h + bias). */
int pdk_mxfp4_moe_down(const void* down_data, const void* down_scale, const void* down_bias, const void* sorted_row,
                       const void* sorted_slot, const void* block_expert, const void* topk_w, const void* hq,
                       const void* hscale, void* part, uint32_t ff, uint32_t embd, uint32_t n_active, uint32_t bm,
                       uint32_t max_blocks, void* stream);

/* No counterpart in the reference.  A few launchers (the small-batch k-quant GEMMs, the NVFP4
 * W4A16 GEMV, the prefill-width NVFP4 GEMM) keep per-call scratch in the library, one slice per
 * (device, stream) for the first two streams of a device that make such calls; further streams
 * take the launchers' scratch-free routes.  Before destroying a stream that made such calls,
 * with the stream idle and its device current, call this so that a later stream can take its
 * slices over.  Thread-safe. */
void pdk_stream_release(void* stream);

/* No counterpart among the reference's exports (it keeps a bench program for the same purpose,
 * packs/cuda/src/gemm/dense_nvf4_tc5.cuh:306-309).  Issue-rate probe of the tensor core: one CTA per
 * SM issues n_mma (8 .. 2^20, a multiple of 4) tcgen05.mma on operands that stay in shared memory - kind 0 bf16
 * M128 N256 K16, 1 e4m3 M128 N256 K32, 2 NVFP4 block-scaled M128 N128 K64, 3 as 2 with the two
 * scale-cell copies a GEMM issues per MMA; 4 and 5: kinds 1 and 3 on pairs of SMs (cta_group::2,
 * M256 per pair, one issuing CTA per pair, flops = pairs * n_mma * 2 * 256 * N * K).  cycles: device u64[SM count] or NULL, SM clocks from
 * first issue to completion per CTA.  Flops of a launch = SMs * n_mma * 2 * 128 * N * K. */
int pdk_tc5_issue_probe(uint32_t kind, uint32_t n_mma, void* cycles, void* stream);

/* No counterpart in the reference (whose mbarrier waits spin without a bound).  Self-test of the
 * bounded wait under every tcgen05 kernel of this pack: one warp waits on a barrier that nothing
 * arrives on; returns 0 when the wait gave up after about budget_us microseconds (1..100000)
 * and the kernel returned normally, after which pdk_device_error() reads 0x507.  scratch = 4
 * bytes of device memory.  Synchronizes the stream. */
int pdk_selftest_bounded_wait(uint32_t budget_us, void* scratch, void* stream);

/* No counterpart in the reference.  Q4_K decode GEMV of one rank's row band whose epilogue stores
 * the band into every rank's full-length y over NVLink (y_ptrs: host array of n_ranks <= 8 device
 * pointers valid on this GPU, own buffer included; rows row0 .. row0 + out_dim) - the all-gather
 * of a row-sharded layer done by the kernel's own stores.  Ordering against consumers on other
 * ranks is the caller's (barrier or flag).  801 outside the GEMV kernel's plan. */
int pdk_q4k_gemv_shard(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                       uint32_t n_ranks, uint32_t row0, uint32_t in_dim, uint32_t out_dim, void* stream);

/* No counterpart in the reference.  pdk_q4k_gemv_shard with a completion signal, so that a step
 * needs no host barrier: once its band is stored in every rank's y, rank `rank` stores the step
 * number into word `rank` of every rank's flag array (flag_ptrs[p]: rank p's array of 16 u32
 * words, zeroed at set-up, mapped like y_ptrs: words 0..7 flags, word 8 the count of waits).
 * ctr: two zeroed u32 words of this rank's own memory, not shared between streams (CTA counter,
 * count of signalled steps).  step != 0 names the step (growing from call to call); step == 0
 * takes the rank's count plus one, so a captured launch can be replayed. */
int pdk_q4k_gemv_shard_sync(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                            const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank,
                            uint32_t row0, uint32_t step, uint32_t in_dim, uint32_t out_dim, void* stream);
/* The same for a loop that rotates THREE or more y buffers, which all share ONE flag array per rank and one
 * pair of counter words.  Nothing is signalled at the end of the kernel (the system-scope fence that takes
 * costs an NVLink round trip per step).  Every launch stores, once the stream's previous kernel and its
 * peer stores are complete, the number of the PREVIOUS launch into the flags, and checks before it ends (at
 * most a second; 0x1c << 8 | rank in the device error word for a rank that is late) that every rank's
 * previous step has arrived here: what sits between launch s and launch s + 1 in the stream may read step
 * s - 1 of every rank (a peer may already be storing step s + 1, hence three buffers).  The loop needs no
 * wait kernel between steps; pdk_peer_flags_post + pdk_peer_flags_wait close it. */
int pdk_q4k_gemv_shard_lagged(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                              const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank,
                              uint32_t row0, uint32_t step, uint32_t in_dim, uint32_t out_dim, void* stream);
/* Closes a pdk_q4k_gemv_shard_lagged loop: signals the stream's last launch (its number is ctr[1]) in
 * word `rank` of every rank's flag array, behind the stream's previous kernel. */
int pdk_peer_flags_post(const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank, void* stream);
/* No counterpart in the reference.  Device-side wait (one small kernel in `stream`) until all
 * n_ranks <= 8 flag words of this rank's flag array have reached the step (`step`; or with
 * step == 0 the array's count of waits plus one; or with step == 0x80000000 | r the step rank r,
 * the caller itself, signalled last); bounded: after budget_us microseconds the
 * kernel records 0x16 << 8 | late-rank in the device error word and returns. */
int pdk_peer_flags_wait(void* flags, uint32_t n_ranks, uint32_t step, uint32_t budget_us, void* stream);

/* ---- MXFP4 expert GEMMs on the block-scaled tensor-core path (no counterpart in the reference,
 * whose B200 MoE kernels are mma.sync on int8 activations, packs/cuda/src/moe/mmq.cuh:139-626).
 * The repacked data plane is used as it is; the E8M0 scale plane is re-expressed once at load time
 * as tiled UE4M3 scale records plus one power-of-two factor per plane; activations are expanded
 * into four NVFP4 terms per token. */

/* scale u8[n_expert][rows][in_dim/32] -> tiled u8[n_expert][ceil(rows/128)][ceil(in_dim/256)][2048]
 * and meta (8 bytes of device memory: u32 largest scale byte, f32 scale2).  in_dim % 64 == 0. */
int pdk_mxfp4_tc5_tile_scales(const void* scale, void* tiled, void* meta, uint32_t rows, uint32_t in_dim,
                              uint32_t n_expert, void* stream);
/* Block positions (pd_moe_align_bm order) -> four NVFP4 term rows each:
 * mode 0: position p = row sorted_row[p] of x f32[rows][dim];  mode 1: position p =
 * swiglu_oai(x[p], up[p]) of raw gate / up outputs f32[positions][dim].
 * Padding positions of used blocks become zero rows; the rows of unused blocks (block_expert = PDK_MOE_PAD),
 * which the GEMMs skip, are left as they are.
 * xq u8[max_blocks*4*bm][dim/2], xs u8[max_blocks][ceil(dim/256)][2048] (scale records, the layout
 * of the tiled weight scales; zero the buffer once), xstep f32[max_blocks*bm]. */
int pdk_moe_prep_act_f4(const void* x, const void* up, const void* sorted_row, const void* block_expert, void* xq,
                        void* xs, void* xstep, uint32_t dim, uint32_t bm, uint32_t max_blocks, uint32_t mode, float alpha, float limit,
                        void* stream);
/* Grouped GEMM of one or two planes (w1_data NULL = one) over the term rows.  scatter 0: out_p
 * f32[max_blocks*bm][out_dim], block order, bias added, no activation function; scatter 1 (one
 * plane): out0 = part f32[rows*n_active][out_dim] at row (sorted_row, sorted_slot), times topk_w.
 * in_dim % 64 == 0, bm = 8 or 32, max_blocks <= 1024 (the block table lives in shared memory). */
int pdk_mxfp4_moe_gemm_tc5(const void* w0_data, const void* w0_sf, const void* w0_meta, const void* w0_bias, void* out0,
                           const void* w1_data, const void* w1_sf, const void* w1_meta, const void* w1_bias, void* out1,
                           const void* xq, const void* xs, const void* xstep, const void* block_expert,
                           const void* sorted_row, const void* sorted_slot, const void* topk_w, uint32_t in_dim,
                           uint32_t out_dim, uint32_t n_expert, uint32_t bm, uint32_t max_blocks, uint32_t n_active,
                           uint32_t scatter, void* stream);

/* ---- NVFP4 expert planes on the same grouped GEMM (plane layout of
 * crates/paddock-engine/src/gpu/types.rs:176-226, Row order: data [expert*rows][in/2], scale e4m3
 * [expert*rows][in/16], scale2 f32[expert]).  No slot: the reference's NVFP4 MoE kernels read its
 * Tiled64 / CutBlk orders. */
/* scale -> tiled records u8[n_expert][ceil(rows/128)][ceil(in_dim/256)][2048]; in_dim % 64 == 0 */
int pdk_nvf4_moe_tile_scales(const void* scale, void* tiled, uint32_t rows, uint32_t in_dim, uint32_t n_expert,
                             void* stream);
/* No counterpart in the reference.  Decode widths: moe_topk_batch + moe_align_bm + pdk_moe_prep_act_f4
 * (mode 0) in one launch - rows * k <= 32 pairs, rows <= 8, n_expert <= 512, max_blocks <= 32.  Leaves
 * the same idx / w / sorted_row / sorted_slot / block_expert and term rows as the three calls. */
int pdk_moe_route_prep_f4(const void* logits, const void* router_bias, const void* x, void* idx, void* w,
                          void* sorted_row, void* sorted_slot, void* block_expert, void* xq, void* xs, void* xstep,
                          uint32_t n_expert, uint32_t k, uint32_t rows, uint32_t dim, uint32_t bm, uint32_t max_blocks,
                          void* stream);
/* pdk_moe_prep_act_f4 with the natural element order of NVFP4 planes.  mode 0 gather; mode 1 gated
 * unit (min(g, limit) * sigmoid(alpha * that)) * (clamp(u, +-limit) + up_add); mode 2 relu(x)^2. */
int pdk_moe_prep_act_f4n(const void* x, const void* up, const void* sorted_row, const void* block_expert, void* xq,
                         void* xs, void* xstep, uint32_t dim, uint32_t bm, uint32_t max_blocks, uint32_t mode,
                         float alpha, float limit, float up_add, void* stream);
/* pdk_mxfp4_moe_gemm_tc5 with w*_sf from pdk_nvf4_moe_tile_scales and w*_scale2 f32[n_expert] */
int pdk_nvf4_moe_gemm_tc5(const void* w0_data, const void* w0_sf, const void* w0_scale2, const void* w0_bias, void* out0,
                          const void* w1_data, const void* w1_sf, const void* w1_scale2, const void* w1_bias, void* out1,
                          const void* xq, const void* xs, const void* xstep, const void* block_expert,
                          const void* sorted_row, const void* sorted_slot, const void* topk_w, uint32_t in_dim,
                          uint32_t out_dim, uint32_t n_expert, uint32_t bm, uint32_t max_blocks, uint32_t n_active,
                          uint32_t scatter, void* stream);

/* No counterpart in the reference.  pdk_mxfp4_moe_down + pd_moe_slot_combine for callers that may
 * not allocate device memory (a serving loop that must stay off the allocator, a plug-in handed
 * pointers by its host, a process with a memory budget fixed at start-up): the per-(token, slot)
 * partial buffer is a 1 MiB static device array inside the library, held by every GPU that loads
 * it.  rows*n_active*embd <= pdk_static_part_capacity() (262144), otherwise refused with
 * cudaErrorInvalidValue (reason in pdk_static_last_refusal()).  The first call on a device resolves
 * the array's address and should come before any stream capture; calls share the array, so calls
 * that overlap on the GPU race. */
int pdk_mxfp4_moe_down_combine_static(const void* down_data, const void* down_scale, const void* down_bias,
                                      const void* sorted_row, const void* sorted_slot, const void* block_expert,
                                      const void* topk_w, const void* hq, const void* hscale, void* residual,
                                      uint32_t ff, uint32_t embd, uint32_t n_active, uint32_t rows, uint32_t bm,
                                      uint32_t max_blocks, void* stream);
uint64_t pdk_static_part_capacity(void);
const char* pdk_static_last_refusal(void);

/* ---- glue the engine's preflight needs ------------------------------------- */

/* slot 6 (crates/paddock-engine/src/gpu/mod.rs:507-528 launches it at start-up): y += x */
int pd_add_inplace_f32(void* y, const void* x, uint32_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif
