/*
 * oracle.h - CPU restatement of Paddock's quantized linear-layer math.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the CUDA path is
 * compared against; the product (libpaddock_b200.so) never links, loads or
 * calls it and has no CPU fallback.  Every function cites the reference file
 * (path inside truespar/paddock) whose arithmetic it restates.
 *
 * Parity status: PINNED.  tests/test_oracle_kat.py replays every known-answer
 * vector the reference's own tests hold for this path (reference/mod.rs,
 * tests/pack_parity.rs, ggml_type.rs, modelopt.rs, gguf_nvfp4.rs).
 */
#ifndef PADDOCK_ORACLE_H
#define PADDOCK_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar codecs ---------------------------------------------------- */
float    orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);            /* IEEE RNE, as half::f16::from_f32 */
float    orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float f);           /* RNE */
float    orc_e8m0_half_to_f32(uint8_t e);    /* reference/mod.rs:28-38 */
float    orc_e2m1_to_f32(uint8_t code);      /* modelopt.rs:384-391 */
float    orc_e4m3_to_f32(uint8_t b);         /* modelopt.rs:393-406 */
uint8_t  orc_f32_to_e4m3(float f);           /* RNE, saturate-to-finite (cuda_fp8 __nv_fp8_e4m3 ctor) */
uint8_t  orc_e2m1_rn(float v);               /* quant/e2m1.cuh:12-26 */

/* ---- dequantizers (return 0 ok, -1 bad input length, -2 bad output length) */
int orc_dequant_mxfp4(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
int orc_dequant_q8_0(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
int orc_dequant_q4_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
int orc_dequant_q5_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
int orc_dequant_q6_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
int orc_dequant_q4_0(const uint8_t* data, size_t n_bytes, float* out, size_t n_out);
void orc_scale_min_k4(const uint8_t* scales12, int j, uint32_t* sc, uint32_t* m);
/* NVFP4 plane: data u8[N][K/2], scale e4m3[N][K/16], scale2; w=(e2m1*e4m3)*scale2 */
void orc_dequant_nvfp4(const uint8_t* data, const uint8_t* scale, float scale2,
                       float* out, uint32_t in_dim, uint32_t out_dim);
/* FP8 per-channel plane: e4m3[N][K] * scale[N] */
void orc_dequant_fp8_channel(const uint8_t* w, const float* scale, float* out,
                             uint32_t in_dim, uint32_t out_dim);

/* ---- quantizers for the synthetic inputs ------------------------------ */
void orc_quantize_q8_0(const float* w, size_t n, uint8_t* out34);
void orc_quantize_q4_k(const float* w, size_t n, uint8_t* out144);
void orc_quantize_fp8_absmax(const float* w, uint32_t rows, uint32_t k, uint8_t* q, float* scale);
void orc_quantize_e4m3_row_pow2(const float* x, uint32_t rows, uint32_t k, uint8_t* q, float* scale);
void orc_quantize_nvf4(const float* x, size_t n, uint8_t* q, uint8_t* scale);
void orc_quantize_nvf4_global(const float* x, size_t n, float scale2, uint8_t* q, uint8_t* scale);
void orc_quantize_mxfp4(const float* w, size_t n, uint8_t* out17);
void orc_quantize_q8_act(const float* x, size_t n, int8_t* q, float* scale, float* sums16);

/* ---- repack restatements (byte-level expectations for the repack kernels) */
void orc_repack_q8_0(const uint8_t* src, uint64_t n_blocks, int8_t* data, uint16_t* scale);
void orc_repack_mxfp4(const uint8_t* src, uint64_t n_blocks, uint8_t* data, uint8_t* scale);

/* ---- linear algebra ---------------------------------------------------- */
/* reference CPU path: scalar f32 matvec, ascending k (reference/tensor.rs:39-54) */
void orc_matvec_f32(const float* w, const float* x, float* y, uint32_t in_dim, uint32_t out_dim);
/* y[m][n] = sum_k w[n][k] x[m][k], f64 accumulate; also optional sum|w x| */
void orc_matmul_f64(const float* w, const float* x, float* y, float* abs_sum,
                    uint32_t in_dim, uint32_t out_dim, uint32_t batch);

/* ---- MoE ---------------------------------------------------------------- */
void orc_moe_topk(const float* logits, const float* bias, uint32_t n_expert, uint32_t k,
                  uint32_t batch, uint32_t* out_idx, float* out_w);
void orc_swiglu_oai(float* gate, const float* up, size_t n, float alpha, float limit);
/* full MXFP4 MoE layer on dequantized experts, f64 accumulate:
 * gate/up/down: 17-byte-block MXFP4 [n_expert][rows][k/32*17]; biases may be NULL */
void orc_moe_mxfp4_layer(const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                         const float* gate_b, const float* up_b, const float* down_b,
                         const float* x, const uint32_t* topk_idx, const float* topk_w,
                         float* out, uint32_t tokens, uint32_t n_active, uint32_t embd,
                         uint32_t ff, float alpha, float limit);

/* ---- synthetic data ---------------------------------------------------- */
/* counter-based N(0, sigma): splitmix64 -> Box-Muller in f64 -> f32 */
void orc_fill_normal(float* out, size_t n, uint64_t seed, float sigma);

/* timing helper for the CPU baseline: threads the library will use */
int orc_num_threads(void);
void orc_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
