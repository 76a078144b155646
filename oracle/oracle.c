/*
 * oracle.c - CPU restatement of Paddock's quantized linear-layer math.
 *
 * TEST INFRASTRUCTURE ONLY (see oracle.h).  Plain C + OpenMP.  Citations are
 * paths inside the truespar/paddock tree.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ======================================================================= */
/* scalar codecs                                                            */
/* ======================================================================= */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float orc_f16_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

uint16_t orc_f32_to_f16(float f) {
    _Float16 v = (_Float16)f; /* IEEE round-to-nearest-even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* quiet NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* crates/paddock-kernels/src/reference/mod.rs:28-38: 2^(e-127) * 0.5, with the
 * e < 2 branch built from raw denormal bit patterns. */
float orc_e8m0_half_to_f32(uint8_t e) {
    uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
    return u2f(bits);
}

/* crates/paddock-models/src/modelopt.rs:381-391 */
float orc_e2m1_to_f32(uint8_t code) {
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = mag[code & 7];
    return (code & 8) ? -m : m;
}

/* crates/paddock-models/src/modelopt.rs:393-406 (e4m3fn: bias 7, no inf,
 * 0x7f / 0xff = NaN) */
float orc_e4m3_to_f32(uint8_t b) {
    if ((b & 0x7f) == 0x7f) return NAN;
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int exp = (b >> 3) & 0xf;
    float mant = (float)(b & 7);
    if (exp == 0) return sign * (mant / 8.0f) * ldexpf(1.0f, -6);
    return sign * (1.0f + mant / 8.0f) * ldexpf(1.0f, exp - 7);
}

/* f32 -> e4m3fn, round-to-nearest-even, saturate to +-448: the conversion the
 * reference's quantizers get from the __nv_fp8_e4m3(float) constructor
 * (packs/cuda/src/gemm/dense_f8_decode.cuh:3154, quant/e2m1.cuh:36). */
uint8_t orc_f32_to_e4m3(float f) {
    uint32_t u = f2u(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    float a = fabsf(f);
    if (a != a) return (uint8_t)(sign | 0x7f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (a < 0.015625f) { /* below 2^-6: subnormal grid, step 2^-9 */
        int q = (int)nearbyintf(a * 512.0f);
        return (uint8_t)(sign | q); /* q == 8 is the first normal, 0x08 */
    }
    int e;
    float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) */
    int q = (int)nearbyintf(m * 16.0f); /* 8..16 */
    e -= 1;                             /* a = (q/8) * 2^e */
    if (q == 16) { q = 8; e += 1; }
    int code = ((e + 7) << 3) | (q - 8);
    if (code > 0x7e) code = 0x7e;
    return (uint8_t)(sign | code);
}

/* packs/cuda/src/quant/e2m1.cuh:12-26: RN-even onto {0,.5,1,1.5,2,3,4,6} */
uint8_t orc_e2m1_rn(float v) {
    uint8_t s = v < 0.0f ? 8 : 0;
    float a = fabsf(v);
    uint8_t m;
    if (a <= 0.25f) m = 0;
    else if (a < 0.75f) m = 1;
    else if (a <= 1.25f) m = 2;
    else if (a < 1.75f) m = 3;
    else if (a <= 2.5f) m = 4;
    else if (a < 3.5f) m = 5;
    else if (a <= 5.0f) m = 6;
    else m = 7;
    return s | m;
}

/* ======================================================================= */
/* dequantizers                                                             */
/* ======================================================================= */

/* crates/paddock-kernels/src/reference/mod.rs:22-24,56-83: doubled FP4 table,
 * halved E8M0 scale; low nibble of qs[j] = element j, high nibble = j+16. */
int orc_dequant_mxfp4(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    static const float fp4[16] = {0.0f, 1.0f, 2.0f, 3.0f, 4.0f, 6.0f, 8.0f, 12.0f,
                                  0.0f, -1.0f, -2.0f, -3.0f, -4.0f, -6.0f, -8.0f, -12.0f};
    if (n_bytes % 17) return -1;
    size_t blocks = n_bytes / 17;
    if (n_out != blocks * 32) return -2;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < blocks; ++i) {
        const uint8_t* b = data + i * 17;
        float d = orc_e8m0_half_to_f32(b[0]);
        float* y = out + i * 32;
        for (int j = 0; j < 16; ++j) {
            y[j] = fp4[b[1 + j] & 0x0f] * d;
            y[j + 16] = fp4[b[1 + j] >> 4] * d;
        }
    }
    return 0;
}

/* crates/paddock-kernels/src/reference/mod.rs:88-115: f16 scale + 32 int8 */
int orc_dequant_q8_0(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 34) return -1;
    size_t blocks = n_bytes / 34;
    if (n_out != blocks * 32) return -2;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < blocks; ++i) {
        const uint8_t* b = data + i * 34;
        float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float* y = out + i * 32;
        for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)b[2 + j] * d;
    }
    return 0;
}

/* crates/paddock-engine/tests/gpu_kquant_parity.rs:27-36 and
 * packs/cuda/src/quant/kquant.cuh:121-132 (get_scale_min_k4) */
void orc_scale_min_k4(const uint8_t* s, int j, uint32_t* sc, uint32_t* m) {
    if (j < 4) {
        *sc = s[j] & 63u;
        *m = s[j + 4] & 63u;
    } else {
        *sc = (uint32_t)(s[j + 4] & 0xF) | ((uint32_t)(s[j - 4] >> 6) << 4);
        *m = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

/* crates/paddock-engine/tests/gpu_kquant_parity.rs:39-69 (Q4_K arm): per
 * sub-block j of 32: y = (d*sc_j)*q - (dmin*m_j), separate f32 multiply and
 * subtract (no fused multiply-add). */
int orc_dequant_q4_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 144) return -1;
    size_t n_super = n_bytes / 144;
    if (n_out != n_super * 256) return -2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_super; ++b) {
        const uint8_t* s = data + b * 144;
        float d = orc_f16_to_f32((uint16_t)(s[0] | (s[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(s[2] | (s[3] << 8)));
        const uint8_t* scales = s + 4;
        const uint8_t* qs = s + 16;
        for (int j = 0; j < 8; ++j) {
            uint32_t sc, m;
            orc_scale_min_k4(scales, j, &sc, &m);
            float dj = d * (float)sc;
            float mj = dmin * (float)m;
            const uint8_t* qg = qs + (j >> 1) * 32;
            for (int l = 0; l < 32; ++l) {
                uint32_t v = (j & 1) ? (uint32_t)(qg[l] >> 4) : (uint32_t)(qg[l] & 0xF);
                float p = dj * (float)v;
                out[b * 256 + j * 32 + l] = p - mj;
            }
        }
    }
    return 0;
}

/* crates/paddock-engine/tests/gpu_kquant_parity.rs:39-69 (Q5_K arm): the Q4_K walk with a
 * fifth bit per weight; source order is d, dmin, scales[12], qh[32], qs[128] (176 bytes). */
int orc_dequant_q5_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 176) return -1;
    size_t n_super = n_bytes / 176;
    if (n_out != n_super * 256) return -2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_super; ++b) {
        const uint8_t* s = data + b * 176;
        float d = orc_f16_to_f32((uint16_t)(s[0] | (s[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(s[2] | (s[3] << 8)));
        const uint8_t* scales = s + 4;
        const uint8_t* qh = s + 16;
        const uint8_t* qs = s + 48;
        for (int j = 0; j < 8; ++j) {
            uint32_t sc, m;
            orc_scale_min_k4(scales, j, &sc, &m);
            float dj = d * (float)sc;
            float mj = dmin * (float)m;
            const uint8_t* qg = qs + (j >> 1) * 32;
            for (int l = 0; l < 32; ++l) {
                uint32_t v = (j & 1) ? (uint32_t)(qg[l] >> 4) : (uint32_t)(qg[l] & 0xF);
                if ((qh[l] >> j) & 1) v += 16;
                float p = dj * (float)v;
                out[b * 256 + j * 32 + l] = p - mj;
            }
        }
    }
    return 0;
}

/* gpu_kquant_parity.rs:70-94 (Q6_K arm): ql[128], qh[64], i8 scales[16], f16 d (210 bytes);
 * y = (d * scale) * q with q in [-32, 31], two separate f32 multiplies. */
int orc_dequant_q6_k(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 210) return -1;
    size_t n_super = n_bytes / 210;
    if (n_out != n_super * 256) return -2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_super; ++b) {
        const uint8_t* s = data + b * 210;
        const uint8_t *ql = s, *qh = s + 128;
        const int8_t* sc = (const int8_t*)(s + 192);
        float d = orc_f16_to_f32((uint16_t)(s[208] | (s[209] << 8)));
        for (int nh = 0; nh < 2; ++nh)
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                uint8_t qlo = ql[nh * 64 + l], qlh = ql[nh * 64 + 32 + l], h = qh[nh * 32 + l];
                int q[4] = {((qlo & 0xF) | ((h & 3) << 4)) - 32, ((qlh & 0xF) | (((h >> 2) & 3) << 4)) - 32,
                            ((qlo >> 4) | (((h >> 4) & 3) << 4)) - 32, ((qlh >> 4) | (((h >> 6) & 3) << 4)) - 32};
                for (int r = 0; r < 4; ++r) {
                    float ds = d * (float)sc[nh * 8 + r * 2 + is];
                    out[b * 256 + nh * 128 + r * 32 + l] = ds * (float)q[r];
                }
            }
    }
    return 0;
}

/* gpu_kquant_parity.rs:117-128 (Q4_0 arm): 32-weight blocks { f16 d, 16 nibble bytes };
 * byte k holds weight k (low) and k + 16 (high); value = d * (q - 8). */
int orc_dequant_q4_0(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 18) return -1;
    size_t n_blk = n_bytes / 18;
    if (n_out != n_blk * 32) return -2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_blk; ++b) {
        const uint8_t* s = data + b * 18;
        float d = orc_f16_to_f32((uint16_t)(s[0] | (s[1] << 8)));
        for (int k = 0; k < 16; ++k) {
            out[b * 32 + k] = d * (float)((int)(s[2 + k] & 0xF) - 8);
            out[b * 32 + 16 + k] = d * (float)((int)(s[2 + k] >> 4) - 8);
        }
    }
    return 0;
}

/* gpu_kquant_parity.rs:19-21, 96-115 (IQ4_XS arm): super-block of 136 bytes { f16 d, u16 scales_h,
 * u8 scales_l[4], u8 qs[128] }.  Sub-block ib of 32 weights: ls = 4 bits of scales_l | 2 bits of
 * scales_h << 4, dl = d * (ls - 32); byte j of the sub-block holds weight j (low nibble) and 16 + j
 * (high), each an index into ggml's 16-entry non-linear code book; value = dl * book[index]. */
static const int8_t orc_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
int orc_dequant_iq4_xs(const uint8_t* data, size_t n_bytes, float* out, size_t n_out) {
    if (n_bytes % 136) return -1;
    size_t n_super = n_bytes / 136;
    if (n_out != n_super * 256) return -2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_super; ++b) {
        const uint8_t* s = data + b * 136;
        float d = orc_f16_to_f32((uint16_t)(s[0] | (s[1] << 8)));
        unsigned sh = (unsigned)(s[2] | (s[3] << 8));
        const uint8_t *sl = s + 4, *qs = s + 8;
        for (int ib = 0; ib < 8; ++ib) {
            int ls = (int)(((sl[ib >> 1] >> (4 * (ib & 1))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
            float dl = d * (float)ls;
            for (int j = 0; j < 16; ++j) {
                out[b * 256 + ib * 32 + j] = dl * (float)orc_iq4nl[qs[ib * 16 + j] & 0xF];
                out[b * 256 + ib * 32 + 16 + j] = dl * (float)orc_iq4nl[qs[ib * 16 + j] >> 4];
            }
        }
    }
    return 0;
}

/* crates/paddock-models/src/modelopt.rs:408-424: op order (e2m1*e4m3)*scale2;
 * byte j holds elements 2j (low nibble) and 2j+1 (high nibble). */
void orc_dequant_nvfp4(const uint8_t* data, const uint8_t* scale, float scale2, float* out,
                       uint32_t in_dim, uint32_t out_dim) {
    size_t kh = in_dim / 2, ks = in_dim / 16;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < out_dim; ++r) {
        const uint8_t* p = data + r * kh;
        const uint8_t* sr = scale + r * ks;
        float* y = out + r * (size_t)in_dim;
        for (size_t j = 0; j < kh; ++j) {
            float s = orc_e4m3_to_f32(sr[(2 * j) / 16]);
            float a = orc_e2m1_to_f32(p[j] & 0x0f) * s;
            float b = orc_e2m1_to_f32(p[j] >> 4) * s;
            y[2 * j] = a * scale2;
            y[2 * j + 1] = b * scale2;
        }
    }
}

/* crates/paddock-models/src/modelopt.rs:343-352: e4m3 * row_scale */
void orc_dequant_fp8_channel(const uint8_t* w, const float* scale, float* out, uint32_t in_dim,
                             uint32_t out_dim) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < out_dim; ++r)
        for (size_t k = 0; k < in_dim; ++k)
            out[r * in_dim + k] = orc_e4m3_to_f32(w[r * in_dim + k]) * scale[r];
}

/* ======================================================================= */
/* quantizers for the synthetic inputs                                      */
/* ======================================================================= */

/* crates/paddock-engine/src/gpu_model/laguna/dflash.rs:233-253: d = amax/127
 * in f32, id = 1/d, q = round-half-away(v*id), d stored as f16. */
void orc_quantize_q8_0(const float* w, size_t n, uint8_t* out) {
    size_t blocks = n / 32;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < blocks; ++b) {
        const float* v = w + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        float d = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        uint16_t h = orc_f32_to_f16(d);
        uint8_t* o = out + b * 34;
        o[0] = (uint8_t)(h & 0xff);
        o[1] = (uint8_t)(h >> 8);
        for (int i = 0; i < 32; ++i) o[2 + i] = (uint8_t)(int8_t)roundf(v[i] * id);
    }
}

/* The reference tree holds no Q4_K quantizer (only dequant is pinned), so the
 * synthetic-input quantizer is this build's own: per sub-block of 32 a min/max
 * fit (scale = (max-min)/15, min clamped <= 0); per super-block d = max
 * scale/63 and dmin = max(-min)/63 rounded to f16; 6-bit sc/m; nibble =
 * clamp(RN((w + dmin*m)/(d*sc)), 0, 15).  Layout: ggml block_q4_K, 144 bytes
 * (f16 d, f16 dmin, 12 packed scale bytes, 128 nibble bytes). */
void orc_quantize_q4_k(const float* w, size_t n, uint8_t* out) {
    size_t n_super = n / 256;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < n_super; ++b) {
        const float* v = w + b * 256;
        float scale[8], mn[8];
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) {
            float lo = 0.0f, hi = -INFINITY;
            for (int l = 0; l < 32; ++l) {
                lo = fminf(lo, v[j * 32 + l]);
                hi = fmaxf(hi, v[j * 32 + l]);
            }
            if (hi < lo) hi = lo;
            scale[j] = (hi - lo) / 15.0f;
            mn[j] = 0.0f - lo;
            max_scale = fmaxf(max_scale, scale[j]);
            max_min = fmaxf(max_min, mn[j]);
        }
        uint16_t hd = orc_f32_to_f16(max_scale / 63.0f);
        uint16_t hm = orc_f32_to_f16(max_min / 63.0f);
        float d = orc_f16_to_f32(hd), dmin = orc_f16_to_f32(hm);
        uint32_t sc[8], m[8];
        for (int j = 0; j < 8; ++j) {
            int s = d > 0.0f ? (int)nearbyintf(scale[j] / d) : 0;
            int mm = dmin > 0.0f ? (int)nearbyintf(mn[j] / dmin) : 0;
            sc[j] = (uint32_t)(s < 0 ? 0 : (s > 63 ? 63 : s));
            m[j] = (uint32_t)(mm < 0 ? 0 : (mm > 63 ? 63 : mm));
        }
        uint8_t* o = out + b * 144;
        o[0] = (uint8_t)(hd & 0xff); o[1] = (uint8_t)(hd >> 8);
        o[2] = (uint8_t)(hm & 0xff); o[3] = (uint8_t)(hm >> 8);
        uint8_t* s12 = o + 4;
        for (int j = 0; j < 4; ++j) {
            s12[j] = (uint8_t)((sc[j] & 63u) | ((sc[j + 4] >> 4) << 6));
            s12[j + 4] = (uint8_t)((m[j] & 63u) | ((m[j + 4] >> 4) << 6));
            s12[j + 8] = (uint8_t)((sc[j + 4] & 0xFu) | ((m[j + 4] & 0xFu) << 4));
        }
        uint8_t* qs = o + 16;
        for (int g = 0; g < 4; ++g) {
            for (int l = 0; l < 32; ++l) {
                uint32_t nib[2];
                for (int h = 0; h < 2; ++h) {
                    int j = 2 * g + h;
                    float dj = d * (float)sc[j], mj = dmin * (float)m[j];
                    int q = dj > 0.0f ? (int)nearbyintf((v[j * 32 + l] + mj) / dj) : 0;
                    nib[h] = (uint32_t)(q < 0 ? 0 : (q > 15 ? 15 : q));
                }
                qs[g * 32 + l] = (uint8_t)(nib[0] | (nib[1] << 4));
            }
        }
    }
}

/* The FP8 benchmark recipe: per row s = absmax/448 (f32), q = e4m3_rn(w/s) */
void orc_quantize_fp8_absmax(const float* w, uint32_t rows, uint32_t k, uint8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const float* v = w + r * (size_t)k;
        float amax = 0.0f;
        for (uint32_t i = 0; i < k; ++i) amax = fmaxf(amax, fabsf(v[i]));
        float s = amax / 448.0f;
        scale[r] = s;
        for (uint32_t i = 0; i < k; ++i)
            q[r * (size_t)k + i] = s > 0.0f ? orc_f32_to_e4m3(v[i] / s) : 0;
    }
}

/* packs/cuda/src/gemm/dense_f8_decode.cuh:3210-3235 (quantize_e4m3_row): power
 * of two row scale 2^e with e = ex - 9 + (fr > 0.875), amax/2^e <= 448. */
void orc_quantize_e4m3_row_pow2(const float* x, uint32_t rows, uint32_t k, uint8_t* q,
                                float* scale) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const float* v = x + r * (size_t)k;
        float amax = 0.0f;
        for (uint32_t i = 0; i < k; ++i) amax = fmaxf(amax, fabsf(v[i]));
        int e = 0;
        if (amax > 0.0f) {
            int ex;
            float fr = frexpf(amax, &ex);
            e = ex - 9 + (fr > 0.875f ? 1 : 0);
        }
        scale[r] = ldexpf(1.0f, e);
        float inv = ldexpf(1.0f, -e);
        for (uint32_t i = 0; i < k; ++i) q[r * (size_t)k + i] = orc_f32_to_e4m3(v[i] * inv);
    }
}

/* packs/cuda/src/quant/e2m1.cuh:30-41 + quant/nvf4.cuh:381-403: per 16 block,
 * scale byte = RN_e4m3(amax/6) (min subnormal 1 when amax > 0), inv = 1/scale,
 * nibble = e2m1_rn(v*inv), packed adjacent (low nibble = even element). */
void orc_quantize_nvf4(const float* x, size_t n, uint8_t* q, uint8_t* scale) {
    orc_quantize_nvf4_global(x, n, 1.0f, q, scale);
}

/* Same with a per-tensor global scale (the checkpoint's and the NVFP4 benchmark's form):
 * block scale byte = RN_e4m3(amax/(6*scale2)), element = e2m1_rn(v/(e4m3*scale2)). */
void orc_quantize_nvf4_global(const float* x, size_t n, float scale2, uint8_t* q, uint8_t* scale) {
    size_t blocks = n / 16;
    float inv2 = scale2 == 1.0f ? 1.0f : 1.0f / scale2;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < blocks; ++b) {
        const float* v = x + b * 16;
        float amax = 0.0f;
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i] * inv2));
        uint8_t sb = 0;
        float inv = 0.0f;
        if (amax > 0.0f) {
            sb = orc_f32_to_e4m3(amax * (1.0f / 6.0f));
            if (sb == 0) sb = 1;
            inv = 1.0f / orc_e4m3_to_f32(sb);
        }
        scale[b] = sb;
        for (int i = 0; i < 8; ++i) {
            uint8_t lo = orc_e2m1_rn((v[2 * i] * inv2) * inv);
            uint8_t hi = orc_e2m1_rn((v[2 * i + 1] * inv2) * inv);
            q[b * 8 + i] = (uint8_t)(lo | (hi << 4));
        }
    }
}

/* packs/cuda/src/gemm/dense_fp4_w8.cuh:27-50: per 32 block the smallest power
 * of two with amax/2^e <= 6, byte e+127, nibble RN-even on the OCP grid,
 * split order (element j low nibble, j+16 high nibble), 17-byte blocks
 * (scale byte first) as ggml stores them. */
void orc_quantize_mxfp4(const float* w, size_t n, uint8_t* out) {
    size_t blocks = n / 32;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < blocks; ++b) {
        const float* v = w + b * 32;
        float a = 0.0f;
        for (int i = 0; i < 32; ++i) a = fmaxf(a, fabsf(v[i]));
        int e = 0;
        if (a > 0.0f) {
            int ex;
            float m = frexpf(a, &ex);
            e = ex - 3 + (m > 0.75f ? 1 : 0);
        }
        float inv = ldexpf(1.0f, -e);
        uint8_t* o = out + b * 17;
        o[0] = (uint8_t)(e + 127);
        for (int j = 0; j < 16; ++j)
            o[1 + j] = (uint8_t)(orc_e2m1_rn(v[j] * inv) | (orc_e2m1_rn(v[j + 16] * inv) << 4));
    }
}

/* packs/cuda/src/attn/decode.cuh:2981-3004 and 3041-3068: per 32 block
 * scale = amax*(1/127), q = clamp(rint(v/scale), +-127); per-16 integer sums
 * as f32 (sums16 may be NULL). */
void orc_quantize_q8_act(const float* x, size_t n, int8_t* q, float* scale, float* sums16) {
    size_t blocks = n / 32;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < blocks; ++b) {
        const float* v = x + b * 32;
        float a = 0.0f;
        for (int i = 0; i < 32; ++i) a = fmaxf(a, fabsf(v[i]));
        float scl = a * (1.0f / 127.0f);
        scale[b] = scl;
        float inv = scl > 0.0f ? 1.0f / scl : 0.0f;
        int s[2] = {0, 0};
        for (int i = 0; i < 32; ++i) {
            int qi = (int)nearbyintf(v[i] * inv);
            qi = qi < -127 ? -127 : (qi > 127 ? 127 : qi);
            q[b * 32 + i] = (int8_t)qi;
            s[i >> 4] += qi;
        }
        if (sums16) {
            sums16[b * 2] = (float)s[0];
            sums16[b * 2 + 1] = (float)s[1];
        }
    }
}

/* ======================================================================= */
/* repack restatements                                                      */
/* ======================================================================= */

/* packs/cuda/src/deltanet/core.cuh:2552-2565: 34-byte blocks -> int8 plane
 * [n_blocks*32] + f16 scale plane [n_blocks]. */
void orc_repack_q8_0(const uint8_t* src, uint64_t n_blocks, int8_t* data, uint16_t* scale) {
    for (uint64_t b = 0; b < n_blocks; ++b) {
        const uint8_t* s = src + b * 34;
        scale[b] = (uint16_t)(s[0] | (s[1] << 8));
        memcpy(data + b * 32, s + 2, 32);
    }
}

/* packs/cuda/src/attn/decode.cuh:2294-2304: 17-byte blocks -> 16-byte nibble
 * plane + 1-byte scale plane. */
void orc_repack_mxfp4(const uint8_t* src, uint64_t n_blocks, uint8_t* data, uint8_t* scale) {
    for (uint64_t b = 0; b < n_blocks; ++b) {
        scale[b] = src[b * 17];
        memcpy(data + b * 16, src + b * 17 + 1, 16);
    }
}

/* ======================================================================= */
/* linear algebra                                                           */
/* ======================================================================= */

/* crates/paddock-engine/src/reference/tensor.rs:39-54: out[o] = dot(row o, x),
 * scalar f32, ascending k.  Rows are independent, so they run across threads;
 * each row's arithmetic order is the reference's. */
void orc_matvec_f32(const float* w, const float* x, float* y, uint32_t in_dim, uint32_t out_dim) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; ++o) {
        const float* row = w + o * (size_t)in_dim;
        float acc = 0.0f;
        for (uint32_t k = 0; k < in_dim; ++k) {
            float p = row[k] * x[k];
            acc = acc + p;
        }
        y[o] = acc;
    }
}

/* f64-accumulated matmul of dequantized operands (the comparison target of the
 * reference's GPU parity tests, tests/gpu_kquant_parity.rs:369-383) plus the
 * condition number term sum_k |w x| (tests/gpu_nvfp4_oracle.rs:140-153). */
void orc_matmul_f64(const float* w, const float* x, float* y, float* abs_sum, uint32_t in_dim,
                    uint32_t out_dim, uint32_t batch) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; ++o) {
        const float* row = w + o * (size_t)in_dim;
        for (uint32_t c = 0; c < batch; ++c) {
            const float* xr = x + c * (size_t)in_dim;
            double acc = 0.0, ab = 0.0;
            for (uint32_t k = 0; k < in_dim; ++k) {
                double p = (double)row[k] * (double)xr[k];
                acc += p;
                ab += fabs(p);
            }
            y[c * (size_t)out_dim + o] = (float)acc;
            if (abs_sum) abs_sum[c * (size_t)out_dim + o] = (float)ab;
        }
    }
}

/* ======================================================================= */
/* MoE                                                                      */
/* ======================================================================= */

/* packs/cuda/src/attn/decode.cuh:1392-1445: k rounds of argmax over
 * logits+bias, strict > with ties to the lowest index; weights = softmax over
 * the k selected logits (max-subtracted, expf). */
void orc_moe_topk(const float* logits, const float* bias, uint32_t n_expert, uint32_t k,
                  uint32_t batch, uint32_t* out_idx, float* out_w) {
    for (uint32_t b = 0; b < batch; ++b) {
        float* v = (float*)malloc(sizeof(float) * n_expert);
        for (uint32_t i = 0; i < n_expert; ++i)
            v[i] = logits[(size_t)b * n_expert + i] + (bias ? bias[i] : 0.0f);
        float sel[64];
        for (uint32_t s = 0; s < k; ++s) {
            float best = -1e30f;
            uint32_t bi = 0;
            for (uint32_t i = 0; i < n_expert; ++i)
                if (v[i] > best) { best = v[i]; bi = i; }
            sel[s] = best;
            out_idx[(size_t)b * k + s] = bi;
            v[bi] = -1e30f;
        }
        float mm = sel[0];
        for (uint32_t s = 1; s < k; ++s) mm = fmaxf(mm, sel[s]);
        float sum = 0.0f;
        for (uint32_t s = 0; s < k; ++s) {
            float e = expf(sel[s] - mm);
            out_w[(size_t)b * k + s] = e;
            sum += e;
        }
        for (uint32_t s = 0; s < k; ++s) out_w[(size_t)b * k + s] /= sum;
        free(v);
    }
}

/* crates/paddock-kernels/src/reference/ops.rs:27-36 */
void orc_swiglu_oai(float* gate, const float* up, size_t n, float alpha, float limit) {
    for (size_t i = 0; i < n; ++i) {
        float x = fminf(gate[i], limit);
        float y = fminf(fmaxf(up[i], -limit), limit);
        gate[i] = (x / (1.0f + expf(-alpha * x))) * (y + 1.0f);
    }
}

/* MoE block as crates/paddock-engine/src/gpu_model/gpt_oss.rs:2279-2521 walks
 * it: per (token, slot) h = swiglu_oai(Wg x + bg, Wu x + bu); o = Wd h + bd;
 * out[token] = sum over slots in ascending slot order of w_slot * o.  Expert
 * planes are dequantized with orc_dequant_mxfp4; dot products accumulate in
 * f64. */
void orc_moe_mxfp4_layer(const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                         const float* gate_b, const float* up_b, const float* down_b,
                         const float* x, const uint32_t* topk_idx, const float* topk_w,
                         float* out, uint32_t tokens, uint32_t n_active, uint32_t embd,
                         uint32_t ff, float alpha, float limit) {
    size_t gu_bytes = (size_t)ff * (embd / 32) * 17;
    size_t dn_bytes = (size_t)embd * (ff / 32) * 17;
    float* wg = (float*)malloc(sizeof(float) * ff * embd);
    float* wu = (float*)malloc(sizeof(float) * ff * embd);
    float* wd = (float*)malloc(sizeof(float) * ff * embd);
    float* part = (float*)calloc((size_t)tokens * n_active * embd, sizeof(float));
    uint32_t max_e = 0;
    for (size_t i = 0; i < (size_t)tokens * n_active; ++i)
        if (topk_idx[i] > max_e) max_e = topk_idx[i];
    for (uint32_t e = 0; e <= max_e; ++e) {
        int used = 0;
        for (size_t i = 0; i < (size_t)tokens * n_active && !used; ++i) used = topk_idx[i] == e;
        if (!used) continue;
        orc_dequant_mxfp4(gate + e * gu_bytes, gu_bytes, wg, (size_t)ff * embd);
        orc_dequant_mxfp4(up + e * gu_bytes, gu_bytes, wu, (size_t)ff * embd);
        orc_dequant_mxfp4(down + e * dn_bytes, dn_bytes, wd, (size_t)ff * embd);
        for (uint32_t t = 0; t < tokens; ++t) {
            for (uint32_t s = 0; s < n_active; ++s) {
                if (topk_idx[(size_t)t * n_active + s] != e) continue;
                const float* xt = x + (size_t)t * embd;
                float* g = (float*)malloc(sizeof(float) * ff);
                float* u = (float*)malloc(sizeof(float) * ff);
#pragma omp parallel for schedule(static)
                for (size_t f = 0; f < ff; ++f) {
                    double ag = 0.0, au = 0.0;
                    for (uint32_t k = 0; k < embd; ++k) {
                        ag += (double)wg[f * embd + k] * xt[k];
                        au += (double)wu[f * embd + k] * xt[k];
                    }
                    g[f] = (float)ag + (gate_b ? gate_b[(size_t)e * ff + f] : 0.0f);
                    u[f] = (float)au + (up_b ? up_b[(size_t)e * ff + f] : 0.0f);
                }
                orc_swiglu_oai(g, u, ff, alpha, limit);
                float* o = part + ((size_t)t * n_active + s) * embd;
#pragma omp parallel for schedule(static)
                for (size_t r = 0; r < embd; ++r) {
                    double a = 0.0;
                    for (uint32_t k = 0; k < ff; ++k) a += (double)wd[r * ff + k] * g[k];
                    o[r] = (float)a + (down_b ? down_b[(size_t)e * embd + r] : 0.0f);
                }
                free(g);
                free(u);
            }
        }
    }
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t r = 0; r < embd; ++r) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < n_active; ++s)
                acc += topk_w[(size_t)t * n_active + s] * part[((size_t)t * n_active + s) * embd + r];
            out[(size_t)t * embd + r] = acc;
        }
    free(wg); free(wu); free(wd); free(part);
}

/* ======================================================================= */
/* synthetic data                                                           */
/* ======================================================================= */

static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* element pair p = (2p, 2p+1): two uniforms from splitmix64 of the counter,
 * Box-Muller in f64, rounded to f32.  Counter based, so any thread count gives
 * the same array. */
void orc_fill_normal(float* out, size_t n, uint64_t seed, float sigma) {
    size_t pairs = (n + 1) / 2;
#pragma omp parallel for schedule(static)
    for (size_t p = 0; p < pairs; ++p) {
        uint64_t a = splitmix64(seed * 0xD1342543DE82EF95ull + 2 * p);
        uint64_t b = splitmix64(seed * 0xD1342543DE82EF95ull + 2 * p + 1);
        double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0);
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
        double r = sqrt(-2.0 * log(u1));
        double th = 6.283185307179586476925 * u2;
        out[2 * p] = (float)(r * cos(th) * (double)sigma);
        if (2 * p + 1 < n) out[2 * p + 1] = (float)(r * sin(th) * (double)sigma);
    }
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads the following calls may use (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
