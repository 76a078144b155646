// f8_producers.cu - what runs in front of the row-scaled e4m3 GEMM: the activation row quantizer
// and its fused forms (RMSNorm, residual add + RMSNorm, SwiGLU), each one pass over the row.
//
// One CTA per row; thread t holds the row's float4 number t, t + T, t + 2T, ... in registers from
// the first load to the last store, so every access of a warp is one contiguous 512-byte run and
// the row leaves DRAM once.  The quantizer is that of slot 183: amax = fr * 2^ex, e = ex - 9 +
// (fr > 0.875), scale = 2^e (so that amax / scale <= 448), q = RN_e4m3(v / scale), saturating.
#include <cuda_fp8.h>

#include "pdk_common.cuh"

namespace {

constexpr uint32_t kRowMaxThreads = 1024;

enum RowMode : int {
    kQuantOnly = 0,     // q, scale = quantize(x)
    kNormQuant = 1,     // xn = rmsnorm(x) * w; q, scale = quantize(xn)
    kAddNormQuant = 2,  // x += pscale * proj (written back); then as kNormQuant
    kSwigluQuant = 3    // h = silu(gate) * up; q, scale = quantize(h)
};

__device__ __forceinline__ uint32_t e4m3x4(const float4& v, float inv) {
    return (uint32_t)__nv_cvt_float_to_fp8(v.x * inv, __NV_SATFINITE, __NV_E4M3) |
           (uint32_t)__nv_cvt_float_to_fp8(v.y * inv, __NV_SATFINITE, __NV_E4M3) << 8 |
           (uint32_t)__nv_cvt_float_to_fp8(v.z * inv, __NV_SATFINITE, __NV_E4M3) << 16 |
           (uint32_t)__nv_cvt_float_to_fp8(v.w * inv, __NV_SATFINITE, __NV_E4M3) << 24;
}
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// a: x (modes 0-2) or gate (mode 3); b: proj (mode 2) or up (mode 3); w, xn: modes 1-2
template <int kChunks, int kMode>
__global__ void __launch_bounds__(kRowMaxThreads)
f8_row_producer_kernel(float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ w,
                       float* __restrict__ xn, uint8_t* __restrict__ q, float* __restrict__ rscale, uint32_t n, float eps,
                       float pscale) {
    __shared__ double warp_sq[32];
    __shared__ float warp_max[32];
    const uint32_t t = threadIdx.x, width = blockDim.x, n4 = n >> 2, lane = t & 31u, warp = t >> 5;
    const size_t row4 = (size_t)blockIdx.x * n4;
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();

    float4 held[kChunks];
    double sq = 0.0;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const uint32_t at = (uint32_t)c * width + t;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (at < n4) {
            v = (reinterpret_cast<const float4*>(a) + row4)[at];
            if (kMode == kAddNormQuant) {
                const float4 p = (reinterpret_cast<const float4*>(b) + row4)[at];
                v.x = fmaf(pscale, p.x, v.x); v.y = fmaf(pscale, p.y, v.y);
                v.z = fmaf(pscale, p.z, v.z); v.w = fmaf(pscale, p.w, v.w);
                (reinterpret_cast<float4*>(a) + row4)[at] = v;
            }
            if (kMode == kSwigluQuant) {
                const float4 u = (reinterpret_cast<const float4*>(b) + row4)[at];
                v = make_float4(silu_mul(v.x, u.x), silu_mul(v.y, u.y), silu_mul(v.z, u.z), silu_mul(v.w, u.w));
            }
        }
        held[c] = v;
        if (kMode == kNormQuant || kMode == kAddNormQuant)
            sq += (double)(v.x * v.x) + (double)(v.y * v.y) + (double)(v.z * v.z) + (double)(v.w * v.w);
    }
    if (kMode == kNormQuant || kMode == kAddNormQuant) {
        // mean square: f32 products, f64 sums (per thread, per warp, then over the warps in warp order)
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
        if (lane == 0u) warp_sq[warp] = sq;
        __syncthreads();
        double total = 0.0;
        for (uint32_t i = 0; i < (width >> 5); ++i) total += warp_sq[i];
        const float norm = 1.0f / sqrtf((float)(total / (double)n) + eps);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const uint32_t at = (uint32_t)c * width + t;
            if (at < n4) {
                const float4 g = reinterpret_cast<const float4*>(w)[at];
                const float4 v = held[c];
                const float4 r = make_float4(v.x * norm * g.x, v.y * norm * g.y, v.z * norm * g.z, v.w * norm * g.w);
                (reinterpret_cast<float4*>(xn) + row4)[at] = r;
                held[c] = r;
            }
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c)
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(held[c].x), fabsf(held[c].y)), fmaxf(fabsf(held[c].z), fabsf(held[c].w))));
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if (lane == 0u) warp_max[warp] = amax;
    __syncthreads();
    float m = 0.0f;
    for (uint32_t i = 0; i < (width >> 5); ++i) m = fmaxf(m, warp_max[i]);
    int e = 0;
    if (m > 0.0f) {
        int ex;
        const float fr = frexpf(m, &ex);
        e = ex - 9 + (fr > 0.875f ? 1 : 0);
    }
    if (t == 0u) rscale[blockIdx.x] = ldexpf(1.0f, e);
    const float inv = ldexpf(1.0f, -e);
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q + (size_t)blockIdx.x * n);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const uint32_t at = (uint32_t)c * width + t;
        if (at < n4) qrow[at] = e4m3x4(held[c], inv);
    }
}

template <int kMode>
int launch_rows(float* a, const float* b, const float* w, float* xn, uint8_t* q, float* rscale, uint32_t n, float eps,
                float pscale, uint32_t batch, cudaStream_t st) {
    const uint32_t n4 = n >> 2;
    uint32_t chunks = 1;
    while (chunks < 16u && (n4 + chunks - 1u) / chunks > kRowMaxThreads) chunks <<= 1;
    const uint32_t width = ((n4 + chunks - 1u) / chunks + 31u) & ~31u;
    if (width > kRowMaxThreads) return -1;   // rows beyond 65536 elements
#define PDK_ROW_CASE(C)                                                                                              \
    case C:                                                                                                          \
        return pdk_launch_pdl(f8_row_producer_kernel<C, kMode>, dim3(batch), dim3(width), 0, st, a, b, w, xn, q, rscale, n, \
                              eps, pscale)
    switch (chunks) {
        PDK_ROW_CASE(1);
        PDK_ROW_CASE(2);
        PDK_ROW_CASE(4);
        PDK_ROW_CASE(8);
        PDK_ROW_CASE(16);
    }
#undef PDK_ROW_CASE
    return -1;
}

bool rows_ok(uint32_t n, const void* p0, const void* p1, const void* p2, const void* p3, const void* q, const void* rs) {
    return (n & 3u) == 0u && pdk_aligned(p0, 16) && pdk_aligned(p1, 16) && pdk_aligned(p2, 16) && pdk_aligned(p3, 16) &&
           pdk_aligned(q, 4) && pdk_aligned(rs, 4) && (((size_t)n) & 3u) == 0u;
}

}  // namespace

// The single-pass form of slot 183 for rows of whole float4 (the launcher in fp8_quant.cu falls back
// to its two-pass kernel otherwise); -1 = not this route.
int pdk_quantize_e4m3_row_1p(const float* x, uint8_t* q, float* rscale, uint32_t n, uint32_t batch, cudaStream_t st) {
    if (!rows_ok(n, x, nullptr, nullptr, nullptr, q, rscale)) return -1;
    return launch_rows<kQuantOnly>(const_cast<float*>(x), nullptr, nullptr, nullptr, q, rscale, n, 0.0f, 0.0f, batch, st);
}

// slot 511, packs/cuda/src/exports.cuh:380-500: h = silu(gate) * up in f32 (g / (1 + expf(-g)) * u),
// q e4m3 [batch][n] + one power-of-two f32 scale per row.
PDK_EXPORT int pd_swiglu_quant_e4m3_row(const void* gate, const void* up, void* q, void* rscale, uint32_t n, uint32_t batch,
                                        void* stream) {
    if (n == 0 || batch == 0) return 0;
    if ((n & 31u) != 0u || !rows_ok(n, gate, up, nullptr, nullptr, q, rscale)) return cudaErrorInvalidValue;
    const int rc = launch_rows<kSwigluQuant>((float*)const_cast<void*>(gate), (const float*)up, nullptr, nullptr, (uint8_t*)q,
                                             (float*)rscale, n, 0.0f, 0.0f, batch, (cudaStream_t)stream);
    return rc == -1 ? (int)cudaErrorNotSupported : rc;
}

// slot 512, packs/cuda/src/gemm/dense_f8_decode.cuh:4357-4555: xn = x * (1 / sqrtf(mean(x^2) + eps)) * w
// (multiplied in that order), then the row quantizer on xn.  The reference declines (status 100)
// from 64 rows on and beyond 16384 elements; this kernel takes every batch and rows up to 65536.
PDK_EXPORT int pd_rmsnorm_quant_e4m3_row(const void* x, const void* w, void* xn, void* q, void* rscale, uint32_t n, float eps,
                                         uint32_t batch, void* stream) {
    if (n == 0 || batch == 0) return 0;
    if ((n & 31u) != 0u || !rows_ok(n, x, w, xn, nullptr, q, rscale)) return cudaErrorInvalidValue;
    const int rc = launch_rows<kNormQuant>((float*)const_cast<void*>(x), nullptr, (const float*)w, (float*)xn, (uint8_t*)q,
                                           (float*)rscale, n, eps, 0.0f, batch, (cudaStream_t)stream);
    return rc == -1 ? 100 : rc;
}

// slot 513, packs/cuda/src/gemm/dense_f8_decode.cuh:4448-4575: x += pscale * proj (one fused
// multiply-add per element, written back), then as slot 512.
PDK_EXPORT int pd_add_rmsnorm_scaled_quant_e4m3_row(void* x, const void* proj, const void* w, void* xn, void* q, void* rscale,
                                                    uint32_t n, float eps, float pscale, uint32_t batch, void* stream) {
    if (n == 0 || batch == 0) return 0;
    if ((n & 31u) != 0u || proj == nullptr || !rows_ok(n, x, proj, w, xn, q, rscale)) return cudaErrorInvalidValue;
    const int rc = launch_rows<kAddNormQuant>((float*)x, (const float*)proj, (const float*)w, (float*)xn, (uint8_t*)q,
                                              (float*)rscale, n, eps, pscale, batch, (cudaStream_t)stream);
    return rc == -1 ? 100 : rc;
}
