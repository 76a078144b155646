// kquant.cu - Q4_K: dequant, repack and the exact-f32 decode GEMV / small-batch
// GEMM over the repacked planes.
//
// Repacked layout (the byte budget the engine allocates: 128 B + 24 B per
// 256-weight super-block):
//   data   : the 128 nibble bytes verbatim - group g (32 bytes) byte l holds
//            element g*64 + l in its low nibble and g*64 + 32 + l in its high;
//   scales : 24-byte record {f16 d, f16 dmin, u8 sc[8], u8 m[8], 4 pad bytes}
//            with the 6-bit (scale, min) pairs unpacked to bytes.
// Dequant value of element l of sub-block j: (d*sc_j)*q - (dmin*m_j).
#include "pdk_common.cuh"

namespace {

// ggml get_scale_min_k4: unpack 6-bit pair j of the 12 packed scale bytes.
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, uint32_t j, uint32_t* sc, uint32_t* m) {
    if (j < 4u) {
        *sc = s[j] & 63u;
        *m = s[j + 4u] & 63u;
    } else {
        *sc = (s[j + 4u] & 0xFu) | ((uint32_t)(s[j - 4u] >> 6) << 4);
        *m = (uint32_t)(s[j + 4u] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

// One warp per super-block; lane l writes element l of each of the 8
// sub-blocks, so every store instruction covers one 128-byte line.
__global__ void q4k_dequant_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, uint64_t n_super) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint8_t* s = src + b * 144u;
    const float d = __half2float(*reinterpret_cast<const __half*>(s));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(s + 2));
    float* y = dst + b * 256u;
#pragma unroll
    for (uint32_t j = 0; j < 8u; ++j) {
        uint32_t sc, m;
        scale_min_k4(s + 4, j, &sc, &m);
        const float dj = __fmul_rn(d, (float)sc), mj = __fmul_rn(dmin, (float)m);
        const uint32_t q = s[16u + (j >> 1) * 32u + lane];
        const uint32_t v = (j & 1u) ? (q >> 4) : (q & 0xFu);
        y[j * 32u + lane] = __fsub_rn(__fmul_rn(dj, (float)v), mj);
    }
}

// One warp per super-block: lanes copy the 128 nibble bytes as 32 words (the
// source payload at 144*b + 16 is 4-byte aligned when the plane is); lane 0..7
// unpack one (sc, m) pair each into the 24-byte record.
__global__ void q4k_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst_data,
                                  uint8_t* __restrict__ dst_scales, uint64_t n_super) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint8_t* s = src + b * 144u;
    reinterpret_cast<uint32_t*>(dst_data + b * 128u)[lane] = reinterpret_cast<const uint32_t*>(s + 16)[lane];
    uint8_t* rec = dst_scales + b * 24u;
    if (lane < 8u) {
        uint32_t sc, m;
        scale_min_k4(s + 4, lane, &sc, &m);
        rec[4u + lane] = (uint8_t)sc;
        rec[12u + lane] = (uint8_t)m;
    } else if (lane < 12u) {
        rec[lane - 8u] = s[lane - 8u];  // f16 d, f16 dmin
    } else if (lane < 16u) {
        rec[8u + lane] = 0;             // pad bytes 20..23
    }
}

constexpr uint32_t kWarps = 8;

// Exact-f32 GEMV / small-batch GEMM.  A warp owns one output row at a time and
// reads each super-block's 128 nibble bytes as one coalesced 128-byte line:
// lane l = (group g = l/8, word w = l%8) holds four low nibbles (sub-block 2g,
// elements 4w..4w+3) and four high nibbles (sub-block 2g+1).  Per sub-block
// the partial is (d*sc)*sum(q*x) - (dmin*m)*sum(x), all f32.
template <uint32_t TOK, uint32_t UNROLL>
__global__ void __launch_bounds__(kWarps * 32)
q4k_gemv_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim, uint32_t out_dim,
                uint32_t batch0) {
    extern __shared__ __align__(16) float xs[];  // [TOK][in_dim]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float* xg = x + (size_t)batch0 * in_dim;
    for (uint32_t i = tid * 4u; i < TOK * in_dim; i += blockDim.x * 4u)
        *reinterpret_cast<float4*>(xs + i) = *reinterpret_cast<const float4*>(xg + i);
    __syncthreads();

    const uint32_t n_super = in_dim >> 8;
    const uint32_t g = lane >> 3, w = lane & 7u;
    const uint32_t koff = g * 64u + w * 4u;  // first low-nibble element inside the super-block
    for (uint32_t row = blockIdx.x * kWarps + warp; row < out_dim; row += gridDim.x * kWarps) {
        const uint8_t* drow = data + (size_t)row * n_super * 128u;
        const uint8_t* srow = scales + (size_t)row * n_super * 24u;
        float acc[TOK];
#pragma unroll
        for (uint32_t t = 0; t < TOK; ++t) acc[t] = 0.0f;
        for (uint32_t sb0 = 0; sb0 < n_super; sb0 += UNROLL) {
            uint32_t q[UNROLL];
            uint32_t dd[UNROLL];
            uint32_t scm[UNROLL];
#pragma unroll
            for (uint32_t u = 0; u < UNROLL; ++u) {
                const uint32_t sb = sb0 + u;
                if (sb < n_super) {
                    q[u] = pdk_ldg_stream4(drow + sb * 128u + lane * 4u);
                    const uint8_t* rec = srow + sb * 24u;
                    dd[u] = *reinterpret_cast<const uint32_t*>(rec);
                    const uint32_t s2 = *reinterpret_cast<const uint16_t*>(rec + 4u + 2u * g);
                    const uint32_t m2 = *reinterpret_cast<const uint16_t*>(rec + 12u + 2u * g);
                    scm[u] = s2 | (m2 << 16);
                } else {
                    q[u] = 0u; dd[u] = 0u; scm[u] = 0u;
                }
            }
#pragma unroll
            for (uint32_t u = 0; u < UNROLL; ++u) {
                const uint32_t sb = sb0 + u;
                if (sb >= n_super) break;
                const __half2 dh = *reinterpret_cast<const __half2*>(&dd[u]);
                const float d = __low2float(dh), dmin = __high2float(dh);
                const float d_lo = d * (float)(scm[u] & 0xffu), d_hi = d * (float)((scm[u] >> 8) & 0xffu);
                const float m_lo = dmin * (float)((scm[u] >> 16) & 0xffu), m_hi = dmin * (float)(scm[u] >> 24);
                const uint32_t k = sb * 256u + koff;
#pragma unroll
                for (uint32_t t = 0; t < TOK; ++t) {
                    const float4 xl = *reinterpret_cast<const float4*>(xs + t * in_dim + k);
                    const float4 xh = *reinterpret_cast<const float4*>(xs + t * in_dim + k + 32u);
                    float sl = (float)(q[u] & 0xFu) * xl.x;
                    sl = fmaf((float)((q[u] >> 8) & 0xFu), xl.y, sl);
                    sl = fmaf((float)((q[u] >> 16) & 0xFu), xl.z, sl);
                    sl = fmaf((float)((q[u] >> 24) & 0xFu), xl.w, sl);
                    float sh = (float)((q[u] >> 4) & 0xFu) * xh.x;
                    sh = fmaf((float)((q[u] >> 12) & 0xFu), xh.y, sh);
                    sh = fmaf((float)((q[u] >> 20) & 0xFu), xh.z, sh);
                    sh = fmaf((float)(q[u] >> 28), xh.w, sh);
                    const float xsl = (xl.x + xl.y) + (xl.z + xl.w);
                    const float xsh = (xh.x + xh.y) + (xh.z + xh.w);
                    acc[t] += (d_lo * sl - m_lo * xsl) + (d_hi * sh - m_hi * xsh);
                }
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < TOK; ++t) {
            const float v = pdk_warp_sum(acc[t]);
            if (lane == 0) y[(size_t)(batch0 + t) * out_dim + row] = v;
        }
    }
}

template <uint32_t TOK>
int launch(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
           uint32_t batch0, cudaStream_t st) {
    const size_t smem = (size_t)TOK * in_dim * sizeof(float);
    auto kern = q4k_gemv_kernel<TOK, 10>;
    if (smem > 48u * 1024u) {
        if (smem > 200u * 1024u) return cudaErrorNotSupported;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)(kWarps * 32u), smem) != cudaSuccess ||
        per_sm < 1)
        per_sm = 1;
    uint32_t grid = (uint32_t)pdk_sm_count() * (uint32_t)per_sm;
    const uint32_t need = (out_dim + kWarps - 1u) / kWarps;
    if (grid > need) grid = need;
    kern<<<grid, kWarps * 32u, smem, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim, out_dim, batch0);
    return pdk_launch_status();
}

int check_gemv(const void* data, const void* scales, const void* x, const void* y, uint32_t in_dim, uint32_t dtype) {
    if (dtype != PDK_KQ_Q4K) {
        if (dtype == PDK_KQ_Q5K || dtype == PDK_KQ_Q6K || dtype == PDK_KQ_IQ4XS || dtype == PDK_KQ_Q4_0)
            return cudaErrorNotSupported;
        return cudaErrorInvalidValue;
    }
    if (in_dim == 0u || (in_dim & 255u) != 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(scales, 8) || !pdk_aligned(x, 16) || !pdk_aligned(y, 4))
        return cudaErrorInvalidValue;
    return 0;
}

}  // namespace

PDK_EXPORT int pd_kquant_dequant(const void* src, void* dst, uint64_t n_super, uint32_t dtype, void* stream) {
    if (n_super == 0) return 0;
    if (dtype != PDK_KQ_Q4K)
        return (dtype == PDK_KQ_Q5K || dtype == PDK_KQ_Q6K || dtype == PDK_KQ_IQ4XS || dtype == PDK_KQ_Q4_0)
                   ? cudaErrorNotSupported : cudaErrorInvalidValue;
    if (!pdk_aligned(src, 2) || !pdk_aligned(dst, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    q4k_dequant_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (float*)dst, n_super);
    return pdk_launch_status();
}

PDK_EXPORT int pd_kquant_repack(const void* src, void* dst_data, void* dst_scales, uint64_t n_super, uint32_t dtype,
                                void* stream) {
    if (n_super == 0) return 0;
    if (dtype != PDK_KQ_Q4K)
        return (dtype == PDK_KQ_Q5K || dtype == PDK_KQ_Q6K || dtype == PDK_KQ_IQ4XS || dtype == PDK_KQ_Q4_0)
                   ? cudaErrorNotSupported : cudaErrorInvalidValue;
    if (!pdk_aligned(src, 4) || !pdk_aligned(dst_data, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    q4k_repack_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst_data, (uint8_t*)dst_scales, n_super);
    return pdk_launch_status();
}

PDK_EXPORT int pd_kquant_gemv(const void* data, const void* scales, const void* x, void* y, uint32_t in_dim,
                              uint32_t out_dim, uint32_t dtype, void* stream) {
    if (out_dim == 0) return 0;
    if (int rc = check_gemv(data, scales, x, y, in_dim, dtype)) return rc;
    return launch<1>(data, scales, (const float*)x, (float*)y, in_dim, out_dim, 0u, (cudaStream_t)stream);
}

PDK_EXPORT int pdk_kquant_gemm_f32(const void* data, const void* scales, const void* x, void* y, uint32_t in_dim,
                                   uint32_t out_dim, uint32_t batch, uint32_t dtype, void* stream) {
    if (out_dim == 0 || batch == 0) return 0;
    if (batch > 64u) return cudaErrorInvalidValue;
    if (int rc = check_gemv(data, scales, x, y, in_dim, dtype)) return rc;
    const float* xf = (const float*)x;
    float* yf = (float*)y;
    auto st = (cudaStream_t)stream;
    uint32_t b = 0;
    for (; b + 4u <= batch; b += 4u)
        if (int rc = launch<4>(data, scales, xf, yf, in_dim, out_dim, b, st)) return rc;
    for (; b + 2u <= batch; b += 2u)
        if (int rc = launch<2>(data, scales, xf, yf, in_dim, out_dim, b, st)) return rc;
    for (; b < batch; ++b)
        if (int rc = launch<1>(data, scales, xf, yf, in_dim, out_dim, b, st)) return rc;
    return 0;
}
