// q8_0.cu - Q8_0 launchers and the plain-load f32 GEMV / small-batch GEMM over the repacked planes
// (int8 data [out][in] + f16 scale [out][in/32]).
//
// HBM-bound: 8.5 bits per weight are streamed once.  A warp owns one output
// row at a time; every lane issues all of its 16-byte weight loads for the
// row before the first use, so a resident CTA keeps (in_dim) bytes per warp
// in flight.  Activations sit in shared memory as f32; the 16-term inner
// products and the scale application are exact f32 (reduction order differs
// from a scalar walk, nothing else).
#include <cstdlib>

#include "pdk_common.cuh"

int pdk_q8_0_gemm_i8(const void* data, const void* scale, const float* bias, const float* x, float* y, uint32_t in_dim,
                     uint32_t out_dim, uint32_t batch, cudaStream_t st);
int pdk_q8_0_gemv_i8(const void* data, const void* scale, const float* bias, const float* x, float* y,
                     uint32_t in_dim, uint32_t out_dim, cudaStream_t st);

namespace {

// PDK_Q8_PLAIN=1 forces the plain-load f32 kernel (A/B switch, read once).
bool force_plain() {
    static const bool v = [] {
        const char* e = getenv("PDK_Q8_PLAIN");
        return e && e[0] == '1';
    }();
    return v;
}

constexpr uint32_t kWarps = 8;         // warps per CTA
constexpr uint32_t kMaxChunks = 16;    // 16 * 512 = 8192 elements per register pass

__device__ __forceinline__ float dot16(const uint4 w, const float* __restrict__ xs) {
    const float4 x0 = *reinterpret_cast<const float4*>(xs);
    const float4 x1 = *reinterpret_cast<const float4*>(xs + 4);
    const float4 x2 = *reinterpret_cast<const float4*>(xs + 8);
    const float4 x3 = *reinterpret_cast<const float4*>(xs + 12);
    float a = 0.0f;
#define PDK_B(word, sh) (float)(int8_t)(((word) >> (sh)) & 0xffu)
    a = fmaf(PDK_B(w.x, 0), x0.x, a);  a = fmaf(PDK_B(w.x, 8), x0.y, a);
    a = fmaf(PDK_B(w.x, 16), x0.z, a); a = fmaf(PDK_B(w.x, 24), x0.w, a);
    a = fmaf(PDK_B(w.y, 0), x1.x, a);  a = fmaf(PDK_B(w.y, 8), x1.y, a);
    a = fmaf(PDK_B(w.y, 16), x1.z, a); a = fmaf(PDK_B(w.y, 24), x1.w, a);
    a = fmaf(PDK_B(w.z, 0), x2.x, a);  a = fmaf(PDK_B(w.z, 8), x2.y, a);
    a = fmaf(PDK_B(w.z, 16), x2.z, a); a = fmaf(PDK_B(w.z, 24), x2.w, a);
    a = fmaf(PDK_B(w.w, 0), x3.x, a);  a = fmaf(PDK_B(w.w, 8), x3.y, a);
    a = fmaf(PDK_B(w.w, 16), x3.z, a); a = fmaf(PDK_B(w.w, 24), x3.w, a);
#undef PDK_B
    return a;
}

// x for `TOK` tokens is staged once per CTA into shared memory; each warp then
// walks rows warp_id, warp_id + stride, ...  CH = ceil(in_dim / 512) chunks of
// 512 elements are held in registers per row.
template <uint32_t CH, uint32_t TOK>
__global__ void __launch_bounds__(kWarps * 32)
q8_gemv_kernel(const int8_t* __restrict__ data, const __half* __restrict__ scale,
               const float* __restrict__ bias, const float* __restrict__ x, float* __restrict__ y,
               uint32_t in_dim, uint32_t out_dim, uint32_t batch0) {
    extern __shared__ __align__(16) float xs[];  // [TOK][in_dim]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float* xg = x + (size_t)batch0 * in_dim;
    for (uint32_t i = tid * 4u; i < TOK * in_dim; i += blockDim.x * 4u)
        *reinterpret_cast<float4*>(xs + i) = *reinterpret_cast<const float4*>(xg + i);
    __syncthreads();

    const uint32_t nb = in_dim >> 5;
    for (uint32_t row = blockIdx.x * kWarps + warp; row < out_dim; row += gridDim.x * kWarps) {
        const int8_t* wrow = data + (size_t)row * in_dim;
        const __half* srow = scale + (size_t)row * nb;
        uint4 w[CH];
        float sc[CH];
#pragma unroll
        for (uint32_t c = 0; c < CH; ++c) {
            const uint32_t k = c * 512u + lane * 16u;
            if (k < in_dim) {
                w[c] = pdk_ldg_stream16(wrow + k);
                sc[c] = __half2float(srow[k >> 5]);
            } else {
                w[c] = make_uint4(0u, 0u, 0u, 0u);
                sc[c] = 0.0f;
            }
        }
        float acc[TOK];
#pragma unroll
        for (uint32_t t = 0; t < TOK; ++t) acc[t] = 0.0f;
#pragma unroll
        for (uint32_t c = 0; c < CH; ++c) {
            const uint32_t k = c * 512u + lane * 16u;
            if (k < in_dim) {
#pragma unroll
                for (uint32_t t = 0; t < TOK; ++t) acc[t] = fmaf(sc[c], dot16(w[c], xs + t * in_dim + k), acc[t]);
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < TOK; ++t) {
            float v = pdk_warp_sum(acc[t]);
            if (lane == 0) {
                if (bias) v += bias[row];
                y[(size_t)(batch0 + t) * out_dim + row] = v;
            }
        }
    }
}

template <uint32_t CH, uint32_t TOK>
int launch(const void* data, const void* scale, const void* bias, const float* x, float* y, uint32_t in_dim,
           uint32_t out_dim, uint32_t batch0, cudaStream_t st) {
    const size_t smem = (size_t)TOK * in_dim * sizeof(float);
    auto kern = q8_gemv_kernel<CH, TOK>;
    if (smem > 48u * 1024u) {
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
    kern<<<grid, kWarps * 32u, smem, st>>>((const int8_t*)data, (const __half*)scale, (const float*)bias, x, y,
                                           in_dim, out_dim, batch0);
    return pdk_launch_status();
}

template <uint32_t TOK>
int dispatch(const void* data, const void* scale, const void* bias, const float* x, float* y, uint32_t in_dim,
             uint32_t out_dim, uint32_t batch0, cudaStream_t st) {
    const uint32_t ch = (in_dim + 511u) / 512u;
    if (ch <= 2u) return launch<2, TOK>(data, scale, bias, x, y, in_dim, out_dim, batch0, st);
    if (ch <= 4u) return launch<4, TOK>(data, scale, bias, x, y, in_dim, out_dim, batch0, st);
    if (ch <= 6u) return launch<6, TOK>(data, scale, bias, x, y, in_dim, out_dim, batch0, st);
    if (ch <= 10u) return launch<10, TOK>(data, scale, bias, x, y, in_dim, out_dim, batch0, st);
    if (ch <= kMaxChunks) return launch<kMaxChunks, TOK>(data, scale, bias, x, y, in_dim, out_dim, batch0, st);
    return cudaErrorNotSupported;
}

int check(const void* data, const void* scale, const void* x, const void* y, uint32_t in_dim) {
    if ((in_dim & 31u) != 0u || in_dim == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(scale, 2) || !pdk_aligned(x, 16) || !pdk_aligned(y, 4))
        return cudaErrorInvalidValue;
    if ((in_dim & 15u) != 0u) return cudaErrorInvalidValue;
    return 0;
}

}  // namespace

PDK_EXPORT int pd_q8_0_gemv_repacked(const void* data, const void* scale, const void* bias, const void* x, void* y,
                                     uint32_t in_dim, uint32_t out_dim, void* stream) {
    if (out_dim == 0) return 0;
    if (int rc = check(data, scale, x, y, in_dim)) return rc;
    if (!force_plain()) {
        const int rc = pdk_q8_0_gemv_i8(data, scale, (const float*)bias, (const float*)x, (float*)y, in_dim, out_dim,
                                        (cudaStream_t)stream);
        if (rc != -1) return rc;
    }
    return dispatch<1>(data, scale, bias, (const float*)x, (float*)y, in_dim, out_dim, 0u, (cudaStream_t)stream);
}

PDK_EXPORT int pd_q8_0_gemm_repacked(const void* data, const void* scale, const void* bias, const void* x, void* y,
                                     uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream) {
    if (out_dim == 0 || batch == 0) return 0;
    if (int rc = check(data, scale, x, y, in_dim)) return rc;
    const float* xf = (const float*)x;
    float* yf = (float*)y;
    auto st = (cudaStream_t)stream;
    if (!force_plain()) {
        // two or more tokens: the tokens-as-columns kernel on the TMA ring (one weight pass per eight
        // tokens); shapes outside its plan take one decode GEMV per token, which still beats the plain
        // f32 kernel below (169 us per four tokens against 18 us per token at K=5120 N=17408)
        int rc = batch >= 2u ? pdk_q8_0_gemm_i8(data, scale, (const float*)bias, xf, yf, in_dim, out_dim, batch, st) : -1;
        if (rc != -1) return rc;
        rc = 0;
        for (uint32_t t = 0; t < batch && rc == 0; ++t)
            rc = pdk_q8_0_gemv_i8(data, scale, (const float*)bias, xf + (size_t)t * in_dim, yf + (size_t)t * out_dim, in_dim,
                                  out_dim, st);
        if (rc != -1) return rc;  // -1 can only come from the first call: the plan depends on the shape alone
    }
    uint32_t b = 0;
    for (; b + 4u <= batch; b += 4u)
        if (int rc = dispatch<4>(data, scale, bias, xf, yf, in_dim, out_dim, b, st)) return rc;
    for (; b + 2u <= batch; b += 2u)
        if (int rc = dispatch<2>(data, scale, bias, xf, yf, in_dim, out_dim, b, st)) return rc;
    for (; b < batch; ++b)
        if (int rc = dispatch<1>(data, scale, bias, xf, yf, in_dim, out_dim, b, st)) return rc;
    return 0;
}
