// nvf4_elem.cu - NVFP4 element kernels: activation quantizer, dequant, the
// weight-scale tiler for the tcgen05 GEMM, and the W4A16 decode GEMV.
//
// NVFP4 plane (ModelOpt / llm-compressor checkpoints):
//   data   u8  [out][in/2]   e2m1 nibbles, low nibble = even element
//   scale  u8  [out][in/16]  e4m3 per 16 elements
//   scale2 f32               per tensor;  w = (e2m1 * e4m3) * scale2
#include <cuda_fp8.h>

#include "pdk_common.cuh"

int pdk_nvf4_gemv_tc5(const void* data, const void* scale, const void* bias, const void* x, void* y, float scale2,
                      uint32_t in_dim, uint32_t out_dim, cudaStream_t st);

namespace {

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 stored doubled, one per byte
    const uint64_t mags2 = 0x0C08060403020100ull;
    const float m = 0.5f * (float)(uint32_t)((mags2 >> ((code & 7u) * 8u)) & 0xffu);
    return (code & 8u) ? -m : m;
}

// RN-even onto {0, .5, 1, 1.5, 2, 3, 4, 6}; ties go to the even mantissa.
__device__ __forceinline__ uint32_t e2m1_rn(float v) {
    const uint32_t s = v < 0.0f ? 8u : 0u;
    const float a = fabsf(v);
    uint32_t m;
    if (a <= 0.25f) m = 0u;
    else if (a < 0.75f) m = 1u;
    else if (a <= 1.25f) m = 2u;
    else if (a < 1.75f) m = 3u;
    else if (a <= 2.5f) m = 4u;
    else if (a < 3.5f) m = 5u;
    else if (a <= 5.0f) m = 6u;
    else m = 7u;
    return s | m;
}

// The NVFP4 rule for one 16-element block (packs/cuda/src/quant/e2m1.cuh): scale byte =
// RN_e4m3(amax / 6), raised to the smallest subnormal when amax > 0 rounds to zero; elements =
// e2m1_rn(v / decode(scale byte)).  A block whose amax is 0 stores scale 0 and codes 0.
struct Nvf4BlockScale {
    uint32_t byte;   // the e4m3 scale as stored
    float recip;     // 1 / its value, 0 for an all-zero block
};
__device__ __forceinline__ Nvf4BlockScale nvf4_block_scale(float amax) {
    Nvf4BlockScale s = {0u, 0.0f};
    if (amax > 0.0f) {
        s.byte = (uint32_t)__nv_cvt_float_to_fp8(amax * (1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3);
        if (s.byte == 0u) s.byte = 1u;
        s.recip = 1.0f / e4m3_to_f32((uint8_t)s.byte);
    }
    return s;
}
__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}
// four values -> four e2m1 codes, first value in the low nibble
__device__ __forceinline__ uint32_t nvf4_codes4(const float4& v, float recip) {
    return e2m1_rn(v.x * recip) | e2m1_rn(v.y * recip) << 4 | e2m1_rn(v.z * recip) << 8 | e2m1_rn(v.w * recip) << 12;
}

// One thread per 8 elements (half a block); the lane pair closes the 16-element amax.
__global__ void quantize_nvf4_kernel(const float* __restrict__ x, uint8_t* __restrict__ q,
                                     uint8_t* __restrict__ scale, uint32_t n) {
    const uint32_t i = (blockIdx.x * 256u + threadIdx.x) * 8u;
    if (i >= n) return;  // n % 32 == 0: lane pairs leave together
    const float4 a = *reinterpret_cast<const float4*>(x + i);
    const float4 b = *reinterpret_cast<const float4*>(x + i + 4u);
    const uint32_t lane = threadIdx.x & 31u;
    float amax = fmaxf(amax4(a), amax4(b));
    amax = fmaxf(amax, __shfl_xor_sync(0x3u << (lane & 30u), amax, 1));
    const Nvf4BlockScale s = nvf4_block_scale(amax);
    *reinterpret_cast<uint32_t*>(q + (i >> 1)) = nvf4_codes4(a, s.recip) | nvf4_codes4(b, s.recip) << 16;
    if ((lane & 1u) == 0u) scale[i >> 4] = (uint8_t)s.byte;
}

// SwiGLU in front of the quantizer: h = (g / (1 + expf(-g))) * u in f32, then quantize_nvf4_kernel's
// blocks.  gate / up: two planes of n elements (stride 0), or the two halves of fused rows
// [rows][2 * ff] (stride = ff: element i of the output is row i / ff, column i % ff).
__device__ __forceinline__ float silu_times(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
__global__ void quantize_nvf4_swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                            uint8_t* __restrict__ q, uint8_t* __restrict__ scale, uint32_t n, uint32_t ff) {
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    const uint32_t i = (blockIdx.x * 256u + threadIdx.x) * 8u;
    if (i >= n) return;  // n % 32 == 0: lane pairs leave together
    size_t src = i;
    if (ff != 0u) src = (size_t)(i / ff) * 2u * ff + i % ff;   // ff % 32 == 0: the 8 elements stay in one row
    const float4 g0 = *reinterpret_cast<const float4*>(gate + src), g1 = *reinterpret_cast<const float4*>(gate + src + 4u);
    const float4 u0 = *reinterpret_cast<const float4*>(up + src), u1 = *reinterpret_cast<const float4*>(up + src + 4u);
    const float4 a = make_float4(silu_times(g0.x, u0.x), silu_times(g0.y, u0.y), silu_times(g0.z, u0.z), silu_times(g0.w, u0.w));
    const float4 b = make_float4(silu_times(g1.x, u1.x), silu_times(g1.y, u1.y), silu_times(g1.z, u1.z), silu_times(g1.w, u1.w));
    const uint32_t lane = threadIdx.x & 31u;
    float amax = fmaxf(amax4(a), amax4(b));
    amax = fmaxf(amax, __shfl_xor_sync(0x3u << (lane & 30u), amax, 1));
    const Nvf4BlockScale s = nvf4_block_scale(amax);
    *reinterpret_cast<uint32_t*>(q + (i >> 1)) = nvf4_codes4(a, s.recip) | nvf4_codes4(b, s.recip) << 16;
    if ((lane & 1u) == 0u) scale[i >> 4] = (uint8_t)s.byte;
}

// Fused producer in front of an NVFP4 GEMM (the contract of packs/cuda/src/quant/nvf4.cuh:545-571):
// x += proj, out = rmsnorm(x) * w, q / scale = the NVFP4 planes of out.  One CTA per row, and the
// summed row never leaves the register file: thread t holds the row's float4 number t, t + T,
// t + 2T, ... (T threads, kChunks of them), so every load and store of a warp is one contiguous
// 512-byte run and nothing is staged in shared memory.  Mean square: f32 products accumulated in
// f64, per thread, then per warp, then over the warps in warp order; scale = 1 / sqrtf((float)
// (sum / n) + eps); out = v * scale * w, multiplied in that order.  A 16-element NVFP4 block is
// four neighbouring float4, i.e. four neighbouring lanes: two shuffles close its amax and each
// lane emits its own four codes.
constexpr uint32_t kNormMaxThreads = 384;
template <int kChunks>
__global__ void __launch_bounds__(kChunks <= 8 ? 1024 : kNormMaxThreads)
add_rmsnorm_quant_nvf4_kernel(float* __restrict__ x, const float* __restrict__ proj, const float* __restrict__ w,
                              float* __restrict__ out, uint8_t* __restrict__ q, uint8_t* __restrict__ scale, uint32_t n,
                              float eps) {
    __shared__ double warp_sq[32];
    const uint32_t t = threadIdx.x, width = blockDim.x, n4 = n >> 2;   // width % 32 == 0, n4 % 4 == 0
    const size_t row4 = (size_t)blockIdx.x * n4;
    float4* x4 = reinterpret_cast<float4*>(x) + row4;
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();

    float4 held[kChunks];
    double sq = 0.0;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const uint32_t at = (uint32_t)c * width + t;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (at < n4) {
            v = x4[at];
            if (proj != nullptr) {
                const float4 add = (reinterpret_cast<const float4*>(proj) + row4)[at];
                v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
                x4[at] = v;
            }
        }
        held[c] = v;
        sq += (double)(v.x * v.x) + (double)(v.y * v.y) + (double)(v.z * v.z) + (double)(v.w * v.w);
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
    if ((t & 31u) == 0u) warp_sq[t >> 5] = sq;
    __syncthreads();
    double total = 0.0;
    for (uint32_t i = 0; i < (width >> 5); ++i) total += warp_sq[i];   // every thread, same order: no second barrier
    const float norm = 1.0f / sqrtf((float)(total / (double)n) + eps);

    float4* out4 = reinterpret_cast<float4*>(out) + row4;
    uint16_t* codes = reinterpret_cast<uint16_t*>(q + (size_t)blockIdx.x * (n >> 1));
    uint8_t* srow = scale + (size_t)blockIdx.x * (n >> 4);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const uint32_t at = (uint32_t)c * width + t;
        const bool live = at < n4;   // the same for the four lanes of a block: n4 and width are multiples of 4
        float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (live) {
            const float4 g = reinterpret_cast<const float4*>(w)[at];
            const float4 v = held[c];
            r = make_float4(v.x * norm * g.x, v.y * norm * g.y, v.z * norm * g.z, v.w * norm * g.w);
            out4[at] = r;
        }
        float amax = amax4(r);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const Nvf4BlockScale s = nvf4_block_scale(amax);
        if (live) {
            codes[at] = (uint16_t)nvf4_codes4(r, s.recip);
            if ((t & 3u) == 0u) srow[at >> 2] = (uint8_t)s.byte;
        }
    }
}

// One CTA per output row; (e2m1 * e4m3) * scale2 with two separate roundings.
__global__ void nvf4_dequant_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scale, float scale2,
                                    float* __restrict__ y, uint32_t in_dim) {
    const uint32_t o = blockIdx.x, kh = in_dim >> 1;
    const uint8_t* row = data + (size_t)o * kh;
    const uint8_t* srow = scale + (size_t)o * (in_dim >> 4);
    float* yrow = y + (size_t)o * in_dim;
    for (uint32_t j = threadIdx.x; j < kh; j += blockDim.x) {
        const uint32_t b = row[j];
        const float s = e4m3_to_f32(srow[j >> 3]);
        float2 out;
        out.x = __fmul_rn(__fmul_rn(e2m1_to_f32(b & 15u), s), scale2);
        out.y = __fmul_rn(__fmul_rn(e2m1_to_f32(b >> 4), s), scale2);
        *reinterpret_cast<float2*>(yrow + 2u * j) = out;
    }
}

// Weight scales [out][in/16] -> the tensor core's scale-cell order.  For row
// tile rt (128 rows) and K slab kb (256 elements) a 2048-byte record of four
// 512-byte cells, one per 64-element MMA step j:
//   byte l*16 + c*4 + b  of cell j  =  scale[rt*128 + c*32 + l][kb*16 + j*4 + b]
// (rows past out_dim read as 0).  One thread per 4-byte word of the output.
__global__ void nvf4_tile_scales_kernel(const uint8_t* __restrict__ scale, uint32_t* __restrict__ tiled,
                                        uint32_t in_dim, uint32_t out_dim, uint64_t n_words) {
    const uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= n_words) return;
    const uint32_t n_slab = in_dim >> 8, kb16 = in_dim >> 4;
    const uint32_t c = (uint32_t)(w & 3u), l = (uint32_t)((w >> 2) & 31u), j = (uint32_t)((w >> 7) & 3u);
    const uint64_t rec = w >> 9;
    const uint32_t kb = (uint32_t)(rec % n_slab), rt = (uint32_t)(rec / n_slab);
    const uint32_t row = rt * 128u + c * 32u + l;
    uint32_t v = 0u;
    if (row < out_dim) v = *reinterpret_cast<const uint32_t*>(scale + (size_t)row * kb16 + kb * 16u + j * 4u);
    tiled[w] = v;
}

// W4A16 decode GEMV, f32 activations: a warp per output row, 8 rows per CTA.
// Lane l owns elements 32l'.. in steps of 1024: 16 packed bytes (32 elements,
// two scale blocks) per step.
__global__ void __launch_bounds__(256)
nvf4_gemv_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scale, const float* __restrict__ bias,
                 const float* __restrict__ x, float* __restrict__ y, float scale2, uint32_t in_dim, uint32_t out_dim) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (row >= out_dim) return;
    const uint8_t* drow = data + (size_t)row * (in_dim >> 1);
    const uint8_t* srow = scale + (size_t)row * (in_dim >> 4);
    float acc = 0.0f;
    for (uint32_t e = lane * 32u; e < in_dim; e += 1024u) {
        const uint4 q = pdk_ldg_stream16(drow + (e >> 1));
        const uint32_t ss = *reinterpret_cast<const uint16_t*>(srow + (e >> 4));
        const float s0 = e4m3_to_f32((uint8_t)(ss & 0xffu)), s1 = e4m3_to_f32((uint8_t)(ss >> 8));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        float part[2] = {0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 xa = *reinterpret_cast<const float4*>(x + e + 8 * i);
            const float4 xb = *reinterpret_cast<const float4*>(x + e + 8 * i + 4);
            float t = e2m1_to_f32(w[i] & 15u) * xa.x;
            t = fmaf(e2m1_to_f32((w[i] >> 4) & 15u), xa.y, t);
            t = fmaf(e2m1_to_f32((w[i] >> 8) & 15u), xa.z, t);
            t = fmaf(e2m1_to_f32((w[i] >> 12) & 15u), xa.w, t);
            t = fmaf(e2m1_to_f32((w[i] >> 16) & 15u), xb.x, t);
            t = fmaf(e2m1_to_f32((w[i] >> 20) & 15u), xb.y, t);
            t = fmaf(e2m1_to_f32((w[i] >> 24) & 15u), xb.z, t);
            t = fmaf(e2m1_to_f32(w[i] >> 28), xb.w, t);
            part[i >> 1] += t;
        }
        acc = fmaf(s0, part[0], acc);
        acc = fmaf(s1, part[1], acc);
    }
    acc = pdk_warp_sum(acc);
    if (lane == 0) y[row] = fmaf(acc, scale2, bias ? bias[row] : 0.0f);
}

}  // namespace

// slot 119, packs/cuda/src/quant/nvf4.cuh:405-421
PDK_EXPORT int pd_quantize_nvf4(const void* x, void* q, void* scale, uint32_t n, void* stream) {
    if (n == 0) return 0;
    if ((n & 31u) != 0u || !pdk_aligned(x, 16) || !pdk_aligned(q, 4)) return cudaErrorInvalidValue;
    quantize_nvf4_kernel<<<(n / 8u + 255u) / 256u, 256, 0, (cudaStream_t)stream>>>((const float*)x, (uint8_t*)q,
                                                                                    (uint8_t*)scale, n);
    return pdk_launch_status();
}

// slot 436, packs/cuda/src/quant/nvf4.cuh:545-571: x f32 [batch][n] += proj (proj may be null),
// out f32 [batch][n] = rmsnorm(x) * w, q / scale = pd_quantize_nvf4 of each row of out.
PDK_EXPORT int pd_add_rmsnorm_quant_nvf4_batch(void* x, const void* proj, const void* w, void* out, void* q, void* scale,
                                               uint32_t n, float eps, uint32_t batch, void* stream) {
    if (n == 0 || batch == 0) return 0;
    if ((n & 31u) != 0u || !pdk_aligned(x, 16) || !pdk_aligned(proj, 16) || !pdk_aligned(w, 16) || !pdk_aligned(out, 16) ||
        !pdk_aligned(q, 4))
        return cudaErrorInvalidValue;
    // the fewest float4 per thread (a power of two) that fits the row into one CTA: up to 1024
    // threads while a thread holds at most 8 float4, kNormMaxThreads beyond.  5120 -> 2 per thread,
    // 640 threads (measured at 4096 rows of 5120: 2 per thread 64 us, 4 70 us, 8 84 us, 16 131 us)
    const uint32_t n4 = n >> 2;
    uint32_t chunks = 1;
    while (chunks < 32u && (n4 + chunks - 1u) / chunks > (chunks <= 8u ? 1024u : kNormMaxThreads)) chunks <<= 1;
    static const uint32_t forced = getenv("PDK_NORM_CHUNKS") ? (uint32_t)atoi(getenv("PDK_NORM_CHUNKS")) : 0u;   // A/B switch
    if (forced != 0u && forced <= 32u && (forced & (forced - 1u)) == 0u &&
        (n4 + forced - 1u) / forced <= (forced <= 8u ? 1024u : kNormMaxThreads))
        chunks = forced;
    const uint32_t width = ((n4 + chunks - 1u) / chunks + 31u) & ~31u;
    if (width > (chunks <= 8u ? 1024u : kNormMaxThreads)) return cudaErrorNotSupported;   // rows beyond 49152 elements
#define PDK_NORM_CASE(C)                                                                                          \
    case C:                                                                                                       \
        return pdk_launch_pdl(add_rmsnorm_quant_nvf4_kernel<C>, dim3(batch), dim3(width), 0, (cudaStream_t)stream, \
                              (float*)x, (const float*)proj, (const float*)w, (float*)out, (uint8_t*)q,           \
                              (uint8_t*)scale, n, eps)
    switch (chunks) {
        PDK_NORM_CASE(1);
        PDK_NORM_CASE(2);
        PDK_NORM_CASE(4);
        PDK_NORM_CASE(8);
        PDK_NORM_CASE(16);
        PDK_NORM_CASE(32);
    }
#undef PDK_NORM_CASE
    return cudaErrorNotSupported;
}

// slot 861, packs/cuda/src/exports.cuh:505-520: the decode tick's pre-FFN norm feeding the W4A4 GEMM -
// slot 436's contract with proj required.
PDK_EXPORT int pd_add_rmsnorm_nvf4_batch(void* x, const void* proj, const void* w, void* out, void* q, void* qs, uint32_t n,
                                         float eps, uint32_t batch, void* stream) {
    if (n == 0 || batch == 0) return 0;
    if (proj == nullptr) return cudaErrorInvalidValue;
    return pd_add_rmsnorm_quant_nvf4_batch(x, proj, w, out, q, qs, n, eps, batch, stream);
}

// slot 120, packs/cuda/src/quant/nvf4.cuh:714-735, 1023-1030: h = silu(gate) * up, NVFP4 planes of h
PDK_EXPORT int pd_quantize_nvf4_swiglu(const void* gate, const void* up, void* q, void* scale, uint32_t n, void* stream) {
    if (n == 0) return 0;
    if ((n & 31u) != 0u || !pdk_aligned(gate, 16) || !pdk_aligned(up, 16) || !pdk_aligned(q, 4)) return cudaErrorInvalidValue;
    return pdk_launch_pdl(quantize_nvf4_swiglu_kernel, dim3((n / 8u + 255u) / 256u), dim3(256), 0, (cudaStream_t)stream,
                          (const float*)gate, (const float*)up, (uint8_t*)q, (uint8_t*)scale, n, 0u);
}

// slot 516, packs/cuda/src/quant/nvf4.cuh:737-775: the same over fused rows [n_rows][2 * ff] (gate | up)
PDK_EXPORT int pd_swiglu_fused_nvf4(const void* fused, void* q, void* scale, uint32_t ff, uint32_t n_rows, void* stream) {
    if (n_rows == 0 || ff == 0) return 0;
    if ((ff & 31u) != 0u || (uint64_t)n_rows * ff > 0xffffffffull || !pdk_aligned(fused, 16) || !pdk_aligned(q, 4))
        return cudaErrorInvalidValue;
    const uint32_t n = n_rows * ff;
    return pdk_launch_pdl(quantize_nvf4_swiglu_kernel, dim3((n / 8u + 255u) / 256u), dim3(256), 0, (cudaStream_t)stream,
                          (const float*)fused, (const float*)fused + ff, (uint8_t*)q, (uint8_t*)scale, n, ff);
}

// slot 393, packs/cuda/src/quant/nvf4.cuh:4365-4403
PDK_EXPORT int pd_nvf4_dequant(const void* data, const void* scale, float scale2, void* y, uint32_t in_dim,
                               uint32_t out_dim, void* stream) {
    if (out_dim == 0) return 0;
    if ((in_dim & 31u) != 0u || !pdk_aligned(y, 8)) return cudaErrorInvalidValue;
    nvf4_dequant_kernel<<<out_dim, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)data, (const uint8_t*)scale, scale2,
                                                                   (float*)y, in_dim);
    return pdk_launch_status();
}

// slot 853, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:845-861,981-994
PDK_EXPORT int pd_nvf4_tc5_tile_scales(const void* scale, void* tiled, uint32_t in_dim, uint32_t out_dim,
                                       void* stream) {
    if (out_dim == 0 || in_dim == 0) return 0;
    if ((in_dim & 255u) != 0u || !pdk_aligned(scale, 4) || !pdk_aligned(tiled, 16)) return cudaErrorInvalidValue;
    const uint64_t n_words = (uint64_t)((out_dim + 127u) / 128u) * (in_dim >> 8) * 512u;
    const uint64_t blocks = (n_words + 255u) / 256u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    nvf4_tile_scales_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)scale,
                                                                                (uint32_t*)tiled, in_dim, out_dim,
                                                                                n_words);
    return pdk_launch_status();
}

// slot 394, packs/cuda/src/quant/nvf4.cuh:4436-4779
PDK_EXPORT int pd_nvf4_gemv(const void* data, const void* scale, const void* bias, const void* x, void* y,
                            float scale2, uint32_t in_dim, uint32_t out_dim, void* stream) {
    if (out_dim == 0) return 0;
    if ((in_dim & 31u) != 0u || in_dim == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(scale, 2) || !pdk_aligned(x, 16)) return cudaErrorInvalidValue;
    // tensor-core route (activations as four NVFP4 terms, moe_tc5.cu); PDK_NVF4_GEMV_PLAIN=1 keeps the
    // plain kernel (A/B switch, read once)
    static const bool plain = [] {
        const char* e = getenv("PDK_NVF4_GEMV_PLAIN");
        return e && e[0] == '1';
    }();
    if (!plain) {
        const int rc = pdk_nvf4_gemv_tc5(data, scale, bias, x, y, scale2, in_dim, out_dim, (cudaStream_t)stream);
        if (rc >= 0) return rc;
    }
    nvf4_gemv_kernel<<<(out_dim + 7u) / 8u, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)data, (const uint8_t*)scale, (const float*)bias, (const float*)x, (float*)y, scale2, in_dim,
        out_dim);
    return pdk_launch_status();
}
