// elementwise.cu - dequantizers and repackers that touch every byte once.
//
// All of these are pure HBM streams: the kernels are laid out so that each
// warp reads and writes whole 128-byte lines, and the arithmetic reproduces
// the reference's per-element products bit for bit (single f32 multiplies, no
// fused multiply-add where the reference rounds twice).
#include "pdk_common.cuh"

// ---------------------------------------------------------------- add_inplace
__global__ void pdk_add_inplace_kernel(float* __restrict__ y, const float* __restrict__ x, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += x[i];
}

PDK_EXPORT int pd_add_inplace_f32(void* y, const void* x, uint32_t n, void* stream) {
    if (n == 0) return 0;
    pdk_add_inplace_kernel<<<(n + 255u) / 256u, 256, 0, (cudaStream_t)stream>>>((float*)y, (const float*)x, n);
    return pdk_launch_status();
}

// ---------------------------------------------------------------- Q8_0 dequant
// One thread per element: block b = i/32 is {f16 d, int8 q[32]} at byte 34*b
// (2-byte aligned).  y = float(q) * float(d), one rounding.
__global__ void pdk_q8_0_dequant_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, uint64_t total) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    uint64_t b = i >> 5;
    uint32_t j = (uint32_t)(i & 31u);
    const uint8_t* s = in + b * 34u;
    const float d = __half2float(*reinterpret_cast<const __half*>(s));
    out[i] = __fmul_rn((float)(int8_t)s[2u + j], d);
}

PDK_EXPORT int pd_q8_0_dequant_f32(const void* in, void* out, uint64_t n_blocks, void* stream) {
    const uint64_t total = n_blocks * 32ull;
    if (total == 0) return 0;
    if (!pdk_aligned(in, 2) || !pdk_aligned(out, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (total + 255u) / 256u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    pdk_q8_0_dequant_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)in, (float*)out, total);
    return pdk_launch_status();
}

// ---------------------------------------------------------------- Q8_0 repack
// Eight threads per block, one 4-byte word of the int8 payload each (read as
// two u16: the payload sits at 34*b + 2, only 2-byte aligned); a warp covers
// four blocks = 136 contiguous source bytes and writes 128 contiguous bytes.
__global__ void pdk_q8_0_repack_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst_data,
                                       uint16_t* __restrict__ dst_scale, uint64_t n_blocks) {
    uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t b = t >> 3;
    if (b >= n_blocks) return;
    uint32_t w = (uint32_t)(t & 7u);
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src + b * 34u);
    uint32_t lo = s[1u + 2u * w], hi = s[2u + 2u * w];
    dst_data[b * 8u + w] = lo | (hi << 16);
    if (w == 0) dst_scale[b] = s[0];
}

PDK_EXPORT int pd_q8_0_repack(const void* src, void* dst_data, void* dst_scale, uint64_t n_blocks, void* stream) {
    if (n_blocks == 0) return 0;
    if (!pdk_aligned(src, 2) || !pdk_aligned(dst_data, 4) || !pdk_aligned(dst_scale, 2)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_blocks * 8u + 255u) / 256u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    pdk_q8_0_repack_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint32_t*)dst_data, (uint16_t*)dst_scale, n_blocks);
    return pdk_launch_status();
}

// ---------------------------------------------------------------- MXFP4 dequant
// ggml's MXFP4 convention: nibble values doubled, E8M0 scale halved.  The
// scale is built from bit patterns so bytes 0 and 1 give the f32 denormals
// 2^-128 and 2^-127 exactly.
__device__ __forceinline__ float pdk_e8m0_half(uint32_t e) {
    return __uint_as_float(e < 2u ? (0x00200000u << e) : ((e - 1u) << 23));
}
__device__ __forceinline__ float pdk_fp4_doubled(uint32_t nib) {
    // magnitudes 0,1,2,3,4,6,8,12 packed one per byte; sign in bit 3
    const uint64_t mags = 0x0C08060403020100ull;
    float m = (float)(uint32_t)((mags >> ((nib & 7u) * 8u)) & 0xffu);
    return (nib & 8u) ? 0.0f - m : m;  // code 8 is +0.0 in the ggml table
}

// One thread per element: i -> block b, element j; byte 1 + (j & 15), low
// nibble for j < 16, high nibble otherwise.
__global__ void pdk_mxfp4_dequant_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, uint64_t total) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    uint64_t b = i >> 5;
    uint32_t j = (uint32_t)(i & 31u);
    const uint8_t* s = in + b * 17u;
    const float d = pdk_e8m0_half(s[0]);
    const uint32_t q = s[1u + (j & 15u)];
    out[i] = __fmul_rn(pdk_fp4_doubled(j < 16u ? (q & 15u) : (q >> 4)), d);
}

PDK_EXPORT int pd_mxfp4_dequant_f32(const void* in, void* out, uint64_t n_blocks, void* stream) {
    const uint64_t total = n_blocks * 32ull;
    if (total == 0) return 0;
    if (!pdk_aligned(out, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (total + 255u) / 256u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    pdk_mxfp4_dequant_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)in, (float*)out, total);
    return pdk_launch_status();
}

// ---------------------------------------------------------------- MXFP4 repack
// 17-byte blocks -> 16-byte nibble plane + 1-byte scale plane.  Sixteen
// threads per block move one payload byte each (the source has no alignment).
__global__ void pdk_mxfp4_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst_data,
                                        uint8_t* __restrict__ dst_scale, uint64_t n_blocks) {
    uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t b = t >> 4;
    if (b >= n_blocks) return;
    uint32_t j = (uint32_t)(t & 15u);
    const uint8_t* s = src + b * 17u;
    dst_data[b * 16u + j] = s[1u + j];
    if (j == 0) dst_scale[b] = s[0];
}

PDK_EXPORT int pd_mxfp4_repack(const void* src, void* dst_data, void* dst_scale, uint64_t n_blocks, void* stream) {
    if (n_blocks == 0) return 0;
    const uint64_t blocks = (n_blocks * 16u + 255u) / 256u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    pdk_mxfp4_repack_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst_data, (uint8_t*)dst_scale, n_blocks);
    return pdk_launch_status();
}
