// fp8_quant.cu - row-scaled e4m3 quantizers (weights from bf16, activations from
// f32) and the host side of the TMA tensor maps.
//
// Scale rule of both quantizers: a power of two 2^e per row with
// e = ex - 9 + (fr > 0.875) for amax = fr * 2^ex, so that amax / 2^e <= 448;
// values are multiplied by 2^-e (exact) and rounded to e4m3 with
// round-to-nearest-even and saturation to +-448.
#include <cuda_fp8.h>

#include "tc5.cuh"

static __device__ unsigned int g_pdk_device_error = 0;

// Device address of the error word on the current device (resolved once per device).
unsigned int* pdk_error_word() {
    static unsigned int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_pdk_device_error) != cudaSuccess) return nullptr;
        cached[dev] = (unsigned int*)p;
    }
    return cached[dev];
}

// Reads and clears the device error word of the current device (0 = none).
// Synchronizes the device.
PDK_EXPORT unsigned int pdk_device_error(void) {
    unsigned int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return 0xffffffffu;
    cudaMemcpyFromSymbol(&v, g_pdk_device_error, sizeof(v));
    cudaMemcpyToSymbol(g_pdk_device_error, &zero, sizeof(zero));
    return v;
}

int pdk_quantize_e4m3_row_1p(const float* x, uint8_t* q, float* rscale, uint32_t n, uint32_t batch, cudaStream_t st);

namespace {

__device__ __forceinline__ uint8_t to_e4m3(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float block_max(float a, float* wmax) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
    if ((threadIdx.x & 31u) == 0u) wmax[threadIdx.x >> 5] = a;
    __syncthreads();
    float m = 0.0f;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) m = fmaxf(m, wmax[w]);
    return m;
}

__device__ __forceinline__ int pow2_exponent(float amax) {
    if (!(amax > 0.0f)) return 0;
    int ex;
    const float fr = frexpf(amax, &ex);
    return ex - 9 + (fr > 0.875f ? 1 : 0);
}

// One CTA per row; 8 elements per thread per pass, 16-byte loads, 8-byte stores.
template <typename TI>
__global__ void __launch_bounds__(256) quantize_row_kernel(const TI* __restrict__ x, uint8_t* __restrict__ q,
                                                           float* __restrict__ rscale, uint32_t n_dim) {
    __shared__ float wmax[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const TI* xr = x + (size_t)row * n_dim;
    float a = 0.0f;
    for (uint32_t i = tid; i < n_dim; i += 256u) a = fmaxf(a, fabsf((float)xr[i]));
    const float amax = block_max(a, wmax);
    const int e = pow2_exponent(amax);
    if (tid == 0) rscale[row] = ldexpf(1.0f, e);
    const float inv = ldexpf(1.0f, -e);
    uint8_t* qr = q + (size_t)row * n_dim;
    for (uint32_t i = tid; i < n_dim; i += 256u) qr[i] = to_e4m3((float)xr[i] * inv);
}

}  // namespace

// slot 183, packs/cuda/src/gemm/dense_f8_decode.cuh:3179-3235
PDK_EXPORT int pd_quantize_e4m3_row(const void* x, void* q, void* rscale, uint32_t n_dim, uint32_t batch,
                                    void* stream) {
    if (n_dim == 0 || batch == 0) return 0;
    if (!pdk_aligned(x, 4) || !pdk_aligned(rscale, 4)) return cudaErrorInvalidValue;
    // rows of whole, aligned float4: one pass with the row in registers (f8_producers.cu)
    const int rc = pdk_quantize_e4m3_row_1p((const float*)x, (uint8_t*)q, (float*)rscale, n_dim, batch, (cudaStream_t)stream);
    if (rc != -1) return rc;
    quantize_row_kernel<float><<<batch, 256, 0, (cudaStream_t)stream>>>((const float*)x, (uint8_t*)q, (float*)rscale,
                                                                        n_dim);
    return pdk_launch_status();
}

// slot 375, packs/cuda/src/gemm/dense_fp4_w8.cuh:627-677
PDK_EXPORT int pd_bf16_to_f8row(const void* bf16, void* f8_data, void* row_scale, uint32_t in_dim, uint32_t out_dim,
                                void* stream) {
    if (in_dim == 0 || out_dim == 0) return 0;
    if (!pdk_aligned(bf16, 2) || !pdk_aligned(row_scale, 4)) return cudaErrorInvalidValue;
    quantize_row_kernel<__nv_bfloat16><<<out_dim, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)bf16, (uint8_t*)f8_data, (float*)row_scale, in_dim);
    return pdk_launch_status();
}

// ---- host: tensor maps --------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &st) !=
                cudaSuccess || st != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            p = nullptr;
        }
        return (EncodeTiledFn)p;
    }();
    return fn;
}

int pdk_make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                     uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    if (((uintptr_t)base & 15u) || (pitch & 15u) || box_inner * elem_bytes > 128u || box_rows > 256u)
        return cudaErrorInvalidValue;
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstride[1] = {pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estride[2] = {1u, 1u};
    const CUresult r = enc(map, dtype, 2u, const_cast<void*>(base), gdim, gstride, box, estride,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
}

int pdk_make_tmap_2d_dense(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                           uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    if (((uintptr_t)base & 15u) || (pitch & 15u) || box_inner > 256u || ((box_inner * elem_bytes) & 15u) || box_rows > 256u)
        return cudaErrorInvalidValue;
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstride[1] = {pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estride[2] = {1u, 1u};
    const CUresult r = enc(map, dtype, 2u, const_cast<void*>(base), gdim, gstride, box, estride,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
}

// ---------------------------------------------------------------- bounded-wait self-test
namespace {
// One warp waits on a barrier that nothing ever arrives on.  The wait must give up after
// `budget_ns`, record kErrTestWait in the error word and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(unsigned long long budget_ns, unsigned int* err_word, unsigned int* done) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tc5::mbar_init(&bar, 1);
        abort_flag = 0;
        tc5::mbar_fence_init();
    }
    __syncthreads();
    const tc5::WaitCtx ctx{&abort_flag, err_word};
    const bool ok = tc5::mbar_wait(&bar, 0u, ctx, tc5::kErrTestWait, 7u, budget_ns);
    __syncthreads();
    if (threadIdx.x == 0) *done = ok ? 2u : 1u;  // 1 = gave up as designed
}
}  // namespace

// No counterpart in the reference (whose mbarrier waits are unbounded).  Runs the timed-out
// path of the wait every tcgen05 kernel here is built on: returns 0 when the wait gave up after
// about budget_us microseconds (1..100000) and the kernel exited normally; pdk_device_error()
// then reads (kErrTestWait << 8 | 7).  `scratch` is 4 bytes of device memory.  Synchronizes.
PDK_EXPORT int pdk_selftest_bounded_wait(uint32_t budget_us, void* scratch, void* stream) {
    if (budget_us == 0 || budget_us > 100000u || scratch == nullptr) return cudaErrorInvalidValue;
    auto st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(scratch, 0, 4, st);
    if (e != cudaSuccess) return (int)e;
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>((unsigned long long)budget_us * 1000ull, pdk_error_word(),
                                                   (unsigned int*)scratch);
    if (int rc = pdk_launch_status()) return rc;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    unsigned int done = 0;
    e = cudaMemcpy(&done, scratch, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    return done == 1u ? 0 : (int)cudaErrorUnknown;
}
