// fp8_gemm.cu - row-scaled e4m3 prefill GEMM on tcgen05.
//
//   y[t][n] = ( sum_k e4m3(Xq[t][k]) * e4m3(W[n][k]) ) * xs[t] * ws[n]
//
// Compute-bound (2*M*N*K flops against M*K + N*K + M*N bytes).  One persistent
// CTA per SM, warp-specialized:
//   warp 0      TMA producer: 128-byte-swizzled boxes of Xq (128 tokens x 128 K
//               bytes) and W (256 channels x 128 K bytes) into a 4-stage ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::f8f6f4
//               (M=128 tokens, N=256 channels, K=32 per instruction), f32
//               accumulators in tensor memory, two 256-column buffers so the
//               next tile's MMAs run under this tile's epilogue
//   warps 2..5  epilogue: tcgen05.ld 32 columns at a time, scale by xs[t]*ws[n],
//               store f32 or bf16; a lane owns one token row, so every store is a
//               contiguous run of that row
// Tokens are the MMA's M dimension because y is token-major.  Tiles are walked
// token-tile fastest so the CTAs of a wave share a few W tiles through L2.
// Scales touch only the epilogue: the accumulation is the exact product sum.
#include <cstdlib>

#include "tc5.cuh"

// fp8_gemm2.cu: the same GEMM on pairs of SMs
int pdk_f8row_gemm_pair_f32(const void*, const void*, const void*, const void*, void*, uint32_t, uint32_t, uint32_t, cudaStream_t);
int pdk_f8row_gemm_pair_bf16(const void*, const void*, const void*, const void*, void*, uint32_t, uint32_t, uint32_t, cudaStream_t);

namespace {

constexpr uint32_t BM = 128, BN = 256, BK = 128;  // BK in bytes = e4m3 elements
constexpr uint32_t kStages = 4;
constexpr uint32_t kABytes = BM * BK, kBBytes = BN * BK, kStageBytes = kABytes + kBBytes;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kTmemCols = 512;

struct Shared {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

template <typename TO>
__device__ __forceinline__ void store_chunk(TO* dst, const float (&v)[32], uint32_t valid);

template <>
__device__ __forceinline__ void store_chunk<float>(float* dst, const float (&v)[32], uint32_t valid) {
    if (valid == 32u && (((uintptr_t)dst) & 15u) == 0u) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if ((uint32_t)i < valid) dst[i] = v[i];
    }
}

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], uint32_t valid) {
    if (valid == 32u && (((uintptr_t)dst) & 15u) == 0u) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 w;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
            w.x = *reinterpret_cast<uint32_t*>(&p0);
            w.y = *reinterpret_cast<uint32_t*>(&p1);
            w.z = *reinterpret_cast<uint32_t*>(&p2);
            w.w = *reinterpret_cast<uint32_t*>(&p3);
            reinterpret_cast<uint4*>(dst)[i] = w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if ((uint32_t)i < valid) dst[i] = __float2bfloat16_rn(v[i]);
    }
}

template <typename TO>
__global__ void __launch_bounds__(kThreads, 1)
f8row_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                  const float* __restrict__ w_scale, const float* __restrict__ x_scale, TO* __restrict__ y,
                  uint32_t in_dim, uint32_t out_dim, uint32_t batch, unsigned int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * kStageBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_m = (batch + BM - 1u) / BM, tiles_n = (out_dim + BN - 1u) / BN;
    const uint32_t n_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (in_dim + BK - 1u) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], 1);
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 4);
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_x);
        tc5::tma_prefetch_desc(&tmap_w);
    }
    if (warp == 1) {
        tc5::tmem_alloc(&sh->tmem_base, kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, err_word};
    pdk_pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (whole warp, one lane issues)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        // The weights depend on nothing the previous kernel in the stream writes: the first
        // tile's first stages take their weight box before the wait for that kernel.
        auto issue_w = [&](uint32_t stg, uint32_t n0, uint32_t kb) {
            uint8_t* a = tiles + stg * kStageBytes;
            tc5::mbar_arrive_expect_tx_elect(&sh->full[stg], kStageBytes);
            tc5::tma_load_2d_elect(a + kABytes, &tmap_w, &sh->full[stg], (int32_t)(kb * BK), (int32_t)n0);
        };
        uint32_t pre = 0;
        if (blockIdx.x < n_tiles) {
            pre = min(num_kb, kStages);
            for (uint32_t i = 0; i < pre; ++i) issue_w(i, (blockIdx.x / tiles_m) * BN, i);
        }
        pdk_pdl_wait();
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const uint32_t m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const bool early = tile == blockIdx.x && kb < pre;
                if (!early) {
                    ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    issue_w(stage, n0, kb);
                }
                tc5::tma_load_2d_elect(tiles + stage * kStageBytes, &tmap_x, &sh->full[stage], (int32_t)(kb * BK),
                                       (int32_t)m0);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) {
            // copies already issued still land in this CTA's shared memory: give
            // them time before the CTA may exit
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        constexpr uint32_t idesc = tc5::idesc_f32acc(0u, 0u, BM, BN);
        uint32_t stage = 0, phase = 0, iter = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            ok = tc5::mbar_wait(&sh->tmem_empty[buf], aphase ^ 1u, ctx, tc5::kErrTmemEmptyWait, buf);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc5::fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                ok = tc5::mbar_wait(&sh->full[stage], phase, ctx, tc5::kErrFullWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc5::fence_after_sync();
                const uint32_t a_addr = tc5::smem_u32(tiles + stage * kStageBytes);
                const uint64_t a_desc = tc5::smem_desc_sw128(a_addr);
                const uint64_t b_desc = tc5::smem_desc_sw128(a_addr + kABytes);
                static_assert(BK == 128u, "one group of four 32-byte K steps per stage");
                tc5::mma_f8f6f4_x4_elect(d_tmem, a_desc, b_desc, idesc, kb != 0u);
                tc5::mma_commit_elect(&sh->empty[stage]);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) tc5::mma_commit_elect(&sh->tmem_full[buf]);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
        uint32_t iter = 0;
        bool ok = true;
        pdk_pdl_wait();  // scales and y may still be in use by the previous kernel
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            const uint32_t m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            ok = tc5::mbar_wait(&sh->tmem_full[buf], aphase, ctx, tc5::kErrTmemFullWait, buf);
            if (!ok) break;
            tc5::fence_after_sync();
            const uint32_t t = m0 + quarter * 32u + lane;
            const float xs = t < batch ? x_scale[t] : 0.0f;
            TO* yrow = y + (size_t)t * out_dim + n0;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32u; ++c) {
                uint32_t r[32];
                tc5::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + buf * BN + c * 32u, r);
                tc5::tmem_ld_wait();
                const uint32_t nc = n0 + c * 32u;
                if (nc < out_dim && t < batch) {
                    const uint32_t valid = min(32u, out_dim - nc);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float ws = (uint32_t)i < valid ? __ldg(w_scale + nc + i) : 0.0f;
                        v[i] = __uint_as_float(r[i]) * (xs * ws);
                    }
                    store_chunk<TO>(yrow + c * 32u, v, valid);
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(&sh->tmem_empty[buf]);
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// PDK_F8_PAIR=0 keeps every call on the one-SM kernel (A/B switch, read once).
bool pair_enabled() {
    static const bool v = [] {
        const char* e = getenv("PDK_F8_PAIR");
        return !(e && e[0] == '0');
    }();
    return v;
}

template <typename TO>
int launch(const void* data, const void* w_scale, const void* xq, const void* x_scale, void* y, uint32_t in_dim,
           uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    if (out_dim == 0 || batch == 0) return 0;
    if (in_dim == 0 || (in_dim & 15u) != 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(xq, 16) || !pdk_aligned(w_scale, 4) || !pdk_aligned(x_scale, 4) ||
        !pdk_aligned(y, sizeof(TO)))
        return cudaErrorInvalidValue;
    // prefill widths: 256-token tiles on pairs of SMs (fp8_gemm2.cu), when there are enough of them to
    // give every pair work
    if (pair_enabled() && batch > BM &&
        (uint64_t)((batch + 2u * BM - 1u) / (2u * BM)) * ((out_dim + BN - 1u) / BN) >= (uint64_t)pdk_sm_count() / 2u) {
        if constexpr (sizeof(TO) == 4) return pdk_f8row_gemm_pair_f32(data, w_scale, xq, x_scale, y, in_dim, out_dim, batch, st);
        else return pdk_f8row_gemm_pair_bf16(data, w_scale, xq, x_scale, y, in_dim, out_dim, batch, st);
    }
    CUtensorMap tx, tw;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, in_dim, batch, in_dim, BK, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, in_dim, out_dim, in_dim, BK, BN))
        return rc;
    const size_t smem = (size_t)kStages * kStageBytes + sizeof(Shared) + 1024u;
    auto kern = f8row_gemm_kernel<TO>;
    static const cudaError_t attr_rc =  // once per process; one caller thread by the pack's contract
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr_rc != cudaSuccess) return (int)attr_rc;
    const uint32_t n_tiles = ((batch + BM - 1u) / BM) * ((out_dim + BN - 1u) / BN);
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_tiles) grid = n_tiles;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, tx, tw, (const float*)w_scale,
                          (const float*)x_scale, (TO*)y, in_dim, out_dim, batch, pdk_error_word());
}

}  // namespace

// slot 184, packs/cuda/src/gemm/dense_f8_decode.cuh:4638-4722: f32 output
PDK_EXPORT int pd_f8row_gemm(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale,
                             void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream) {
    return launch<float>(data, w_rowscale, xq, x_rowscale, y, in_dim, out_dim, batch, (cudaStream_t)stream);
}

// slot 855, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:1480-1515: same contract
PDK_EXPORT int pd_f8row_gemm_tc5x(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale,
                                  void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream) {
    return launch<float>(data, w_rowscale, xq, x_rowscale, y, in_dim, out_dim, batch, (cudaStream_t)stream);
}

// No slot: the same GEMM with bf16 output (halves the store traffic of a prefill)
PDK_EXPORT int pdk_f8row_gemm_bf16(const void* data, const void* w_rowscale, const void* xq, const void* x_rowscale,
                                   void* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, void* stream) {
    return launch<__nv_bfloat16>(data, w_rowscale, xq, x_rowscale, y, in_dim, out_dim, batch, (cudaStream_t)stream);
}
