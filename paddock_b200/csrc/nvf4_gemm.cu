// nvf4_gemm.cu - NVFP4 x NVFP4 GEMM on tcgen05 with hardware block scaling.
//
//   y[t][n] = scale2 * sum over 16-element blocks b of
//             e4m3(ws[n][b]) * e4m3(xs[t][b]) * sum_{k in b} e2m1(W[n][k]) * e2m1(X[t][k])   (+ bias[n])
//
// tcgen05.mma kind::mxf4nvf4 reads packed e2m1 operands straight from shared
// memory (K = 64 per instruction) and applies both operands' per-16 UE4M3
// scales from tensor memory, so no weight ever passes through a register: at
// decode widths the kernel is a pure HBM stream (4.5 bits per weight), at
// prefill widths it is tensor-bound.
//
// Tile: 128 weight rows (the MMA's M, one TMEM lane each) x 128 tokens (N); K
// in slabs of 256, two slabs per pipeline stage.  Weights are the A operand so that a decode batch
// is a single token tile and the epilogue writes, per token, 128 consecutive
// channels.  One persistent CTA per SM:
//   warp 0      producer: TMA boxes of W and X (128 rows x 128 bytes, 128-byte
//               swizzle), one 2 KB bulk copy of the pre-tiled weight scale cells,
//               and a 32-lane cp.async gather of the activation scale cells into
//               the same cell order, arriving on the stage barrier asynchronously
//   warp 1      MMA issuer (converged warp, one elected lane): per slab 8 tcgen05.cp
//               (scale cells -> TMEM) + 4 MMAs, one commit per stage
//   warps 2..5  epilogue: TMEM -> registers -> y (f32 or bf16), * scale2 + bias
// Accumulators are double buffered (2 x 128 TMEM columns); scale cells take
// 32 columns per slab.
#include <cstdlib>

#include "nvf4_tc5.cuh"

// nvf4_gemm2.cu: prefill widths on pairs of SMs
int pdk_nvf4_gemm_pair_f32(const void*, const void*, const void*, const void*, const void*, void*, float, uint32_t, uint32_t,
                           uint32_t, cudaStream_t);
int pdk_nvf4_gemm_pair_bf16(const void*, const void*, const void*, const void*, const void*, void*, float, uint32_t, uint32_t,
                            uint32_t, cudaStream_t);

namespace {

using namespace nvf4tc5;

// PDK_NVF4_PAIR=0 keeps every call on the one-SM kernel (A/B switch, read once).
bool pair_enabled() {
    static const bool v = [] {
        const char* e = getenv("PDK_NVF4_PAIR");
        return !(e && e[0] == '0');
    }();
    return v;
}

template <typename TO>
__device__ __forceinline__ void store_one(TO* p, float v);
template <>
__device__ __forceinline__ void store_one<float>(float* p, float v) { __stcs(p, v); }  // streaming: written once
template <>
__device__ __forceinline__ void store_one<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    __stcs(reinterpret_cast<unsigned short*>(p), __bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
template <typename TO>
__device__ __forceinline__ void store_one_smem(TO* p, float v);
template <>
__device__ __forceinline__ void store_one_smem<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_one_smem<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// XT: the activation scales come pre-tiled (the weight scales' record layout, one record
// per 128 tokens and slab) and are bulk-copied; otherwise they are row-major and gathered.
template <uint32_t BN, typename TO, bool XT>
__global__ void __launch_bounds__(kThreads, 1)
nvf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const uint8_t* __restrict__ w_sf_tiled, const uint8_t* __restrict__ x_sf,
                 const float* __restrict__ bias, TO* __restrict__ y, float scale2, uint32_t in_dim, uint32_t out_dim,
                 uint32_t batch, unsigned int* err_word, const __grid_constant__ CUtensorMap tmap_y,
                 const uint32_t tma_out) {
    constexpr uint32_t kStages = Cfg<BN>::kStages, kBBytes = Cfg<BN>::kBBytes, kStageBytes = Cfg<BN>::kStageBytes;
    constexpr uint32_t kSfCol0 = Cfg<BN>::kSfCol0, kIdesc = Cfg<BN>::kIdesc, kSfCols = Cfg<BN>::kSfCols;
    constexpr uint32_t kOffB = Cfg<BN>::kOffB, kOffSfa = Cfg<BN>::kOffSfa, kOffSfb = Cfg<BN>::kOffSfb;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * kStageBytes);
    // tma_out: output staging [32 tokens][128 channels] behind the control block (16-byte aligned)
    TO* stage_out = reinterpret_cast<TO*>(tiles + kStages * kStageBytes + 128u);
    static_assert(sizeof(Shared) <= 128u, "control block");

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_w = (out_dim + BM - 1u) / BM, tiles_t = (batch + BN - 1u) / BN;
    const uint32_t n_tiles = tiles_w * tiles_t;
    const uint32_t num_kb = in_dim >> 8;       // 256-element slabs (in_dim % 256 == 0)
    const uint32_t num_ks = (num_kb + KS - 1u) / KS;  // stages per tile; the last may hold fewer slabs
    const uint32_t sf_row = in_dim >> 4;       // activation scale bytes per token

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], XT ? 1 : 33);  // expect_tx arrival (+ 32 lanes' cp.async arrivals)
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 4);
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_w);
        tc5::tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        tc5::tmem_alloc(&sh->tmem_base, kTmemCols);
        tc5::tmem_relinquish();
    }
    // activation scale cells: the gather writes only the rows a token tile has; the rest stay zero
    for (uint32_t i = threadIdx.x; i < kStages * (KS * kSfBytes / 16u); i += kThreads) {
        const uint32_t s = i / (KS * kSfBytes / 16u), o = i % (KS * kSfBytes / 16u);
        reinterpret_cast<uint4*>(tiles + s * kStageBytes + kOffSfb)[o] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, err_word};
    pdk_pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ producer (whole warp)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        // Activation scale cells of one stage: word (j, l, c) of the 2 KB record is
        // xs[t0 + c*32 + l][kb*16 + 4j .. 4j+3].  Each lane issues its words as 4-byte
        // cp.async copies (zero-filled past the batch) and then an asynchronous arrive on
        // the stage's barrier, so the producer never waits for a load.
        constexpr uint32_t kRowGroups = BN / 32u;  // this lane's rows: t0 + c*32 + lane, c < BN/32
        const uint8_t* sf_src[kRowGroups];          // row base of the current token tile
        uint32_t sf_size[kRowGroups];               // 4, or 0 past the batch (zero fill)
        auto set_sf_rows = [&](uint32_t t0) {
#pragma unroll
            for (uint32_t c = 0; c < kRowGroups; ++c) {
                const uint32_t t = t0 + c * 32u + lane;
                sf_src[c] = x_sf + (size_t)min(t, batch - 1u) * sf_row;
                sf_size[c] = t < batch ? 4u : 0u;
            }
        };
        auto gather_sf = [&](uint8_t* sfb, uint64_t* bar, uint32_t kb0, uint32_t nsl) {
            const uint32_t dst0 = tc5::smem_u32(sfb) + lane * 16u;
#pragma unroll
            for (uint32_t u = 0; u < KS; ++u)
                if (u < nsl)
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j)
#pragma unroll
                        for (uint32_t c = 0; c < kRowGroups; ++c)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst0 + u * kSfBytes +
                                                                                            j * 512u + c * 4u),
                                         "l"(sf_src[c] + (kb0 + u) * 16u + j * 4u), "r"(sf_size[c])
                                         : "memory");
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(tc5::smem_u32(bar)) : "memory");
        };
        // weight half of a stage: the expected bytes of the whole stage, the W boxes and their
        // scale records (consecutive slabs' records are contiguous: one bulk copy)
        const uint64_t stream_once = tc5::l2_policy_evict_first();
        auto issue_w = [&](uint32_t stg, uint32_t tile_w, uint32_t ks) {
            uint8_t* a = tiles + stg * kStageBytes;
            const uint32_t kb0 = ks * KS, nsl = min(KS, num_kb - kb0);
            tc5::mbar_arrive_expect_tx_elect(&sh->full[stg], nsl * (kABytes + kBBytes + kSfBytes + (XT ? kSfBytes : 0u)));
#pragma unroll
            for (uint32_t u = 0; u < KS; ++u)
                if (u < nsl) {
                    // decode widths have one token tile: a weight box is read once per launch and need not stay in L2
                    if constexpr (BN < 128u)
                        tc5::tma_load_2d_hint_elect(a + u * kABytes, &tmap_w, &sh->full[stg], (int32_t)((kb0 + u) * BKB),
                                                    (int32_t)(tile_w * BM), stream_once);
                    else
                        tc5::tma_load_2d_elect(a + u * kABytes, &tmap_w, &sh->full[stg], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(tile_w * BM));
                }
            tc5::bulk_load_elect(a + kOffSfa, w_sf_tiled + ((size_t)tile_w * num_kb + kb0) * kSfBytes, nsl * kSfBytes,
                                 &sh->full[stg]);
        };
        // The weights depend on nothing the previous kernel in the stream writes: the first
        // tile's first stages stream in before the wait for that kernel; activations after it.
        uint32_t pre = 0;
        if (blockIdx.x < n_tiles) {
            pre = min(num_ks, kStages);
            for (uint32_t i = 0; i < pre; ++i) issue_w(i, blockIdx.x / tiles_t, i);
        }
        pdk_pdl_wait();
        // Tiles are walked token-tile fastest: the CTAs of a wave share a few weight tiles
        // across all token tiles, so a weight tile streams from DRAM once while the small
        // activation plane stays in L2.  (Weight-tile fastest re-read the whole weight
        // plane once per token tile under the output stream's L2 churn.)
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const uint32_t tile_w = tile / tiles_t, t0 = (tile % tiles_t) * BN;
            if (!XT) set_sf_rows(t0);
            for (uint32_t ks = 0; ks < num_ks; ++ks) {
                const bool early = tile == blockIdx.x && ks < pre;  // first use of the stage, W already issued
                if (!early) {
                    ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    issue_w(stage, tile_w, ks);
                }
                uint8_t* a = tiles + stage * kStageBytes;
                const uint32_t kb0 = ks * KS, nsl = min(KS, num_kb - kb0);
#pragma unroll
                for (uint32_t u = 0; u < KS; ++u)
                    if (u < nsl)
                        tc5::tma_load_2d_elect(a + kOffB + u * kBBytes, &tmap_x, &sh->full[stage],
                                               (int32_t)((kb0 + u) * BKB), (int32_t)t0);
                if (XT)
                    tc5::bulk_load_elect(a + kOffSfb, x_sf + ((size_t)(tile % tiles_t) * num_kb + kb0) * kSfBytes,
                                         nsl * kSfBytes, &sh->full[stage]);
                else
                    gather_sf(a + kOffSfb, &sh->full[stage], kb0, nsl);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) {
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        uint32_t stage = 0, phase = 0, iter = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            ok = tc5::mbar_wait(&sh->tmem_empty[buf], aphase ^ 1u, ctx, tc5::kErrTmemEmptyWait, buf);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc5::fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t ks = 0; ks < num_ks; ++ks) {
                ok = tc5::mbar_wait(&sh->full[stage], phase, ctx, tc5::kErrFullWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc5::fence_after_sync();
                if (!XT) fence_proxy_async_smem();  // the gathered cells were written through the generic proxy
                const uint32_t a_addr = tc5::smem_u32(tiles + stage * kStageBytes);
                const uint32_t nsl = min(KS, num_kb - ks * KS);
#pragma unroll
                for (uint32_t u = 0; u < KS; ++u) {
                    if (u >= nsl) break;
                    const uint32_t sfa_addr = a_addr + kOffSfa + u * kSfBytes, sfb_addr = a_addr + kOffSfb + u * kSfBytes;
                    const uint32_t sfa_t = tmem_base + kSfCol0 + stage * kSfCols + u * 32u, sfb_t = sfa_t + 16u;
                    const uint64_t a_desc = tc5::smem_desc_sw128(a_addr + u * kABytes);
                    const uint64_t b_desc = tc5::smem_desc_sw128(a_addr + kOffB + u * kBBytes);
                    // four MMAs of 64 e2m1 (32 bytes of K) each, the two scale-cell copies of each in front of it
                    slab_nvf4<true>(d_tmem, a_desc, b_desc, kIdesc, (ks | u) != 0u, sfa_t, sfb_t, sfa_addr, sfb_addr, 4u);
                }
                tc5::mma_commit_elect(&sh->empty[stage]);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) tc5::mma_commit_elect(&sh->tmem_full[buf]);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quarter = warp & 3u;
        uint32_t iter = 0;
        bool ok = true;
        pdk_pdl_wait();  // y and bias may still be in use by the previous kernel
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            const uint32_t w0 = (tile / tiles_t) * BM, t0 = (tile % tiles_t) * BN;
            ok = tc5::mbar_wait(&sh->tmem_full[buf], aphase, ctx, tc5::kErrTmemFullWait, buf);
            if (!ok) break;
            tc5::fence_after_sync();
            const uint32_t n = w0 + quarter * 32u + lane;
            const float b = (bias != nullptr && n < out_dim) ? bias[n] : 0.0f;
            const uint32_t n_tok = min(BN, batch - t0);
#pragma unroll 1
            for (uint32_t c = 0; c * 32u < n_tok; ++c) {
                uint32_t r[32];
                tc5::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + buf * BN + c * 32u, r);
                tc5::tmem_ld_wait();
                if (tma_out) {
                    // the four epilogue warps fill a dense [32 tokens][128 channels] box, one thread
                    // stores it with TMA (whole lines; rows and channels past the end are clipped)
                    if (threadIdx.x == 64u) tc5::tma_store_wait_read();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                    for (uint32_t i = 0; i < 32u; ++i)
                        store_one_smem<TO>(stage_out + i * BM + quarter * 32u + lane,
                                           fmaf(__uint_as_float(r[i]), scale2, b));
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (threadIdx.x == 64u) tc5::tma_store_2d(&tmap_y, stage_out, (int32_t)w0, (int32_t)(t0 + c * 32u));
                    continue;
                }
                if (n < out_dim) {
#pragma unroll
                    for (uint32_t i = 0; i < 32u; ++i) {
                        const uint32_t t = c * 32u + i;
                        if (t < n_tok) store_one<TO>(y + (size_t)(t0 + t) * out_dim + n, fmaf(__uint_as_float(r[i]), scale2, b));
                    }
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(&sh->tmem_empty[buf]);
        }
    }

    if (tma_out && threadIdx.x == 64u) tc5::tma_store_wait_all();  // the staging box is read until then
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <uint32_t BN, typename TO, bool XT>
int launch_bn(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs, void* y,
              float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    CUtensorMap tw, tx;
    const uint32_t kbytes = in_dim >> 1;
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, kbytes, out_dim, kbytes, BKB, BM))
        return rc;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, kbytes, batch, kbytes, BKB, BN)) return rc;
    // bf16 outputs at prefill width leave through a staged TMA store (whole 256-byte rows)
    // when y qualifies for a tensor map; everything else stores from registers
    CUtensorMap ty = tw;
    uint32_t tma_out = 0u;
    if (BN == 128u && sizeof(TO) == 2u && pdk_aligned(y, 16) && (out_dim & 7u) == 0u &&
        pdk_make_tmap_2d_dense(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, out_dim, batch, (uint64_t)out_dim * 2u, BM,
                               32u) == 0)
        tma_out = 1u;
    const size_t smem = (size_t)Cfg<BN>::kStages * Cfg<BN>::kStageBytes + 128u + (BN == 128u ? 32u * BM * 2u : 0u) + 1024u;
    auto kern = nvf4_gemm_kernel<BN, TO, XT>;
    static const cudaError_t attr_rc =  // once per process; one caller thread by the pack's contract
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr_rc != cudaSuccess) return (int)attr_rc;
    const uint32_t n_tiles = ((out_dim + BM - 1u) / BM) * ((batch + BN - 1u) / BN);
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_tiles) grid = n_tiles;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, tw, tx, (const uint8_t*)scale_tiled,
                          (const uint8_t*)xs, (const float*)bias, (TO*)y, scale2, in_dim, out_dim, batch,
                          pdk_error_word(), ty, tma_out);
}

// Scratch for the re-tiled activation scales of prefill-width calls: a 4-byte gather per
// token row and 64 K-elements cost the L2 as many requests again as the operand boxes, one
// 2 KB bulk copy per slab does not.  The buffer lives in the library (the pack allocates
// nothing at run time); one slice per stream, for the first kXsfLanes streams that make
// such calls - further streams, and calls too large for a slice, use the gather.
constexpr size_t kXsfSliceBytes = 8u << 20;  // batch * in_dim / 16 bytes, padded to 128 tokens
constexpr int kXsfLanes = 2;
__device__ __align__(1024) uint8_t g_xsf_scratch[kXsfLanes][kXsfSliceBytes];

PDK_SLICE_TABLE(xsf_slice_table, g_xsf_scratch, kXsfSliceBytes, kXsfLanes);
uint8_t* xsf_slice(cudaStream_t st, size_t need) {
    if (need > kXsfSliceBytes) return nullptr;
    return xsf_slice_table.slice(st);
}

template <typename TO>
int launch(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs, void* y,
           float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    if (out_dim == 0 || batch == 0) return 0;
    if (in_dim == 0 || (in_dim & 255u) != 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(xq, 16) || !pdk_aligned(scale_tiled, 16) || !pdk_aligned(xs, 4) ||
        !pdk_aligned(y, sizeof(TO)))
        return cudaErrorInvalidValue;
    if (batch <= 32u)
        return launch_bn<32, TO, false>(data, scale_tiled, bias, xq, xs, y, scale2, in_dim, out_dim, batch, st);
    if (batch <= 64u)
        return launch_bn<64, TO, false>(data, scale_tiled, bias, xq, xs, y, scale2, in_dim, out_dim, batch, st);
    const size_t need = (size_t)((batch + 127u) / 128u) * (in_dim >> 8) * kSfBytes;
    if (uint8_t* xt = xsf_slice(st, need)) {
        if (int rc = pd_nvf4_tc5_tile_scales(xs, xt, in_dim, batch, st)) return rc;
        // enough 256-row x 128-token tiles to give every pair of SMs work: the pair kernel
        if (pair_enabled() &&
            (uint64_t)((out_dim + 2u * BM - 1u) / (2u * BM)) * ((batch + 127u) / 128u) >= (uint64_t)pdk_sm_count() / 2u) {
            if constexpr (sizeof(TO) == 4) return pdk_nvf4_gemm_pair_f32(data, scale_tiled, bias, xq, xt, y, scale2, in_dim, out_dim, batch, st);
            else return pdk_nvf4_gemm_pair_bf16(data, scale_tiled, bias, xq, xt, y, scale2, in_dim, out_dim, batch, st);
        }
        return launch_bn<128, TO, true>(data, scale_tiled, bias, xq, xt, y, scale2, in_dim, out_dim, batch, st);
    }
    return launch_bn<128, TO, false>(data, scale_tiled, bias, xq, xs, y, scale2, in_dim, out_dim, batch, st);
}

}  // namespace

// slot 852, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:1216-1263.  `part` / `part_floats`
// (the reference's K-split partial planes) are accepted and unused: this kernel
// never splits K.
PDK_EXPORT int pd_nvf4_gemm_tc5w(const void* data, const void* scale_tiled, const void* bias, const void* xq,
                                 const void* xs, void* y, float scale2, uint32_t in_dim, uint32_t out_dim,
                                 uint32_t batch, void* part, uint64_t part_floats, void* stream) {
    (void)part;
    (void)part_floats;
    return launch<float>(data, scale_tiled, bias, xq, xs, y, scale2, in_dim, out_dim, batch, (cudaStream_t)stream);
}

// No slot: slot 852 with bf16 output.
PDK_EXPORT int pdk_nvf4_gemm_bf16(const void* data, const void* scale_tiled, const void* bias, const void* xq,
                                  const void* xs, void* y, float scale2, uint32_t in_dim, uint32_t out_dim,
                                  uint32_t batch, void* stream) {
    return launch<__nv_bfloat16>(data, scale_tiled, bias, xq, xs, y, scale2, in_dim, out_dim, batch,
                                 (cudaStream_t)stream);
}
