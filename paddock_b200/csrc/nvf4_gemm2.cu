// nvf4_gemm2.cu - the NVFP4 x NVFP4 prefill GEMM of nvf4_gemm.cu on pairs of SMs.
//
// At prefill widths the one-SM kernel is paced by its L2 feed: 36 KB per 256-element K slab
// (128 weight rows, 128 tokens, two 2 KB scale records) for four MMAs, and L2 delivers about
// 116 GB/s to one SM.  Two CTAs of a cluster share a tile of 256 weight rows x 128 tokens
// (tcgen05 cta_group::2): each loads its own 128 weight rows and their scale record, HALF of the
// token tile's data, and the whole token tile's scale record (every tensor core needs all 128
// tokens' scales) - 28 KB per slab - and the leader's instructions drive both tensor cores and
// both CTAs' scale-cell copies.
//
//   CTA r of a pair (r = rank in the cluster, 0 leads):
//   warp 0      producer: four tiled TMA copies per slab (W box, X half box, two scale records
//               as [8 rows][256 bytes] boxes), all counted on the LEADER's full barrier
//   warp 1      leader only: per slab one asm block of 8 tcgen05.cp + 4 tcgen05.mma, cta_group::2;
//               commits arrive on both CTAs' barriers
//   warps 2..5  epilogue of the CTA's own 128 channels x 128 tokens
// The activation scales come pre-tiled (pd_nvf4_tc5_tile_scales over xs).  No multicast loads;
// every wait is bounded.
#include "nvf4_tc5.cuh"

namespace {

using namespace nvf4tc5;
using namespace tc5::pair;

constexpr uint32_t BN = 128;                       // tokens per pair tile
constexpr uint32_t BNH = 64;                       // tokens whose data one CTA loads
constexpr uint32_t kBHalf = BNH * BKB;             // 8 KB
constexpr uint32_t kSlab = kABytes + kBHalf + 2u * kSfBytes;   // 28 KB per CTA and slab
constexpr uint32_t kStagesP = 3;
// a stage = KS slabs: [W boxes][X half boxes][W scale records][X scale records]
constexpr uint32_t kOffB = KS * kABytes, kOffSfa = kOffB + KS * kBHalf, kOffSfb = kOffSfa + KS * kSfBytes;
constexpr uint32_t kStageBytes = kOffSfb + KS * kSfBytes;
static_assert(kStageBytes == KS * kSlab, "stage layout");
constexpr uint32_t kSfCol0 = 2u * BN, kSfCols = KS * 32u;
// e2m1 x e2m1, UE4M3 scales, M = 256 over the pair
constexpr uint32_t kIdescPair = (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | (((2u * BM) >> 4) << 24);

// slab_nvf4 (nvf4_tc5.cuh) for a pair of CTAs: the copies and the MMAs act in both
__device__ __forceinline__ void slab_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t acc_first, uint32_t sfa_t, uint32_t sfb_t, uint32_t sfa_smem,
                                               uint32_t sfb_smem, uint32_t steps) {
    const uint64_t cell_a = (uint64_t)((sfa_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    const uint64_t cell_b = (uint64_t)((sfb_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
#define PDK_NV4_STEP2(J, PRED)                                                                                        \
    "setp.gt.and.u32 ej, %9, " #J ", e;\n\t"                                                                          \
    "add.u64 a, %1, " #J "*2;\n\tadd.u64 b, %2, " #J "*2;\n\tadd.u32 sa, %5, " #J "*4;\n\tadd.u32 sb, %6, " #J "*4;\n\t" \
    "add.u64 ca, %7, " #J "*32;\n\tadd.u64 cb, %8, " #J "*32;\n\t"                                                    \
    "@ej tcgen05.cp.cta_group::2.32x128b.warpx4 [sa], ca;\n\t@ej tcgen05.cp.cta_group::2.32x128b.warpx4 [sb], cb;\n\t" \
    "@ej tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], a, b, %3, [sa], [sb], " PRED ";\n\t"
    asm volatile(
        "{\n\t.reg .pred e, p, q, ej;\n\t.reg .b64 a, b, ca, cb;\n\t.reg .b32 sa, sb;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        PDK_NV4_STEP2(0, "p") PDK_NV4_STEP2(1, "q") PDK_NV4_STEP2(2, "q") PDK_NV4_STEP2(3, "q") "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first), "r"(sfa_t), "r"(sfb_t), "l"(cell_a), "l"(cell_b), "r"(steps)
        : "memory");
#undef PDK_NV4_STEP2
}

template <typename TO>
__device__ __forceinline__ void store_one2(TO* p, float v);
template <>
__device__ __forceinline__ void store_one2<float>(float* p, float v) { __stcs(p, v); }
template <>
__device__ __forceinline__ void store_one2<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    __stcs(reinterpret_cast<unsigned short*>(p), __bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
template <typename TO>
__device__ __forceinline__ void store_smem2(TO* p, float v);
template <>
__device__ __forceinline__ void store_smem2<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_smem2<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TO>
__global__ void __launch_bounds__(kThreads, 1)
nvf4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_wsf, const __grid_constant__ CUtensorMap tmap_xsf,
                      const float* __restrict__ bias, TO* __restrict__ y, float scale2, uint32_t in_dim, uint32_t out_dim,
                      uint32_t batch, unsigned int* err_word, const __grid_constant__ CUtensorMap tmap_y,
                      const uint32_t tma_out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStagesP * kStageBytes);
    TO* stage_out = reinterpret_cast<TO*>(tiles + kStagesP * kStageBytes + 128u);   // [32 tokens][128 channels]
    static_assert(sizeof(Shared) <= 128u, "control block");

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0u;
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t tiles_w = (out_dim + 2u * BM - 1u) / (2u * BM), tiles_t = (batch + BN - 1u) / BN;
    const uint32_t n_tiles = tiles_w * tiles_t;
    const uint32_t num_kb = in_dim >> 8;
    const uint32_t num_ks = (num_kb + KS - 1u) / KS;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStagesP; ++s) {
            tc5::mbar_init(&sh->full[s], 1);
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 8);   // in the leader: 4 epilogue warps of each CTA
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_w);
        tc5::tma_prefetch_desc(&tmap_x);
        tc5::tma_prefetch_desc(&tmap_wsf);
        tc5::tma_prefetch_desc(&tmap_xsf);
    }
    if (warp == 1) {
        tmem_alloc2(&sh->tmem_base, kTmemCols);
        tmem_relinquish2();
    }
    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, err_word};
    pdk_pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        pdk_pdl_wait();
        for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
            // token tile fastest: the pairs of a wave share a few weight tiles
            const uint32_t tile_w = (tile / tiles_t) * 2u + rank, tile_t = tile % tiles_t;
            for (uint32_t ks = 0; ks < num_ks; ++ks) {
                ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* a = tiles + stage * kStageBytes;
                const uint32_t kb0 = ks * KS, nsl = min(KS, num_kb - kb0);
                // the scale boxes always span KS records (rows past the plane read as zero and count)
                if (leader) tc5::mbar_arrive_expect_tx_elect(&sh->full[stage], 2u * (nsl * (kABytes + kBHalf) + 2u * KS * kSfBytes));
#pragma unroll
                for (uint32_t u = 0; u < KS; ++u)
                    if (u < nsl) {
                        tma_load_2d_pair_elect(a + u * kABytes, &tmap_w, &sh->full[stage], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(tile_w * BM));
                        tma_load_2d_pair_elect(a + kOffB + u * kBHalf, &tmap_x, &sh->full[stage], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(tile_t * BN + rank * BNH));
                    }
                tma_load_2d_pair_elect(a + kOffSfa, &tmap_wsf, &sh->full[stage], 0, (int32_t)((tile_w * num_kb + kb0) * 8u));
                tma_load_2d_pair_elect(a + kOffSfb, &tmap_xsf, &sh->full[stage], 0, (int32_t)((tile_t * num_kb + kb0) * 8u));
                if (++stage == kStagesP) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) {
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (leader) {
            // -------------------------------------------------------- MMA issuer (leader)
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++iter) {
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
                    const uint32_t a_addr = tc5::smem_u32(tiles + stage * kStageBytes);
                    const uint32_t nsl = min(KS, num_kb - ks * KS);
#pragma unroll
                    for (uint32_t u = 0; u < KS; ++u) {
                        if (u >= nsl) break;
                        const uint32_t sfa_t = tmem_base + kSfCol0 + stage * kSfCols + u * 32u, sfb_t = sfa_t + 16u;
                        slab_nvf4_pair(d_tmem, tc5::smem_desc_sw128(a_addr + u * kABytes),
                                       tc5::smem_desc_sw128(a_addr + kOffB + u * kBHalf), kIdescPair, (ks | u) != 0u, sfa_t, sfb_t,
                                       a_addr + kOffSfa + u * kSfBytes, a_addr + kOffSfb + u * kSfBytes, 4u);
                    }
                    mma_commit_pair_elect(&sh->empty[stage]);
                    if (++stage == kStagesP) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit_pair_elect(&sh->tmem_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 channels)
        const uint32_t quarter = warp & 3u;
        uint32_t iter = 0;
        bool ok = true;
        pdk_pdl_wait();
        for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            const uint32_t w0 = ((tile / tiles_t) * 2u + rank) * BM, t0 = (tile % tiles_t) * BN;
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
                    if (threadIdx.x == 64u) tc5::tma_store_wait_read();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                    for (uint32_t i = 0; i < 32u; ++i)
                        store_smem2<TO>(stage_out + i * BM + quarter * 32u + lane, fmaf(__uint_as_float(r[i]), scale2, b));
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (threadIdx.x == 64u && w0 < out_dim) tc5::tma_store_2d(&tmap_y, stage_out, (int32_t)w0, (int32_t)(t0 + c * 32u));
                    continue;
                }
                if (n < out_dim) {
#pragma unroll
                    for (uint32_t i = 0; i < 32u; ++i) {
                        const uint32_t t = c * 32u + i;
                        if (t < n_tok) store_one2<TO>(y + (size_t)(t0 + t) * out_dim + n, fmaf(__uint_as_float(r[i]), scale2, b));
                    }
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&sh->tmem_empty[buf]);
        }
    }

    if (tma_out && threadIdx.x == 64u) tc5::tma_store_wait_all();
    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc5::fence_after_sync();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}

template <typename TO>
int launch_pair(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled, void* y,
                float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    CUtensorMap tw, tx, twsf, txsf;
    const uint32_t kbytes = in_dim >> 1, num_kb = in_dim >> 8;
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, kbytes, out_dim, kbytes, BKB, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, kbytes, batch, kbytes, BKB, BNH)) return rc;
    // scale records (2048 bytes each) as rows of 256 bytes, eight per record; a box spans KS records
    const uint64_t w_recs = (uint64_t)((out_dim + BM - 1u) / BM) * num_kb, x_recs = (uint64_t)((batch + BN - 1u) / BN) * num_kb;
    if (int rc = pdk_make_tmap_2d_dense(&twsf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale_tiled, 256u, w_recs * 8u, 256u, 256u, 8u * KS))
        return rc;
    if (int rc = pdk_make_tmap_2d_dense(&txsf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xs_tiled, 256u, x_recs * 8u, 256u, 256u, 8u * KS))
        return rc;
    CUtensorMap ty = tw;
    uint32_t tma_out = 0u;
    if (sizeof(TO) == 2u && pdk_aligned(y, 16) && (out_dim & 7u) == 0u &&
        pdk_make_tmap_2d_dense(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, out_dim, batch, (uint64_t)out_dim * 2u, BM, 32u) == 0)
        tma_out = 1u;
    const size_t smem = (size_t)kStagesP * kStageBytes + 128u + 32u * BM * sizeof(TO) + 1024u;
    auto kern = nvf4_gemm_pair_kernel<TO>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = ((out_dim + 2u * BM - 1u) / (2u * BM)) * ((batch + BN - 1u) / BN);
    uint32_t pairs = (uint32_t)pdk_sm_count() / 2u;
    if (pairs > n_tiles) pairs = n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdk_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    e = cudaLaunchKernelEx(&cfg, kern, tw, tx, twsf, txsf, (const float*)bias, (TO*)y, scale2, in_dim, out_dim, batch,
                           pdk_error_word(), ty, tma_out);
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}

}  // namespace

// Prefill widths on pairs of SMs; xs_tiled = the activation scales in the weight scales' record
// layout (one record per 128 tokens and slab).
int pdk_nvf4_gemm_pair_f32(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled,
                           void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair<float>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
}
int pdk_nvf4_gemm_pair_bf16(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled,
                            void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair<__nv_bfloat16>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
}
