// nvf4_gemm2.cu - the NVFP4 x NVFP4 prefill GEMM of nvf4_gemm.cu on pairs of SMs.
//
// At prefill widths this GEMM is bound by shared-memory bandwidth (128 bytes per cycle and SM),
// which every byte crosses twice or more: written once by TMA, read by the tensor core once per
// MMA that uses it, and a token box additionally by the partner SM's tensor core.  Two CTAs of a
// cluster share a tile of 256 weight rows x BN tokens (tcgen05 cta_group::2): each loads its own
// 128 weight rows and their scale record, HALF of the token tile's data, and the whole token
// tile's scale records (every tensor core needs all tokens' scales); the leader's instructions
// drive both tensor cores and both CTAs' scale-cell copies.  Per CTA and 256-element K slab:
//   BN = 128   28 KB written + 4 MMAs x (4 KB weights + 2 KB own tokens + 2 KB served to the
//              partner) read + 4 KB scale cells = 64 KB = 500 cycles for 256 tensor cycles
//              (measured: 505 per slab; stages of two slabs, two accumulators)
//   BN = 256   38 KB + 4 x (4 + 4 + 4) KB + 6 KB = 92 KB = 720 cycles for 512 tensor cycles
//              (stages of one slab; ONE accumulator, two would fill tensor memory and leave the
//              scale cells no room, so the tensor core idles from its last MMA of a tile until the
//              epilogue has the accumulator in registers: measured 875 per slab overall)
// The one-SM kernel of nvf4_gemm.cu (128 x 128, 36 KB written per slab) needs 560.
//
//   CTA r of a pair (r = rank in the cluster, 0 leads):
//   warp 0      producer: tiled TMA copies per slab (W box, X half box, the scale records as
//               [8 rows][256 bytes] boxes), all counted on the LEADER's full barrier
//   warp 1      leader only: per slab one asm block of the scale-cell copies + 4 tcgen05.mma,
//               cta_group::2; commits arrive on both CTAs' barriers
//   warps 2..9  epilogue of the CTA's own 128 channels x BN tokens, two warps per 32 channels
// The activation scales come pre-tiled (pd_nvf4_tc5_tile_scales over xs).  No multicast loads;
// every wait is bounded.
#include "nvf4_tc5.cuh"

namespace {

using namespace nvf4tc5;
using namespace tc5::pair;

template <uint32_t BN_>
struct PairCfg {
    static constexpr uint32_t BN = BN_;                  // tokens per pair tile
    static constexpr uint32_t BNH = BN / 2u;             // tokens whose data one CTA loads
    static constexpr uint32_t kRec = BN / 128u;          // token scale records per slab
    static constexpr uint32_t kSlabs = BN == 128u ? 2u : 1u;   // slabs per pipeline stage
    static constexpr uint32_t kStages = BN == 128u ? 3u : 4u;   // + the output tile: 200 / 216 KB
    static constexpr uint32_t kAcc = BN == 128u ? 2u : 1u;     // accumulators in tensor memory
    static constexpr uint32_t kBHalf = BNH * BKB;
    // a stage: [W boxes][X half boxes][W scale records][X scale records]
    static constexpr uint32_t kOffB = kSlabs * kABytes, kOffSfa = kOffB + kSlabs * kBHalf;
    static constexpr uint32_t kOffSfb = kOffSfa + kSlabs * kSfBytes;
    static constexpr uint32_t kStageBytes = kOffSfb + kSlabs * kRec * kSfBytes;
    // tensor-memory columns: the accumulators, then per stage and slab 4 steps x (4 + 4 * kRec) scale columns
    static constexpr uint32_t kSfCol0 = kAcc * BN, kSlabCols = 16u + 16u * kRec, kSfCols = kSlabs * kSlabCols;
    static_assert(kSfCol0 + kStages * kSfCols <= kTmemCols, "tensor memory");
    // e2m1 x e2m1, UE4M3 scales, M = 256 over the pair
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | (((2u * BM) >> 4) << 24);
};
constexpr uint32_t kMaxStagesP = 5;
constexpr uint32_t kThreadsP = 320;   // producer, issuer, 8 epilogue warps (two per lane quarter)

struct SharedP {
    uint64_t full[kMaxStagesP];
    uint64_t empty[kMaxStagesP];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

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

// The same for 256 tokens: the token scales are two records (tokens 0..127, 128..255), two cells of four
// columns side by side per step.
__device__ __forceinline__ void slab_nvf4_pair256(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t acc_first, uint32_t sfa_t, uint32_t sfb_t, uint32_t sfa_smem,
                                                  uint32_t sfb_smem) {
    const uint64_t cell_a = (uint64_t)((sfa_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    const uint64_t cell_b = (uint64_t)((sfb_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    const uint64_t cell_b2 = (uint64_t)(((sfb_smem + kSfBytes) >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
#define PDK_NV4_STEP3(J, PRED)                                                                                        \
    "add.u64 a, %1, " #J "*2;\n\tadd.u64 b, %2, " #J "*2;\n\tadd.u32 sa, %5, " #J "*4;\n\tadd.u32 sb, %6, " #J "*8;\n\t" \
    "add.u32 sc, sb, 4;\n\tadd.u64 ca, %7, " #J "*32;\n\tadd.u64 cb, %8, " #J "*32;\n\tadd.u64 cc, %9, " #J "*32;\n\t"   \
    "@e tcgen05.cp.cta_group::2.32x128b.warpx4 [sa], ca;\n\t@e tcgen05.cp.cta_group::2.32x128b.warpx4 [sb], cb;\n\t" \
    "@e tcgen05.cp.cta_group::2.32x128b.warpx4 [sc], cc;\n\t"                                                        \
    "@e tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], a, b, %3, [sa], [sb], " PRED ";\n\t"
    asm volatile(
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 a, b, ca, cb, cc;\n\t.reg .b32 sa, sb, sc;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        PDK_NV4_STEP3(0, "p") PDK_NV4_STEP3(1, "q") PDK_NV4_STEP3(2, "q") PDK_NV4_STEP3(3, "q") "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first), "r"(sfa_t), "r"(sfb_t), "l"(cell_a), "l"(cell_b), "l"(cell_b2)
        : "memory");
#undef PDK_NV4_STEP3
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

// A = the operand whose rows are the accumulator's lanes (256 per pair tile: the weights), B = the one whose
// rows are its columns (BN per pair tile: the tokens).  (Tokens as lanes, each epilogue thread writing 16-byte
// pieces of its token's row straight to global memory, measured 14 % slower at 8192 tokens.)
template <typename TO, uint32_t BN>
__global__ void __launch_bounds__(kThreadsP, 1)
nvf4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_wsf, const __grid_constant__ CUtensorMap tmap_xsf,
                      const float* __restrict__ bias, TO* __restrict__ y, float scale2, uint32_t in_dim, uint32_t a_rows,
                      uint32_t b_rows, unsigned int* err_word, const __grid_constant__ CUtensorMap tmap_y,
                      const uint32_t tma_out) {
    using C = PairCfg<BN>;
    constexpr uint32_t kSlabs = C::kSlabs, kStages = C::kStages, kStageBytes = C::kStageBytes, kAcc = C::kAcc;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    SharedP* sh = reinterpret_cast<SharedP*>(tiles + kStages * kStageBytes);
    uint8_t* stage_out = tiles + kStages * kStageBytes + 128u;   // [BN tokens][128 channels] bf16 (tensor-map output only)
    static_assert(sizeof(SharedP) <= 128u, "control block");

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0u;
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t tiles_a = (a_rows + 2u * BM - 1u) / (2u * BM), tiles_b = (b_rows + BN - 1u) / BN;
    const uint32_t n_tiles = tiles_a * tiles_b;
    const uint32_t num_kb = in_dim >> 8;
    const uint32_t num_ks = (num_kb + kSlabs - 1u) / kSlabs;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], 1);
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 16);   // in the leader: 8 epilogue warps of each CTA
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
            // B tile fastest: the pairs of a wave share a few A tiles
            const uint32_t tile_a = (tile / tiles_b) * 2u + rank, tile_b = tile % tiles_b;
            for (uint32_t ks = 0; ks < num_ks; ++ks) {
                ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* a = tiles + stage * kStageBytes;
                const uint32_t kb0 = ks * kSlabs, nsl = min(kSlabs, num_kb - kb0);
                // the scale boxes always span kSlabs records (rows past the plane read as zero and count)
                if (leader)
                    tc5::mbar_arrive_expect_tx_elect(&sh->full[stage],
                                                     2u * (nsl * (kABytes + C::kBHalf) + (1u + C::kRec) * kSlabs * kSfBytes));
#pragma unroll
                for (uint32_t u = 0; u < kSlabs; ++u)
                    if (u < nsl) {
                        tma_load_2d_pair_elect(a + u * kABytes, &tmap_w, &sh->full[stage], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(tile_a * BM));
                        tma_load_2d_pair_elect(a + C::kOffB + u * C::kBHalf, &tmap_x, &sh->full[stage], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(tile_b * BN + rank * C::BNH));
                    }
                tma_load_2d_pair_elect(a + C::kOffSfa, &tmap_wsf, &sh->full[stage], 0, (int32_t)((tile_a * num_kb + kb0) * 8u));
#pragma unroll
                for (uint32_t j = 0; j < C::kRec; ++j)   // one box of kSlabs records per 128 tokens
                    tma_load_2d_pair_elect(a + C::kOffSfb + j * kSlabs * kSfBytes, &tmap_xsf, &sh->full[stage], 0,
                                           (int32_t)(((tile_b * C::kRec + j) * num_kb + kb0) * 8u));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
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
                const uint32_t buf = iter % kAcc, aphase = (iter / kAcc) & 1u;
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
                    const uint32_t nsl = min(kSlabs, num_kb - ks * kSlabs);
#pragma unroll
                    for (uint32_t u = 0; u < kSlabs; ++u) {
                        if (u >= nsl) break;
                        const uint32_t sfa_t = tmem_base + C::kSfCol0 + stage * C::kSfCols + u * C::kSlabCols, sfb_t = sfa_t + 16u;
                        const uint64_t a_desc = tc5::smem_desc_sw128(a_addr + u * kABytes);
                        const uint64_t b_desc = tc5::smem_desc_sw128(a_addr + C::kOffB + u * C::kBHalf);
                        if constexpr (BN == 128u)
                            slab_nvf4_pair(d_tmem, a_desc, b_desc, C::kIdesc, (ks | u) != 0u, sfa_t, sfb_t,
                                           a_addr + C::kOffSfa + u * kSfBytes, a_addr + C::kOffSfb + u * kSfBytes, 4u);
                        else
                            slab_nvf4_pair256(d_tmem, a_desc, b_desc, C::kIdesc, (ks | u) != 0u, sfa_t, sfb_t,
                                              a_addr + C::kOffSfa + u * kSfBytes, a_addr + C::kOffSfb + u * kSfBytes);
                    }
                    mma_commit_pair_elect(&sh->empty[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit_pair_elect(&sh->tmem_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 channels)
        // The accumulator is read 64 token columns at a time and handed back to the MMA issuer as soon
        // as the last columns sit in registers; with a bf16 tensor map the whole [BN tokens][128 channels]
        // tile is staged in shared memory and leaves as ONE tiled store (one proxy fence and two
        // barriers per tile; the store drains while the next tile accumulates).
        const uint32_t quarter = warp & 3u, half = (warp - 2u) >> 2;   // this warp: every second group of 64 tokens
        uint32_t iter = 0;
        bool ok = true;
        TO* out_box = reinterpret_cast<TO*>(stage_out);
        pdk_pdl_wait();
        for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++iter) {
            const uint32_t buf = iter % kAcc, aphase = (iter / kAcc) & 1u;
            const uint32_t a0 = ((tile / tiles_b) * 2u + rank) * BM, b0 = (tile % tiles_b) * BN;
            const uint32_t n = a0 + quarter * 32u + lane;
            const uint32_t n_b = min(BN, b_rows - b0), n_grp = (n_b + 63u) / 64u;
            const float b = (bias != nullptr && n < a_rows) ? bias[n] : 0.0f;
            if (tma_out) {   // the previous tile's store has read the box
                if (threadIdx.x == 64u) tc5::tma_store_wait_read();
                asm volatile("bar.sync 2, 256;" ::: "memory");
            }
            ok = tc5::mbar_wait(&sh->tmem_full[buf], aphase, ctx, tc5::kErrTmemFullWait, buf);
            if (!ok) break;
            tc5::fence_after_sync();
            auto put_group = [&](uint32_t g, const uint32_t (&ra)[32], const uint32_t (&rb)[32]) {
                if (tma_out) {
#pragma unroll
                    for (uint32_t i = 0; i < 64u; ++i)
                        store_smem2<TO>(out_box + (g * 64u + i) * BM + quarter * 32u + lane,
                                        fmaf(__uint_as_float(i < 32u ? ra[i & 31u] : rb[i & 31u]), scale2, b));
                } else if (n < a_rows) {
#pragma unroll
                    for (uint32_t i = 0; i < 64u; ++i) {
                        const uint32_t t = g * 64u + i;
                        if (t < n_b)
                            store_one2<TO>(y + (size_t)(b0 + t) * a_rows + n,
                                           fmaf(__uint_as_float(i < 32u ? ra[i & 31u] : rb[i & 31u]), scale2, b));
                    }
                }
            };
            auto hand_back = [&]() {   // every column this warp reads is in registers
                tc5::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(&sh->tmem_empty[buf]);
            };
            const uint32_t col0 = tmem_base + ((quarter * 32u) << 16) + buf * BN;
            if constexpr (BN == 256u) {
                // this warp's two groups (half, half + 2) are read before either is stored: the accumulator goes back
                // to the issuer after two load latencies instead of after the first group's 64 stores
                uint32_t ra0[32], rb0[32], ra1[32], rb1[32];
                const bool has0 = half < n_grp, has1 = half + 2u < n_grp;   // warp-uniform
                if (has0) {
                    tc5::tmem_ld_32x32(col0 + half * 64u, ra0);
                    tc5::tmem_ld_32x32(col0 + half * 64u + 32u, rb0);
                }
                if (has1) {
                    tc5::tmem_ld_32x32(col0 + (half + 2u) * 64u, ra1);
                    tc5::tmem_ld_32x32(col0 + (half + 2u) * 64u + 32u, rb1);
                }
                tc5::tmem_ld_wait();
                hand_back();
                if (has0) put_group(half, ra0, rb0);
                if (has1) put_group(half + 2u, ra1, rb1);
            } else {
                if (half >= n_grp) hand_back();   // a ragged tile with nothing for this warp to read
#pragma unroll 1
                for (uint32_t g = half; g < n_grp; g += 2u) {
                    uint32_t ra[32], rb[32];
                    tc5::tmem_ld_32x32(col0 + g * 64u, ra);
                    tc5::tmem_ld_32x32(col0 + g * 64u + 32u, rb);
                    tc5::tmem_ld_wait();
                    if (g + 2u >= n_grp) hand_back();
                    put_group(g, ra, rb);
                }
            }
            if (tma_out) {
                fence_proxy_async_smem();
                asm volatile("bar.sync 2, 256;" ::: "memory");
                // rows past the batch (stale rows of a ragged tile) and channels past a_rows are clipped
                if (threadIdx.x == 64u && a0 < a_rows) tc5::tma_store_2d(&tmap_y, out_box, (int32_t)a0, (int32_t)b0);
            }
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

template <typename TO, uint32_t BN>
int launch_pair(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled, void* y,
                float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    using C = PairCfg<BN>;
    CUtensorMap ta, tb, tasf, tbsf;
    const uint32_t kbytes = in_dim >> 1, num_kb = in_dim >> 8;
    const void *a_data = data, *b_data = xq, *a_sf = scale_tiled, *b_sf = xs_tiled;
    const uint32_t a_rows = out_dim, b_rows = batch;
    if (int rc = pdk_make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_data, kbytes, a_rows, kbytes, BKB, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_data, kbytes, b_rows, kbytes, BKB, C::BNH)) return rc;
    // scale records (2048 bytes each, one per 128 rows and slab) as rows of 256 bytes, eight per record; a box
    // spans a stage's records
    const uint64_t a_recs = (uint64_t)((a_rows + 127u) / 128u) * num_kb, b_recs = (uint64_t)((b_rows + 127u) / 128u) * num_kb;
    if (int rc = pdk_make_tmap_2d_dense(&tasf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_sf, 256u, a_recs * 8u, 256u, 256u, 8u * C::kSlabs))
        return rc;
    if (int rc = pdk_make_tmap_2d_dense(&tbsf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_sf, 256u, b_recs * 8u, 256u, 256u, 8u * C::kSlabs))
        return rc;
    CUtensorMap ty = ta;
    uint32_t tma_out = 0u;
    if (sizeof(TO) == 2u && pdk_aligned(y, 16) && (out_dim & 7u) == 0u &&
        pdk_make_tmap_2d_dense(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, out_dim, batch, (uint64_t)out_dim * 2u, BM, BN) == 0)
        tma_out = 1u;
    const size_t smem = (size_t)C::kStages * C::kStageBytes + 128u + (tma_out ? BN * BM * sizeof(TO) : 0u) + 1024u;
    auto kern = nvf4_gemm_pair_kernel<TO, BN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = ((a_rows + 2u * BM - 1u) / (2u * BM)) * ((b_rows + BN - 1u) / BN);
    uint32_t pairs = (uint32_t)pdk_sm_count() / 2u;
    if (pairs > n_tiles) pairs = n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * pairs);
    cfg.blockDim = dim3(kThreadsP);
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
    e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tasf, tbsf, (const float*)bias, (TO*)y, scale2, in_dim, a_rows, b_rows,
                           pdk_error_word(), ty, tma_out);
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}

// 256-token tiles once every pair of SMs gets at least one of them (PDK_NVF4_PAIR_BN=128 / 256 forces
// one; read per call: a launch of tens to hundreds of microseconds).
template <typename TO>
int launch_pair_any(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled, void* y,
                    float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    const char* env = getenv("PDK_NVF4_PAIR_BN");
    const int forced = env ? atoi(env) : 0;
    const uint32_t tiles256 = ((out_dim + 2u * BM - 1u) / (2u * BM)) * ((batch + 255u) / 256u);
    const bool wide = forced == 256 || (forced != 128 && tiles256 >= (uint32_t)pdk_sm_count() / 2u);
    if (wide) return launch_pair<TO, 256u>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
    return launch_pair<TO, 128u>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
}

}  // namespace

// Prefill widths on pairs of SMs; xs_tiled = the activation scales in the weight scales' record
// layout (one record per 128 tokens and slab).
int pdk_nvf4_gemm_pair_f32(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled,
                           void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair_any<float>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
}
int pdk_nvf4_gemm_pair_bf16(const void* data, const void* scale_tiled, const void* bias, const void* xq, const void* xs_tiled,
                            void* y, float scale2, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair_any<__nv_bfloat16>(data, scale_tiled, bias, xq, xs_tiled, y, scale2, in_dim, out_dim, batch, st);
}
