// nvf4_tc5.cuh - what the block-scaled e2m1 tcgen05 kernels share: the tile and
// pipeline geometry, the shared-memory control block, the scale-cell copy and the
// kind::mxf4nvf4 MMA issue.  (Used by the dense NVFP4 GEMM and by the grouped
// MXFP4 expert GEMM.)
#pragma once
#include "tc5.cuh"

namespace nvf4tc5 {

constexpr uint32_t BM = 128;            // weight rows per tile
constexpr uint32_t BKB = 128;           // bytes of K per stage = 256 e2m1
constexpr uint32_t kABytes = BM * BKB, kSfBytes = 2048;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kMaxStages = 4;
// Slabs per pipeline stage.  A stage hand-off (barrier wait, fences, commit) costs the
// issuing warp about as long as the tensor pipe needs for half a slab, and nothing
// overlaps it; two slabs per hand-off halve that.
constexpr uint32_t KS = 2;

// Token tile BN: 128 for prefill widths (3 stages of two slabs); 32 or 64 for decode
// widths, where the smaller activation box leaves room for 4 stages (8 slabs, 144 KB of
// weights in flight per SM).
template <uint32_t BN>
struct Cfg {
    static constexpr uint32_t kStages = BN == 128u ? 3u : 4u;
    static constexpr uint32_t kBBytes = BN * BKB;
    // a stage = KS slabs: [W boxes][X boxes][W scale records][X scale records]
    static constexpr uint32_t kOffB = KS * kABytes, kOffSfa = kOffB + KS * kBBytes, kOffSfb = kOffSfa + KS * kSfBytes;
    static constexpr uint32_t kStageBytes = kOffSfb + KS * kSfBytes;
    static constexpr uint32_t kSfCol0 = 2u * BN;  // scale cells start after the two accumulators
    static constexpr uint32_t kSfCols = KS * 32u; // TMEM columns of one stage's scale cells
    // e2m1 x e2m1 (format code 1 in the mxf4 encoding), UE4M3 scales, scale ids 0
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);
};

struct Shared {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 512-byte scale cell (32 rows x 16 bytes, no swizzle) -> 4 TMEM columns, broadcast to the 4 lane quarters
// (called by a converged warp; one elected lane issues)
__device__ __forceinline__ void sf_copy(uint32_t taddr, uint32_t saddr) {
    const uint64_t desc = (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    asm volatile(TC5_ELECT "@e tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(taddr), "l"(desc)
                 : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(TC5_ELECT
                 ".reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "@e tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(
                     d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
                 : "memory");
}
// One 256-element K slab of a block-scaled tile: `steps` (1..4) MMAs of 64 elements each, every
// one preceded - when kCopies - by the copies of its two 512-byte scale cells from shared memory
// (sfa_smem / sfb_smem: the slab's 2048-byte records) into tensor memory (sfa_t / sfb_t, four
// columns per step).  One election, descriptors and addresses stepped inside the asm block:
// issued this way the pair (two copies + MMA) takes the tensor core 92 cycles, the MMA alone 64;
// one wrapper call per copy and per MMA took the issuing warp 200.
template <bool kCopies>
__device__ __forceinline__ void slab_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t acc_first, uint32_t sfa_t, uint32_t sfb_t, uint32_t sfa_smem,
                                          uint32_t sfb_smem, uint32_t steps) {
    const uint64_t cell_a = (uint64_t)((sfa_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    const uint64_t cell_b = (uint64_t)((sfb_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
#define PDK_NV4_STEP(J, PRED)                                                                                        \
    "setp.gt.and.u32 ej, %10, " #J ", e;\n\tsetp.gt.and.u32 cj, %10, " #J ", c;\n\t"                                  \
    "add.u64 a, %1, " #J "*2;\n\tadd.u64 b, %2, " #J "*2;\n\tadd.u32 sa, %5, " #J "*4;\n\tadd.u32 sb, %6, " #J "*4;\n\t" \
    "add.u64 ca, %7, " #J "*32;\n\tadd.u64 cb, %8, " #J "*32;\n\t"                                                    \
    "@cj tcgen05.cp.cta_group::1.32x128b.warpx4 [sa], ca;\n\t@cj tcgen05.cp.cta_group::1.32x128b.warpx4 [sb], cb;\n\t" \
    "@ej tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], a, b, %3, [sa], [sb], " PRED ";\n\t"
    asm volatile(
        "{\n\t.reg .pred e, p, q, c, ej, cj;\n\t.reg .b64 a, b, ca, cb;\n\t.reg .b32 sa, sb;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "setp.ne.and.b32 c, %9, 0, e;\n\t"
        PDK_NV4_STEP(0, "p") PDK_NV4_STEP(1, "q") PDK_NV4_STEP(2, "q") PDK_NV4_STEP(3, "q") "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first), "r"(sfa_t), "r"(sfb_t), "l"(cell_a), "l"(cell_b),
        "r"(kCopies ? 1u : 0u), "r"(steps)
        : "memory");
#undef PDK_NV4_STEP
}
}  // namespace nvf4tc5
