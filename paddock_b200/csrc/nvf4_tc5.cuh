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
}  // namespace nvf4tc5
