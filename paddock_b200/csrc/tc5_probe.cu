// tc5_probe.cu - how fast one SM's tensor core takes tcgen05.mma of each operand kind when
// nothing else is in the way: operands resident in shared memory, no loads, no epilogue.
// The figure is the denominator the FP8 / NVFP4 GEMMs are judged against (the reference keeps
// the same kind of probe beside its kernels, packs/cuda/src/gemm/dense_nvf4_tc5.cuh:306-309).
#include "nvf4_tc5.cuh"
#include "pdk_common.cuh"
#include "tc5.cuh"

namespace {

constexpr uint32_t kProbeThreads = 128;
constexpr uint32_t kProbeA = 128u * 128u;        // 128 rows of 128 bytes, 128-byte swizzle atoms
constexpr uint32_t kProbeB = 256u * 128u;        // up to 256 rows
constexpr uint32_t kProbeSf = 2u * 2048u;        // four 512-byte scale cells for each operand
constexpr uint32_t kProbeSmem = kProbeA + kProbeB + kProbeSf + 1024u;
constexpr uint32_t kErrProbeWait = 0x17;

// kind 0: bf16 x bf16 (M128 N256 K16)   1: e4m3 x e4m3 (M128 N256 K32)
//      2: e2m1 x e2m1 with UE4M3 block-16 scales (M128 N128 K64), scales left in tensor memory
//      3: as 2, each MMA preceded by the two scale-cell copies a GEMM needs for it
// One warp issues n_mma instructions in groups of four K steps over the same 128-byte rows,
// groups alternating between two accumulators; one commit at the end, one bounded wait.
// cycles[cta] = SM clocks from the first issue to the completion of the last MMA.
template <int kKind>
__global__ void __launch_bounds__(kProbeThreads)
tc5_issue_probe_kernel(uint32_t n_mma, unsigned int* err, unsigned long long* cycles) {
    extern __shared__ uint8_t probe_raw[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    uint8_t* base = (uint8_t*)(((uintptr_t)probe_raw + 1023u) & ~(uintptr_t)1023u);
    uint8_t* a_tile = base;
    uint8_t* b_tile = base + kProbeA;
    uint8_t* sf = b_tile + kProbeB;
    const uint32_t t = threadIdx.x, warp = t >> 5;

    // any finite operands do: bytes below 0x38 are small positive numbers in every format used here
    for (uint32_t i = t; i < (kProbeA + kProbeB) / 4u; i += kProbeThreads) {
        uint32_t h = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15;
        reinterpret_cast<uint32_t*>(base)[i] = h & 0x37373737u;
    }
    for (uint32_t i = t; i < kProbeSf / 4u; i += kProbeThreads) reinterpret_cast<uint32_t*>(sf)[i] = 0x38383838u;  // 1.0
    if (t == 0) {
        tc5::mbar_init(&done_bar, 1);
        abort_flag = 0;
        tc5::mbar_fence_init();
    }
    nvf4tc5::fence_proxy_async_smem();
    __syncthreads();
    if (warp == 0) {
        tc5::tmem_alloc(&tmem_slot, 512);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        const uint64_t a_desc = tc5::smem_desc_sw128(tc5::smem_u32(a_tile));
        const uint64_t b_desc = tc5::smem_desc_sw128(tc5::smem_u32(b_tile));
        constexpr uint32_t n_cols = kKind >= 2 ? 128u : 256u;
        constexpr uint32_t idesc = kKind == 0   ? tc5::idesc_f32acc(1u, 1u, 128u, 256u)
                                   : kKind == 1 ? tc5::idesc_f32acc(0u, 0u, 128u, 256u)
                                                : nvf4tc5::Cfg<128>::kIdesc;
        const uint32_t sfa_t = tmem + 256u, sfb_t = sfa_t + 16u;
        if (kKind >= 2)
            for (uint32_t j = 0; j < 4u; ++j) {
                nvf4tc5::sf_copy(sfa_t + j * 4u, tc5::smem_u32(sf) + j * 512u);
                nvf4tc5::sf_copy(sfb_t + j * 4u, tc5::smem_u32(sf) + 2048u + j * 512u);
            }
        const long long t0 = clock64();
#pragma unroll 2
        for (uint32_t g = 0; g < (n_mma >> 2); ++g) {
            const uint32_t d = tmem + (g & 1u) * n_cols;
            const uint32_t acc = g >= 2u ? 1u : 0u;
            // the issue sequences of the GEMMs themselves (tc5.cuh, nvf4_tc5.cuh)
            if (kKind == 0) tc5::mma_f16_x4_elect(d, a_desc, b_desc, idesc, acc);
            else if (kKind == 1) tc5::mma_f8f6f4_x4_elect(d, a_desc, b_desc, idesc, acc);
            else nvf4tc5::slab_nvf4<kKind == 3>(d, a_desc, b_desc, idesc, acc, sfa_t, sfb_t, tc5::smem_u32(sf), tc5::smem_u32(sf) + 2048u, 4u);
        }
        tc5::mma_commit_elect(&done_bar);
        const tc5::WaitCtx ctx{&abort_flag, err};
        tc5::mbar_wait(&done_bar, 0u, ctx, kErrProbeWait, (unsigned)kKind);
        const long long t1 = clock64();
        if (t == 0 && cycles != nullptr) cycles[blockIdx.x] = (unsigned long long)(t1 - t0);
    }
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc5::tmem_dealloc(tmem, 512);
}

// The same for a pair of CTAs (cta_group::2): kind 4 e4m3 M256 N256 K32, kind 5 NVFP4 M256 N128
// K64 with its scale-cell copies.  Each CTA holds its A tile, half of B and its scale cells; the
// leader issues, the commit arrives in both CTAs.
__device__ __forceinline__ void probe_group_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t acc_first) {
    asm volatile(
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 a, b;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t"
        "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t"
        "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first)
        : "memory");
}
__device__ __forceinline__ void probe_group_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t acc_first, uint32_t sfa_t, uint32_t sfb_t, uint32_t sfa_smem,
                                                      uint32_t sfb_smem) {
    const uint64_t cell_a = (uint64_t)((sfa_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
    const uint64_t cell_b = (uint64_t)((sfb_smem >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)8u << 32);
#define PDK_PROBE_NV4P(J, PRED)                                                                                       \
    "add.u64 a, %1, " #J "*2;\n\tadd.u64 b, %2, " #J "*2;\n\tadd.u32 sa, %5, " #J "*4;\n\tadd.u32 sb, %6, " #J "*4;\n\t" \
    "add.u64 ca, %7, " #J "*32;\n\tadd.u64 cb, %8, " #J "*32;\n\t"                                                    \
    "@e tcgen05.cp.cta_group::2.32x128b.warpx4 [sa], ca;\n\t@e tcgen05.cp.cta_group::2.32x128b.warpx4 [sb], cb;\n\t"  \
    "@e tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], a, b, %3, [sa], [sb], " PRED ";\n\t"
    asm volatile(
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 a, b, ca, cb;\n\t.reg .b32 sa, sb;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        PDK_PROBE_NV4P(0, "p") PDK_PROBE_NV4P(1, "q") PDK_PROBE_NV4P(2, "q") PDK_PROBE_NV4P(3, "q") "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first), "r"(sfa_t), "r"(sfb_t), "l"(cell_a), "l"(cell_b)
        : "memory");
#undef PDK_PROBE_NV4P
}

template <int kKind>
__global__ void __launch_bounds__(kProbeThreads)
tc5_issue_probe_pair_kernel(uint32_t n_mma, unsigned int* err, unsigned long long* cycles) {
    using namespace tc5::pair;
    extern __shared__ uint8_t probe_raw[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    uint8_t* base = (uint8_t*)(((uintptr_t)probe_raw + 1023u) & ~(uintptr_t)1023u);
    uint8_t* a_tile = base;
    uint8_t* b_tile = base + kProbeA;
    uint8_t* sf = b_tile + kProbeB;
    const uint32_t t = threadIdx.x, warp = t >> 5;
    const bool leader = cluster_ctarank() == 0u;
    for (uint32_t i = t; i < (kProbeA + kProbeB) / 4u; i += kProbeThreads) {
        uint32_t h = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15;
        reinterpret_cast<uint32_t*>(base)[i] = h & 0x37373737u;
    }
    for (uint32_t i = t; i < kProbeSf / 4u; i += kProbeThreads) reinterpret_cast<uint32_t*>(sf)[i] = 0x38383838u;
    if (t == 0) {
        tc5::mbar_init(&done_bar, 1);
        abort_flag = 0;
        tc5::mbar_fence_init();
    }
    nvf4tc5::fence_proxy_async_smem();
    __syncthreads();
    if (warp == 0) {
        tmem_alloc2(&tmem_slot, 512);
        tmem_relinquish2();
    }
    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();
    tc5::fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (warp == 0) {
        const long long t0 = clock64();
        if (leader) {
            const uint64_t a_desc = tc5::smem_desc_sw128(tc5::smem_u32(a_tile));
            const uint64_t b_desc = tc5::smem_desc_sw128(tc5::smem_u32(b_tile));
            constexpr uint32_t n_cols = kKind == 4 ? 256u : 128u;
            constexpr uint32_t idesc = kKind == 4 ? tc5::idesc_f32acc(0u, 0u, 256u, 256u)
                                                  : ((1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((256u >> 4) << 24));
            const uint32_t sfa_t = tmem + 256u, sfb_t = sfa_t + 16u;
#pragma unroll 2
            for (uint32_t g = 0; g < (n_mma >> 2); ++g) {
                const uint32_t d = tmem + (g & 1u) * n_cols;
                const uint32_t acc = g >= 2u ? 1u : 0u;
                if (kKind == 4) probe_group_f8_pair(d, a_desc, b_desc, idesc, acc);
                else probe_group_nvf4_pair(d, a_desc, b_desc, idesc, acc, sfa_t, sfb_t, tc5::smem_u32(sf), tc5::smem_u32(sf) + 2048u);
            }
            mma_commit_pair_elect(&done_bar);
        }
        const tc5::WaitCtx ctx{&abort_flag, err};
        tc5::mbar_wait(&done_bar, 0u, ctx, kErrProbeWait, (unsigned)kKind);
        const long long t1 = clock64();
        if (t == 0 && cycles != nullptr) cycles[blockIdx.x] = (unsigned long long)(t1 - t0);
    }
    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (warp == 0) tmem_dealloc2(tmem, 512);
}

template <int kKind>
int launch_probe_pair(uint32_t n_mma, void* cycles, cudaStream_t st) {
    auto kern = tc5_issue_probe_pair_kernel<kKind>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kProbeSmem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((uint32_t)pdk_sm_count() & ~1u);
    cfg.blockDim = dim3(kProbeThreads);
    cfg.dynamicSmemBytes = kProbeSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, n_mma, pdk_error_word(), (unsigned long long*)cycles);
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}

template <int kKind>
int launch_probe(uint32_t n_mma, void* cycles, cudaStream_t st) {
    cudaError_t e = cudaFuncSetAttribute(tc5_issue_probe_kernel<kKind>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kProbeSmem);
    if (e != cudaSuccess) return (int)e;
    tc5_issue_probe_kernel<kKind><<<pdk_sm_count(), kProbeThreads, kProbeSmem, st>>>(n_mma, pdk_error_word(),
                                                                                      (unsigned long long*)cycles);
    return pdk_launch_status();
}

}  // namespace

// No counterpart among the reference's exports (its probe is a bench program,
// bench/tc5_mma_rate.cu).  Launches one CTA per SM, each issuing n_mma (8 .. 2^20, a multiple of 4)
// tcgen05.mma of `kind` (0 bf16 M128 N256 K16, 1 e4m3 M128 N256 K32, 2 NVFP4 block-scaled
// M128 N128 K64, 3 as 2 with the scale-cell copies of a GEMM; on pairs of SMs, one issuing CTA
// per pair: 4 e4m3 M256 N256 K32, 5 NVFP4 M256 N128 K64 with scale-cell copies) on operands that
// stay in shared memory.  cycles: device u64[SM count] (may be NULL), SM clocks per CTA.  Time the launch with
// events: flops = SMs * n_mma * 2 * 128 * N * K.
PDK_EXPORT int pdk_tc5_issue_probe(uint32_t kind, uint32_t n_mma, void* cycles, void* stream) {
    if (kind > 5u || n_mma < 8u || n_mma > (1u << 20) || (n_mma & 3u)) return cudaErrorInvalidValue;
    auto st = (cudaStream_t)stream;
    switch (kind) {
        case 0: return launch_probe<0>(n_mma, cycles, st);
        case 1: return launch_probe<1>(n_mma, cycles, st);
        case 2: return launch_probe<2>(n_mma, cycles, st);
        case 3: return launch_probe<3>(n_mma, cycles, st);
        case 4: return launch_probe_pair<4>(n_mma, cycles, st);
        default: return launch_probe_pair<5>(n_mma, cycles, st);
    }
}
