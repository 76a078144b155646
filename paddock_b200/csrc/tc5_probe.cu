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
// M128 N128 K64, 3 as 2 with the scale-cell copies of a GEMM) on operands that stay in shared
// memory.  cycles: device u64[SM count] (may be NULL), SM clocks per CTA.  Time the launch with
// events: flops = SMs * n_mma * 2 * 128 * N * K.
PDK_EXPORT int pdk_tc5_issue_probe(uint32_t kind, uint32_t n_mma, void* cycles, void* stream) {
    if (kind > 3u || n_mma < 8u || n_mma > (1u << 20) || (n_mma & 3u)) return cudaErrorInvalidValue;
    auto st = (cudaStream_t)stream;
    switch (kind) {
        case 0: return launch_probe<0>(n_mma, cycles, st);
        case 1: return launch_probe<1>(n_mma, cycles, st);
        case 2: return launch_probe<2>(n_mma, cycles, st);
        default: return launch_probe<3>(n_mma, cycles, st);
    }
}
