// fp8_gemm2.cu - the row-scaled e4m3 prefill GEMM of fp8_gemm.cu on pairs of SMs.
//
// The one-SM kernel moves 48 KB from L2 per K stage (128 tokens + 256 channels of 128 bytes) for
// four MMAs that take the tensor core 512 cycles, and L2 delivers to one SM about 61 bytes per
// cycle: the feed, not the tensor core, sets its pace.  Here two CTAs of a cluster share a
// 256 x 256 tile (tcgen05 cta_group::2): each loads its own 128 tokens (A) and HALF of the 256
// channels (B), 32 KB per stage, and one instruction of the leader CTA drives both tensor cores,
// each reading B's other half out of its partner's shared memory.  Same flops per SM and stage,
// two thirds of the bytes, and the 32 KB stages leave room for six of them.
//
//   CTA r of a pair (r = rank in the cluster, 0 leads):
//   warp 0      TMA producer: its A box and its half of the B box, completion counted on the
//               LEADER's full barrier (which expects both CTAs' bytes)
//   warp 1      leader only: MMA issuer, M = 256 (128 per CTA) x N = 256 x K = 32 per
//               instruction; its commits arrive on both CTAs' barriers (stage free, accumulator full)
//   warps 2..5  epilogue of the CTA's own 128 tokens x 256 channels, out of its own tensor
//               memory; "accumulator drained" is counted on the leader's barrier by all eight
//               epilogue warps of the pair
// No multicast loads.  Every wait is bounded; a CTA that gives up raises its abort flag, its
// partner runs into its own bounded waits, and both leave through the closing cluster barrier.
#include "tc5.cuh"

namespace {

using namespace tc5::pair;

constexpr uint32_t BM = 128;            // tokens per CTA (256 per pair)
constexpr uint32_t BN = 256;            // channels per pair
constexpr uint32_t BNH = 128;           // channels whose weights one CTA loads
constexpr uint32_t BK = 128;            // bytes of K per stage
constexpr uint32_t kStages = 6;
constexpr uint32_t kABytes = BM * BK, kBBytes = BNH * BK, kStageBytes = kABytes + kBBytes;
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
__device__ __forceinline__ void store_chunk2(TO* dst, const float (&v)[32], uint32_t valid);
template <>
__device__ __forceinline__ void store_chunk2<float>(float* dst, const float (&v)[32], uint32_t valid) {
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
__device__ __forceinline__ void store_chunk2<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], uint32_t valid) {
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
f8row_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                       const float* __restrict__ w_scale, const float* __restrict__ x_scale, TO* __restrict__ y,
                       uint32_t in_dim, uint32_t out_dim, uint32_t batch, unsigned int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * kStageBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0u;
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t tiles_m = (batch + 2u * BM - 1u) / (2u * BM), tiles_n = (out_dim + BN - 1u) / BN;
    const uint32_t n_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (in_dim + BK - 1u) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], 1);     // the leader's arrive.expect_tx; both CTAs' bytes
            tc5::mbar_init(&sh->empty[s], 1);    // the leader's commit, delivered to both CTAs
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 8);   // used in the leader: 4 epilogue warps of each CTA
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_x);
        tc5::tma_prefetch_desc(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc2(&sh->tmem_base, kTmemCols);
        tmem_relinquish2();
    }
    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();          // the partner's barriers exist before anything arrives on them
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, err_word};
    pdk_pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        pdk_pdl_wait();
        for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs) {
            const uint32_t m0 = (tile % tiles_m) * 2u * BM + rank * BM, n0 = (tile / tiles_m) * BN + rank * BNH;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* a = tiles + stage * kStageBytes;
                if (leader) tc5::mbar_arrive_expect_tx_elect(&sh->full[stage], 2u * kStageBytes);
                tma_load_2d_pair_elect(a, &tmap_x, &sh->full[stage], (int32_t)(kb * BK), (int32_t)m0);
                tma_load_2d_pair_elect(a + kABytes, &tmap_w, &sh->full[stage], (int32_t)(kb * BK), (int32_t)n0);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) {
            for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies in flight still land in this CTA
        }
    } else if (warp == 1) {
        if (leader) {
            // -------------------------------------------------------- MMA issuer (leader; whole warp, one lane issues)
            constexpr uint32_t idesc = tc5::idesc_f32acc(0u, 0u, 2u * BM, BN);
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++iter) {
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
                    mma_f8f6f4_x4_pair_elect(d_tmem, tc5::smem_desc_sw128(a_addr), tc5::smem_desc_sw128(a_addr + kABytes), idesc,
                                             kb != 0u);
                    mma_commit_pair_elect(&sh->empty[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit_pair_elect(&sh->tmem_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 tokens)
        const uint32_t quarter = warp & 3u;
        uint32_t iter = 0;
        bool ok = true;
        pdk_pdl_wait();
        for (uint32_t tile = pair; tile < n_tiles && ok; tile += n_pairs, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            const uint32_t m0 = (tile % tiles_m) * 2u * BM + rank * BM, n0 = (tile / tiles_m) * BN;
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
                    store_chunk2<TO>(yrow + c * 32u, v, valid);
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&sh->tmem_empty[buf]);
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    cluster_sync();          // neither CTA leaves while its partner may still read its shared memory or signal it
    if (warp == 1) {
        tc5::fence_after_sync();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}

template <typename TO>
int launch_pair(const void* data, const void* w_scale, const void* xq, const void* x_scale, void* y, uint32_t in_dim,
                uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    CUtensorMap tx, tw;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, in_dim, batch, in_dim, BK, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, in_dim, out_dim, in_dim, BK, BNH)) return rc;
    const size_t smem = (size_t)kStages * kStageBytes + sizeof(Shared) + 1024u;
    auto kern = f8row_gemm_pair_kernel<TO>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = ((batch + 2u * BM - 1u) / (2u * BM)) * ((out_dim + BN - 1u) / BN);
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
    e = cudaLaunchKernelEx(&cfg, kern, tx, tw, (const float*)w_scale, (const float*)x_scale, (TO*)y, in_dim, out_dim, batch,
                           pdk_error_word());
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}

}  // namespace

// The pair kernel for problems that fill pairs of SMs with 256-token tiles; -1 = not this route.
int pdk_f8row_gemm_pair_f32(const void* data, const void* w_scale, const void* xq, const void* x_scale, void* y,
                            uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair<float>(data, w_scale, xq, x_scale, y, in_dim, out_dim, batch, st);
}
int pdk_f8row_gemm_pair_bf16(const void* data, const void* w_scale, const void* xq, const void* x_scale, void* y,
                             uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    return launch_pair<__nv_bfloat16>(data, w_scale, xq, x_scale, y, in_dim, out_dim, batch, st);
}
