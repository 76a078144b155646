// moe_route.cu - MoE routing around the grouped expert GEMMs: top-k router,
// expert alignment (token permutation into expert-contiguous blocks),
// activation preparation for the expert GEMMs, and the fixed-order
// slot combine.
#include <cuda_fp8.h>

#include "moe_route.cuh"
#include "pdk_common.cuh"

namespace {

// ---------------------------------------------------------------- top-k router (moe_route.cuh)
__global__ void moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, uint32_t n_expert,
                                uint32_t k, uint32_t* __restrict__ out_idx, float* __restrict__ out_w,
                                uint32_t batch) {
    // dependent launch: may start while the previous kernel of the stream drains; its results are awaited here
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    const uint32_t token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= batch) return;
    moe_route::topk_warp(logits + (size_t)token * n_expert, bias, n_expert, k, threadIdx.x & 31u,
                         out_idx + (size_t)token * k, out_w + (size_t)token * k);
}

// ---------------------------------------------------------------- expert alignment
// Groups the (token, slot) pairs by expert into blocks of `bm` entries, padding
// each expert's last block.  One CTA; a warp owns experts warp, warp+nwarps, ...
// and walks the pair list in order with ballots, so entries inside an expert
// keep ascending pair order (the layout is a pure function of the routing).
//   sorted_row[b*bm + i]  source token row, or PDK_MOE_PAD
//   sorted_slot[b*bm + i] which of the token's k picks
//   block_expert[b]       expert of block b, PDK_MOE_PAD past the used blocks
__global__ void __launch_bounds__(1024)
moe_align_kernel(const uint32_t* __restrict__ idx, uint32_t* __restrict__ sorted_row,
                 uint32_t* __restrict__ sorted_slot, uint32_t* __restrict__ block_expert, uint32_t rows,
                 uint32_t n_active, uint32_t n_expert, uint32_t bm, uint32_t max_blocks, uint32_t staged) {
    extern __shared__ uint32_t ash[];
    uint32_t* count = ash;               // [n_expert]
    uint32_t* boff = ash + n_expert;     // [n_expert + 1] first block of each expert
    uint32_t* sidx = boff + n_expert + 1u;  // [npairs] when `staged`: every warp rescans the whole list
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const uint32_t npairs = rows * n_active;
    for (uint32_t e = tid; e < n_expert; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (uint32_t p = tid; p < npairs; p += blockDim.x) {
        const uint32_t e = idx[p];
        if (staged) sidx[p] = e;
        if (e < n_expert) atomicAdd(&count[e], 1u);
    }
    __syncthreads();
    const uint32_t* pick = staged ? sidx : idx;
    if (tid == 0) {
        uint32_t b = 0;
        for (uint32_t e = 0; e < n_expert; ++e) {
            boff[e] = b;
            b += (count[e] + bm - 1u) / bm;
        }
        boff[n_expert] = b;
    }
    __syncthreads();
    const uint32_t used = min(boff[n_expert], max_blocks);
    for (uint32_t b = used + tid; b < max_blocks; b += blockDim.x) block_expert[b] = PDK_MOE_PAD;
    for (uint32_t e = warp; e < n_expert; e += nwarp) {
        const uint32_t b0 = boff[e], nb = boff[e + 1] - b0;
        for (uint32_t b = lane; b < nb; b += 32u)
            if (b0 + b < max_blocks) block_expert[b0 + b] = e;
        uint32_t pos = b0 * bm;
        for (uint32_t base = 0; base < npairs; base += 32u) {
            const uint32_t p = base + lane;
            const bool mine = p < npairs && pick[p] == e;
            const uint32_t m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const uint32_t at = pos + __popc(m & ((1u << lane) - 1u));
                if (at < max_blocks * bm) {
                    sorted_row[at] = p / n_active;
                    sorted_slot[at] = p % n_active;
                }
            }
            pos += __popc(m);
        }
        const uint32_t end = (b0 + nb) * bm;
        for (uint32_t at = pos + lane; at < end; at += 32u)
            if (at < max_blocks * bm) {
                sorted_row[at] = PDK_MOE_PAD;
                sorted_slot[at] = 0;
            }
    }
}

// Same layout, linear work: the pair list is walked in chunks of one pair per thread; a
// pair's place among its expert's entries is (entries of earlier chunks) + (entries of
// earlier warps of this chunk) + (earlier lanes of its warp with the same expert, from
// __match_any_sync).  Needs a [warps][n_expert] table in shared memory.
__global__ void __launch_bounds__(1024)
moe_align_rank_kernel(const uint32_t* __restrict__ idx, uint32_t* __restrict__ sorted_row,
                      uint32_t* __restrict__ sorted_slot, uint32_t* __restrict__ block_expert, uint32_t rows,
                      uint32_t n_active, uint32_t n_expert, uint32_t bm, uint32_t max_blocks) {
    extern __shared__ uint32_t ash[];
    uint32_t* count = ash;                    // [n_expert] entries per expert
    uint32_t* boff = count + n_expert;        // [n_expert + 1] first block of each expert
    uint32_t* cursor = boff + n_expert + 1u;  // [n_expert] entries placed by earlier chunks
    uint32_t* table = cursor + n_expert;      // [nwarp][n_expert]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const uint32_t npairs = rows * n_active, cap = max_blocks * bm;
    // dependent launch: may start while the previous kernel of the stream drains; its results are awaited here
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    for (uint32_t e = tid; e < n_expert; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (uint32_t p = tid; p < npairs; p += blockDim.x) {
        const uint32_t e = idx[p];
        if (e < n_expert) atomicAdd(&count[e], 1u);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the block counts, 32 experts at a time
        uint32_t carry = 0;
        for (uint32_t e0 = 0; e0 < n_expert; e0 += 32u) {
            const uint32_t e = e0 + lane;
            const uint32_t nb = e < n_expert ? (count[e] + bm - 1u) / bm : 0u;
            uint32_t inc = nb;
#pragma unroll
            for (uint32_t d = 1; d < 32u; d <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, inc, d);
                if (lane >= d) inc += up;
            }
            if (e < n_expert) boff[e] = carry + inc - nb;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) boff[n_expert] = carry;
    }
    __syncthreads();
    const uint32_t used = min(boff[n_expert], max_blocks);
    for (uint32_t b = used + tid; b < max_blocks; b += blockDim.x) block_expert[b] = PDK_MOE_PAD;
    for (uint32_t e = tid; e < n_expert; e += blockDim.x) {
        for (uint32_t b = boff[e]; b < boff[e + 1] && b < max_blocks; ++b) block_expert[b] = e;
        // padding of the expert's last block
        for (uint32_t at = boff[e] * bm + count[e]; at < boff[e + 1] * bm && at < cap; ++at) {
            sorted_row[at] = PDK_MOE_PAD;
            sorted_slot[at] = 0;
        }
    }
    for (uint32_t base = 0; base < npairs; base += blockDim.x) {
        for (uint32_t i = tid; i < nwarp * n_expert; i += blockDim.x) table[i] = 0;
        __syncthreads();
        const uint32_t p = base + tid;
        const uint32_t e = p < npairs ? idx[p] : 0xFFFFFFFFu;
        const bool live = e < n_expert;
        const uint32_t peers = __match_any_sync(0xffffffffu, live ? e : 0xFFFFFFFFu);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        if (live && rank == 0u) table[warp * n_expert + e] = __popc(peers);
        __syncthreads();
        for (uint32_t x = tid; x < n_expert; x += blockDim.x) {  // per expert: prefix over the warps
            uint32_t run = cursor[x];
            for (uint32_t w = 0; w < nwarp; ++w) {
                const uint32_t t = table[w * n_expert + x];
                table[w * n_expert + x] = run;
                run += t;
            }
            cursor[x] = run;
        }
        __syncthreads();
        if (live) {
            const uint32_t at = boff[e] * bm + table[warp * n_expert + e] + rank;
            if (at < cap) {
                sorted_row[at] = p / n_active;
                sorted_slot[at] = p % n_active;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------- activation prep
// f32 rows -> the B operand of the expert GEMMs: f16 with one power-of-two step
// 2^e per row chosen so that amax / 2^e lies in [2^14, 2^15).  bf16 activations
// are carried exactly (8 significant bits fit in f16's 11); general f32 ones are
// rounded to 11 significant bits.
// Layout per row and 32-element block, 64 bytes: for t = 0..3 the eight halves
//   [x(4t), x(4t+2), x(4t+1), x(4t+3), x(16+4t), x(16+4t+2), x(16+4t+1), x(16+4t+3)]
// which is one lane's B registers for the block's two mmas.
__global__ void __launch_bounds__(256)
moe_prep_act_kernel(const float* __restrict__ x, uint8_t* __restrict__ xq, float* __restrict__ xscale, uint32_t dim) {
    __shared__ float wmax[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t)row * dim;
    float a = 0.0f;
    for (uint32_t i = tid; i < dim; i += 256u) {
        const float v = fabsf(xr[i]);
        a = fmaxf(a, v == v ? v : 0.0f);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
    if ((tid & 31u) == 0u) wmax[tid >> 5] = a;
    __syncthreads();
    float amax = 0.0f;
    for (int w = 0; w < 8; ++w) amax = fmaxf(amax, wmax[w]);
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        (void)frexpf(amax, &e);   // amax in [2^(e-1), 2^e)
        e -= 15;                  // amax / 2^e in [2^14, 2^15)
        e = max(e, -100);
    }
    const float inv = ldexpf(1.0f, -e);
    if (tid == 0) xscale[row] = ldexpf(1.0f, e);
    uint8_t* out = xq + (size_t)row * dim * 2u;
    for (uint32_t u = tid; u < (dim >> 3); u += 256u) {  // one thread per (block, t): 8 elements -> 16 bytes
        const uint32_t blk = u >> 2, t = u & 3u;
        const float4 p = *reinterpret_cast<const float4*>(xr + blk * 32u + 4u * t);
        const float4 q = *reinterpret_cast<const float4*>(xr + blk * 32u + 16u + 4u * t);
        const __half2 h0 = __floats2half2_rn(p.x * inv, p.z * inv), h1 = __floats2half2_rn(p.y * inv, p.w * inv);
        const __half2 h2 = __floats2half2_rn(q.x * inv, q.z * inv), h3 = __floats2half2_rn(q.y * inv, q.w * inv);
        uint4 o;
        o.x = *reinterpret_cast<const uint32_t*>(&h0);
        o.y = *reinterpret_cast<const uint32_t*>(&h1);
        o.z = *reinterpret_cast<const uint32_t*>(&h2);
        o.w = *reinterpret_cast<const uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(out + (size_t)blk * 64u + t * 16u) = o;
    }
}

// ---------------------------------------------------------------- slot combine
__global__ void moe_slot_combine_kernel(const float4* __restrict__ part, float4* __restrict__ residual,
                                        uint32_t embd4, uint32_t n_active, uint32_t rows) {
    // dependent launch: may start while the previous kernel of the stream drains; its results are awaited here
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * embd4) return;
    const size_t t = i / embd4, r = i % embd4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < n_active; ++k) {  // fixed slot order: bit-reproducible
        const float4 p = part[(t * n_active + k) * embd4 + r];
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    float4 d = residual[i];
    d.x += acc.x; d.y += acc.y; d.z += acc.z; d.w += acc.w;
    residual[i] = d;
}

}  // namespace

// slot 29, packs/cuda/src/attn/decode.cuh:1392-1500 (launcher gemm/f32_qkv.cuh:1137-1150)
PDK_EXPORT int pd_moe_topk_batch(const void* logits, const void* bias, uint32_t n_expert, uint32_t k, void* out_idx,
                                 void* out_w, uint32_t batch, void* stream) {
    if (batch == 0) return 0;
    if (n_expert == 0 || n_expert > 512u || k == 0 || k > 16u || k > n_expert) return cudaErrorInvalidValue;
    return pdk_launch_pdl(moe_topk_kernel, dim3((batch + 3u) / 4u), dim3(128), 0, (cudaStream_t)stream,
                          (const float*)logits, (const float*)bias, n_expert, k, (uint32_t*)out_idx, (float*)out_w, batch);
}

// slot 146, packs/cuda/src/gemm/f32_qkv.cuh:1269-1279 (kernel attn/decode.cuh:2316-2396)
PDK_EXPORT int pd_moe_align_bm(const void* idx, void* sorted_row, void* sorted_slot, void* block_expert,
                               uint32_t rows, uint32_t n_active, uint32_t n_expert, uint32_t bm, uint32_t max_blocks,
                               void* stream) {
    if (rows == 0 || n_expert == 0) return 0;
    if (bm == 0 || (bm & (bm - 1u)) || n_expert > 4096u) return cudaErrorInvalidValue;
    static const cudaError_t attr_rank =
        cudaFuncSetAttribute(moe_align_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const size_t rank_smem = ((size_t)3u * n_expert + 1u + (size_t)32u * n_expert) * sizeof(uint32_t);
    if (attr_rank == cudaSuccess && rank_smem <= 200u * 1024u) {
        return pdk_launch_pdl(moe_align_rank_kernel, dim3(1), dim3(1024), rank_smem, (cudaStream_t)stream,
                              (const uint32_t*)idx, (uint32_t*)sorted_row, (uint32_t*)sorted_slot,
                              (uint32_t*)block_expert, rows, n_active, n_expert, bm, max_blocks);
    }
    // many experts: the scan kernel, one warp per expert
    size_t shmem = (size_t)(2u * n_expert + 1u) * sizeof(uint32_t);
    // the pick list is staged in shared memory when it fits (up to 200 KB)
    const size_t list = (size_t)rows * n_active * sizeof(uint32_t);
    const uint32_t staged = shmem + list <= 200u * 1024u ? 1u : 0u;
    if (staged) shmem += list;
    static const cudaError_t attr_rc =
        cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (attr_rc != cudaSuccess) return (int)attr_rc;
    moe_align_kernel<<<1, 1024, shmem, (cudaStream_t)stream>>>((const uint32_t*)idx, (uint32_t*)sorted_row,
                                                               (uint32_t*)sorted_slot, (uint32_t*)block_expert, rows,
                                                               n_active, n_expert, bm, max_blocks, staged);
    return pdk_launch_status();
}

// slot 34, packs/cuda/src/attn/decode.cuh:2316-2396: blocks of 32 entries
PDK_EXPORT int pd_moe_align(const void* idx, void* sorted_row, void* sorted_slot, void* block_expert, uint32_t rows,
                            uint32_t n_active, uint32_t n_expert, uint32_t max_blocks, void* stream) {
    return pd_moe_align_bm(idx, sorted_row, sorted_slot, block_expert, rows, n_active, n_expert, 32u, max_blocks,
                           stream);
}

// No slot: the activation step in front of the expert GEMMs (the reference's
// chain quantizes to int8 here, packs/cuda/src/attn/decode.cuh:2981-3004).
// x f32[rows][dim] -> xq f16[rows][dim] (fragment order) + xscale f32[rows]; dim % 32 == 0.
PDK_EXPORT int pdk_moe_prep_act(const void* x, void* xq, void* xscale, uint32_t dim, uint32_t rows, void* stream) {
    if (rows == 0 || dim == 0) return 0;
    if ((dim & 31u) != 0u || !pdk_aligned(x, 16) || !pdk_aligned(xq, 16)) return cudaErrorInvalidValue;
    moe_prep_act_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((const float*)x, (uint8_t*)xq, (float*)xscale, dim);
    return pdk_launch_status();
}

// slot 91, packs/cuda/src/moe/mmq.cuh:447-483
PDK_EXPORT int pd_moe_slot_combine(const void* part, void* residual, uint32_t embd, uint32_t n_active, uint32_t rows,
                                   void* stream) {
    if (rows == 0 || embd == 0) return 0;
    if ((embd & 3u) != 0u || !pdk_aligned(part, 16) || !pdk_aligned(residual, 16)) return cudaErrorInvalidValue;
    const size_t total = (size_t)rows * (embd >> 2);
    return pdk_launch_pdl(moe_slot_combine_kernel, dim3((uint32_t)((total + 255u) / 256u)), dim3(256), 0,
                          (cudaStream_t)stream, (const float4*)part, (float4*)residual, embd >> 2, n_active, rows);
}
