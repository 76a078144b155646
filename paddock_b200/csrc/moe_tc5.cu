// moe_tc5.cu - MXFP4 expert GEMMs on the block-scaled tcgen05 path.
//
// An MXFP4 plane needs no weight transformation to run on kind::mxf4nvf4:
//   * the repacked data plane is already 16 packed e2m1 bytes per 32 weights.  The
//     tensor core reads byte j of a block as the element pair (2j, 2j+1) where ggml
//     means (j, j+16); a dot product does not care as long as the activations are
//     packed in the same order, and the whole block shares one scale;
//   * the E8M0 block scale 2^(s-127) becomes two equal UE4M3 per-16 scales
//     2^(s - emax + 8) plus one per-plane factor scale2 = 2^(emax - 135), emax being
//     the largest scale byte of the plane.  Powers of two from 2^-9 to 2^8 are exact in
//     UE4M3, so every block within 17 binades of the plane's largest is exact; smaller
//     ones flush to zero (below 2^-17 of the largest weight block).
// Activations keep more than 4 bits by being expanded into four NVFP4 terms,
//   x * 2^-e = t0 + t1/16 + t2/256 + t3/4096,  t_k = nvfp4(16^k * residual_k),
// which sit side by side in the token dimension of one MMA (8 tokens x 4 terms = N 32,
// 32 tokens x 4 terms = N 128); the epilogue adds the four column groups.  What is
// left of a 16-element group after four terms is below 1e-3 of the group's largest
// element.  No weight passes through a register: at decode widths the kernel is a
// pure stream of 4.25 bits per weight.
//
// Launch order of one MoE block (host side in planes.py):
//   pdk_moe_prep_act_f4 (gather by sorted_row)  ->  pdk_mxfp4_moe_gemm_tc5 (gate and up, raw)
//   pdk_moe_prep_act_f4 (SwiGLU of gate/up)     ->  pdk_mxfp4_moe_gemm_tc5 (down, scattered to
//   (token, slot) rows and multiplied by the routing weight)  ->  pd_moe_slot_combine
#include <cuda_fp8.h>

#include "moe_route.cuh"
#include "nvf4_tc5.cuh"

namespace {

using namespace nvf4tc5;

// ---------------------------------------------------------------- weight scale planes

__global__ void mxfp4_emax_kernel(const uint8_t* __restrict__ scale, uint64_t n, uint32_t* __restrict__ meta) {
    uint32_t m = 0u;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        m = max(m, (uint32_t)scale[i]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31u) == 0u && m) atomicMax(meta, m);
}

// E8M0 byte relative to the plane's largest -> UE4M3 byte of 2^(s - emax + 8)
__device__ __forceinline__ uint32_t e8m0_to_ue4m3(uint32_t s, uint32_t emax) {
    const int k = (int)s - (int)emax + 8;  // <= 8
    if (k >= -6) return (uint32_t)(k + 7) << 3;
    if (k >= -9) return 1u << (k + 9);     // subnormals 2^-9, 2^-8, 2^-7
    return 0u;
}

// scale u8 [expert][rows][nblk]  ->  tiled [expert][row tile][slab][2048]: for row tile rt
// (128 rows) and slab kb (256 elements = 8 blocks) four 512-byte cells, one per MMA step j:
//   byte l*16 + c*4 + b of cell j = ue4m3 of block kb*8 + j*2 + b/2 of row rt*128 + c*32 + l
// (rows past `rows` and blocks past nblk read as 0).  One thread per 4-byte word.
__global__ void mxfp4_tile_scales_kernel(const uint8_t* __restrict__ scale, uint32_t* __restrict__ tiled,
                                         uint32_t rows, uint32_t nblk, uint32_t row_tiles, uint32_t num_kb,
                                         uint32_t* __restrict__ meta) {
    const uint32_t emax = meta[0];
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
        reinterpret_cast<float*>(meta)[1] = emax >= 9u ? __uint_as_float((emax - 8u) << 23) : 0.0f;  // 2^(emax - 135)
    const uint32_t expert = blockIdx.y;
    const uint32_t words = row_tiles * num_kb * 512u;
    for (uint32_t w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
        const uint32_t c = w & 3u, l = (w >> 2) & 31u, j = (w >> 7) & 3u, rec = w >> 9;
        const uint32_t kb = rec % num_kb, rt = rec / num_kb;
        const uint32_t row = rt * 128u + c * 32u + l;
        uint32_t out = 0u;
        if (row < rows) {
            const uint8_t* srow = scale + ((size_t)expert * rows + row) * nblk;
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                const uint32_t blk = kb * 8u + j * 2u + h;
                if (blk < nblk) out |= (e8m0_to_ue4m3(srow[blk], emax) * 0x0101u) << (16u * h);
            }
        }
        tiled[(size_t)expert * words + w] = out;
    }
}

// NVFP4 expert planes carry UE4M3 per-16 scales already: scale u8 [expert][rows][in_dim/16]
// -> the same records, byte l*16 + c*4 + b of cell j = scale[row rt*128 + c*32 + l][kb*16 + j*4 + b].
__global__ void nvf4_moe_tile_scales_kernel(const uint8_t* __restrict__ scale, uint32_t* __restrict__ tiled,
                                            uint32_t rows, uint32_t sf_row, uint32_t row_tiles, uint32_t num_kb) {
    const uint32_t expert = blockIdx.y;
    const uint32_t words = row_tiles * num_kb * 512u;
    for (uint32_t w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
        const uint32_t c = w & 3u, l = (w >> 2) & 31u, j = (w >> 7) & 3u, rec = w >> 9;
        const uint32_t kb = rec % num_kb, rt = rec / num_kb;
        const uint32_t row = rt * 128u + c * 32u + l, off = kb * 16u + j * 4u;
        uint32_t out = 0u;
        if (row < rows && off < sf_row)  // sf_row % 4 == 0
            out = *reinterpret_cast<const uint32_t*>(scale + ((size_t)expert * rows + row) * sf_row + off);
        tiled[(size_t)expert * words + w] = out;
    }
}

// ---------------------------------------------------------------- activations: four NVFP4 terms

__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}
// Two f32 -> one byte of two e2m1 codes (RN-even, saturating; low nibble = lo), and the
// byte's two values back as f32.
__device__ __forceinline__ uint32_t e2m1x2_rn(float lo, float hi, float& back_lo, float& back_hi) {
    uint16_t byte;
    asm("{\n\t.reg .b8 q;\n\tcvt.rn.satfinite.e2m1x2.f32 q, %1, %2;\n\tmov.b16 %0, {q, 0};\n\t}"
        : "=h"(byte)
        : "f"(hi), "f"(lo));
    uint32_t h2;
    asm("{\n\t.reg .b8 q, z;\n\tmov.b16 {q, z}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, q;\n\t}" : "=r"(h2) : "h"(byte));
    const __half2 v = *reinterpret_cast<const __half2*>(&h2);
    back_lo = __low2float(v);
    back_hi = __high2float(v);
    return byte;
}

struct PrepArgs {
    const float* x;              // mode 0: [src rows][dim]; mode 1: gate [positions][dim]
    const float* up;             // mode 1: up [positions][dim]
    const uint32_t* sorted_row;  // [positions]; PDK_MOE_PAD = padding (zeros are written)
    const uint32_t* block_expert;  // [blocks]; PDK_MOE_PAD = unused block (its sorted_row entries are not defined; its rows are left as they are)
    uint8_t* xq;                 // [blocks][4*bm][dim/2]
    uint8_t* xs;                 // tiled: [blocks][slab][4 cells][512], the weight scale records' layout
    float* xstep;                // [positions] power of two the row was divided by
    uint32_t dim, bm, mode;  // mode 0 gather, 1 gated (x = gate, up), 2 relu(x)^2 of x [positions][dim],
                             // 3 one row: position 0 = x, the rest padding; the kernel writes the tables itself
    uint32_t* tables;        // mode 3: sorted_row[bm], block_expert[1] (written here), then f32 scale2 = table_scale2
    float table_scale2;
    uint32_t natural;        // 0: ggml MXFP4 element order (byte j = elements j, j+16); 1: byte j = elements 2j, 2j+1
    float alpha, limit, up_add;
};

// One CTA per block position.  Position (block b, token i) writes the four term rows
// b*4*bm + k*bm + i.  A 16-element scale group of the tensor core's element order is the
// two 8-runs (h*8 .. h*8+7) and (16 + h*8 .. 16 + h*8+7) of a 32-element block.
__device__ __forceinline__ void prep_position(const PrepArgs& a, uint32_t pos, uint32_t src) {
    const uint32_t b = pos / a.bm, i = pos % a.bm;
    const uint32_t tid = threadIdx.x;
    const uint32_t groups = a.dim >> 4, kh = a.dim >> 1;
    __shared__ float s_red[8];
    const bool pad = src == PDK_MOE_PAD;
    const float* row = (a.mode == 0u || a.mode == 3u) ? a.x + (size_t)(pad ? 0u : src) * a.dim : a.x + (size_t)pos * a.dim;
    const float* urow = a.up + (size_t)pos * a.dim;

    auto load8 = [&](uint32_t off, float (&v)[8]) {
        const float4 p = *reinterpret_cast<const float4*>(row + off);
        const float4 q = *reinterpret_cast<const float4*>(row + off + 4u);
        v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
        if (a.mode == 1u) {
            const float4 r = *reinterpret_cast<const float4*>(urow + off);
            const float4 t = *reinterpret_cast<const float4*>(urow + off + 4u);
            const float u[8] = {r.x, r.y, r.z, r.w, t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                // gated unit: (xg * sigmoid(alpha * xg)) * (yu + up_add); OpenAI variant (reference/ops.rs:27-36)
                // = alpha 1.702, limit 7, up_add 1; plain SwiGLU = alpha 1, limit inf, up_add 0
                const float xg = fminf(v[k], a.limit);
                const float yu = fminf(fmaxf(u[k], -a.limit), a.limit);
                v[k] = (xg / (1.0f + __expf(-a.alpha * xg))) * (yu + a.up_add);
            }
        } else if (a.mode == 2u) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float r = fmaxf(v[k], 0.0f);
                v[k] = r * r;
            }
        }
    };
    // first element of scale group g's two 8-runs
    auto run_base = [&](uint32_t g, uint32_t& lo_at, uint32_t& hi_at) {
        if (a.natural) { lo_at = g * 16u; hi_at = g * 16u + 8u; }
        else { lo_at = (g >> 1) * 32u + (g & 1u) * 8u; hi_at = lo_at + 16u; }
    };

    // ---- the row's largest magnitude -> the power of two that brings it into [256, 512).
    // When the CTA has a thread per group (dim <= 4096) the row is read once and kept in
    // registers across the reduction.
    const uint32_t num_kb = (a.dim + 255u) >> 8;
    const bool single = num_kb * 16u <= blockDim.x;
    float lo0[8], hi0[8];
    float amax = 0.0f;
    if (!pad)
        for (uint32_t g = tid; g < groups; g += blockDim.x) {
            uint32_t lo_at, hi_at;
            run_base(g, lo_at, hi_at);
            load8(lo_at, lo0);
            load8(hi_at, hi0);
#pragma unroll
            for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fmaxf(fabsf(lo0[k]), fabsf(hi0[k])));
        }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31u) == 0u) s_red[tid >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) amax = fmaxf(amax, s_red[w]);
    // amax = m * 2^ex with m in [1, 2): divide by 2^(ex - 8)
    const int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
    const bool live = !pad && amax > 0.0f && ex > -110 && ex < 120;
    const float inv_step = live ? __uint_as_float((uint32_t)(127 - (ex - 8)) << 23) : 0.0f;
    if (tid == 0) a.xstep[pos] = live ? __uint_as_float((uint32_t)(127 + (ex - 8)) << 23) : 0.0f;

    // ---- four terms per 16-element group
    const size_t r0 = (size_t)b * 4u * a.bm + i;
    uint8_t* xs_blk = a.xs + (size_t)b * num_kb * 2048u;
    if (!live) {
        // padding (half of the positions when most experts hold a ragged block) and all-zero rows: zero
        // term rows and scale bytes, none of the term arithmetic
        for (uint32_t g = tid; g < num_kb * 16u; g += blockDim.x) {
            uint8_t* xs_g = xs_blk + (size_t)(g >> 4) * 2048u + ((g >> 2) & 3u) * 512u + (g & 3u);
#pragma unroll
            for (uint32_t term = 0; term < 4u; ++term) {
                const uint32_t rr = term * a.bm + i;
                xs_g[(rr & 31u) * 16u + (rr >> 5) * 4u] = 0;
                if (g < groups) *reinterpret_cast<uint2*>(a.xq + (r0 + (size_t)term * a.bm) * kh + (size_t)g * 8u) = make_uint2(0u, 0u);
            }
        }
        return;
    }
    for (uint32_t g = tid; g < num_kb * 16u; g += blockDim.x) {
        // scale byte of group g and term row r: record g/16, cell (g/4)%4, byte (r%32)*16 + (r/32)*4 + g%4
        uint8_t* xs_g = xs_blk + (size_t)(g >> 4) * 2048u + ((g >> 2) & 3u) * 512u + (g & 3u);
        if (g >= groups) {  // past K: the record's cells must read as zero
#pragma unroll
            for (uint32_t term = 0; term < 4u; ++term) {
                const uint32_t r = term * a.bm + i;
                xs_g[(r & 31u) * 16u + (r >> 5) * 4u] = 0;
            }
            continue;
        }
        float lo[8], hi[8];
        if (live && !single) {
            uint32_t lo_at, hi_at;
            run_base(g, lo_at, hi_at);
            load8(lo_at, lo0);
            load8(hi_at, hi0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            lo[k] = live ? lo0[k] * inv_step : 0.0f;
            hi[k] = live ? hi0[k] * inv_step : 0.0f;
        }
#pragma unroll
        for (uint32_t term = 0; term < 4u; ++term) {
            float m = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) m = fmaxf(m, fmaxf(fabsf(lo[k]), fabsf(hi[k])));
            uint32_t sb = 0u;
            float sc = 0.0f, inv = 0.0f;
            if (m > 0.0f) {
                sb = (uint32_t)__nv_cvt_float_to_fp8(m * (1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3);
                if (sb == 0u) sb = 1u;
                sc = e4m3_to_f32(sb);
                inv = 1.0f / sc;
            }
            uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
            if (!a.natural) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {  // byte k = (lo run k, hi run k)
                    float bl, bh;
                    const uint32_t byte = e2m1x2_rn(lo[k] * inv, hi[k] * inv, bl, bh);
                    if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
                    lo[k] = (lo[k] - bl * sc) * 16.0f;
                    hi[k] = (hi[k] - bh * sc) * 16.0f;
                }
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {  // byte k = lo run (2k, 2k+1); byte 4+k = hi run (2k, 2k+1)
                    float b0, b1;
                    uint32_t byte = e2m1x2_rn(lo[2 * k] * inv, lo[2 * k + 1] * inv, b0, b1);
                    w0 |= byte << (8 * k);
                    lo[2 * k] = (lo[2 * k] - b0 * sc) * 16.0f;
                    lo[2 * k + 1] = (lo[2 * k + 1] - b1 * sc) * 16.0f;
                    byte = e2m1x2_rn(hi[2 * k] * inv, hi[2 * k + 1] * inv, b0, b1);
                    w1 |= byte << (8 * k);
                    hi[2 * k] = (hi[2 * k] - b0 * sc) * 16.0f;
                    hi[2 * k + 1] = (hi[2 * k + 1] - b1 * sc) * 16.0f;
                }
            }
            const size_t r = r0 + (size_t)term * a.bm;
            *reinterpret_cast<uint2*>(a.xq + r * kh + (size_t)g * 8u) = make_uint2(w0, w1);
            const uint32_t rr = term * a.bm + i;
            xs_g[(rr & 31u) * 16u + (rr >> 5) * 4u] = (uint8_t)sb;
        }
    }
}

__global__ void __launch_bounds__(256) moe_prep_f4_kernel(const PrepArgs a) {
    // dependent launch: may start while the previous kernel of the stream drains; its results are awaited here
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    const uint32_t pos = blockIdx.x;
    uint32_t src;
    if (a.mode == 3u) {
        src = pos == 0u ? 0u : PDK_MOE_PAD;
        if (threadIdx.x == 0) {
            a.tables[pos] = src;
            if (pos == 0u) {
                a.tables[a.bm] = 0u;  // block 0 belongs to expert 0
                reinterpret_cast<float*>(a.tables)[a.bm + 1u] = a.table_scale2;
            }
        }
    } else {
        if (a.block_expert[pos / a.bm] == PDK_MOE_PAD) return;   // an unused block: the GEMMs skip it, nothing reads its rows
        src = a.sorted_row[pos];
    }
    prep_position(a, pos, src);
}

// Decode widths (rows * k <= 32 pairs): routing, alignment and the first activation preparation in
// one launch.  Every CTA (one per block position, as above) routes the few tokens itself - a warp
// per token for the top-k, one warp for the alignment of at most 32 pairs: rank inside an expert
// from __match_any_sync, first block of an expert from the block counts of the lower experts - and
// then prepares its own position; CTA 0 also leaves the routing tables in global memory for the
// GEMMs and the combine.  The layout is moe_align's: blocks in ascending expert order, a block's
// entries in ascending pair order, unused blocks marked PDK_MOE_PAD.
struct RouteArgs {
    const float* logits;     // [rows][n_expert]
    const float* bias;       // [n_expert] or null
    uint32_t* idx;           // out [rows][k]
    float* w;                // out [rows][k]
    uint32_t* sorted_row;    // out [max_blocks * bm]
    uint32_t* sorted_slot;   // out [max_blocks * bm]
    uint32_t* block_expert;  // out [max_blocks]
    uint32_t rows, k, n_expert, max_blocks;
};
constexpr uint32_t kRouteMaxPos = 32u * 32u;

__global__ void __launch_bounds__(256) moe_route_prep_f4_kernel(const PrepArgs a, const RouteArgs r) {
    __shared__ uint32_t s_idx[32];
    __shared__ float s_w[32];
    __shared__ uint32_t s_row[kRouteMaxPos], s_slot[kRouteMaxPos], s_bexp[32];
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t npairs = r.rows * r.k, n_pos = r.max_blocks * a.bm;
    if (warp < r.rows) moe_route::topk_warp(r.logits + (size_t)warp * r.n_expert, r.bias, r.n_expert, r.k, lane, s_idx + warp * r.k, s_w + warp * r.k);
    for (uint32_t p = tid; p < n_pos; p += blockDim.x) { s_row[p] = PDK_MOE_PAD; s_slot[p] = 0u; }
    if (tid < 32u) s_bexp[tid] = PDK_MOE_PAD;
    __syncthreads();
    if (warp == 0u) {
        const bool valid = lane < npairs;
        const uint32_t e = valid ? s_idx[lane] : 0xfffffff0u + lane;     // idle lanes: distinct keys that match nobody
        const uint32_t grp = __match_any_sync(0xffffffffu, e);
        const uint32_t rank = __popc(grp & ((1u << lane) - 1u)), cnt = __popc(grp);
        const uint32_t nblk = (valid && rank == 0u) ? (cnt + a.bm - 1u) / a.bm : 0u;   // counted once, by the group's first lane
        uint32_t first = 0u;
        for (uint32_t q = 0; q < 32u; ++q) {
            const uint32_t eq = __shfl_sync(0xffffffffu, e, q), nq = __shfl_sync(0xffffffffu, nblk, q);
            if (eq < e) first += nq;
        }
        if (valid) {
            const uint32_t blk = first + rank / a.bm, at = blk * a.bm + rank % a.bm;
            if (blk < r.max_blocks) {
                s_row[at] = lane / r.k;
                s_slot[at] = lane % r.k;
                if (rank % a.bm == 0u) s_bexp[blk] = e;
            }
        }
    }
    __syncthreads();
    if (blockIdx.x == 0u) {
        if (tid < npairs) { r.idx[tid] = s_idx[tid]; r.w[tid] = s_w[tid]; }
        for (uint32_t p = tid; p < n_pos; p += blockDim.x) { r.sorted_row[p] = s_row[p]; r.sorted_slot[p] = s_slot[p]; }
        if (tid < r.max_blocks) r.block_expert[tid] = s_bexp[tid];
    }
    const uint32_t pos = blockIdx.x;
    if (s_bexp[pos / a.bm] == PDK_MOE_PAD) return;   // an unused block
    prep_position(a, pos, s_row[pos]);
}

// ---------------------------------------------------------------- grouped GEMM

struct GemmArgs {
    const uint8_t* w_sf[2];      // tiled UE4M3 weight scales per plane
    const float* scale2[2];      // per-plane factor (device memory), or per expert when scale2_per_expert
    const float* bias[2];        // [expert][out_dim] or null
    float* out[2];               // gate / up: [positions][out_dim]; down: part [(row, slot)][out_dim]
    const uint8_t* x_sf;         // tiled [blocks][slab][2048]
    const float* xstep;          // [positions]
    const uint32_t* block_expert;
    const uint32_t* sorted_row;
    const uint32_t* sorted_slot;  // down only
    const float* topk_w;          // down only
    uint32_t in_dim, out_dim, max_blocks, n_planes, n_active, scatter, scale2_per_expert;
    unsigned int* err_word;
};

// One tile = (block of BN/4 tokens, plane, 128 weight rows of the block's expert), walked
// by persistent CTAs.  Roles as in the dense NVFP4 GEMM: warp 0 producer (TMA boxes of W
// and of the block's term rows, bulk copies of both operands' scale records), warp 1 MMA issuer, warps 2..5 epilogue.
// WG: the weight scales are the row-major plane [rows][in_dim/16] (one expert) and the producer
// gathers them with 4-byte cp.async copies instead of bulk-copying pre-tiled records - for
// callers whose slot hands over the checkpoint's own scale plane (the W4A16 decode GEMV).
template <uint32_t BN, bool WG>
__global__ void __launch_bounds__(kThreads, 1)
moe_tc5_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1,
                    const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
    constexpr uint32_t kStages = Cfg<BN>::kStages, kBBytes = Cfg<BN>::kBBytes, kStageBytes = Cfg<BN>::kStageBytes;
    constexpr uint32_t kSfCol0 = Cfg<BN>::kSfCol0, kIdesc = Cfg<BN>::kIdesc, kSfCols = Cfg<BN>::kSfCols;
    constexpr uint32_t kOffB = Cfg<BN>::kOffB, kOffSfa = Cfg<BN>::kOffSfa, kOffSfb = Cfg<BN>::kOffSfb;
    constexpr uint32_t BT = BN / 4u;  // tokens per block
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * kStageBytes);
    uint32_t* s_expert = reinterpret_cast<uint32_t*>(sh + 1);  // block_expert[], read once per tile by every role

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row_tiles = (a.out_dim + BM - 1u) / BM, per_block = a.n_planes * row_tiles;
    const uint32_t n_tiles = a.max_blocks * per_block;
    const uint32_t n_mma = a.in_dim >> 6;                 // 64-element MMA steps (in_dim % 64 == 0)
    const uint32_t num_kb = (n_mma + 3u) >> 2;            // 256-element slabs, the last may be partial
    const uint32_t num_ks = (num_kb + KS - 1u) / KS;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], WG ? 33 : 1);  // expect_tx arrival (+ 32 lanes' cp.async arrivals)
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 4);
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_w0);
        tc5::tma_prefetch_desc(&tmap_w1);
        tc5::tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        tc5::tmem_alloc(&sh->tmem_base, kTmemCols);
        tc5::tmem_relinquish();
    }
    // dependent launch: barriers and tensor memory are set up while the previous kernel drains;
    // everything below reads what it wrote
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();
    for (uint32_t i = threadIdx.x; i < a.max_blocks; i += kThreads) s_expert[i] = a.block_expert[i];
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, a.err_word};

    if (warp == 0) {
        // ------------------------------------------------------------ producer (whole warp)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const uint32_t blk = tile / per_block, rem = tile % per_block;
            const uint32_t plane = rem / row_tiles, rt = rem % row_tiles;
            const uint32_t expert = s_expert[blk];
            if (expert == PDK_MOE_PAD) continue;
            const CUtensorMap* tw = plane ? &tmap_w1 : &tmap_w0;
            const uint8_t* wsf = a.w_sf[plane] + ((size_t)expert * row_tiles + rt) * num_kb * kSfBytes;
            const uint8_t* xsf = a.x_sf + (size_t)blk * num_kb * kSfBytes;
            for (uint32_t ks = 0; ks < num_ks; ++ks) {
                ok = tc5::mbar_wait(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* st = tiles + stage * kStageBytes;
                const uint32_t kb0 = ks * KS, nsl = min(KS, num_kb - kb0);
                tc5::mbar_arrive_expect_tx_elect(&sh->full[stage], nsl * (kABytes + kBBytes + (WG ? 1u : 2u) * kSfBytes));
#pragma unroll
                for (uint32_t u = 0; u < KS; ++u)
                    if (u < nsl) {
                        tc5::tma_load_2d_elect(st + u * kABytes, tw, &sh->full[stage], (int32_t)((kb0 + u) * BKB),
                                               (int32_t)(expert * a.out_dim + rt * BM));
                        tc5::tma_load_2d_elect(st + kOffB + u * kBBytes, &tmap_x, &sh->full[stage],
                                               (int32_t)((kb0 + u) * BKB), (int32_t)(blk * BN));
                    }
                if (!WG) {
                    tc5::bulk_load_elect(st + kOffSfa, wsf + (size_t)kb0 * kSfBytes, nsl * kSfBytes, &sh->full[stage]);
                } else {
                    // cell j of slab u: byte l*16 + c*4 + b = scale[rt*128 + c*32 + l][(kb0+u)*16 + j*4 + b]
                    const uint32_t sf_row = a.in_dim >> 4;
                    const uint32_t dst0 = tc5::smem_u32(st + kOffSfa) + lane * 16u;
#pragma unroll
                    for (uint32_t u = 0; u < KS; ++u)
                        if (u < nsl)
#pragma unroll
                            for (uint32_t j = 0; j < 4u; ++j) {
                                const uint32_t off = (kb0 + u) * 16u + j * 4u;
#pragma unroll
                                for (uint32_t c = 0; c < 4u; ++c) {
                                    const uint32_t row = rt * BM + c * 32u + lane;
                                    const uint32_t size = (row < a.out_dim && off < sf_row) ? 4u : 0u;
                                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(
                                                     dst0 + u * kSfBytes + j * 512u + c * 4u),
                                                 "l"(a.w_sf[plane] + (size ? (size_t)row * sf_row + off : 0u)), "r"(size)
                                                 : "memory");
                                }
                            }
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(
                                     tc5::smem_u32(&sh->full[stage]))
                                 : "memory");
                }
                tc5::bulk_load_elect(st + kOffSfb, xsf + (size_t)kb0 * kSfBytes, nsl * kSfBytes, &sh->full[stage]);
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
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            if (s_expert[tile / per_block] == PDK_MOE_PAD) continue;
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            ++iter;
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
                if (WG) fence_proxy_async_smem();  // the gathered cells were written through the generic proxy
                const uint32_t a_addr = tc5::smem_u32(tiles + stage * kStageBytes);
                const uint32_t nsl = min(KS, num_kb - ks * KS);
#pragma unroll
                for (uint32_t u = 0; u < KS; ++u) {
                    if (u >= nsl) break;
                    const uint32_t kb = ks * KS + u, steps = min(4u, n_mma - kb * 4u);
                    const uint32_t sfa_addr = a_addr + kOffSfa + u * kSfBytes, sfb_addr = a_addr + kOffSfb + u * kSfBytes;
                    const uint32_t sfa_t = tmem_base + kSfCol0 + stage * kSfCols + u * 32u, sfb_t = sfa_t + 16u;
                    const uint64_t a_desc = tc5::smem_desc_sw128(a_addr + u * kABytes);
                    const uint64_t b_desc = tc5::smem_desc_sw128(a_addr + kOffB + u * kBBytes);
                    slab_nvf4<true>(d_tmem, a_desc, b_desc, kIdesc, (ks | u) != 0u, sfa_t, sfb_t, sfa_addr, sfb_addr, steps);
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
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const uint32_t blk = tile / per_block, rem = tile % per_block;
            const uint32_t plane = rem / row_tiles, rt = rem % row_tiles;
            const uint32_t expert = s_expert[blk];
            if (expert == PDK_MOE_PAD) continue;
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            ++iter;
            ok = tc5::mbar_wait(&sh->tmem_full[buf], aphase, ctx, tc5::kErrTmemFullWait, buf);
            if (!ok) break;
            tc5::fence_after_sync();
            // lane = weight row; columns = term * BT + token
            float v[BT];
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + buf * BN;
            if (BN == 32u) {
                uint32_t r[32];
                tc5::tmem_ld_32x32(taddr, r);
                tc5::tmem_ld_wait();
#pragma unroll
                for (uint32_t i = 0; i < BT; ++i)
                    v[i] = __uint_as_float(r[i]) + __uint_as_float(r[BT + i]) * 0.0625f +
                           __uint_as_float(r[2u * BT + i]) * 0.00390625f +
                           __uint_as_float(r[3u * BT + i]) * 0.000244140625f;
            } else {
                float c = 1.0f;
#pragma unroll
                for (uint32_t term = 0; term < 4u; ++term) {
                    uint32_t r[32];
                    tc5::tmem_ld_32x32(taddr + term * 32u, r);
                    tc5::tmem_ld_wait();
#pragma unroll
                    for (uint32_t i = 0; i < 32u; ++i)
                        if (i < BT) v[i] = term == 0u ? __uint_as_float(r[i]) : fmaf(__uint_as_float(r[i]), c, v[i]);
                    c *= 0.0625f;
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(&sh->tmem_empty[buf]);  // the accumulator is in registers now

            // lane i < BT fetches token i's routing data once; the loop below broadcasts it
            const uint32_t my_pos = blk * BT + min(lane, BT - 1u);
            const uint32_t my_src = a.sorted_row[my_pos];
            uint32_t my_row = my_pos;  // output row: block position, or the (token, slot) pair
            float my_wgt = 1.0f;       // routing weight when scattering
            if (a.scatter && my_src != PDK_MOE_PAD) {
                my_row = my_src * a.n_active + a.sorted_slot[my_pos];
                my_wgt = a.topk_w[my_row];
            }
            const float my_mul = a.xstep[my_pos] * a.scale2[plane][a.scale2_per_expert ? expert : 0u] * my_wgt;
            const uint32_t n = rt * BM + quarter * 32u + lane;
            float bias = 0.0f;
            if (n < a.out_dim && a.bias[plane]) bias = a.bias[plane][(size_t)expert * a.out_dim + n];
            float* out = a.out[plane];
#pragma unroll
            for (uint32_t i = 0; i < BT; ++i) {
                const uint32_t src = __shfl_sync(0xffffffffu, my_src, i);
                const uint32_t row = __shfl_sync(0xffffffffu, my_row, i);
                const float mul = __shfl_sync(0xffffffffu, my_mul, i);
                const float wgt = __shfl_sync(0xffffffffu, my_wgt, i);
                if (src == PDK_MOE_PAD || n >= a.out_dim) continue;
                // (acc * scale2 * step + bias) * routing weight
                out[(size_t)row * a.out_dim + n] = fmaf(v[i], mul, bias * wgt);
            }
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, kTmemCols);
    }
}

constexpr uint32_t kMaxBlocks = 1024;  // block_expert[] is kept in shared memory

template <uint32_t BN, bool WG = false>
int launch_gemm(const CUtensorMap& tw0, const CUtensorMap& tw1, const CUtensorMap& tx, const GemmArgs& a,
                cudaStream_t st) {
    const size_t smem = (size_t)Cfg<BN>::kStages * Cfg<BN>::kStageBytes + sizeof(Shared) + kMaxBlocks * 4u + 1024u;
    auto kern = moe_tc5_gemm_kernel<BN, WG>;
    static const cudaError_t attr_rc =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr_rc != cudaSuccess) return (int)attr_rc;
    const uint32_t n_tiles = a.max_blocks * a.n_planes * ((a.out_dim + BM - 1u) / BM);
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_tiles) grid = n_tiles;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, tw0, tw1, tx, a);
}

}  // namespace

// No counterpart in the reference (its B200 MoE kernels run mma.sync on int8 activations):
// E8M0 scale plane [n_expert][rows][in_dim/32] -> tiled UE4M3 scale records
// [n_expert][ceil(rows/128)][ceil(in_dim/256)][2048] for pdk_mxfp4_moe_gemm_tc5, plus
// meta = {u32 largest scale byte, f32 scale2 = 2^(largest - 135)} (8 bytes, device memory).
// Load-time call; three launches on `stream`.
PDK_EXPORT int pdk_mxfp4_tc5_tile_scales(const void* scale, void* tiled, void* meta, uint32_t rows, uint32_t in_dim,
                                         uint32_t n_expert, void* stream) {
    if (rows == 0 || n_expert == 0) return 0;
    if (in_dim == 0 || (in_dim & 63u) != 0u || !pdk_aligned(tiled, 16) || !pdk_aligned(meta, 8))
        return cudaErrorInvalidValue;
    auto st = (cudaStream_t)stream;
    const uint32_t nblk = in_dim >> 5, row_tiles = (rows + 127u) / 128u, num_kb = (in_dim + 255u) >> 8;
    cudaError_t e = cudaMemsetAsync(meta, 0, 8, st);
    if (e != cudaSuccess) return (int)e;
    const uint64_t n = (uint64_t)n_expert * rows * nblk;
    const uint64_t want = (n + 1023u) / 1024u;
    mxfp4_emax_kernel<<<(uint32_t)(want < 1184u ? want : 1184u), 256, 0, st>>>((const uint8_t*)scale, n, (uint32_t*)meta);
    const uint32_t words = row_tiles * num_kb * 512u;
    mxfp4_tile_scales_kernel<<<dim3((words + 255u) / 256u < 64u ? (words + 255u) / 256u : 64u, n_expert), 256, 0, st>>>(
        (const uint8_t*)scale, (uint32_t*)tiled, rows, nblk, row_tiles, num_kb, (uint32_t*)meta);
    return pdk_launch_status();
}

// No counterpart in the reference: block positions -> four NVFP4 term rows each.
//   mode 0: position p takes row sorted_row[p] of x f32 [rows][dim]            (`up` unused)
//   mode 1: position p takes swiglu(x[p], up[p]) of the raw gate / up outputs f32 [positions][dim]
// Writes xq u8 [max_blocks*4*bm][dim/2], xs u8 [max_blocks][ceil(dim/256)][2048] (scale records in the
// weight scale records' layout; bytes of term rows a block does not have are left alone), xstep f32 [max_blocks*bm].
// dim % 32 == 0, bm 8 or 32.
static int prep_impl(const void* x, const void* up, const void* sorted_row, const void* block_expert, void* xq, void* xs,
                     void* xstep, uint32_t dim, uint32_t bm, uint32_t max_blocks, uint32_t mode, uint32_t natural,
                     float alpha, float limit, float up_add, void* stream) {
    if (max_blocks == 0) return 0;
    if (dim == 0 || (dim & 31u) != 0u || (bm != 8u && bm != 32u) || mode > 2u) return cudaErrorInvalidValue;
    if (!pdk_aligned(x, 16) || !pdk_aligned(xq, 16) || (mode == 1u && !pdk_aligned(up, 16))) return cudaErrorInvalidValue;
    PrepArgs a{};
    a.x = (const float*)x; a.up = (const float*)up; a.sorted_row = (const uint32_t*)sorted_row;
    a.block_expert = (const uint32_t*)block_expert;
    a.xq = (uint8_t*)xq; a.xs = (uint8_t*)xs; a.xstep = (float*)xstep;
    a.dim = dim; a.bm = bm; a.mode = mode; a.natural = natural; a.alpha = alpha; a.limit = limit; a.up_add = up_add;
    const uint32_t per_row = ((dim + 255u) >> 8) * 16u;  // scale groups incl. the zero tail of the last record
    return pdk_launch_pdl(moe_prep_f4_kernel, dim3(max_blocks * bm),
                          dim3(per_row <= 256u ? (per_row + 31u) & ~31u : 256u), 0, (cudaStream_t)stream, a);
}

PDK_EXPORT int pdk_moe_prep_act_f4(const void* x, const void* up, const void* sorted_row, const void* block_expert,
                                   void* xq, void* xs, void* xstep, uint32_t dim, uint32_t bm, uint32_t max_blocks,
                                   uint32_t mode, float alpha, float limit, void* stream) {
    if (mode > 1u) return cudaErrorInvalidValue;
    return prep_impl(x, up, sorted_row, block_expert, xq, xs, xstep, dim, bm, max_blocks, mode, 0u, alpha, limit, 1.0f,
                     stream);
}

// No counterpart in the reference.  moe_topk_batch + moe_align_bm + pdk_moe_prep_act_f4 (mode 0) in one
// launch for decode widths: rows * k <= 32 pairs, rows <= 8, n_expert <= 512, max_blocks <= 32.  Writes
// the same idx / w / sorted_row / sorted_slot / block_expert the three calls would, and the term rows.
PDK_EXPORT int pdk_moe_route_prep_f4(const void* logits, const void* router_bias, const void* x, void* idx, void* w,
                                     void* sorted_row, void* sorted_slot, void* block_expert, void* xq, void* xs, void* xstep,
                                     uint32_t n_expert, uint32_t k, uint32_t rows, uint32_t dim, uint32_t bm,
                                     uint32_t max_blocks, void* stream) {
    if (rows == 0 || max_blocks == 0) return 0;
    if (rows > 8u || k == 0 || k > 16u || rows * k > 32u || n_expert == 0 || n_expert > 512u || k > n_expert ||
        max_blocks > 32u || (bm != 8u && bm != 32u) || max_blocks * bm > kRouteMaxPos || dim == 0 || (dim & 31u) != 0u)
        return cudaErrorInvalidValue;
    if (!pdk_aligned(x, 16) || !pdk_aligned(xq, 16) || !pdk_aligned(xs, 16) || !pdk_aligned(logits, 4)) return cudaErrorInvalidValue;
    PrepArgs a{};
    a.x = (const float*)x;
    a.xq = (uint8_t*)xq; a.xs = (uint8_t*)xs; a.xstep = (float*)xstep;
    a.dim = dim; a.bm = bm; a.mode = 0u; a.natural = 0u; a.alpha = 1.0f; a.limit = 0.0f; a.up_add = 0.0f;
    RouteArgs r{};
    r.logits = (const float*)logits; r.bias = (const float*)router_bias;
    r.idx = (uint32_t*)idx; r.w = (float*)w;
    r.sorted_row = (uint32_t*)sorted_row; r.sorted_slot = (uint32_t*)sorted_slot; r.block_expert = (uint32_t*)block_expert;
    r.rows = rows; r.k = k; r.n_expert = n_expert; r.max_blocks = max_blocks;
    return pdk_launch_pdl(moe_route_prep_f4_kernel, dim3(max_blocks * bm), dim3(256), 0, (cudaStream_t)stream, a, r);
}

// The same for NVFP4 expert planes: term rows packed in the natural element order (byte j = elements
// 2j, 2j+1, as ModelOpt checkpoints store their weights).  mode 0 gather; mode 1 gated unit
// (min(g, limit) * sigmoid(alpha * that)) * (clamp(u, +-limit) + up_add) - plain SwiGLU is alpha 1,
// limit inf, up_add 0; mode 2 relu(x)^2 of x f32 [positions][dim] (the non-gated experts).
PDK_EXPORT int pdk_moe_prep_act_f4n(const void* x, const void* up, const void* sorted_row, const void* block_expert,
                                    void* xq, void* xs, void* xstep, uint32_t dim, uint32_t bm, uint32_t max_blocks,
                                    uint32_t mode, float alpha, float limit, float up_add, void* stream) {
    return prep_impl(x, up, sorted_row, block_expert, xq, xs, xstep, dim, bm, max_blocks, mode, 1u, alpha, limit, up_add,
                     stream);
}

// No counterpart in the reference (slots 88 / 89 are its mma.sync kernels on int8 activations):
// grouped expert GEMM over blocks aligned with block size bm.  Plane p (w*_data repacked MXFP4
// data [n_expert][out_dim][in_dim/2], w*_sf / w*_meta from pdk_mxfp4_tc5_tile_scales, bias
// [n_expert][out_dim] or NULL) times the term rows of pdk_moe_prep_act_f4.
//   scatter 0: out_p f32 [max_blocks*bm][out_dim] in block order, raw (bias added); one or two planes
//              (w1_data NULL = one)
//   scatter 1: out0 = part f32 [rows*n_active][out_dim], row (sorted_row, sorted_slot), times topk_w
// in_dim % 64 == 0, max_blocks <= 1024.
static int gemm_impl(const void* w0_data, const void* w0_sf, const float* w0_scale2, const void* w0_bias, void* out0,
                     const void* w1_data, const void* w1_sf, const float* w1_scale2, const void* w1_bias, void* out1,
                     const void* xq, const void* xs, const void* xstep, const void* block_expert, const void* sorted_row,
                     const void* sorted_slot, const void* topk_w, uint32_t in_dim, uint32_t out_dim, uint32_t n_expert,
                     uint32_t bm, uint32_t max_blocks, uint32_t n_active, uint32_t scatter, uint32_t scale2_per_expert,
                     void* stream) {
    if (max_blocks == 0 || out_dim == 0 || n_expert == 0) return 0;
    if (in_dim == 0 || (in_dim & 63u) != 0u || (bm != 8u && bm != 32u) || max_blocks > kMaxBlocks)
        return cudaErrorInvalidValue;
    if (!pdk_aligned(w0_data, 16) || !pdk_aligned(w0_sf, 16) || !pdk_aligned(xq, 16) || !pdk_aligned(xs, 4) ||
        !pdk_aligned(w0_scale2, 4) || (w1_data && (!pdk_aligned(w1_data, 16) || !pdk_aligned(w1_sf, 16))))
        return cudaErrorInvalidValue;
    if (scatter && (w1_data || !sorted_slot || !topk_w)) return cudaErrorInvalidValue;
    const uint32_t bn = 4u * bm, kbytes = in_dim >> 1;
    CUtensorMap tw0, tw1, tx;
    const uint64_t wrows = (uint64_t)n_expert * out_dim;
    if (int rc = pdk_make_tmap_2d(&tw0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w0_data, kbytes, wrows, kbytes, BKB, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tw1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w1_data ? w1_data : w0_data, kbytes, wrows,
                                  kbytes, BKB, BM))
        return rc;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, kbytes, (uint64_t)max_blocks * bn, kbytes,
                                  BKB, bn))
        return rc;
    GemmArgs a{};
    a.w_sf[0] = (const uint8_t*)w0_sf; a.w_sf[1] = (const uint8_t*)(w1_data ? w1_sf : w0_sf);
    a.scale2[0] = w0_scale2; a.scale2[1] = w1_data ? w1_scale2 : w0_scale2;
    a.scale2_per_expert = scale2_per_expert;
    a.bias[0] = (const float*)w0_bias; a.bias[1] = (const float*)w1_bias;
    a.out[0] = (float*)out0; a.out[1] = (float*)out1;
    a.x_sf = (const uint8_t*)xs; a.xstep = (const float*)xstep;
    a.block_expert = (const uint32_t*)block_expert; a.sorted_row = (const uint32_t*)sorted_row;
    a.sorted_slot = (const uint32_t*)sorted_slot; a.topk_w = (const float*)topk_w;
    a.in_dim = in_dim; a.out_dim = out_dim; a.max_blocks = max_blocks; a.n_planes = w1_data ? 2u : 1u;
    a.n_active = n_active; a.scatter = scatter; a.err_word = pdk_error_word();
    auto st = (cudaStream_t)stream;
    return bm == 8u ? launch_gemm<32>(tw0, tw1, tx, a, st) : launch_gemm<128>(tw0, tw1, tx, a, st);
}

PDK_EXPORT int pdk_mxfp4_moe_gemm_tc5(const void* w0_data, const void* w0_sf, const void* w0_meta, const void* w0_bias,
                                      void* out0, const void* w1_data, const void* w1_sf, const void* w1_meta,
                                      const void* w1_bias, void* out1, const void* xq, const void* xs,
                                      const void* xstep, const void* block_expert, const void* sorted_row,
                                      const void* sorted_slot, const void* topk_w, uint32_t in_dim, uint32_t out_dim,
                                      uint32_t n_expert, uint32_t bm, uint32_t max_blocks, uint32_t n_active,
                                      uint32_t scatter, void* stream) {
    if (!pdk_aligned(w0_meta, 8) || w0_meta == nullptr || (w1_data && w1_meta == nullptr)) return cudaErrorInvalidValue;
    return gemm_impl(w0_data, w0_sf, (const float*)w0_meta + 1, w0_bias, out0, w1_data, w1_sf,
                     w1_meta ? (const float*)w1_meta + 1 : nullptr, w1_bias, out1, xq, xs, xstep, block_expert, sorted_row,
                     sorted_slot, topk_w, in_dim, out_dim, n_expert, bm, max_blocks, n_active, scatter, 0u, stream);
}

// ---- NVFP4 expert planes (crates/paddock-engine/src/gpu/types.rs:176-226: data [expert*rows][in/2],
// scale e4m3 [expert*rows][in/16], scale2 f32 [expert]) on the same grouped GEMM.  No counterpart slot
// is served: the reference's NVFP4 MoE kernels take its Tiled64 / CutBlk plane orders.

// scale -> tiled records [n_expert][ceil(rows/128)][ceil(in_dim/256)][2048].  in_dim % 64 == 0.
PDK_EXPORT int pdk_nvf4_moe_tile_scales(const void* scale, void* tiled, uint32_t rows, uint32_t in_dim,
                                        uint32_t n_expert, void* stream) {
    if (rows == 0 || n_expert == 0) return 0;
    if (in_dim == 0 || (in_dim & 63u) != 0u || !pdk_aligned(tiled, 16) || !pdk_aligned(scale, 4))
        return cudaErrorInvalidValue;
    const uint32_t row_tiles = (rows + 127u) / 128u, num_kb = (in_dim + 255u) >> 8;
    const uint32_t words = row_tiles * num_kb * 512u;
    nvf4_moe_tile_scales_kernel<<<dim3((words + 255u) / 256u < 64u ? (words + 255u) / 256u : 64u, n_expert), 256, 0,
                                  (cudaStream_t)stream>>>((const uint8_t*)scale, (uint32_t*)tiled, rows, in_dim >> 4,
                                                          row_tiles, num_kb);
    return pdk_launch_status();
}

// pdk_mxfp4_moe_gemm_tc5 with NVFP4 planes: w*_sf from pdk_nvf4_moe_tile_scales, w*_scale2 f32 [n_expert],
// term rows from pdk_moe_prep_act_f4n.
PDK_EXPORT int pdk_nvf4_moe_gemm_tc5(const void* w0_data, const void* w0_sf, const void* w0_scale2, const void* w0_bias,
                                     void* out0, const void* w1_data, const void* w1_sf, const void* w1_scale2,
                                     const void* w1_bias, void* out1, const void* xq, const void* xs, const void* xstep,
                                     const void* block_expert, const void* sorted_row, const void* sorted_slot,
                                     const void* topk_w, uint32_t in_dim, uint32_t out_dim, uint32_t n_expert,
                                     uint32_t bm, uint32_t max_blocks, uint32_t n_active, uint32_t scatter,
                                     void* stream) {
    if (w0_scale2 == nullptr || (w1_data && w1_scale2 == nullptr)) return cudaErrorInvalidValue;
    return gemm_impl(w0_data, w0_sf, (const float*)w0_scale2, w0_bias, out0, w1_data, w1_sf, (const float*)w1_scale2,
                     w1_bias, out1, xq, xs, xstep, block_expert, sorted_row, sorted_slot, topk_w, in_dim, out_dim,
                     n_expert, bm, max_blocks, n_active, scatter, 1u, stream);
}

// ---------------------------------------------------------------- W4A16 decode GEMV on the same kernels
// pd_nvf4_gemv (slot 394) hands over the checkpoint's NVFP4 plane (row-major scales) and one f32
// activation vector.  On the tensor-core route the vector becomes four NVFP4 term rows (one
// "block" of one token) in a library-resident scratch slice and the grouped GEMM runs with one
// expert, gathering the weight scales from the row-major plane.  Two launches; the plane is
// streamed once at 4.5 bits per weight.  One scratch slice per stream for the first two streams
// that come here (the pack allocates nothing); other callers get -1 and take the plain kernel.
namespace {
constexpr uint32_t kGemvMaxK = 16384;
constexpr size_t kGemvXs = 128, kGemvXq = kGemvXs + (size_t)(kGemvMaxK / 256u) * 2048u;
constexpr size_t kGemvSlice = ((kGemvXq + 32u * (kGemvMaxK / 2u)) + 1023u) & ~(size_t)1023u;
constexpr int kGemvLanes = 2;
__device__ __align__(1024) uint8_t g_gemv_scratch[kGemvLanes][kGemvSlice];

PDK_SLICE_TABLE(gemv_slice_table, g_gemv_scratch, kGemvSlice, kGemvLanes);
uint8_t* gemv_slice(cudaStream_t st) { return gemv_slice_table.slice(st); }
}  // namespace

// 0 / cudaError_t, or -1 when the route does not apply (in_dim not a multiple of 64 or above 16384,
// no scratch slice for this stream) and the caller should use its own kernel.
int pdk_nvf4_gemv_tc5(const void* data, const void* scale, const void* bias, const void* x, void* y, float scale2,
                      uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    if ((in_dim & 63u) != 0u || in_dim > kGemvMaxK || !pdk_aligned(data, 16) || !pdk_aligned(scale, 4) ||
        !pdk_aligned(x, 16))
        return -1;
    uint8_t* sl = gemv_slice(st);
    if (sl == nullptr) return -1;
    uint32_t* tables = reinterpret_cast<uint32_t*>(sl);          // sorted_row[8], block_expert[1], f32 scale2
    float* xstep = reinterpret_cast<float*>(sl + 64);
    uint8_t* xs = sl + kGemvXs;
    uint8_t* xq = sl + kGemvXq;
    PrepArgs pa{};
    pa.x = (const float*)x; pa.xq = xq; pa.xs = xs; pa.xstep = xstep;
    pa.dim = in_dim; pa.bm = 8u; pa.mode = 3u; pa.natural = 1u; pa.tables = tables; pa.table_scale2 = scale2;
    const uint32_t per_row = ((in_dim + 255u) >> 8) * 16u;
    if (int rc = pdk_launch_pdl(moe_prep_f4_kernel, dim3(8), dim3(per_row <= 256u ? (per_row + 31u) & ~31u : 256u), 0,
                                st, pa))
        return rc;
    const uint32_t kbytes = in_dim >> 1;
    CUtensorMap tw, tx;
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, kbytes, out_dim, kbytes, BKB, BM)) return rc;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, kbytes, 32u, kbytes, BKB, 32u)) return rc;
    GemmArgs a{};
    a.w_sf[0] = a.w_sf[1] = (const uint8_t*)scale;
    a.scale2[0] = a.scale2[1] = reinterpret_cast<const float*>(tables) + 9;
    a.bias[0] = (const float*)bias;
    a.out[0] = (float*)y;
    a.x_sf = xs; a.xstep = xstep;
    a.block_expert = tables + 8; a.sorted_row = tables;
    a.in_dim = in_dim; a.out_dim = out_dim; a.max_blocks = 1u; a.n_planes = 1u; a.n_active = 1u;
    a.err_word = pdk_error_word();
    return launch_gemm<32, true>(tw, tw, tx, a, st);
}
