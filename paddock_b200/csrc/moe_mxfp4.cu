// moe_mxfp4.cu - MXFP4 expert GEMMs over expert-aligned token blocks
// (gate + up + SwiGLU, then down), the MoE half of the quantized linear path.
//
// HBM-bound at decode widths: a routed expert's 13 MB of 4.25-bit weights are read
// once for a handful of tokens.  Weights stay packed until they are in registers.
// An e2m1 nibble (s e1 e0 m) placed at bits (15 | 11 10 | 9) of an f16 is exactly
// e2m1 * 2^-14 - the f16 subnormal range continues the e2m1 grid, so codes 0 and 1
// need no special case - which costs two shifts and two logic ops per nibble pair
// and no lookup.  The products run on the tensor cores (mma m16n8k16 f16 -> f32).
// A ggml MXFP4 block keeps element j in the low nibble of byte j and element j+16
// in the high nibble; lane t takes word t of each 16-byte block (elements 4t..4t+3
// and 16+4t..16+4t+3) and the activation operand is stored in the matching order,
// so the k permutation costs nothing.
// Activations arrive as f16 with one power-of-two step per row (pdk_moe_prep_act):
// bf16 activations are carried exactly, general f32 ones to 11 significant bits.
// Lane t of a row loads whole 16-byte blocks (block 4*group + t), so the four
// lanes of a row read 64 contiguous bytes per step.  Each block is multiplied in
// f16 by 2^(its E8M0 exponent - the largest of the warp's K slice) - exact - so
// every mma of the slice accumulates into one tile; the common scale, the row
// step, bias, SwiGLU and the routing weight are applied in the epilogue.
//
// A CTA works on one aligned block of BM = 8*NT tokens.  NT = 1 (BM = 8) is the
// decode shape: 4 row tiles x 4 K slices per CTA, several CTAs per SM.  NT = 4
// (BM = 32) is the prefill shape: each expert's weights are read once per 32
// routed tokens, 16 row tiles per CTA, one CTA per SM.
#include "pdk_common.cuh"

namespace {

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1, const float (&)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Word of 8 nibbles n0..n7 -> four f16x2 registers holding (n0,n4), (n2,n6), (n1,n5), (n3,n7)
// as e2m1 * 2^-14: magnitude bits to f16 bits 9..11, sign bit to bit 15.
__device__ __forceinline__ void nib_to_f16x2(uint32_t w, uint32_t& p04, uint32_t& p26, uint32_t& p15, uint32_t& p37) {
    constexpr uint32_t M = 0x0E000E00u, S = 0x80008000u;
    p04 = ((w << 9) & M) | ((w << 12) & S);
    p15 = ((w << 5) & M) | ((w << 8) & S);
    p26 = ((w << 1) & M) | ((w << 4) & S);
    p37 = ((w >> 3) & M) | (w & S);
}
// E8M0 byte s -> 2^(s - 127) * 2^14 (the f16 values carry e2m1 * 2^-14)
__device__ __forceinline__ float e8m0_x2p14(uint32_t s) { return __uint_as_float(min(s + 14u, 254u) << 23); }

struct Args {
    const uint8_t* w0_data;   // gate (or down) nibbles  [expert][rows][nblk*16]
    const uint8_t* w0_scale;  //                 scales  [expert][rows][nblk]
    const float* w0_bias;     // [expert][rows] or null
    const uint8_t* w1_data;   // up planes (GATED only)
    const uint8_t* w1_scale;
    const float* w1_bias;
    const uint32_t* sorted_row;
    const uint32_t* sorted_slot;
    const uint32_t* block_expert;
    const float* topk_w;      // down only
    const uint8_t* xq;        // f16 [src rows][in_dim] in fragment order
    const float* xscale;      // [src rows]
    float* out;               // GATED: h [max_blocks*BM][out_dim];  else part [rows*n_active][out_dim]
    uint32_t in_dim, out_dim, n_active;
    float alpha, limit;
};

// GATED: two planes + SwiGLU, activations gathered through sorted_row, output
// in block order.  !GATED: one plane, activations already in block order,
// output scattered to (token, slot) rows and scaled by the routing weight.
template <uint32_t NT, uint32_t SLOTS, uint32_t KS, bool GATED>
__global__ void __launch_bounds__(SLOTS * KS * 32)
moe_mxfp4_kernel(const Args a) {
    constexpr uint32_t BM = NT * 8u;
    constexpr uint32_t NP = GATED ? 2u : 1u;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t block = blockIdx.y;
    const uint32_t expert = a.block_expert[block];
    if (expert == PDK_MOE_PAD) return;

    const uint32_t in_dim = a.in_dim, out_dim = a.out_dim, nblk = in_dim >> 5;
    const uint32_t pitch = in_dim * 2u + 64u;  // bytes per staged token: keeps the 8 columns on distinct banks
    uint8_t* xs = smem;                                              // [BM][pitch]
    float* red = reinterpret_cast<float*>(smem + (size_t)BM * pitch);  // [2][SLOTS][KS][32][NP*NT*4]
    __shared__ uint32_t s_src[BM];
    __shared__ float s_scale[BM];

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / KS, slice = warp % KS;

    // ---- stage the block's activations
    if (tid < BM) {
        const uint32_t pos = block * BM + tid;
        const uint32_t src = GATED ? a.sorted_row[pos] : (a.sorted_row[pos] == PDK_MOE_PAD ? PDK_MOE_PAD : pos);
        s_src[tid] = src;
        s_scale[tid] = src == PDK_MOE_PAD ? 0.0f : a.xscale[src];
    }
    __syncthreads();
    {
        const uint32_t chunks = in_dim >> 3;  // 16-byte chunks per token
        for (uint32_t i = tid; i < BM * chunks; i += blockDim.x) {
            const uint32_t tok = i / chunks, c = i % chunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (s_src[tok] != PDK_MOE_PAD)
                v = *reinterpret_cast<const uint4*>(a.xq + (size_t)s_src[tok] * in_dim * 2u + (size_t)c * 16u);
            *reinterpret_cast<uint4*>(xs + (size_t)tok * pitch + (size_t)c * 16u) = v;
        }
    }
    __syncthreads();

    // K is walked in groups of four 32-element blocks; lane t owns block 4*grp + t of its rows
    const uint32_t n_grp = (nblk + 3u) >> 2;
    const uint32_t grp_lo = slice * n_grp / KS, grp_hi = (slice + 1u) * n_grp / KS;
    const size_t plane_rows = (size_t)expert * out_dim;
    const uint8_t* xs_lane = xs + (size_t)g * pitch;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    uint32_t iter = 0;

    for (uint32_t tile = blockIdx.x * SLOTS + slot; tile < n_tiles; tile += gridDim.x * SLOTS, ++iter) {
        const uint32_t r0 = min(tile * 16u + g, out_dim - 1u), r1 = min(tile * 16u + g + 8u, out_dim - 1u);
        const uint8_t* d[NP][2];
        const uint8_t* s[NP][2];
        d[0][0] = a.w0_data + (plane_rows + r0) * nblk * 16u;
        d[0][1] = a.w0_data + (plane_rows + r1) * nblk * 16u;
        s[0][0] = a.w0_scale + (plane_rows + r0) * nblk;
        s[0][1] = a.w0_scale + (plane_rows + r1) * nblk;
        if (GATED) {
            d[NP - 1][0] = a.w1_data + (plane_rows + r0) * nblk * 16u;
            d[NP - 1][1] = a.w1_data + (plane_rows + r1) * nblk * 16u;
            s[NP - 1][0] = a.w1_scale + (plane_rows + r0) * nblk;
            s[NP - 1][1] = a.w1_scale + (plane_rows + r1) * nblk;
        }
        float acc[NP][NT][4];
#pragma unroll
        for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
            for (uint32_t n = 0; n < NT; ++n) acc[p][n][0] = acc[p][n][1] = acc[p][n][2] = acc[p][n][3] = 0.0f;

        // Common power of two of this warp's K slice, per plane and row: the largest E8M0
        // byte among the slice's blocks.  Every block is brought to it in f16 (a
        // power-of-two multiply, exact for blocks within 24 binades of the largest; what
        // smaller blocks lose is below 2^-28 of the largest block, under f32 resolution), so all mmas of the slice
        // accumulate into one tile and the scale is applied once, in the epilogue.
        uint32_t smax[NP][2];
#pragma unroll
        for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
            for (uint32_t r = 0; r < 2u; ++r) {
                uint32_t m = 0u;
                for (uint32_t kb = grp_lo * 4u + t; kb < min(grp_hi * 4u, nblk); kb += 4u)
                    m = max(m, (uint32_t)__ldg(s[p][r] + kb));
                m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
                smax[p][r] = m;
            }

        // Register prefetch, DEPTH groups ahead: one 16-byte block per lane, row and plane;
        // the four lanes of a row bring four consecutive blocks.
        constexpr uint32_t DEPTH = (GATED && NT == 4) ? 2 : 3;  // what fits in 128 registers
        uint4 wq[DEPTH][NP][2];
        uint32_t sq[DEPTH][NP][2];
        auto fetch = [&](uint32_t slot_i, uint32_t grp) {
            const uint32_t kb = grp * 4u + t;
            const bool have = kb < nblk;
#pragma unroll
            for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
                for (uint32_t r = 0; r < 2u; ++r) {
                    wq[slot_i][p][r] = have ? pdk_ldg_stream16(d[p][r] + (size_t)kb * 16u) : make_uint4(0u, 0u, 0u, 0u);
                    sq[slot_i][p][r] = have ? (uint32_t)__ldg(s[p][r] + kb) : 0u;
                }
        };
#pragma unroll
        for (uint32_t i = 0; i < DEPTH; ++i)
            if (grp_lo + i < grp_hi) fetch(i, grp_lo + i);

        for (uint32_t g0 = grp_lo; g0 < grp_hi; g0 += DEPTH) {
#pragma unroll
            for (uint32_t i = 0; i < DEPTH; ++i) {
                const uint32_t grp = g0 + i;
                if (grp >= grp_hi) break;
                // block value in f16 = e2m1 * 2^-14 * 2^(sb - smax + 15) (the largest multiplier f16 holds):
                // at most 12, exact for blocks within 24 binades of the largest, rounded to 2^-24 below
                __half2 h2[NP][2];
                uint32_t w[NP][2][4];
#pragma unroll
                for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
                    for (uint32_t r = 0; r < 2u; ++r) {
                        const int e = (int)sq[i][p][r] - (int)smax[p][r] + 15;
                        h2[p][r] = __half2half2(
                            __float2half_rn(e >= -24 ? __uint_as_float((uint32_t)(e + 127) << 23) : 0.0f));
                        // lane t walks its block's words in the order k ^ t, so that the four lanes'
                        // activation reads of one step fall on different shared-memory banks
                        uint32_t* ww = w[p][r];
                        ww[0] = wq[i][p][r].x; ww[1] = wq[i][p][r].y; ww[2] = wq[i][p][r].z; ww[3] = wq[i][p][r].w;
                        if (t & 1u) { const uint32_t a0 = ww[0], a2 = ww[2]; ww[0] = ww[1]; ww[1] = a0; ww[2] = ww[3]; ww[3] = a2; }
                        if (t & 2u) { const uint32_t a0 = ww[0], a1 = ww[1]; ww[0] = ww[2]; ww[2] = a0; ww[1] = ww[3]; ww[3] = a1; }
                    }
                if (grp + DEPTH < grp_hi) fetch(i, grp + DEPTH);
                const uint32_t kb = min(grp * 4u + t, nblk - 1u);  // lanes past the end hold zero weights
#pragma unroll
                for (uint32_t k = 0; k < 4u; ++k) {
                    // word k of both rows and planes -> scaled f16x2 pairs (e0,e2) (e1,e3) (e16,e18) (e17,e19)
                    uint32_t qa[NP][2][4];
#pragma unroll
                    for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
                        for (uint32_t r = 0; r < 2u; ++r) {
                            uint32_t c[4];
                            nib_to_f16x2(w[p][r][k], c[0], c[1], c[2], c[3]);
#pragma unroll
                            for (uint32_t u = 0; u < 4u; ++u) {
                                const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&c[u]), h2[p][r]);
                                qa[p][r][u] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                        }
#pragma unroll
                    for (uint32_t n = 0; n < NT; ++n) {
                        const uint4 b = *reinterpret_cast<const uint4*>(xs_lane + (size_t)n * 8u * pitch +
                                                                        (size_t)kb * 64u + ((k ^ t) * 16u));
#pragma unroll
                        for (uint32_t p = 0; p < NP; ++p) {
                            mma_f16(acc[p][n], qa[p][0][0], qa[p][1][0], qa[p][0][1], qa[p][1][1], b.x, b.y, acc[p][n]);
                            mma_f16(acc[p][n], qa[p][0][2], qa[p][1][2], qa[p][0][3], qa[p][1][3], b.z, b.w, acc[p][n]);
                        }
                    }
                }
            }
        }
        // true weight = stored * 2^(smax - 128)
#pragma unroll
        for (uint32_t p = 0; p < NP; ++p) {
            const float f0 = smax[p][0] >= 2u ? __uint_as_float((smax[p][0] - 1u) << 23) : 0.0f;
            const float f1 = smax[p][1] >= 2u ? __uint_as_float((smax[p][1] - 1u) << 23) : 0.0f;
#pragma unroll
            for (uint32_t n = 0; n < NT; ++n) {
                acc[p][n][0] *= f0; acc[p][n][1] *= f0;
                acc[p][n][2] *= f1; acc[p][n][3] *= f1;
            }
        }

        // ---- fold the K slices in shared memory (fixed order), slice 0 finishes the tile
        if (KS > 1u) {
            constexpr uint32_t PER = NP * NT * 4u;
            float* rb = red + ((size_t)(iter & 1u) * SLOTS + slot) * (KS * 32u * PER);
            if (slice != 0u) {
                float* mine = rb + ((size_t)slice * 32u + lane) * PER;
#pragma unroll
                for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
                    for (uint32_t n = 0; n < NT; ++n)
                        *reinterpret_cast<float4*>(mine + (p * NT + n) * 4u) =
                            make_float4(acc[p][n][0], acc[p][n][1], acc[p][n][2], acc[p][n][3]);
            }
            bar_sync(1u + slot, KS * 32u);
            if (slice != 0u) continue;
#pragma unroll
            for (uint32_t sl = 1; sl < KS; ++sl) {
                const float* other = rb + ((size_t)sl * 32u + lane) * PER;
#pragma unroll
                for (uint32_t p = 0; p < NP; ++p)
#pragma unroll
                    for (uint32_t n = 0; n < NT; ++n) {
                        const float4 v = *reinterpret_cast<const float4*>(other + (p * NT + n) * 4u);
                        acc[p][n][0] += v.x; acc[p][n][1] += v.y; acc[p][n][2] += v.z; acc[p][n][3] += v.w;
                    }
            }
        }

        // ---- epilogue: lane holds rows (g, g+8) x tokens (n*8 + 2t, +1)
#pragma unroll
        for (uint32_t n = 0; n < NT; ++n)
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                const uint32_t row = tile * 16u + g + (q >> 1) * 8u;
                const uint32_t tok = n * 8u + 2u * t + (q & 1u);
                if (row >= out_dim || s_src[tok] == PDK_MOE_PAD) continue;
                const float xsc = s_scale[tok];
                float v0 = acc[0][n][q] * xsc;
                if (a.w0_bias) v0 += a.w0_bias[plane_rows + row];
                if (GATED) {
                    float v1 = acc[NP - 1][n][q] * xsc;
                    if (a.w1_bias) v1 += a.w1_bias[plane_rows + row];
                    // SwiGLU, OpenAI variant: gate clamped from above, up symmetrically, up + 1
                    const float xg = fminf(v0, a.limit);
                    const float yu = fminf(fmaxf(v1, -a.limit), a.limit);
                    const float h = (xg / (1.0f + __expf(-a.alpha * xg))) * (yu + 1.0f);
                    a.out[((size_t)block * BM + tok) * out_dim + row] = h;
                } else {
                    const uint32_t pos = block * BM + tok;
                    const uint32_t pair = a.sorted_row[pos] * a.n_active + a.sorted_slot[pos];
                    a.out[(size_t)pair * out_dim + row] = a.topk_w[pair] * v0;
                }
            }
    }
}

template <uint32_t NT, uint32_t SLOTS, uint32_t KS, bool GATED>
int launch_cfg(const Args& a, uint32_t max_blocks, cudaStream_t st, uint32_t waves = 2u) {
    constexpr uint32_t BM = NT * 8u, NP = GATED ? 2u : 1u;
    const size_t smem = (size_t)BM * (a.in_dim * 2u + 64u) + (KS > 1u ? (size_t)2u * SLOTS * KS * 32u * NP * NT * 4u * 4u : 0u);
    if (smem > 220u * 1024u) return cudaErrorNotSupported;
    auto kern = moe_mxfp4_kernel<NT, SLOTS, KS, GATED>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = (a.out_dim + 15u) / 16u;
    // enough row groups that the used blocks fill the machine about `waves` times
    uint32_t groups = (waves * (uint32_t)pdk_sm_count() + max_blocks - 1u) / max_blocks;
    const uint32_t max_groups = (n_tiles + SLOTS - 1u) / SLOTS;
    if (groups > max_groups) groups = max_groups;
    if (groups < 1u) groups = 1u;
    kern<<<dim3(groups, max_blocks), SLOTS * KS * 32u, smem, st>>>(a);
    return pdk_launch_status();
}

// Decode blocks (8 tokens): with few blocks a CTA splits K over four warps per tile so that
// even one token's four experts fill the machine; with many blocks each warp walks the whole
// K of its tile - one pipeline fill per tile instead of four, no cross-warp fold.
bool wide_decode(const Args& a, uint32_t max_blocks) {
    static const int force = [] {
        const char* e = getenv("PDK_MOE_DECODE_CFG");
        return e ? atoi(e) : -1;
    }();
    if (force >= 0) return force == 1;
    const uint32_t n_tiles = (a.out_dim + 15u) / 16u;
    return max_blocks * ((n_tiles + 15u) / 16u) >= 2u * (uint32_t)pdk_sm_count();
}

int check_common(const Args& a, uint32_t bm, uint32_t max_blocks) {
    if (bm != 8u && bm != 32u) return cudaErrorInvalidValue;
    if (a.in_dim == 0u || (a.in_dim & 31u) != 0u || a.out_dim == 0u || max_blocks == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(a.w0_data, 4) || !pdk_aligned(a.xq, 16) || !pdk_aligned(a.out, 4)) return cudaErrorInvalidValue;
    if (max_blocks > 65535u) return cudaErrorInvalidValue;
    return 0;
}

}  // namespace

// No slot (the reference's counterpart is slot 88, packs/cuda/src/moe/mmq.cuh:550-590, whose
// activation operands are int8): gate + up + SwiGLU over blocks aligned with block size bm
// (8 or 32).  h f32 [max_blocks*bm][ff] in block order; rows of padding entries are not written.
PDK_EXPORT int pdk_mxfp4_moe_gate_up(const void* gate_data, const void* gate_scale, const void* gate_bias,
                                     const void* up_data, const void* up_scale, const void* up_bias,
                                     const void* sorted_row, const void* block_expert, const void* xq,
                                     const void* xscale, void* h, uint32_t in_dim, uint32_t ff, uint32_t bm,
                                     uint32_t max_blocks, float alpha, float limit, void* stream) {
    Args a{};
    a.w0_data = (const uint8_t*)gate_data; a.w0_scale = (const uint8_t*)gate_scale; a.w0_bias = (const float*)gate_bias;
    a.w1_data = (const uint8_t*)up_data; a.w1_scale = (const uint8_t*)up_scale; a.w1_bias = (const float*)up_bias;
    a.sorted_row = (const uint32_t*)sorted_row; a.block_expert = (const uint32_t*)block_expert;
    a.xq = (const uint8_t*)xq; a.xscale = (const float*)xscale; a.out = (float*)h;
    a.in_dim = in_dim; a.out_dim = ff; a.alpha = alpha; a.limit = limit;
    if (max_blocks == 0) return 0;
    if (int rc = check_common(a, bm, max_blocks)) return rc;
    if (!pdk_aligned(up_data, 4)) return cudaErrorInvalidValue;
    auto st = (cudaStream_t)stream;
    if (bm == 8u) return wide_decode(a, max_blocks) ? launch_cfg<1, 16, 1, true>(a, max_blocks, st, 4u)
                                                      : launch_cfg<1, 4, 4, true>(a, max_blocks, st);
    return launch_cfg<4, 16, 1, true>(a, max_blocks, st);
}

// No slot (reference counterpart slot 89, packs/cuda/src/moe/mmq.cuh:592-626): down projection of
// h (prepared with pdk_moe_prep_act, block order) into per-(token, slot) rows
// part f32 [rows*n_active][embd], each already times its routing weight.
PDK_EXPORT int pdk_mxfp4_moe_down(const void* down_data, const void* down_scale, const void* down_bias,
                                  const void* sorted_row, const void* sorted_slot, const void* block_expert,
                                  const void* topk_w, const void* hq, const void* hscale, void* part, uint32_t ff,
                                  uint32_t embd, uint32_t n_active, uint32_t bm, uint32_t max_blocks, void* stream) {
    Args a{};
    a.w0_data = (const uint8_t*)down_data; a.w0_scale = (const uint8_t*)down_scale; a.w0_bias = (const float*)down_bias;
    a.sorted_row = (const uint32_t*)sorted_row; a.sorted_slot = (const uint32_t*)sorted_slot;
    a.block_expert = (const uint32_t*)block_expert; a.topk_w = (const float*)topk_w;
    a.xq = (const uint8_t*)hq; a.xscale = (const float*)hscale; a.out = (float*)part;
    a.in_dim = ff; a.out_dim = embd; a.n_active = n_active;
    if (max_blocks == 0) return 0;
    if (int rc = check_common(a, bm, max_blocks)) return rc;
    auto st = (cudaStream_t)stream;
    if (bm == 8u) return wide_decode(a, max_blocks) ? launch_cfg<1, 16, 1, false>(a, max_blocks, st, 4u)
                                                      : launch_cfg<1, 4, 4, false>(a, max_blocks, st);
    return launch_cfg<4, 16, 1, false>(a, max_blocks, st);
}
