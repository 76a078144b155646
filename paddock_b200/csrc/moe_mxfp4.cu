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
    // ---- the reference's slot operands (pd_mxfp4_moe_*_mmq / *_dp4a_b), all zero on the pdk_ entry points
    const int8_t* xq8;        // int8 activations [src rows][in_dim] with xs32 f32 [src rows][in_dim/32] instead of xq / xscale
    const float* xs32;
    int8_t* out8;             // GATED: h as int8 [max_blocks*BM][out_dim] with outs f32 [..][out_dim/32] instead of `out`
    float* outs;
    uint32_t w0_pitch, w1_pitch;  // bytes between the rows of the data planes (0 = in_dim/2: a plain plane)
    uint32_t direct;          // 1: block b is pair b (one token), its expert block_expert[b], its source row b / n_active
                              // (GATED) or b (down), its output row b
    float up_add;             // SwiGLU: (up + up_add)
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
    __shared__ float s_inv[BM];
    __shared__ uint32_t s_amax[BM];

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / KS, slice = warp % KS;

    // ---- stage the block's activations
    if (tid < BM) {
        const uint32_t pos = block * BM + tid;
        uint32_t src;
        if (a.direct) src = tid == 0u ? (GATED ? block / a.n_active : block) : PDK_MOE_PAD;
        else src = GATED ? a.sorted_row[pos] : (a.sorted_row[pos] == PDK_MOE_PAD ? PDK_MOE_PAD : pos);
        s_src[tid] = src;
        s_scale[tid] = (src == PDK_MOE_PAD || a.xq8) ? 0.0f : a.xscale[src];
        s_amax[tid] = 0u;
    }
    __syncthreads();
    if (a.xq8 == nullptr) {
        const uint32_t chunks = in_dim >> 3;  // 16-byte chunks per token
        for (uint32_t i = tid; i < BM * chunks; i += blockDim.x) {
            const uint32_t tok = i / chunks, c = i % chunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (s_src[tok] != PDK_MOE_PAD)
                v = *reinterpret_cast<const uint4*>(a.xq + (size_t)s_src[tok] * in_dim * 2u + (size_t)c * 16u);
            *reinterpret_cast<uint4*>(xs + (size_t)tok * pitch + (size_t)c * 16u) = v;
        }
    } else {
        // int8 activations with one f32 scale per 32: the row's largest |q * s| picks a power-of-two
        // step for the row, then q * s / step is rounded to f16 (11 bits against the operand's 7) and
        // laid out in fragment order, as pdk_moe_prep_act would have
        for (uint32_t i = tid; i < BM * nblk; i += blockDim.x) {
            const uint32_t tok = i / nblk, kb = i % nblk, src = s_src[tok];
            if (src == PDK_MOE_PAD) continue;
            const int4 q0 = *reinterpret_cast<const int4*>(a.xq8 + (size_t)src * in_dim + (size_t)kb * 32u);
            const int4 q1 = *reinterpret_cast<const int4*>(a.xq8 + (size_t)src * in_dim + (size_t)kb * 32u + 16u);
            const int w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            int m = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int b = 0; b < 4; ++b) m = max(m, abs((int)(int8_t)(w[j] >> (8 * b))));
            const float v = (float)m * fabsf(a.xs32[(size_t)src * nblk + kb]);
            if (v == v && v < 3.0e38f) atomicMax(&s_amax[tok], __float_as_uint(v));
        }
        __syncthreads();
        if (tid < BM) {
            const float amax = __uint_as_float(s_amax[tid]);
            int e = 0;
            if (amax > 0.0f) e = max((int)(__float_as_uint(amax) >> 23) - 126 - 15, -100);   // amax / 2^e in [2^14, 2^15)
            s_scale[tid] = s_src[tid] == PDK_MOE_PAD ? 0.0f : __uint_as_float((uint32_t)(e + 127) << 23);
            s_inv[tid] = __uint_as_float((uint32_t)(127 - e) << 23);
        }
        __syncthreads();
        for (uint32_t i = tid; i < BM * nblk * 4u; i += blockDim.x) {   // one thread per (token, block, t): 8 elements
            const uint32_t tok = i / (nblk * 4u), r = i % (nblk * 4u), kb = r >> 2, tt = r & 3u, src = s_src[tok];
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (src != PDK_MOE_PAD) {
                const int8_t* q = a.xq8 + (size_t)src * in_dim + (size_t)kb * 32u;
                const int lo = *reinterpret_cast<const int*>(q + 4u * tt), hi = *reinterpret_cast<const int*>(q + 16u + 4u * tt);
                const float f = a.xs32[(size_t)src * nblk + kb] * s_inv[tok];
                auto el = [&](int wv, int b) { return (float)(int8_t)(wv >> (8 * b)) * f; };
                const __half2 h0 = __floats2half2_rn(el(lo, 0), el(lo, 2)), h1 = __floats2half2_rn(el(lo, 1), el(lo, 3));
                const __half2 h2 = __floats2half2_rn(el(hi, 0), el(hi, 2)), h3 = __floats2half2_rn(el(hi, 1), el(hi, 3));
                o.x = *reinterpret_cast<const uint32_t*>(&h0);
                o.y = *reinterpret_cast<const uint32_t*>(&h1);
                o.z = *reinterpret_cast<const uint32_t*>(&h2);
                o.w = *reinterpret_cast<const uint32_t*>(&h3);
            }
            *reinterpret_cast<uint4*>(xs + (size_t)tok * pitch + (size_t)kb * 64u + tt * 16u) = o;
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
        const size_t p0 = a.w0_pitch ? a.w0_pitch : nblk * 16u, p1 = a.w1_pitch ? a.w1_pitch : nblk * 16u;
        d[0][0] = a.w0_data + (plane_rows + r0) * p0;
        d[0][1] = a.w0_data + (plane_rows + r1) * p0;
        s[0][0] = a.w0_scale + (plane_rows + r0) * nblk;
        s[0][1] = a.w0_scale + (plane_rows + r1) * nblk;
        if (GATED) {
            d[NP - 1][0] = a.w1_data + (plane_rows + r0) * p1;
            d[NP - 1][1] = a.w1_data + (plane_rows + r1) * p1;
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
        float hv[NT][4];
#pragma unroll
        for (uint32_t n = 0; n < NT; ++n)
#pragma unroll
            for (uint32_t q = 0; q < 4u; ++q) {
                const uint32_t row = tile * 16u + g + (q >> 1) * 8u;
                const uint32_t tok = n * 8u + 2u * t + (q & 1u);
                hv[n][q] = 0.0f;
                if (row >= out_dim || s_src[tok] == PDK_MOE_PAD) continue;
                const float xsc = s_scale[tok];
                float v0 = acc[0][n][q] * xsc;
                if (a.w0_bias) v0 += a.w0_bias[plane_rows + row];
                const size_t orow = a.direct ? block : (size_t)block * BM + tok;
                if (GATED) {
                    float v1 = acc[NP - 1][n][q] * xsc;
                    if (a.w1_bias) v1 += a.w1_bias[plane_rows + row];
                    // SwiGLU, OpenAI variant: gate clamped from above, up symmetrically, up + up_add
                    const float xg = fminf(v0, a.limit);
                    const float yu = fminf(fmaxf(v1, -a.limit), a.limit);
                    const float h = (xg / (1.0f + __expf(-a.alpha * xg))) * (yu + a.up_add);
                    hv[n][q] = h;
                    if (a.out8 == nullptr) a.out[orow * out_dim + row] = h;
                } else {
                    const uint32_t pos = block * BM + tok;
                    const uint32_t pair = a.direct ? block : a.sorted_row[pos] * a.n_active + a.sorted_slot[pos];
                    a.out[(size_t)pair * out_dim + row] = a.topk_w[pair] * v0;
                }
            }
        if (GATED && KS == 1u && a.out8 != nullptr) {
            // h leaves as int8 with one f32 scale per 32 consecutive rows of a token (the slot's
            // hand-off to the down GEMM): tiles 2j and 2j + 1 belong to neighbouring warps, which
            // exchange their per-token maxima through shared memory (out_dim % 32 == 0, so both
            // take the same trips round this loop)
            float cm[NT][2];
#pragma unroll
            for (uint32_t n = 0; n < NT; ++n)
#pragma unroll
                for (uint32_t j = 0; j < 2u; ++j) {
                    float m = fmaxf(fabsf(hv[n][j]), fabsf(hv[n][2u + j]));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
                    cm[n][j] = m;
                }
            float* pb = red + ((size_t)(iter & 1u) * SLOTS + slot) * BM;       // `red` is unused when KS == 1
            const float* partner = red + ((size_t)(iter & 1u) * SLOTS + (slot ^ 1u)) * BM;
            if (g == 0u)
#pragma unroll
                for (uint32_t n = 0; n < NT; ++n) {
                    pb[n * 8u + 2u * t] = cm[n][0];
                    pb[n * 8u + 2u * t + 1u] = cm[n][1];
                }
            bar_sync(8u + (slot >> 1), 64u);
            const uint32_t nb32 = out_dim >> 5;
#pragma unroll
            for (uint32_t n = 0; n < NT; ++n)
#pragma unroll
                for (uint32_t j = 0; j < 2u; ++j) {
                    const uint32_t tok = n * 8u + 2u * t + j;
                    if (s_src[tok] == PDK_MOE_PAD) continue;
                    const float amax = fmaxf(cm[n][j], partner[tok]);
                    const float d = amax / 127.0f, id = d > 0.0f ? 1.0f / d : 0.0f;
                    const size_t orow = (size_t)block * BM + tok;
                    if (g == 0u && (slot & 1u) == 0u) a.outs[orow * nb32 + (tile >> 1)] = d;
#pragma unroll
                    for (uint32_t h = 0; h < 2u; ++h) {
                        const uint32_t row = tile * 16u + g + h * 8u;
                        const int q = max(-127, min(127, __float2int_rn(hv[n][2u * h + j] * id)));
                        a.out8[orow * out_dim + row] = (int8_t)q;
                    }
                }
        }
    }
}

template <uint32_t NT, uint32_t SLOTS, uint32_t KS, bool GATED>
int launch_cfg(const Args& a, uint32_t max_blocks, cudaStream_t st, uint32_t waves = 2u) {
    constexpr uint32_t BM = NT * 8u, NP = GATED ? 2u : 1u;
    const size_t smem = (size_t)BM * (a.in_dim * 2u + 64u) +
                        (KS > 1u ? (size_t)2u * SLOTS * KS * 32u * NP * NT * 4u * 4u : (size_t)2u * SLOTS * BM * 4u);
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
    if (!pdk_aligned(a.w0_data, 4) || !pdk_aligned(a.xq, 16) || !pdk_aligned(a.xq8, 16) || !pdk_aligned(a.out, 4))
        return cudaErrorInvalidValue;
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
    a.in_dim = in_dim; a.out_dim = ff; a.alpha = alpha; a.limit = limit; a.up_add = 1.0f;
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


// ---------------------------------------------------------------------------------------------
// The reference's own MoE slots for MXFP4 experts, served by the kernel above with int8
// activations staged as f16 (11 bits for the operand's 7) and, between gate|up and down, h handed
// over as int8 with one f32 scale per 32, exactly the buffers the engine allocates.
//
// The gate and up planes reach these slots fused into one plane by slot 155, whose contents are
// private to the pack.  This pack's fused row is [gate row | up row | padding to the reference's
// pitch]: both halves stay plain 16-byte-block rows, so the GEMM reads them like any other plane.
// ---------------------------------------------------------------------------------------------
namespace {

__global__ void gu_interleave_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ dst,
                                     uint32_t n_kb, uint64_t total) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte block of gate and of up
    if (i >= total) return;
    const uint64_t r = i / n_kb;
    const uint32_t b = (uint32_t)(i % n_kb);
    const uint64_t pitch16 = (uint64_t)((n_kb + 3u) >> 2) * 8u;           // row pitch in 16-byte units
    dst[r * pitch16 + b] = gate[i];
    dst[r * pitch16 + n_kb + b] = up[i];
}

inline uint32_t fused_pitch(uint32_t in_dim) { return (((in_dim >> 5) + 3u) >> 2) * 128u; }

// per-(device, stream) scratch of the decode pair: part f32 [batch * n_active][embd]
constexpr size_t kPairPartBytes = 1u << 20;
__device__ __align__(256) uint8_t g_pair_part[2][kPairPartBytes];
PDK_SLICE_TABLE(pair_part_table, g_pair_part, kPairPartBytes, 2);

}  // namespace

// slot 155, packs/cuda/src/gemm/f32_qkv.cuh:1474-1505: gate and up planes (16-byte blocks,
// n_kb per row) -> one plane of `rows` rows with the reference's pitch ceil(n_kb / 4) * 128.
PDK_EXPORT int pd_mxfp4_gu_interleave(const void* gate, const void* up, void* dst, uint32_t n_kb, uint64_t rows,
                                      void* stream) {
    if (rows == 0 || n_kb == 0) return 0;
    if (!pdk_aligned(gate, 16) || !pdk_aligned(up, 16) || !pdk_aligned(dst, 16)) return cudaErrorInvalidValue;
    const uint64_t total = rows * n_kb;
    if ((total + 255u) / 256u > 0x7fffffffull) return cudaErrorInvalidValue;
    gu_interleave_kernel<<<(uint32_t)((total + 255u) / 256u), 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)gate, (const uint4*)up, (uint4*)dst, n_kb, total);
    return pdk_launch_status();
}

// slot 88, packs/cuda/src/moe/mmq.cuh:550-571: gate + up + SwiGLU over 32-row expert blocks.
// gate_data = the fused plane of slot 155 (up_data is the engine's 16-byte dummy and is not
// read), xq int8 [tokens][in_dim] with xs f32 per 32, fq int8 [max_blocks*32][ff] with fs f32 per 32.
PDK_EXPORT int pd_mxfp4_moe_gate_up_mmq(const void* gate_data, const void* gate_scale, const void* gate_bias,
                                        const void* up_data, const void* up_scale, const void* up_bias,
                                        const void* sorted_row, const void* block_expert, const void* xq, const void* xs,
                                        void* fq, void* fs, uint32_t in_dim, uint32_t ff, uint32_t max_blocks, float alpha,
                                        float limit, float up_add, void* stream) {
    (void)up_data;
    if (ff == 0 || max_blocks == 0) return 0;
    if ((in_dim & 31u) || (ff & 31u) || in_dim == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(gate_data, 16) || !pdk_aligned(xs, 4) || !pdk_aligned(fq, 4) || !pdk_aligned(fs, 4))
        return cudaErrorInvalidValue;
    Args a{};
    a.w0_data = (const uint8_t*)gate_data; a.w0_scale = (const uint8_t*)gate_scale; a.w0_bias = (const float*)gate_bias;
    a.w1_data = (const uint8_t*)gate_data + (size_t)(in_dim >> 5) * 16u; a.w1_scale = (const uint8_t*)up_scale;
    a.w1_bias = (const float*)up_bias;
    a.w0_pitch = a.w1_pitch = fused_pitch(in_dim);
    a.sorted_row = (const uint32_t*)sorted_row; a.block_expert = (const uint32_t*)block_expert;
    a.xq8 = (const int8_t*)xq; a.xs32 = (const float*)xs; a.out8 = (int8_t*)fq; a.outs = (float*)fs;
    a.out = (float*)fs;   // not written on this path; check_common wants a pointer
    a.in_dim = in_dim; a.out_dim = ff; a.alpha = alpha; a.limit = limit; a.up_add = up_add;
    if (int rc = check_common(a, 32u, max_blocks)) return rc;
    return launch_cfg<4, 16, 1, true>(a, max_blocks, (cudaStream_t)stream);
}

// slot 89, packs/cuda/src/moe/mmq.cuh:592-626: down projection of the int8 h of slot 88 into
// per-(token, slot) rows part f32 [rows * n_active][embd], each times its routing weight.
PDK_EXPORT int pd_mxfp4_moe_down_mmq(const void* down_data, const void* down_scale, const void* down_bias,
                                     const void* sorted_row, const void* sorted_slot, const void* block_expert,
                                     const void* topk_w, const void* fq, const void* fs, void* part, uint32_t ff,
                                     uint32_t embd, uint32_t n_active, uint32_t max_blocks, void* stream) {
    if (embd == 0 || max_blocks == 0) return 0;
    if ((ff & 31u) || ff == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(fs, 4)) return cudaErrorInvalidValue;
    Args a{};
    a.w0_data = (const uint8_t*)down_data; a.w0_scale = (const uint8_t*)down_scale; a.w0_bias = (const float*)down_bias;
    a.sorted_row = (const uint32_t*)sorted_row; a.sorted_slot = (const uint32_t*)sorted_slot;
    a.block_expert = (const uint32_t*)block_expert; a.topk_w = (const float*)topk_w;
    a.xq8 = (const int8_t*)fq; a.xs32 = (const float*)fs; a.out = (float*)part;
    a.in_dim = ff; a.out_dim = embd; a.n_active = n_active;
    if (int rc = check_common(a, 32u, max_blocks)) return rc;
    return launch_cfg<4, 16, 1, false>(a, max_blocks, (cudaStream_t)stream);
}

// slot 92, packs/cuda/src/gemm/f32_qkv.cuh:370-383: the decode form of gate + up + SwiGLU
// (up + 1): no sorting, pair (token, slot) reads expert idx[pair]; out f32 [batch][n_active][ff].
PDK_EXPORT int pd_mxfp4_moe_gate_up_dp4a_b(const void* gate_data, const void* gate_scale, const void* gate_bias,
                                           const void* up_data, const void* up_scale, const void* up_bias, const void* idx,
                                           const void* xq, const void* xs, void* out, uint32_t in_dim, uint32_t ff,
                                           uint32_t n_active, uint32_t batch, float alpha, float limit, void* stream) {
    (void)up_data;
    if (ff == 0 || n_active == 0 || batch == 0) return 0;
    if ((in_dim & 31u) || in_dim == 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(gate_data, 16) || !pdk_aligned(xs, 4)) return cudaErrorInvalidValue;
    Args a{};
    a.w0_data = (const uint8_t*)gate_data; a.w0_scale = (const uint8_t*)gate_scale; a.w0_bias = (const float*)gate_bias;
    a.w1_data = (const uint8_t*)gate_data + (size_t)(in_dim >> 5) * 16u; a.w1_scale = (const uint8_t*)up_scale;
    a.w1_bias = (const float*)up_bias;
    a.w0_pitch = a.w1_pitch = fused_pitch(in_dim);
    a.block_expert = (const uint32_t*)idx;
    a.xq8 = (const int8_t*)xq; a.xs32 = (const float*)xs; a.out = (float*)out;
    a.in_dim = in_dim; a.out_dim = ff; a.n_active = n_active; a.alpha = alpha; a.limit = limit; a.up_add = 1.0f;
    a.direct = 1u;
    const uint32_t pairs = batch * n_active;
    if (int rc = check_common(a, 8u, pairs)) return rc;
    auto st = (cudaStream_t)stream;
    return wide_decode(a, pairs) ? launch_cfg<1, 16, 1, true>(a, pairs, st, 4u) : launch_cfg<1, 4, 4, true>(a, pairs, st);
}

// slot 93, packs/cuda/src/gemm/f32_qkv.cuh:385-398: the decode form of down: residual f32
// [batch][embd] += sum over a token's slots, in slot order, of weight * (W_down h + bias), with h
// int8 [batch * n_active][ff] and one f32 scale per 32.  The per-pair rows pass through a
// library-resident scratch slice (1 MiB per stream, two streams per device: 801 beyond either).
PDK_EXPORT int pd_mxfp4_moe_down_dp4a_b(const void* down_data, const void* down_scale, const void* down_bias,
                                        const void* idx, const void* topk_w, const void* fused_q, const void* fused_s,
                                        void* residual, uint32_t ff, uint32_t embd, uint32_t n_active, uint32_t batch,
                                        void* stream) {
    if (embd == 0 || n_active == 0 || batch == 0) return 0;
    if ((ff & 31u) || ff == 0u || (embd & 3u)) return cudaErrorInvalidValue;
    if (!pdk_aligned(fused_s, 4) || !pdk_aligned(residual, 16)) return cudaErrorInvalidValue;
    const uint64_t pairs = (uint64_t)batch * n_active;
    if (pairs > 65535u || pairs * embd * sizeof(float) > kPairPartBytes) return cudaErrorNotSupported;
    auto st = (cudaStream_t)stream;
    float* part = reinterpret_cast<float*>(pair_part_table.slice(st));
    if (part == nullptr) return cudaErrorNotSupported;
    Args a{};
    a.w0_data = (const uint8_t*)down_data; a.w0_scale = (const uint8_t*)down_scale; a.w0_bias = (const float*)down_bias;
    a.block_expert = (const uint32_t*)idx; a.topk_w = (const float*)topk_w;
    a.xq8 = (const int8_t*)fused_q; a.xs32 = (const float*)fused_s; a.out = part;
    a.in_dim = ff; a.out_dim = embd; a.n_active = n_active; a.direct = 1u;
    if (int rc = check_common(a, 8u, (uint32_t)pairs)) return rc;
    const int rc = wide_decode(a, (uint32_t)pairs) ? launch_cfg<1, 16, 1, false>(a, (uint32_t)pairs, st, 4u)
                                                   : launch_cfg<1, 4, 4, false>(a, (uint32_t)pairs, st);
    if (rc != 0) return rc;
    return pd_moe_slot_combine(part, residual, embd, n_active, batch, stream);
}
