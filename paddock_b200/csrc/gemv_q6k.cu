// gemv_q6k.cu - single-token decode GEMV for repacked Q6_K planes on the int8 tensor path.
//
// Q6_K: 256 weights per super-block as 16 blocks of 16, w = d * sc[block] * (q - 32) with 6-bit
// codes q (low nibbles in ql[128], two high bits in qh[64]), int8 block scales and one f16 d.
// The kernel is gemv_i8.cu's (persistent CTA per SM, 4 row tiles x 4 K slices, block-floating
// 15-bit activations in two int8 limbs, block-diagonal B operand so that an accumulator column
// is one block's integer dot product) with what 16-weight blocks change:
//   * 16 blocks need 16 columns: two accumulator tiles per limb, one per 128-weight half.
//     The mma count per super-block stays 8 per limb (256 weights / 32 k-slots);
//   * lane t of a row reads bytes [8t, 8t+8) of each 32-byte run of ql and qh (48 bytes of the
//     row's 192), i.e. 8 weights of each (half, 32-run); the mma for (half nh, run r) feeds
//     blocks 2r and 2r+1 of tile nh, and lane (g, t) supplies activations for it only when
//     g == 2r + t/2 (that lane's B column is the block its k-slots belong to);
//   * codes stay unsigned (0..63); the -32 goes through the 16-element activation sums.
// After the 8 mmas lane (g, t) holds, for rows g and g+8, blocks 2t and 2t+1 of both tiles -
// the 32-weight runs nh*128 + 32t - and folds them with their four scales in f32.
#include "pdk_common.cuh"

namespace {

constexpr uint32_t kSlots = 4, kSlices = 4, kThreads = kSlots * kSlices * 32, kDepth = 2;

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct Stage {
    uint2 qa[2][2], qb[2][2], qh[2][2];  // [row g / g+8][half]: ql[64 nh + 8t..], ql[64 nh + 32 + 8t..], qh[32 nh + 8t..]
    uint32_t d[2];                        // f16 d of the two rows (low half)
    uint32_t sc[2];                       // sc[2t], sc[2t+1], sc[8+2t], sc[8+2t+1] of the two rows (int8 each)
};

__device__ __forceinline__ void load_stage(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                           const uint8_t* r1, uint32_t t) {
    const uint8_t* dp[2] = {d0, d1};
    const uint8_t* rp[2] = {r0, r1};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
            s.qa[w][nh] = pdk_ldg_stream8(dp[w] + nh * 64u + t * 8u);
            s.qb[w][nh] = pdk_ldg_stream8(dp[w] + nh * 64u + 32u + t * 8u);
            s.qh[w][nh] = pdk_ldg_stream8(dp[w] + 128u + nh * 32u + t * 8u);
        }
        s.d[w] = __ldg(reinterpret_cast<const uint16_t*>(rp[w]));
        s.sc[w] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(rp[w] + 4u + 2u * t)) |
                  ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(rp[w] + 12u + 2u * t)) << 16);
    }
}

// Shared memory: limb planes int8 [2][K] (hi, lo), 32 zero bytes, xmeta float2 [K/32] = {step,
// unused}, x16 f32 [K/16] = step * (sum of the 16 integers), red f32 [2][kSlots][kSlices][16].
__global__ void __launch_bounds__(kThreads, 1)
gemv_q6k_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ recs, const float* __restrict__ x,
                float* __restrict__ y, uint32_t in_dim, uint32_t out_dim) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_blk = in_dim >> 5, n_unit = in_dim >> 8;
    uint8_t* xs_hi = smem;
    uint8_t* xs_lo = smem + in_dim;
    uint8_t* zeros = smem + 2u * (size_t)in_dim;
    float* xstep = reinterpret_cast<float*>(zeros + 32u);
    float* x16 = xstep + n_blk;
    float* red = x16 + 2u * n_blk;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / kSlices, slice = warp % kSlices;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t u_lo = slice * n_unit / kSlices, u_hi = (slice + 1u) * n_unit / kSlices;
    const uint32_t len = u_hi - u_lo;
    const size_t row_data = (size_t)n_unit * 192u, row_rec = (size_t)n_unit * 24u;
    const uint32_t tile0 = slot * gridDim.x + blockIdx.x, tile_stride = gridDim.x * kSlots;
    const uint32_t my_tiles = tile0 < n_tiles ? (n_tiles - tile0 + tile_stride - 1u) / tile_stride : 0u;
    const uint32_t total = my_tiles * len;

    uint32_t l_tile = tile0, l_u = u_lo;
    const uint8_t *p0 = data, *p1 = data, *r0 = recs, *r1 = recs;
    auto set_rows = [&](uint32_t tl) {
        const uint32_t ra = min(tl * 16u + g, out_dim - 1u), rb = min(tl * 16u + g + 8u, out_dim - 1u);
        p0 = data + ra * row_data;
        p1 = data + rb * row_data;
        r0 = recs + ra * row_rec;
        r1 = recs + rb * row_rec;
    };
    auto issue = [&](Stage& s) {
        load_stage(s, p0 + (size_t)l_u * 192u, p1 + (size_t)l_u * 192u, r0 + (size_t)l_u * 24u, r1 + (size_t)l_u * 24u, t);
        if (++l_u == u_hi) {
            l_u = u_lo;
            l_tile += tile_stride;
            if (l_tile < n_tiles) set_rows(l_tile);
        }
    };

    pdk_pdl_launch_dependents();
    Stage st[kDepth];
    if (total > 0u) {
        set_rows(tile0);
        issue(st[0]);
    }
    pdk_pdl_wait();

    // ---- activations -> block floating point limbs (per 32 elements), 8 elements per thread
    for (uint32_t grp = tid; grp < (in_dim >> 3); grp += kThreads) {
        const float4 a = *reinterpret_cast<const float4*>(x + grp * 8u);
        const float4 b = *reinterpret_cast<const float4*>(x + grp * 8u + 4u);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int ex = 0;
        float step = 1.0f, inv = 0.0f;
        if (amax > 0.0f && amax < 3.0e38f) {
            (void)frexpf(amax, &ex);
            ex = max(ex, -110);
            step = ldexpf(1.0f, ex - 14);
            inv = ldexpf(1.0f, 14 - ex);
        }
        uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
        int isum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = __float2int_rn(v[i] * inv);
            q = max(-16384, min(16384, q));
            const int h = (q + 128) >> 8, l = q - (h << 8);
            hi[i >> 2] |= ((uint32_t)h & 0xffu) << (8 * (i & 3));
            lo[i >> 2] |= ((uint32_t)l & 0xffu) << (8 * (i & 3));
            isum += q;
        }
        *reinterpret_cast<uint2*>(xs_hi + (size_t)grp * 8u) = make_uint2(hi[0], hi[1]);
        *reinterpret_cast<uint2*>(xs_lo + (size_t)grp * 8u) = make_uint2(lo[0], lo[1]);
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);  // 16 elements
        if ((grp & 1u) == 0u) x16[grp >> 1] = step * (float)isum;
        if ((grp & 3u) == 0u) xstep[grp >> 2] = step;
    }
    if (tid < 8u) reinterpret_cast<uint32_t*>(zeros)[tid] = 0u;
    __syncthreads();

    // this lane supplies activations to the mmas of run r_mine (both halves), if any
    const int rm2 = (int)g - (int)(t >> 1);
    const uint32_t r_mine = (rm2 >= 0 && (rm2 & 1) == 0) ? (uint32_t)rm2 >> 1 : 99u;

    float acc_g = 0.0f, acc_g8 = 0.0f;
    uint32_t c_u = u_lo, c_tile = tile0, iter = 0;

    auto compute = [&](const Stage& s, auto&& prefetch) {
        int ch[2][4], cl[2][4];
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
#pragma unroll
            for (int i = 0; i < 4; ++i) ch[nh][i] = cl[nh][i] = 0;
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r) {
                const uint32_t sh = (r >> 1) * 4u;
                const uint2 l0 = (r & 1u) ? s.qb[0][nh] : s.qa[0][nh], l1 = (r & 1u) ? s.qb[1][nh] : s.qa[1][nh];
                const uint2 h0 = s.qh[0][nh], h1 = s.qh[1][nh];
                const uint32_t a0 = ((l0.x >> sh) & 0x0F0F0F0Fu) | (((h0.x >> (2u * r)) & 0x03030303u) << 4);
                const uint32_t a2 = ((l0.y >> sh) & 0x0F0F0F0Fu) | (((h0.y >> (2u * r)) & 0x03030303u) << 4);
                const uint32_t a1 = ((l1.x >> sh) & 0x0F0F0F0Fu) | (((h1.x >> (2u * r)) & 0x03030303u) << 4);
                const uint32_t a3 = ((l1.y >> sh) & 0x0F0F0F0Fu) | (((h1.y >> (2u * r)) & 0x03030303u) << 4);
                const uint32_t xoff = c_u * 256u + nh * 128u + r * 32u + t * 8u;
                const uint2 bh = *reinterpret_cast<const uint2*>(r == r_mine ? xs_hi + xoff : zeros);
                const uint2 bl = *reinterpret_cast<const uint2*>(r == r_mine ? xs_lo + xoff : zeros);
                mma_s8(ch[nh], a0, a1, a2, a3, bh.x, bh.y);
                mma_s8(cl[nh], a0, a1, a2, a3, bl.x, bl.y);
            }
        }
        prefetch();
        // blocks 2t, 2t+1 of tile nh = the 32-weight run nh*128 + 32t: one step, two 16-element sums
        float vg = 0.0f, vg8 = 0.0f;
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
            const uint32_t blk = c_u * 8u + nh * 4u + t;
            const float step = xstep[blk];
            const float2 xs = *reinterpret_cast<const float2*>(x16 + 2u * blk);
            const float f0 = (float)(ch[nh][0] * 256 + cl[nh][0]) * step - 32.0f * xs.x;
            const float f1 = (float)(ch[nh][1] * 256 + cl[nh][1]) * step - 32.0f * xs.y;
            const float f2 = (float)(ch[nh][2] * 256 + cl[nh][2]) * step - 32.0f * xs.x;
            const float f3 = (float)(ch[nh][3] * 256 + cl[nh][3]) * step - 32.0f * xs.y;
            const float s0 = (float)(int8_t)((s.sc[0] >> (16u * nh)) & 0xffu), s1 = (float)(int8_t)((s.sc[0] >> (16u * nh + 8u)) & 0xffu);
            const float s2 = (float)(int8_t)((s.sc[1] >> (16u * nh)) & 0xffu), s3 = (float)(int8_t)((s.sc[1] >> (16u * nh + 8u)) & 0xffu);
            vg += s0 * f0 + s1 * f1;
            vg8 += s2 * f2 + s3 * f3;
        }
        acc_g += __half2float(__ushort_as_half((unsigned short)s.d[0])) * vg;
        acc_g8 += __half2float(__ushort_as_half((unsigned short)s.d[1])) * vg8;

        if (++c_u == u_hi) {
            c_u = u_lo;
            float a = acc_g, b = acc_g8;
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            b += __shfl_xor_sync(0xffffffffu, b, 1);
            b += __shfl_xor_sync(0xffffffffu, b, 2);
            float* rbuf = red + ((size_t)(iter & 1u) * kSlots + slot) * (kSlices * 16u);
            if (t == 0u) {
                rbuf[slice * 16u + g] = a;
                rbuf[slice * 16u + g + 8u] = b;
            }
            bar_sync(1u + slot, kSlices * 32u);
            const uint32_t r = slice * 32u + lane;
            if (r < 16u) {
                const float v = (rbuf[r] + rbuf[16u + r]) + (rbuf[32u + r] + rbuf[48u + r]);
                const uint32_t row = c_tile * 16u + r;
                if (row < out_dim) y[row] = v;
            }
            acc_g = acc_g8 = 0.0f;
            c_tile += tile_stride;
            ++iter;
        }
    };

    for (uint32_t q = 0; q < total; q += kDepth) {
#pragma unroll
        for (uint32_t d = 0; d < kDepth; ++d) {
            if (q + d >= total) break;
            compute(st[d], [&] {
                if (q + d + kDepth - 1u < total) issue(st[(d + kDepth - 1u) % kDepth]);
            });
        }
    }
}

}  // namespace

// Returns 0 / a cudaError_t, or -1 when the shape is outside the kernel's plan (K not a multiple
// of 256, fewer than four super-blocks per row, activations too long for shared memory).
int pdk_q6k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                    cudaStream_t st) {
    const uint32_t n_unit = in_dim >> 8;
    if ((in_dim & 255u) != 0u || n_unit < kSlices) return -1;
    const size_t smem = (size_t)in_dim * 2u + 32u + (size_t)(in_dim >> 5) * 12u + 2u * kSlots * kSlices * 16u * 4u;
    if (smem > 200u * 1024u) return -1;
    cudaError_t e = cudaFuncSetAttribute(gemv_q6k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    const uint32_t need = (n_tiles + kSlots - 1u) / kSlots;
    if (grid > need) grid = need;
    return pdk_launch_pdl(gemv_q6k_kernel, dim3(grid), dim3(kThreads), smem, st, (const uint8_t*)data, (const uint8_t*)scales,
                          x, y, in_dim, out_dim);
}
