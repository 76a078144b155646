// q4k_gemv_diag.cu - the single-token Q4_K decode GEMV.
//
// y[o] = sum over super-blocks of  d * sum_j sc_j * (sum_i q_ji x_ji)  -  dmin * sum_j m_j * (sum_i x_ji)
//
// HBM-bound (4.5 bits per weight, read once), so everything else has to stay
// far below one instruction per weight.  The 32-element inner sums run on the
// tensor cores (bf16 mma, f32 accumulate) with the nibbles as exact bf16
// integers 128+q.  With one token an 8-column mma would waste 7 columns, so the
// B operand is made block diagonal instead: the 16 k-slots of every mma are
// spread over the 8 sub-blocks of a super-block (2 slots each) and column c is
// non-zero only in sub-block c's slots.  After the 16 mmas of a super-block the
// accumulator tile holds C[row][c] = sum_i q x over sub-block c: all eight
// partial sums of 16 rows at once, and lane (g,t) owns exactly the two
// sub-blocks (2t, 2t+1) of rows g and g+8 whose scales it then applies in f32.
//
// Lane t of a row reads ggml group t of the super-block (32 contiguous bytes:
// sub-block 2t in the low nibbles, 2t+1 in the high nibbles), so a row's
// 128-byte super-block is one contiguous read by four lanes.
//
// Activations: x is split into bf16 hi + bf16 lo.  When every lo part is zero
// (the activations are bf16 values, the usual case) only the hi column runs;
// otherwise a second accumulator tile takes the lo parts, which keeps general
// f32 activations exact to 2^-17 relative.
#include "pdk_common.cuh"

namespace {

constexpr uint32_t kSlots = 4;    // 16-row tiles in flight per CTA
constexpr uint32_t kSlices = 4;   // K slices per tile, one warp each
constexpr uint32_t kThreads = kSlots * kSlices * 32;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct Stage {        // one super-block of rows g and g+8, as loaded
    uint4 q[4];       // row g bytes 0..15, 16..31 of group t; row g+8 likewise
    uint32_t dd[2];   // {f16 d, f16 dmin} of the two rows
    uint32_t sm[2];   // sc[2t] | sc[2t+1]<<8 | m[2t]<<16 | m[2t+1]<<24
};

// Shared memory: xs bf16 [2][pitch] (hi column, lo column; 8-element groups
// permuted [0,2,1,3,4,6,5,7]), 64 zero bytes, xsum f32 [K/32] (sum of hi+lo per
// sub-block), red f32 [2][kSlots][kSlices][16].
__global__ void __launch_bounds__(kThreads, 1)
q4k_gemv_diag_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                     const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim, uint32_t out_dim) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_sub = in_dim >> 5, n_super = in_dim >> 8;
    const uint32_t pitch = in_dim * 2u;
    uint8_t* xs = smem;
    uint8_t* zeros = smem + 2u * (size_t)pitch;
    float* xsum = reinterpret_cast<float*>(zeros + 64u);
    float* red = xsum + n_sub;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / kSlices, slice = warp % kSlices;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t sb_lo = slice * n_super / kSlices, sb_hi = (slice + 1u) * n_super / kSlices;
    const uint32_t len = sb_hi - sb_lo;
    const size_t row_data = (size_t)n_super * 128u, row_rec = (size_t)n_super * 24u;

    const uint32_t tile0 = blockIdx.x * kSlots + slot, tile_stride = gridDim.x * kSlots;
    const uint32_t my_tiles = tile0 < n_tiles ? (n_tiles - tile0 + tile_stride - 1u) / tile_stride : 0u;
    const uint32_t total = my_tiles * len;

    // ---- load cursor
    uint32_t l_tile = tile0, l_sb = sb_lo;
    const uint8_t *p0 = data, *p1 = data, *r0 = scales, *r1 = scales;
    auto set_rows = [&](uint32_t tl) {
        const uint32_t ra = min(tl * 16u + g, out_dim - 1u), rb = min(tl * 16u + g + 8u, out_dim - 1u);
        p0 = data + ra * row_data + t * 32u;
        p1 = data + rb * row_data + t * 32u;
        r0 = scales + ra * row_rec;
        r1 = scales + rb * row_rec;
    };
    auto issue = [&](Stage& s) {
        const uint8_t* a = p0 + (size_t)l_sb * 128u;
        const uint8_t* b = p1 + (size_t)l_sb * 128u;
        s.q[0] = pdk_ldg_stream16(a);
        s.q[1] = pdk_ldg_stream16(a + 16);
        s.q[2] = pdk_ldg_stream16(b);
        s.q[3] = pdk_ldg_stream16(b + 16);
        const uint8_t* ra = r0 + (size_t)l_sb * 24u;
        const uint8_t* rb = r1 + (size_t)l_sb * 24u;
        s.dd[0] = __ldg(reinterpret_cast<const uint32_t*>(ra));
        s.dd[1] = __ldg(reinterpret_cast<const uint32_t*>(rb));
        s.sm[0] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(ra + 4u + 2u * t)) |
                  ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(ra + 12u + 2u * t)) << 16);
        s.sm[1] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(rb + 4u + 2u * t)) |
                  ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(rb + 12u + 2u * t)) << 16);
        if (++l_sb == sb_hi) {
            l_sb = sb_lo;
            l_tile += tile_stride;
            if (l_tile < n_tiles) set_rows(l_tile);
        }
    };

    Stage st0, st1, st2;
    if (total > 0u) {
        set_rows(tile0);
        issue(st0);
        if (total > 1u) issue(st1);
    }

    // ---- stage the activation vector (hi / lo columns) and its sub-block sums
    int any_lo = 0;
    {
        const uint32_t groups = in_dim >> 3;
        for (uint32_t grp = tid; grp < groups; grp += kThreads) {  // grp = sub-block*4 + chunk
            const float4 a = *reinterpret_cast<const float4*>(x + grp * 8u);
            const float4 b = *reinterpret_cast<const float4*>(x + grp * 8u + 4u);
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            float hi[8], lo[8];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hi[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
                lo[i] = __bfloat162float(__float2bfloat16_rn(v[i] - hi[i]));
                any_lo |= (lo[i] != 0.0f);
                sum += hi[i] + lo[i];
            }
            uint4 wh, wl;
            wh.x = pack_bf16(hi[0], hi[2]); wh.y = pack_bf16(hi[1], hi[3]);
            wh.z = pack_bf16(hi[4], hi[6]); wh.w = pack_bf16(hi[5], hi[7]);
            wl.x = pack_bf16(lo[0], lo[2]); wl.y = pack_bf16(lo[1], lo[3]);
            wl.z = pack_bf16(lo[4], lo[6]); wl.w = pack_bf16(lo[5], lo[7]);
            *reinterpret_cast<uint4*>(xs + (size_t)grp * 16u) = wh;
            *reinterpret_cast<uint4*>(xs + pitch + (size_t)grp * 16u) = wl;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((grp & 3u) == 0u) xsum[grp >> 2] = sum;
        }
        if (tid < 16u) reinterpret_cast<uint32_t*>(zeros)[tid] = 0u;
    }
    const bool has_lo = __syncthreads_or(any_lo) != 0;

    // B operand source of this lane: sub-block 2t feeds k-slots (2t,2t+1) of
    // column 2t, sub-block 2t+1 feeds slots (2t+8,2t+9) of column 2t+1; every
    // other (lane, slot) pair reads the zero line.
    const bool role_a = (g == 2u * t), role_b = (g == 2u * t + 1u);
    const uint32_t off_a = 2u * t * 64u, off_b = (2u * t + 1u) * 64u;

    float acc_g = 0.0f, acc_g8 = 0.0f;
    uint32_t c_sb = sb_lo, c_tile = tile0, iter = 0;

    auto compute = [&](const Stage& s) {
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float e[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint8_t* xb = xs + (size_t)c_sb * 512u;  // 8 sub-blocks x 64 bytes
        const uint8_t* src_a = role_a ? xb + off_a : zeros;
        const uint8_t* src_b = role_b ? xb + off_b : zeros;
        const uint32_t M = 0x000F000Fu, O = 0x43004300u;
#pragma unroll
        for (uint32_t ch = 0; ch < 4u; ++ch) {  // 16-byte chunk of B = words 2ch, 2ch+1 of A
            const uint4 ba = *reinterpret_cast<const uint4*>(src_a + (role_a ? ch * 16u : 0u));
            const uint4 bb = *reinterpret_cast<const uint4*>(src_b + (role_b ? ch * 16u : 0u));
            const uint4& ql = s.q[ch >> 1];
            const uint4& qh = s.q[2u + (ch >> 1)];
            const uint32_t wl0 = (ch & 1u) ? ql.z : ql.x, wl1 = (ch & 1u) ? ql.w : ql.y;
            const uint32_t wh0 = (ch & 1u) ? qh.z : qh.x, wh1 = (ch & 1u) ? qh.w : qh.y;
            mma_bf16(c, (wl0 & M) | O, (wh0 & M) | O, ((wl0 >> 4) & M) | O, ((wh0 >> 4) & M) | O, ba.x, bb.x);
            mma_bf16(c, ((wl0 >> 8) & M) | O, ((wh0 >> 8) & M) | O, ((wl0 >> 12) & M) | O, ((wh0 >> 12) & M) | O,
                     ba.y, bb.y);
            mma_bf16(c, (wl1 & M) | O, (wh1 & M) | O, ((wl1 >> 4) & M) | O, ((wh1 >> 4) & M) | O, ba.z, bb.z);
            mma_bf16(c, ((wl1 >> 8) & M) | O, ((wh1 >> 8) & M) | O, ((wl1 >> 12) & M) | O, ((wh1 >> 12) & M) | O,
                     ba.w, bb.w);
            if (has_lo) {
                const uint4 la = *reinterpret_cast<const uint4*>(src_a + (role_a ? pitch + ch * 16u : 0u));
                const uint4 lb = *reinterpret_cast<const uint4*>(src_b + (role_b ? pitch + ch * 16u : 0u));
                mma_bf16(e, (wl0 & M) | O, (wh0 & M) | O, ((wl0 >> 4) & M) | O, ((wh0 >> 4) & M) | O, la.x, lb.x);
                mma_bf16(e, ((wl0 >> 8) & M) | O, ((wh0 >> 8) & M) | O, ((wl0 >> 12) & M) | O,
                         ((wh0 >> 12) & M) | O, la.y, lb.y);
                mma_bf16(e, (wl1 & M) | O, (wh1 & M) | O, ((wl1 >> 4) & M) | O, ((wh1 >> 4) & M) | O, la.z, lb.z);
                mma_bf16(e, ((wl1 >> 8) & M) | O, ((wh1 >> 8) & M) | O, ((wl1 >> 12) & M) | O,
                         ((wh1 >> 12) & M) | O, la.w, lb.w);
            }
        }
        // f32 fold of this lane's two sub-blocks (2t, 2t+1) for rows g and g+8
        const float2 X = *reinterpret_cast<const float2*>(xsum + c_sb * 8u + 2u * t);
        const float p0v = (c[0] + e[0]) - 128.0f * X.x, p1v = (c[1] + e[1]) - 128.0f * X.y;
        const float p2v = (c[2] + e[2]) - 128.0f * X.x, p3v = (c[3] + e[3]) - 128.0f * X.y;
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[0]);
            const float d = __low2float(dh), dm = __high2float(dh);
            const float s0 = (float)(s.sm[0] & 0xffu), s1 = (float)((s.sm[0] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[0] >> 16) & 0xffu), m1 = (float)(s.sm[0] >> 24);
            acc_g += d * (s0 * p0v + s1 * p1v) - dm * (m0 * X.x + m1 * X.y);
        }
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[1]);
            const float d = __low2float(dh), dm = __high2float(dh);
            const float s0 = (float)(s.sm[1] & 0xffu), s1 = (float)((s.sm[1] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[1] >> 16) & 0xffu), m1 = (float)(s.sm[1] >> 24);
            acc_g8 += d * (s0 * p2v + s1 * p3v) - dm * (m0 * X.x + m1 * X.y);
        }
        // ---- end of this warp's K slice for the tile: fold lanes, then slices
        if (++c_sb == sb_hi) {
            c_sb = sb_lo;
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

    // ---- one pipeline over every (tile, super-block) of this warp, loads two ahead
    for (uint32_t q = 0; q < total; q += 3u) {
        if (q + 2u < total) issue(st2);
        compute(st0);
        if (q + 1u >= total) break;
        if (q + 3u < total) issue(st0);
        compute(st1);
        if (q + 2u >= total) break;
        if (q + 4u < total) issue(st1);
        compute(st2);
    }
}

}  // namespace

// Returns 0 / a cudaError_t, or -1 when the shape is outside this kernel's plan
// (fewer than four super-blocks per row, or activations too long for shared
// memory) and the caller should take another route.
int pdk_q4k_gemv_diag(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                      uint32_t out_dim, cudaStream_t st) {
    const uint32_t n_super = in_dim >> 8;
    if (n_super < kSlices) return -1;
    const size_t smem = (size_t)in_dim * 4u + 64u + (size_t)(in_dim >> 5) * 4u + 2u * kSlots * kSlices * 16u * 4u;
    if (smem > 200u * 1024u) return -1;
    cudaError_t e = cudaFuncSetAttribute(q4k_gemv_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    const uint32_t need = (n_tiles + kSlots - 1u) / kSlots;
    if (grid > need) grid = need;
    q4k_gemv_diag_kernel<<<grid, kThreads, smem, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim,
                                                       out_dim);
    return pdk_launch_status();
}
