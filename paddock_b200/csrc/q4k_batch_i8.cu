// q4k_batch_i8.cu - Q4_K, Q5_K and Q6_K small-batch GEMM (2..16 tokens per launch) on the int8 tensor path.
//
// The decode GEMV of gemv_i8.cu spends its eight mma columns on the eight 32-weight blocks of
// one token.  With several tokens the columns are the tokens, and what differs per block - the
// 6-bit sub-block scale sc[row][b] - is applied to the integer tile of that block:
//
//   * activations of one token are block floating point per 256 elements (one Q4_K super-block,
//     a "unit"): a power-of-two step s[tok][u] and 15-bit integers v = rint(x / s), |v| <= 2^14,
//     kept as two int8 limbs v = 256 hi + lo.  The error is below 2^-15 of the unit's largest
//     element.  A small kernel in front builds the limbs once per call into library-resident
//     scratch, laid out as the GEMM's shared-memory image, and every CTA of the GEMM fetches
//     that image with a few bulk copies (each CTA converting the activations itself cost a
//     third of the GEMM's instructions);
//   * per block b of a unit one mma m16n8k32 (s8 x s8 -> s32) per limb gives
//     T[row][tok] = sum_i q_i v_i over the block's 32 weights for 16 rows x 8 tokens, and the
//     lane adds sc[row][b] * T into integer unit sums U_hi, U_lo (one IMAD per entry);
//   * the min term sum_b m[row][b] * (sum_i v_i) is an integer product of its own: the block
//     sums of v (at most 2^19) are kept as three int8 limbs and one mma per limb, with the
//     6-bit m[row][b] as the A operand and the eight blocks in eight of its k-slots, gives it
//     for the whole unit;
//   * per unit and accumulator entry: y += s[tok][u] * (d[row] * (256 U_hi + U_lo) - dmin[row] * M).
//
// The CTA structure is the GEMV's: one persistent CTA per SM, 4 tiles of 16 rows in flight,
// each tile's K range split over 4 warps that walk their (tile, unit) pairs as one software
// pipeline; the K-slice partials meet in shared memory in a fixed order.  A lane reads bytes
// [8t, 8t+8) of each 32-byte group of its two rows, so that every lane holds 8 elements of
// every block (the four lanes of a row read one contiguous 32-byte run per group).
#include "tc5.cuh"

namespace {

constexpr uint32_t kSlots = 4;    // 16-row tiles in flight per CTA
constexpr uint32_t kSlices = 4;   // K slices per tile, one warp each
constexpr uint32_t kThreads = kSlots * kSlices * 32;

__device__ __forceinline__ void mma_s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    const int z = 0;
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// What a lane holds of one unit (256 weights) of its two rows.
struct Stage {
    uint2 q0[4], q1[4];  // row g / row g+8: bytes [8t, 8t+8) of ggml groups 0..3
    uint32_t dd[2];      // {f16 d, f16 dmin}
    uint32_t sc[2][2];   // sc[0..3], sc[4..7]
    uint32_t mw[2];      // m[4(t&1) .. 4(t&1)+3]
    uint2 h0, h1;        // Q5_K only: high-bit bytes 8t..8t+7 of row g / row g+8 (bit b of byte l = bit 4 of element l of block b)
};

template <bool K5>
__device__ __forceinline__ void load_stage(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                           const uint8_t* r1, uint32_t t) {
#pragma unroll
    for (uint32_t G = 0; G < 4u; ++G) {
        s.q0[G] = pdk_ldg_stream8(d0 + G * 32u + t * 8u);
        s.q1[G] = pdk_ldg_stream8(d1 + G * 32u + t * 8u);
    }
    if constexpr (K5) {
        s.h0 = pdk_ldg_stream8(d0 + 128u + t * 8u);
        s.h1 = pdk_ldg_stream8(d1 + 128u + t * 8u);
    }
    const uint32_t* w0 = reinterpret_cast<const uint32_t*>(r0);
    const uint32_t* w1 = reinterpret_cast<const uint32_t*>(r1);
    s.dd[0] = __ldg(w0);
    s.dd[1] = __ldg(w1);
    s.sc[0][0] = __ldg(w0 + 1);
    s.sc[0][1] = __ldg(w0 + 2);
    s.sc[1][0] = __ldg(w1 + 1);
    s.sc[1][1] = __ldg(w1 + 2);
    s.mw[0] = __ldg(w0 + 3u + (t & 1u));
    s.mw[1] = __ldg(w1 + 3u + (t & 1u));
}

// The activation image (built by q4k_act_limbs_kernel in global scratch, copied verbatim into
// shared memory), NCOLS = 8 NT token columns:
//   planes : [NCOLS][pitch], pitch = 2K + 64 bytes; per 32-element block 64 bytes =
//            4 x {8 hi limbs, 8 lo limbs} (lane t of a row reads its 16 bytes at once; the
//            64 odd bytes per row put the 8 token rows of a quarter-warp read on distinct banks)
//   ustep  : f32  [K/256][NCOLS]          step of (unit, token)
//   isl    : int8 [K/256][3][NCOLS][8]    limbs of the eight block sums of (unit, token)
// For Q6_K (16 blocks of 16 weights per unit, K6): the 64 bytes of a 32-element run are 4 x {4 hi of its
// first block, 4 hi of its second, 4 lo of the first, 4 lo of the second} - lane t's k-slots of two
// m16n8k16 products, one per block - and isl is int8 [K/256][3][NCOLS][16].
// followed in shared memory by red : f32 [2][kSlots][kSlices][16][NCOLS] and the copy's mbarrier.
template <uint32_t NT, uint32_t NBLK = 8u>
struct Plan {
    static constexpr uint32_t NCOLS = NT * 8u;
    static __host__ __device__ uint32_t pitch(uint32_t in_dim) { return 2u * in_dim + 64u; }
    static __host__ __device__ size_t off_step(uint32_t in_dim) { return (size_t)NCOLS * pitch(in_dim); }
    static __host__ __device__ size_t off_isl(uint32_t in_dim) { return off_step(in_dim) + (size_t)(in_dim >> 8) * NCOLS * 4u; }
    static __host__ __device__ size_t image(uint32_t in_dim) { return off_isl(in_dim) + (size_t)(in_dim >> 8) * 3u * NCOLS * NBLK; }
    static __host__ __device__ size_t off_bar(uint32_t in_dim) { return image(in_dim) + 2u * kSlots * kSlices * 16u * NCOLS * 4u; }
    static __host__ __device__ size_t total(uint32_t in_dim) { return off_bar(in_dim) + 16u; }
};

// Activations -> the image above, in global memory.  One warp per (token, unit), 8 elements
// per lane; token columns at and past `batch` are written as zeros.
template <uint32_t NT, bool K6 = false>
__global__ void __launch_bounds__(256)
q4k_act_limbs_kernel(const float* __restrict__ x, const int8_t* __restrict__ xq, const float* __restrict__ xq_scale,
                     uint8_t* __restrict__ img, uint32_t in_dim, uint32_t batch) {
    using P = Plan<NT, K6 ? 16u : 8u>;
    constexpr uint32_t NCOLS = P::NCOLS;
    const uint32_t n_unit = in_dim >> 8, pitch = P::pitch(in_dim);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t task = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    float* ustep = reinterpret_cast<float*>(img + P::off_step(in_dim));
    uint8_t* isl = img + P::off_isl(in_dim);
    pdk_pdl_launch_dependents();
    if (task >= NCOLS * n_unit) return;
    const uint32_t tok = task / n_unit, u = task - tok * n_unit;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    // the scratch may still be read by the previous GEMM in the stream, and x may be its predecessor's output
    pdk_pdl_wait();
    if (tok < batch) {
        const size_t e0 = (size_t)tok * in_dim + u * 256u + lane * 8u;
        if (xq == nullptr) {
            const float4 a = *reinterpret_cast<const float4*>(x + e0);
            const float4 b = *reinterpret_cast<const float4*>(x + e0 + 4u);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            // int8 activations with one f32 scale per 32 (the W4A8 slots' operands)
            const int2 q = *reinterpret_cast<const int2*>(xq + e0);
            const float s = xq_scale[e0 >> 5];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (float)(int8_t)((i < 4 ? q.x >> (8 * i) : q.y >> (8 * (i - 4))) & 0xff) * s;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    // amax < 2^ex  ->  step 2^(ex-14) keeps |v| <= 2^14
    int ex = 0;
    float step = 0.0f, inv = 0.0f;
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
    auto put_limbs = [&](int sum, uint32_t n_blk, uint32_t blk) {
        // block sum -> three signed byte limbs, sum = l0 + 256 l1 + 65536 l2
        const int l0 = (int)(int8_t)(sum & 0xff);
        const int r1v = (sum - l0) >> 8;
        const int l1 = (int)(int8_t)(r1v & 0xff);
        const int l2 = (r1v - l1) >> 8;
        uint8_t* dst = isl + ((size_t)(u * 3u) * NCOLS + tok) * n_blk + blk;
        dst[0] = (uint8_t)l0;
        dst[NCOLS * n_blk] = (uint8_t)l1;
        dst[2u * NCOLS * n_blk] = (uint8_t)l2;
    };
    if constexpr (K6) {
        // lane = 4 * run + t': elements 8t' .. 8t'+7 of the run, all in its block h = t' / 2; elements
        // 8 (t' & 1) + j go to lane slot 2 (t' & 1) + j / 4 of the k16 products, bytes 4h .. (hi), 8 + 4h .. (lo)
        const uint32_t tp = lane & 3u, h = tp >> 1;
        uint8_t* run = img + (size_t)tok * pitch + u * 512u + (lane >> 2) * 64u + 2u * (tp & 1u) * 16u + h * 4u;
        *reinterpret_cast<uint32_t*>(run) = hi[0];
        *reinterpret_cast<uint32_t*>(run + 8u) = lo[0];
        *reinterpret_cast<uint32_t*>(run + 16u) = hi[1];
        *reinterpret_cast<uint32_t*>(run + 24u) = lo[1];
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        if ((lane & 1u) == 0u) put_limbs(isum, 16u, lane >> 1);
    } else {
        // lane = 4 * block + t: 16 bytes {hi, lo} at block * 64 + t * 16
        *reinterpret_cast<uint4*>(img + (size_t)tok * pitch + u * 512u + lane * 16u) = make_uint4(hi[0], hi[1], lo[0], lo[1]);
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        isum += __shfl_xor_sync(0xffffffffu, isum, 2);
        if ((lane & 3u) == 0u) put_limbs(isum, 8u, lane >> 2);
    }
    if (lane == 0u) ustep[u * NCOLS + tok] = step;
}

// K5: the plane is Q5_K repacked (kquant_more.cu) - per super-block 128 bytes of low nibbles in the Q4_K
// convention, then 32 bytes of high bits; the codes become 5-bit and everything else is Q4_K's.
template <uint32_t NT, uint32_t DEPTH, bool EARLY, bool K5>
__global__ void __launch_bounds__(kThreads, 1)
q4k_batch_i8_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ recs, const uint8_t* __restrict__ img,
                    float* __restrict__ y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, unsigned int* err_word) {
    using P = Plan<NT>;
    constexpr uint32_t NCOLS = P::NCOLS;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_unit = in_dim >> 8, pitch = P::pitch(in_dim);
    const float* ustep = reinterpret_cast<const float*>(smem + P::off_step(in_dim));
    const uint8_t* isl = smem + P::off_isl(in_dim);
    float* red = reinterpret_cast<float*>(smem + P::image(in_dim));
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + P::off_bar(in_dim));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / kSlices, slice = warp % kSlices;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t u_lo = slice * n_unit / kSlices, u_hi = (slice + 1u) * n_unit / kSlices;
    const uint32_t len = u_hi - u_lo;
    constexpr uint32_t kUnitBytes = K5 ? 160u : 128u;
    const size_t row_data = (size_t)n_unit * kUnitBytes, row_rec = (size_t)n_unit * 24u;

    // slot-major tile numbering, as in the decode GEMV
    const uint32_t tile0 = slot * gridDim.x + blockIdx.x, tile_stride = gridDim.x * kSlots;
    const uint32_t my_tiles = tile0 < n_tiles ? (n_tiles - tile0 + tile_stride - 1u) / tile_stride : 0u;
    const uint32_t total = my_tiles * len;

    // ---- load cursor over this warp's (tile, unit) sequence
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
        load_stage<K5>(s, p0 + (size_t)l_u * kUnitBytes, p1 + (size_t)l_u * kUnitBytes, r0 + (size_t)l_u * 24u,
                       r1 + (size_t)l_u * 24u, t);
        if (++l_u == u_hi) {
            l_u = u_lo;
            l_tile += tile_stride;
            if (l_tile < n_tiles) set_rows(l_tile);
        }
    };

    // The first weight loads (weights never depend on the previous kernel in the stream) go in
    // flight before this kernel waits for the previous kernel's results.
    pdk_pdl_launch_dependents();
    Stage st[DEPTH];
    if (total > 0u) {
        set_rows(tile0);
#pragma unroll
        for (uint32_t d = 0; d + 1u < DEPTH; ++d)
            if (d < total) issue(st[d]);
    }
    if (tid == 0u) {
        tc5::mbar_init(bar, 1u);
        *abort_flag = 0;
        tc5::mbar_fence_init();
    }
    __syncthreads();
    pdk_pdl_wait();  // the image is the previous kernel's output

    // ---- the activation image: bulk copies into shared memory, one mbarrier
    if (warp == 0u) {
        tc5::mbar_arrive_expect_tx_elect(bar, (uint32_t)P::image(in_dim));
        for (uint32_t c = 0; c < NCOLS; ++c)
            tc5::bulk_load_elect(smem + (size_t)c * pitch, img + (size_t)c * pitch, pitch, bar);
        tc5::bulk_load_elect(smem + P::off_step(in_dim), img + P::off_step(in_dim),
                             (uint32_t)(P::image(in_dim) - P::off_step(in_dim)), bar);
    }
    const tc5::WaitCtx ctx{abort_flag, err_word};
    const bool landed = tc5::mbar_wait(bar, 0u, ctx, tc5::kErrFullWait, 0x40u);
    if (__syncthreads_or(!landed)) return;  // the copy never landed: error word set, the whole CTA leaves together

    float acc[NT][4];
#pragma unroll
    for (uint32_t nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    uint32_t c_u = u_lo, c_tile = tile0, iter = 0;
    // B operand rows of this lane: token column g of each n-tile, its 16 bytes {hi, lo} of a block
    const uint8_t* bp = smem + (size_t)g * pitch + t * 16u;

    auto compute = [&](const Stage& s, auto&& prefetch) {
        // EARLY: the loads for the stage consumed by the previous unit go out first (a whole unit
        // of distance with two stages); otherwise after the main loop, when this unit's weight
        // registers are dead
        if (EARLY) prefetch();
        int uh[NT][4], ul[NT][4];
#pragma unroll
        for (uint32_t nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) uh[nt][i] = ul[nt][i] = 0;
        const uint8_t* bu = bp + c_u * 512u;
#pragma unroll
        for (uint32_t b = 0; b < 8u; ++b) {
            const uint32_t G = b >> 1, sh = (b & 1u) * 4u;
            uint32_t a0 = (s.q0[G].x >> sh) & 0x0F0F0F0Fu, a2 = (s.q0[G].y >> sh) & 0x0F0F0F0Fu;
            uint32_t a1 = (s.q1[G].x >> sh) & 0x0F0F0F0Fu, a3 = (s.q1[G].y >> sh) & 0x0F0F0F0Fu;
            if constexpr (K5) {
                a0 |= ((s.h0.x >> b) & 0x01010101u) << 4;
                a2 |= ((s.h0.y >> b) & 0x01010101u) << 4;
                a1 |= ((s.h1.x >> b) & 0x01010101u) << 4;
                a3 |= ((s.h1.y >> b) & 0x01010101u) << 4;
            }
            const int sc_g = (int)((s.sc[0][b >> 2] >> (8u * (b & 3u))) & 0xffu);
            const int sc_g8 = (int)((s.sc[1][b >> 2] >> (8u * (b & 3u))) & 0xffu);
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                const uint4 v = *reinterpret_cast<const uint4*>(bu + (size_t)nt * 8u * pitch + b * 64u);
                int th[4], tl[4];
                mma_s8_z(th, a0, a1, a2, a3, v.x, v.y);
                mma_s8_z(tl, a0, a1, a2, a3, v.z, v.w);
                uh[nt][0] += sc_g * th[0];
                uh[nt][1] += sc_g * th[1];
                uh[nt][2] += sc_g8 * th[2];
                uh[nt][3] += sc_g8 * th[3];
                ul[nt][0] += sc_g * tl[0];
                ul[nt][1] += sc_g * tl[1];
                ul[nt][2] += sc_g8 * tl[2];
                ul[nt][3] += sc_g8 * tl[3];
            }
        }
        // min term: A = m[row][block] in k-slots 0..7 (lanes t = 0, 1), B = one limb of the block sums
        const uint32_t am0 = t < 2u ? s.mw[0] : 0u, am1 = t < 2u ? s.mw[1] : 0u;
        const __half2 dh0 = *reinterpret_cast<const __half2*>(&s.dd[0]);
        const __half2 dh1 = *reinterpret_cast<const __half2*>(&s.dd[1]);
        const float d_g = __low2float(dh0), dmin_g = __high2float(dh0);
        const float d_g8 = __low2float(dh1), dmin_g8 = __high2float(dh1);
        if (!EARLY) prefetch();
#pragma unroll
        for (uint32_t nt = 0; nt < NT; ++nt) {
            const uint8_t* ip = isl + ((size_t)(c_u * 3u) * NCOLS + nt * 8u + g) * 8u + (t & 1u) * 4u;
            int m0[4], m1[4], m2[4];
            mma_s8_z(m0, am0, am1, 0u, 0u, *reinterpret_cast<const uint32_t*>(ip), 0u);
            mma_s8_z(m1, am0, am1, 0u, 0u, *reinterpret_cast<const uint32_t*>(ip + NCOLS * 8u), 0u);
            mma_s8_z(m2, am0, am1, 0u, 0u, *reinterpret_cast<const uint32_t*>(ip + 2u * NCOLS * 8u), 0u);
            const float2 stp = *reinterpret_cast<const float2*>(ustep + c_u * NCOLS + nt * 8u + 2u * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mainv = fmaf((float)uh[nt][i], 256.0f, (float)ul[nt][i]);
                const float minv = (float)(m0[i] + 256 * m1[i] + 65536 * m2[i]);
                const float d = i < 2 ? d_g : d_g8, dm = i < 2 ? dmin_g : dmin_g8;
                acc[nt][i] = fmaf((i & 1) ? stp.y : stp.x, d * mainv - dm * minv, acc[nt][i]);
            }
        }

        // ---- end of this warp's K slice for the tile: the four slices meet in shared memory
        if (++c_u == u_hi) {
            c_u = u_lo;
            float* rbuf = red + ((size_t)(iter & 1u) * kSlots + slot) * (kSlices * 16u * NCOLS);
            float* mine = rbuf + (size_t)slice * 16u * NCOLS;
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                *reinterpret_cast<float2*>(mine + g * NCOLS + nt * 8u + 2u * t) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(mine + (g + 8u) * NCOLS + nt * 8u + 2u * t) = make_float2(acc[nt][2], acc[nt][3]);
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
            }
            bar_sync(1u + slot, kSlices * 32u);
            // 128 threads, 16 rows x NCOLS tokens: thread -> (row = idx % 16, token = idx / 16 [+ 8])
            const uint32_t idx = slice * 32u + lane;
            const uint32_t row = c_tile * 16u + (idx & 15u);
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                const uint32_t tok = nt * 8u + (idx >> 4);
                const uint32_t o = (idx & 15u) * NCOLS + tok;
                const float v = (rbuf[o] + rbuf[16u * NCOLS + o]) + (rbuf[32u * NCOLS + o] + rbuf[48u * NCOLS + o]);
                if (row < out_dim && tok < batch) y[(size_t)tok * out_dim + row] = v;
            }
            c_tile += tile_stride;
            ++iter;
        }
    };

    // ---- one pipeline over every (tile, unit) of this warp, loads DEPTH-1 ahead
    for (uint32_t q = 0; q < total; q += DEPTH) {
#pragma unroll
        for (uint32_t d = 0; d < DEPTH; ++d) {
            if (q + d >= total) break;
            compute(st[d], [&] {
                if (q + d + DEPTH - 1u < total) issue(st[(d + DEPTH - 1u) % DEPTH]);
            });
        }
    }
}

// ---------------------------------------------------------------- Q6_K
//
// Q6_K repacked (kquant_more.cu): per super-block 128 bytes ql + 64 bytes qh, record = f16 d at byte 0 and
// int8 sc[16] at bytes 4..19; w = d * sc[block] * (q - 32), 16 blocks of 16.  Lane t of a row reads bytes
// [4t, 4t+4) and [16+4t, 16+4t+4) of each 32-byte run, i.e. four codes of each of the run's two blocks, and
// one m16n8k16 product per block and limb gives T[row][tok] for that block; sc[row][block] * T adds into the
// integer unit sums as for Q4_K.  The -32 goes through the block sums: sum_b sc[row][b] * (sum_i v_i) is one
// k16 product per limb with the sixteen int8 scales as the A operand.
__device__ __forceinline__ void mma_s8_k16_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(z));
}

struct Stage6 {
    uint32_t ql[2][2][2][2];  // [row g / g+8][half][32-byte run of the half: low / high nibbles' bytes][block of the run]
    uint32_t qh[2][2][2];     // [row][half][block]
    uint32_t d[2];            // f16 d (low half)
    uint4 sc[2];              // the sixteen int8 block scales
};

__device__ __forceinline__ void load_stage6(Stage6& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                            const uint8_t* r1, uint32_t t) {
    const uint8_t* dp[2] = {d0, d1};
    const uint8_t* rp[2] = {r0, r1};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                s.ql[w][nh][0][h] = pdk_ldg_stream4(dp[w] + nh * 64u + h * 16u + t * 4u);
                s.ql[w][nh][1][h] = pdk_ldg_stream4(dp[w] + nh * 64u + 32u + h * 16u + t * 4u);
                s.qh[w][nh][h] = pdk_ldg_stream4(dp[w] + 128u + nh * 32u + h * 16u + t * 4u);
            }
        }
        s.d[w] = __ldg(reinterpret_cast<const uint16_t*>(rp[w]));
        const uint32_t* rw = reinterpret_cast<const uint32_t*>(rp[w] + 4u);
        s.sc[w] = make_uint4(__ldg(rw), __ldg(rw + 1), __ldg(rw + 2), __ldg(rw + 3));
    }
}

__device__ __forceinline__ int sc_byte(const uint4& v, uint32_t b) {   // b is a compile-time constant after unrolling
    const uint32_t w = (b >> 2) == 0u ? v.x : (b >> 2) == 1u ? v.y : (b >> 2) == 2u ? v.z : v.w;
    return (int)(int8_t)((w >> (8u * (b & 3u))) & 0xffu);
}

template <uint32_t NT>
__global__ void __launch_bounds__(kThreads, 1)
q6k_batch_i8_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ recs, const uint8_t* __restrict__ img,
                    float* __restrict__ y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, unsigned int* err_word) {
    using P = Plan<NT, 16u>;
    constexpr uint32_t NCOLS = P::NCOLS, DEPTH = 2;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_unit = in_dim >> 8, pitch = P::pitch(in_dim);
    const float* ustep = reinterpret_cast<const float*>(smem + P::off_step(in_dim));
    const uint8_t* isl = smem + P::off_isl(in_dim);
    float* red = reinterpret_cast<float*>(smem + P::image(in_dim));
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + P::off_bar(in_dim));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);

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
    auto issue = [&](Stage6& s) {
        load_stage6(s, p0 + (size_t)l_u * 192u, p1 + (size_t)l_u * 192u, r0 + (size_t)l_u * 24u, r1 + (size_t)l_u * 24u, t);
        if (++l_u == u_hi) {
            l_u = u_lo;
            l_tile += tile_stride;
            if (l_tile < n_tiles) set_rows(l_tile);
        }
    };

    pdk_pdl_launch_dependents();
    Stage6 st[DEPTH];
    if (total > 0u) {
        set_rows(tile0);
        issue(st[0]);
    }
    if (tid == 0u) {
        tc5::mbar_init(bar, 1u);
        *abort_flag = 0;
        tc5::mbar_fence_init();
    }
    __syncthreads();
    pdk_pdl_wait();  // the image is the previous kernel's output
    if (warp == 0u) {
        tc5::mbar_arrive_expect_tx_elect(bar, (uint32_t)P::image(in_dim));
        for (uint32_t c = 0; c < NCOLS; ++c)
            tc5::bulk_load_elect(smem + (size_t)c * pitch, img + (size_t)c * pitch, pitch, bar);
        tc5::bulk_load_elect(smem + P::off_step(in_dim), img + P::off_step(in_dim),
                             (uint32_t)(P::image(in_dim) - P::off_step(in_dim)), bar);
    }
    const tc5::WaitCtx ctx{abort_flag, err_word};
    const bool landed = tc5::mbar_wait(bar, 0u, ctx, tc5::kErrFullWait, 0x41u);
    if (__syncthreads_or(!landed)) return;

    float acc[NT][4];
#pragma unroll
    for (uint32_t nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    uint32_t c_u = u_lo, c_tile = tile0, iter = 0;
    const uint8_t* bp = smem + (size_t)g * pitch + t * 16u;

    auto compute = [&](const Stage6& s, auto&& prefetch) {
        prefetch();   // the next unit's loads go out first
        int uh[NT][4], ul[NT][4];
#pragma unroll
        for (uint32_t nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) uh[nt][i] = ul[nt][i] = 0;
        const uint8_t* bu = bp + c_u * 512u;
#pragma unroll
        for (uint32_t R = 0; R < 8u; ++R) {   // 32-element run R = 4 * half + r
            const uint32_t nh = R >> 2, r = R & 3u, sh = (r >> 1) * 4u;
            uint32_t a[2][2];                  // [block of the run][row g / g+8]
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h)
#pragma unroll
                for (uint32_t w = 0; w < 2u; ++w)
                    a[h][w] = ((s.ql[w][nh][r & 1u][h] >> sh) & 0x0F0F0F0Fu) | (((s.qh[w][nh][h] >> (2u * r)) & 0x03030303u) << 4);
            const int sc0_g = sc_byte(s.sc[0], 2u * R), sc1_g = sc_byte(s.sc[0], 2u * R + 1u);
            const int sc0_g8 = sc_byte(s.sc[1], 2u * R), sc1_g8 = sc_byte(s.sc[1], 2u * R + 1u);
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                const uint4 v = *reinterpret_cast<const uint4*>(bu + (size_t)nt * 8u * pitch + R * 64u);
                int t0h[4], t1h[4], t0l[4], t1l[4];
                mma_s8_k16_z(t0h, a[0][0], a[0][1], v.x);
                mma_s8_k16_z(t1h, a[1][0], a[1][1], v.y);
                mma_s8_k16_z(t0l, a[0][0], a[0][1], v.z);
                mma_s8_k16_z(t1l, a[1][0], a[1][1], v.w);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int s0 = i < 2 ? sc0_g : sc0_g8, s1 = i < 2 ? sc1_g : sc1_g8;
                    uh[nt][i] += s0 * t0h[i] + s1 * t1h[i];
                    ul[nt][i] += s0 * t0l[i] + s1 * t1l[i];
                }
            }
        }
        // the -32: A = sc[row][block] in k-slots 0..15 (lane t holds blocks 4t..4t+3), B = one limb of the block sums
        const uint32_t as0 = t == 0u ? s.sc[0].x : t == 1u ? s.sc[0].y : t == 2u ? s.sc[0].z : s.sc[0].w;
        const uint32_t as1 = t == 0u ? s.sc[1].x : t == 1u ? s.sc[1].y : t == 2u ? s.sc[1].z : s.sc[1].w;
        const float d_g = __half2float(__ushort_as_half((unsigned short)s.d[0]));
        const float d_g8 = __half2float(__ushort_as_half((unsigned short)s.d[1]));
#pragma unroll
        for (uint32_t nt = 0; nt < NT; ++nt) {
            const uint8_t* ip = isl + ((size_t)(c_u * 3u) * NCOLS + nt * 8u + g) * 16u + t * 4u;
            int m0[4], m1[4], m2[4];
            mma_s8_k16_z(m0, as0, as1, *reinterpret_cast<const uint32_t*>(ip));
            mma_s8_k16_z(m1, as0, as1, *reinterpret_cast<const uint32_t*>(ip + NCOLS * 16u));
            mma_s8_k16_z(m2, as0, as1, *reinterpret_cast<const uint32_t*>(ip + 2u * NCOLS * 16u));
            const float2 stp = *reinterpret_cast<const float2*>(ustep + c_u * NCOLS + nt * 8u + 2u * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mainv = fmaf((float)uh[nt][i], 256.0f, (float)ul[nt][i]);
                const float offv = (float)(m0[i] + 256 * m1[i] + 65536 * m2[i]);
                acc[nt][i] = fmaf((i & 1) ? stp.y : stp.x, (i < 2 ? d_g : d_g8) * fmaf(-32.0f, offv, mainv), acc[nt][i]);
            }
        }

        if (++c_u == u_hi) {
            c_u = u_lo;
            float* rbuf = red + ((size_t)(iter & 1u) * kSlots + slot) * (kSlices * 16u * NCOLS);
            float* mine = rbuf + (size_t)slice * 16u * NCOLS;
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                *reinterpret_cast<float2*>(mine + g * NCOLS + nt * 8u + 2u * t) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2*>(mine + (g + 8u) * NCOLS + nt * 8u + 2u * t) = make_float2(acc[nt][2], acc[nt][3]);
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
            }
            bar_sync(1u + slot, kSlices * 32u);
            const uint32_t idx = slice * 32u + lane;
            const uint32_t row = c_tile * 16u + (idx & 15u);
#pragma unroll
            for (uint32_t nt = 0; nt < NT; ++nt) {
                const uint32_t tok = nt * 8u + (idx >> 4);
                const uint32_t o = (idx & 15u) * NCOLS + tok;
                const float v = (rbuf[o] + rbuf[16u * NCOLS + o]) + (rbuf[32u * NCOLS + o] + rbuf[48u * NCOLS + o]);
                if (row < out_dim && tok < batch) y[(size_t)tok * out_dim + row] = v;
            }
            c_tile += tile_stride;
            ++iter;
        }
    };

    for (uint32_t q = 0; q < total; q += DEPTH) {
#pragma unroll
        for (uint32_t d = 0; d < DEPTH; ++d) {
            if (q + d >= total) break;
            compute(st[d], [&] {
                if (q + d + DEPTH - 1u < total) issue(st[(d + DEPTH - 1u) % DEPTH]);
            });
        }
    }
}

// Scratch for the activation image: lives in the library (the pack allocates nothing at run
// time), one slice per stream for the first kImgLanes streams that make such calls.
constexpr size_t kImgSliceBytes = 232448;  // the largest image a CTA's shared memory can hold
constexpr int kImgLanes = 2;
__device__ __align__(1024) uint8_t g_q4k_img[kImgLanes][kImgSliceBytes];

PDK_SLICE_TABLE(img_slice_table, g_q4k_img, kImgSliceBytes, kImgLanes);
uint8_t* img_slice(cudaStream_t st) { return img_slice_table.slice(st); }

template <uint32_t NT, uint32_t DEPTH, bool EARLY, bool K5>
int launch(const void* data, const void* recs, const float* x, const int8_t* xq, const float* xq_scale, float* y,
           uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    using P = Plan<NT>;
    const uint32_t n_unit = in_dim >> 8;
    if ((in_dim & 255u) != 0u || n_unit < kSlices) return -1;
    const size_t smem = P::total(in_dim);
    if (smem > 227u * 1024u) return -1;
    uint8_t* img = img_slice(st);
    if (img == nullptr) return -1;
    auto kern = q4k_batch_i8_kernel<NT, DEPTH, EARLY, K5>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t tasks = P::NCOLS * n_unit;
    if (int rc = pdk_launch_pdl(q4k_act_limbs_kernel<NT>, dim3((tasks + 7u) / 8u), dim3(256), 0, st, x, xq, xq_scale, img,
                                in_dim, batch))
        return rc;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    const uint32_t need = (n_tiles + kSlots - 1u) / kSlots;
    if (grid > need) grid = need;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, (const uint8_t*)data, (const uint8_t*)recs,
                          (const uint8_t*)img, y, in_dim, out_dim, batch, pdk_error_word());
}

template <uint32_t NT>
int launch6(const void* data, const void* recs, const float* x, float* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch,
            cudaStream_t st) {
    using P = Plan<NT, 16u>;
    const uint32_t n_unit = in_dim >> 8;
    if ((in_dim & 255u) != 0u || n_unit < kSlices) return -1;
    const size_t smem = P::total(in_dim);
    if (smem > 227u * 1024u) return -1;
    uint8_t* img = img_slice(st);
    if (img == nullptr) return -1;
    auto kern = q6k_batch_i8_kernel<NT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t tasks = P::NCOLS * n_unit;
    if (int rc = pdk_launch_pdl(q4k_act_limbs_kernel<NT, true>, dim3((tasks + 7u) / 8u), dim3(256), 0, st, x,
                                (const int8_t*)nullptr, (const float*)nullptr, img, in_dim, batch))
        return rc;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    const uint32_t need = (n_tiles + kSlots - 1u) / kSlots;
    if (grid > need) grid = need;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, (const uint8_t*)data, (const uint8_t*)recs,
                          (const uint8_t*)img, y, in_dim, out_dim, batch, pdk_error_word());
}

}  // namespace

// Q4_K GEMM for 1 <= batch <= 16 tokens: y f32 [batch][out_dim].  Activations are either f32
// x [batch][in_dim] or (x == nullptr) int8 xq [batch][in_dim] with one f32 scale per 32
// elements, xq_scale [batch][in_dim / 32].  Returns 0 / a cudaError_t, or -1 when the shape is
// outside the kernel's plan (K not a multiple of 256, fewer than four super-blocks per row, the
// limb planes do not fit in shared memory, or more streams than scratch slices) and the caller
// should take another route.  Two launches: the activation image, then the GEMM.
int pdk_q4k_batch_i8(const void* data, const void* scales, const float* x, const int8_t* xq, const float* xq_scale,
                     float* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    if (batch == 0u || batch > 16u) return -1;
    // Two stages with the loads issued first measured the same as three stages with the loads
    // issued after the main loop (21.5 / 53 us against 22.9 / 58 us at 4 / 16 tokens).
    if (batch <= 8u) return launch<1, 2, true, false>(data, scales, x, xq, xq_scale, y, in_dim, out_dim, batch, st);
    return launch<2, 2, true, false>(data, scales, x, xq, xq_scale, y, in_dim, out_dim, batch, st);
}

// The same for a Q5_K plane (f32 activations).
int pdk_q5k_batch_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, cudaStream_t st) {
    if (batch == 0u || batch > 16u) return -1;
    if (batch <= 8u) return launch<1, 2, true, true>(data, scales, x, nullptr, nullptr, y, in_dim, out_dim, batch, st);
    return launch<2, 2, true, true>(data, scales, x, nullptr, nullptr, y, in_dim, out_dim, batch, st);
}

// The same for a Q6_K plane (f32 activations).
int pdk_q6k_batch_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, cudaStream_t st) {
    if (batch == 0u || batch > 16u) return -1;
    // passes of eight token columns: the 16-column form does not fit 128 registers (123 us at 16 tokens against 83)
    for (uint32_t b = 0; b < batch; b += 8u) {
        const uint32_t take = batch - b < 8u ? batch - b : 8u;
        if (int rc = launch6<1>(data, scales, x + (size_t)b * in_dim, y + (size_t)b * out_dim, in_dim, out_dim, take, st))
            return rc;
    }
    return 0;
}
