// gemv_i8.cu - single-token decode GEMV for Q4_K, Q5_K, Q4_0 and Q8_0 planes.
//
// Both formats are integer codes with one f32-class scale per 32 weights, and
// the GEMV is HBM-bound (4.5 / 8.5 bits per weight, each read once), so the
// kernel's job is to stay far below one instruction per weight:
//
//   * The 32-element inner sums run on the tensor cores as exact integer dot
//     products (mma m16n8k32, s8 x s8 -> s32).  Q8_0 bytes are the A operand
//     as loaded; a Q4_K word of eight nibbles becomes two A registers with two
//     logic ops.
//   * The activation vector is turned into block floating point once per CTA:
//     per 32-element block a power-of-two step s and a 15-bit integer
//     v = rint(x/s), |v| <= 2^14, kept as two int8 limbs v = 256*hi + lo.  For
//     bf16-valued activations this is exact unless a block spans more than 7
//     binades; in general the error is below 2^-15 of the block's largest
//     element.  The limbs are two n-tiles of the same mma, so the weights are
//     unpacked once.
//   * One token would use one of an mma's eight columns.  Instead the B operand
//     is block diagonal: the 32 k-slots of each mma are spread over the eight
//     32-weight blocks of a 256-weight unit (4 slots each) and column c is
//     non-zero only in block c's slots.  After the 8 mmas of a unit the
//     accumulator tile holds C[row][c] = sum_i q x over block c for 16 rows and
//     all eight blocks, and lane (g,t) owns exactly blocks (2t, 2t+1) of rows g
//     and g+8, whose scales it applies in f32.
//
// A CTA (one per SM, persistent) runs 4 tiles of 16 rows at a time, each tile's
// K range split over 4 warps; a warp walks all of its (tile, unit) pairs as one
// software pipeline with its loads issued DEPTH-1 units ahead.  Lane t of a
// row reads a contiguous quarter of the row's unit, so the four lanes of a row
// read one contiguous 128-byte (Q4_K) or 256-byte (Q8_0) run.
#include <cstdlib>

#include "gemv_i8_traits.cuh"

namespace {

constexpr uint32_t kSlots = 4;    // 16-row tiles in flight per CTA
constexpr uint32_t kSlices = 4;   // K slices per tile, one warp each
constexpr uint32_t kThreads = kSlots * kSlices * 32;
// One CTA per SM.  Two half-size CTAs per SM (so that under a dependent launch the next kernel's
// CTAs could move into half-SMs as they free up) measured 4 % slower back to back: 18.2 vs 17.4 us.
constexpr uint32_t kCtasPerSm = 1;

__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

using namespace gemv_i8;

// Shared memory: limb planes int8 [2][K] (hi, lo), 32 zero bytes,
// xmeta float2 [K/32] = {step s_j, s_j * sum_i v_ji}, red f32 [2][kSlots][kSlices][16].
template <class F>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
gemv_i8_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ recs, const float* __restrict__ bias,
               const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim, uint32_t out_dim,
               const int8_t* __restrict__ xq, const float* __restrict__ xq_scale, const PeerOut peers) {
    using Stage = typename F::Stage;
    constexpr uint32_t DEPTH = F::kDepth;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_blk = in_dim >> 5, n_unit = in_dim >> 8;
    uint8_t* xs_hi = smem;
    uint8_t* xs_lo = smem + in_dim;
    uint8_t* zeros = smem + 2u * (size_t)in_dim;
    float2* xmeta = reinterpret_cast<float2*>(zeros + 32u);
    float* red = reinterpret_cast<float*>(xmeta + n_blk);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / kSlices, slice = warp % kSlices;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t u_lo = slice * n_unit / kSlices, u_hi = (slice + 1u) * n_unit / kSlices;
    const uint32_t len = u_hi - u_lo;
    const size_t row_data = (size_t)n_unit * F::kDataBytes, row_rec = (size_t)n_unit * F::kRecBytes;

    // slot-major tile numbering: the tiles of the last, partial round land on different
    // CTAs instead of filling the first CTAs' four slots
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
        F::template load<false>(s, p0 + (size_t)l_u * F::kDataBytes, p1 + (size_t)l_u * F::kDataBytes,
                r0 + (size_t)l_u * F::kRecBytes, r1 + (size_t)l_u * F::kRecBytes, t);
        if (++l_u == u_hi) {
            l_u = u_lo;
            l_tile += tile_stride;
            if (l_tile < n_tiles) set_rows(l_tile);
        }
    };

    // Programmatic dependent launch: let the next kernel in the stream start its
    // own prologue as soon as every CTA of this one is running, and put this
    // kernel's first weight loads (weights never depend on the previous kernel) in
    // flight before waiting for the previous kernel's results (x, and y's old
    // contents).  Both instructions are no-ops under an ordinary launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    Stage st[DEPTH];
    if (total > 0u) {
        set_rows(tile0);
#pragma unroll
        for (uint32_t d = 0; d + 1u < DEPTH; ++d)
            if (d < total) issue(st[d]);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t peer_step = 0u;
    const bool peer_deferred = peers.n != 0u && peers.signal == 2u && blockIdx.x == 0u && tid == 0u;
    if (peer_deferred) peer_step = peer_post_previous(peers);

    act_limbs(x, xq, xq_scale, in_dim, xs_hi, xs_lo, zeros, xmeta, tid, kThreads);
    __syncthreads();

    // B operand source of this lane: block 2t feeds k-slots 4t..4t+3 of column
    // 2t, block 2t+1 feeds slots 16+4t.. of column 2t+1; every other
    // (lane, slot) pair reads the zero line.
    const bool role_a = (g == 2u * t), role_b = (g == 2u * t + 1u);

    float acc_g = 0.0f, acc_g8 = 0.0f;
    uint32_t c_u = u_lo, c_tile = tile0, iter = 0;

    auto compute = [&](const Stage& s, auto&& prefetch) {
        int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
        const uint32_t xoff = c_u * 256u;
        if constexpr (F::kSplitBlock) {
            // mma i feeds block 2t + i/4 alone: low nibbles = its elements 4(i&3).., high nibbles = 16 + 4(i&3)..
#pragma unroll
            for (uint32_t half = 0; half < 2u; ++half) {
                const bool mine = half == 0u ? role_a : role_b;
                const uint8_t* hs = mine ? xs_hi + xoff + (2u * t + half) * 32u : zeros;
                const uint8_t* ls = mine ? xs_lo + xoff + (2u * t + half) * 32u : zeros;
                const uint4 bh0 = *reinterpret_cast<const uint4*>(hs), bh1 = *reinterpret_cast<const uint4*>(hs + 16u);
                const uint4 bl0 = *reinterpret_cast<const uint4*>(ls), bl1 = *reinterpret_cast<const uint4*>(ls + 16u);
                const uint32_t vh0[4] = {bh0.x, bh0.y, bh0.z, bh0.w}, vh1[4] = {bh1.x, bh1.y, bh1.z, bh1.w};
                const uint32_t vl0[4] = {bl0.x, bl0.y, bl0.z, bl0.w}, vl1[4] = {bl1.x, bl1.y, bl1.z, bl1.w};
#pragma unroll
                for (uint32_t k = 0; k < 4u; ++k) {
                    uint32_t a0, a1, a2, a3;
                    F::a_regs(s, half * 4u + k, a0, a1, a2, a3);
                    mma_s8(ch, a0, a1, a2, a3, vh0[k], vh1[k]);
                    mma_s8(cl, a0, a1, a2, a3, vl0[k], vl1[k]);
                }
            }
        } else {
        const uint8_t* ha = role_a ? xs_hi + xoff + 2u * t * 32u : zeros;
            const uint8_t* hb = role_b ? xs_hi + xoff + (2u * t + 1u) * 32u : zeros;
            const uint8_t* la = role_a ? xs_lo + xoff + 2u * t * 32u : zeros;
            const uint8_t* lb = role_b ? xs_lo + xoff + (2u * t + 1u) * 32u : zeros;
    #pragma unroll
            for (uint32_t half = 0; half < 2u; ++half) {
                const uint4 bha = *reinterpret_cast<const uint4*>(ha + half * 16u);
                const uint4 bhb = *reinterpret_cast<const uint4*>(hb + half * 16u);
                const uint4 bla = *reinterpret_cast<const uint4*>(la + half * 16u);
                const uint4 blb = *reinterpret_cast<const uint4*>(lb + half * 16u);
                const uint32_t vha[4] = {bha.x, bha.y, bha.z, bha.w}, vhb[4] = {bhb.x, bhb.y, bhb.z, bhb.w};
                const uint32_t vla[4] = {bla.x, bla.y, bla.z, bla.w}, vlb[4] = {blb.x, blb.y, blb.z, blb.w};
    #pragma unroll
                for (uint32_t k = 0; k < 4u; ++k) {
                    uint32_t a0, a1, a2, a3;
                    F::a_regs(s, half * 4u + k, a0, a1, a2, a3);
                    mma_s8(ch, a0, a1, a2, a3, vha[k], vhb[k]);
                    mma_s8(cl, a0, a1, a2, a3, vla[k], vlb[k]);
                }
            }
        }
        // The next loads are issued only now, after every register of this unit
        // has been consumed: a wait on this unit's data can then never be a wait
        // on loads that were issued a moment ago.
        prefetch();
        // this lane's two blocks (2t, 2t+1) for rows g and g+8
        const float4 xm = *reinterpret_cast<const float4*>(xmeta + c_u * 8u + 2u * t);  // {s0, X0, s1, X1}
        float f[4];
        f[0] = (float)(ch[0] * 256 + cl[0]) * xm.x;
        f[1] = (float)(ch[1] * 256 + cl[1]) * xm.z;
        f[2] = (float)(ch[2] * 256 + cl[2]) * xm.x;
        f[3] = (float)(ch[3] * 256 + cl[3]) * xm.z;
        F::fold(s, f, xm.y, xm.w, acc_g, acc_g8);

        // ---- end of this warp's K slice for the tile: fold lanes, then slices
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
                float v = (rbuf[r] + rbuf[16u + r]) + (rbuf[32u + r] + rbuf[48u + r]);
                const uint32_t row = c_tile * 16u + r;
                if (row < out_dim) {
                    if (bias) v += bias[row];
                    if (peers.n == 0u) {
                        y[row] = v;
                    } else {
#pragma unroll
                        for (uint32_t p = 0; p < 8u; ++p)  // constant indices: the pointers stay in the parameter bank
                            if (p < peers.n) peers.ptr[p][peers.row0 + row] = v;
                    }
                }
            }
            acc_g = acc_g8 = 0.0f;
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
    if (peers.n != 0u && peers.signal == 1u) {   // uniform over the grid
        __syncthreads();
        if (tid == 0u) peer_signal(peers);
    }
    if (peer_deferred) peer_check_previous(peers, peer_step, nullptr);
}

// PDK_NO_PDL=1 launches without programmatic stream serialization (A/B switch, read once).
bool pdl_enabled() {
    static const bool v = [] {
        const char* e = getenv("PDK_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return v;
}

template <class F>
int launch(const void* data, const void* recs, const float* bias, const float* x, float* y, uint32_t in_dim,
           uint32_t out_dim, cudaStream_t st, const int8_t* xq = nullptr, const float* xq_scale = nullptr,
           const PeerOut* peers = nullptr) {
    const uint32_t n_unit = in_dim >> 8;
    if ((in_dim & 255u) != 0u || n_unit < kSlices) return -1;
    const size_t smem = (size_t)in_dim * 2u + 32u + (size_t)(in_dim >> 5) * 8u + 2u * kSlots * kSlices * 16u * 4u;
    if (smem > 200u * 1024u) return -1;
    auto kern = gemv_i8_kernel<F>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count() * kCtasPerSm;
    const uint32_t need = (n_tiles + kSlots - 1u) / kSlots;
    if (grid > need) grid = need;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PeerOut po{};
    if (peers) po = *peers;
    e = cudaLaunchKernelEx(&cfg, kern, (const uint8_t*)data, (const uint8_t*)recs, bias, x, y, in_dim, out_dim, xq,
                           xq_scale, po);
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}

}  // namespace

// The register-staged kernel: the route for the shapes the ring kernel (gemv_ring.cu) declines.
// All return 0 / a cudaError_t, or -1 when the shape is outside this kernel's plan too (K not a
// multiple of 256, fewer than four units per row, or activations too long for shared memory).
int pdk_q4k_gemv_i8_regs(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st) {
    return launch<Q4K>(data, scales, nullptr, x, y, in_dim, out_dim, st);
}

int pdk_q4_0_gemv_i8_regs(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                     uint32_t out_dim, cudaStream_t st) {
    return launch<Q40>(data, scales, nullptr, x, y, in_dim, out_dim, st);
}

int pdk_q5k_gemv_i8_regs(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st) {
    return launch<Q5K>(data, scales, nullptr, x, y, in_dim, out_dim, st);
}

int pdk_q8_0_gemv_i8_regs(const void* data, const void* scale, const float* bias, const float* x, float* y,
                     uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    return launch<Q80>(data, scale, bias, x, y, in_dim, out_dim, st);
}

int pdk_iq4xs_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                      cudaStream_t st) {
    return launch<IQ4XS>(data, scales, nullptr, x, y, in_dim, out_dim, st);
}

// Q4_K GEMV on int8 activations (xq int8 [in_dim], one f32 scale per 32): same kernel, the
// activation staging widens q * scale before it builds its limbs.
int pdk_q4k_gemv_i8_q8act_regs(const void* data, const void* scales, const int8_t* xq, const float* xq_scale, float* y,
                          uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    return launch<Q4K>(data, scales, nullptr, nullptr, y, in_dim, out_dim, st, xq, xq_scale);
}

// The Q4_K GEMV of one rank's row band with the peer-store epilogue (see gemv_ring.cu:
// pdk_q4k_gemv_shard); -1 = shape outside this kernel's plan.
int pdk_q4k_gemv_peers_regs(const void* data, const void* scales, const float* x, const gemv_i8::PeerOut* po,
                            uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    return launch<Q4K>(data, scales, nullptr, x, nullptr, in_dim, out_dim, st, nullptr, nullptr, po);
}
