// gemv_ring.cu - single-token decode GEMV for Q4_K, Q4_0 and Q8_0 planes with the weights staged
// in shared memory by TMA, every warp running its own ring.
//
// The arithmetic is that of gemv_i8.cu (integer dot products on mma m16n8k32, activations as two
// int8 limbs of a 15-bit block floating point, block-diagonal B operand, f32 scale fold); what
// differs is how the bytes reach the SM.  A decode GEMV reads every weight once, so its time is
// the time HBM needs, provided enough bytes are in flight: about 7 MB over the chip.  Loads
// issued from registers cap that at (threads x registers spent on staging); here every warp keeps
// D tiled TMA copies outstanding into its own shared-memory stages, 150-190 KB per SM whatever
// the warps hold in registers, and requests them at kernel start, before the wait on the previous
// kernel in the stream (programmatic dependent launch).
//
//   * A CTA (one per SM) owns a contiguous range of 16-row tiles; warp w takes units w, w + W, ...
//     of every tile (unit = 256 weights of a row).  Per (tile, unit) the warp's elected lane issues
//     one 2-D TMA copy of the 16 rows x 128 bytes of packed weights (two for Q8_0's 256 bytes) and
//     one of the rows' scale records.  The planes stay in the byte layout the repack slots write
//     (super-block local: the engine concatenates planes at super-block offsets); the tensor maps
//     describe them as [rows][row bytes].
//   * The weight boxes are written with the 128-byte swizzle, which puts the 16-byte chunks that
//     the eight rows of one mma fragment load touch into eight different bank groups: fragment
//     loads are conflict free, and the shared-memory port carries each byte twice (in and out).
//   * A warp is the only reader of its stages: it waits on its own mbarrier, moves the fragments
//     to registers, and re-arms the stage itself after the mma sequence has consumed them.  No
//     producer warp, no cross-warp hand-shake in the weight path, so a warp that falls behind
//     delays nobody's loads.  When W equals the units of a row (K = 5120: 20 warps) a warp meets
//     the same slice of the activations in every tile and keeps its B operand in registers.
//   * Per tile each warp leaves 16 partial row sums in one of kRedBufs shared buffers and arrives
//     on the buffer's mbarrier without waiting; warp (tile mod W) adds the W partials in warp order
//     once they are all there - it looks once per iteration - and stores y (or, row sharded, the
//     band into every rank's y).
//
// Every wait is bounded (tc5::mbar_wait): a wait that runs out records a code in the device
// error word and raises the CTA's abort flag; every warp then stops computing, and before it
// leaves waits (bounded again) for the copies it still has in flight.
#include <cstdlib>

#include "gemv_i8_traits.cuh"
#include "tc5.cuh"

namespace {

using namespace gemv_i8;

constexpr uint32_t kMaxWarps = 12;
constexpr uint32_t kMaxDepth = 4;
constexpr uint32_t kRedBufs = 8;
constexpr uint32_t kSmemMax = 232448;  // 227 KB per CTA on sm_100
constexpr uint32_t kBoxBytes = 2048;   // 16 rows x 128 bytes

struct RingPlan {
    uint32_t W;          // warps
    uint32_t D;          // stages per warp
    uint32_t invariant;  // W == pairs per row: a warp's pair never changes
    uint32_t off_xmeta, off_red, off_bar, off_rec, off_data, smem_bytes;
};

enum : unsigned int { kErrRingFull = 0x11, kErrRingFold = 0x13, kErrRingDrain = 0x14, kErrRingFree = 0x15 };

// ---------------------------------------------------------------------------
// Ring traits: how a unit of a tile is read back from its boxes.  Stage, fold and kUnsignedA come
// from the shared traits.  The mma scheme differs from gemv_i8.cu's: one mma carries both
// activation limbs.  Its 32 k-slots are 8 weights of each of four blocks (lane t: block
// blk(p, t), slots 4t..4t+3 and 16+4t..16+4t+3), its eight columns are (block, limb) pairs, and
// column 2b + l is non-zero only in block b's slots.  Four mmas (j = 0..3) finish four blocks,
// two passes the unit's eight: 8 mmas per unit, and lane (g, t) ends up holding the high- and
// low-limb sums of blocks blk(0, t) and blk(1, t) for rows g and g + 8, which it folds with
// their scales.
// ---------------------------------------------------------------------------
// Physical offset of 16-byte chunk c of row r in a box written with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }
__device__ __forceinline__ uint32_t word4(const uint4& v, uint32_t i) { return i == 0u ? v.x : i == 1u ? v.y : i == 2u ? v.z : v.w; }

// load_ring arguments: `box` = the unit's first data box, o0 / o1 = swz(g, 2t) / swz(g, 2t + 1)
// (rows g + 8 lie 1024 bytes further), `rec` = row g's record of the unit (row g + 8: 8 box rows on).
struct RQ4K : Q4K {
    static constexpr uint32_t kDataBoxes = 1;
    // pass p of lane t feeds block 2t + p: the low (p = 0) or high nibbles of ggml group t, whose
    // first 16 bytes (chunk 2t) sit in k-slots 4t.. and whose second 16 (chunk 2t+1) in slots 16+4t..
    __device__ static __forceinline__ uint32_t blk(uint32_t p, uint32_t t) { return 2u * t + p; }
    __device__ static __forceinline__ void a_pass(const Stage& s, uint32_t p, uint32_t j, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint32_t mask = p ? 0xF0F0F0F0u : 0x0F0F0F0Fu;  // high nibbles stay in place: 16 x code, shifted back after
        a0 = word4(s.q[0], j) & mask;
        a1 = word4(s.q[2], j) & mask;
        a2 = word4(s.q[1], j) & mask;
        a3 = word4(s.q[3], j) & mask;
    }
    __device__ static __forceinline__ void load_ring(Stage& s, const uint8_t* box, const uint8_t* rec, uint32_t rec8,
                                                     uint32_t o0, uint32_t o1, uint32_t t) {
        s.q[0] = *reinterpret_cast<const uint4*>(box + o0);
        s.q[1] = *reinterpret_cast<const uint4*>(box + o1);
        s.q[2] = *reinterpret_cast<const uint4*>(box + o0 + 1024u);
        s.q[3] = *reinterpret_cast<const uint4*>(box + o1 + 1024u);
        const uint8_t* r1 = rec + rec8;
        s.dd[0] = *reinterpret_cast<const uint32_t*>(rec);
        s.dd[1] = *reinterpret_cast<const uint32_t*>(r1);
        s.sm[0] = (uint32_t)*reinterpret_cast<const uint16_t*>(rec + 4u + 2u * t) |
                  ((uint32_t)*reinterpret_cast<const uint16_t*>(rec + 12u + 2u * t) << 16);
        s.sm[1] = (uint32_t)*reinterpret_cast<const uint16_t*>(r1 + 4u + 2u * t) |
                  ((uint32_t)*reinterpret_cast<const uint16_t*>(r1 + 12u + 2u * t) << 16);
    }
};

struct RQ40 : Q40 {
    static constexpr uint32_t kDataBoxes = 1;
    __device__ static __forceinline__ uint32_t blk(uint32_t p, uint32_t t) { return 2u * t + p; }
    __device__ static __forceinline__ void a_pass(const Stage& s, uint32_t p, uint32_t j, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint32_t mask = p ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
        a0 = word4(s.q[0], j) & mask;
        a1 = word4(s.q[2], j) & mask;
        a2 = word4(s.q[1], j) & mask;
        a3 = word4(s.q[3], j) & mask;
    }
    __device__ static __forceinline__ void load_ring(Stage& s, const uint8_t* box, const uint8_t* rec, uint32_t rec8,
                                                     uint32_t o0, uint32_t o1, uint32_t t) {
        s.q[0] = *reinterpret_cast<const uint4*>(box + o0);
        s.q[1] = *reinterpret_cast<const uint4*>(box + o1);
        s.q[2] = *reinterpret_cast<const uint4*>(box + o0 + 1024u);
        s.q[3] = *reinterpret_cast<const uint4*>(box + o1 + 1024u);
        s.dd[0] = *reinterpret_cast<const uint32_t*>(rec + 4u * t);
        s.dd[1] = *reinterpret_cast<const uint32_t*>(rec + rec8 + 4u * t);
    }
};

struct RQ80 : Q80 {
    static constexpr uint32_t kDataBoxes = 2;  // blocks 0..3 | blocks 4..7 of the unit
    // pass p of lane t feeds block t + 4p: box p holds blocks 4p..4p+3, chunk 2t its block t's first
    // 16 bytes (k-slots 4t..), chunk 2t+1 the second 16 (slots 16+4t..)
    __device__ static __forceinline__ uint32_t blk(uint32_t p, uint32_t t) { return t + 4u * p; }
    __device__ static __forceinline__ void a_pass(const Stage& s, uint32_t p, uint32_t j, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        a0 = word4(s.q[2u * p], j);
        a1 = word4(s.q[4u + 2u * p], j);
        a2 = word4(s.q[2u * p + 1u], j);
        a3 = word4(s.q[5u + 2u * p], j);
    }
    __device__ static __forceinline__ void load_ring(Stage& s, const uint8_t* box, const uint8_t* rec, uint32_t rec8,
                                                     uint32_t o0, uint32_t o1, uint32_t t) {
        s.q[0] = *reinterpret_cast<const uint4*>(box + o0);
        s.q[1] = *reinterpret_cast<const uint4*>(box + o1);
        s.q[2] = *reinterpret_cast<const uint4*>(box + kBoxBytes + o0);
        s.q[3] = *reinterpret_cast<const uint4*>(box + kBoxBytes + o1);
        s.q[4] = *reinterpret_cast<const uint4*>(box + o0 + 1024u);
        s.q[5] = *reinterpret_cast<const uint4*>(box + o1 + 1024u);
        s.q[6] = *reinterpret_cast<const uint4*>(box + kBoxBytes + o0 + 1024u);
        s.q[7] = *reinterpret_cast<const uint4*>(box + kBoxBytes + o1 + 1024u);
        const uint8_t* r0 = rec + 2u * t;  // f16 d[t] | d[t + 4] << 16
        s.dd[0] = (uint32_t)*reinterpret_cast<const uint16_t*>(r0) | ((uint32_t)*reinterpret_cast<const uint16_t*>(r0 + 8u) << 16);
        s.dd[1] = (uint32_t)*reinterpret_cast<const uint16_t*>(r0 + rec8) |
                  ((uint32_t)*reinterpret_cast<const uint16_t*>(r0 + rec8 + 8u) << 16);
    }
};

template <class F>
__global__ void __launch_bounds__(kMaxWarps * 32u, 1)
gemv_ring_kernel(const __grid_constant__ CUtensorMap dmap, const __grid_constant__ CUtensorMap rmap,
                 const float* __restrict__ bias, const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim,
                 uint32_t out_dim, const int8_t* __restrict__ xq, const float* __restrict__ xq_scale, const PeerOut peers,
                 const RingPlan pl, unsigned int* __restrict__ err) {
    using Stage = typename F::Stage;
    constexpr uint32_t kUnitData = F::kDataBoxes * kBoxBytes;       // one unit's boxes
    constexpr uint32_t kRecRow = 2u * F::kRecBytes;                 // a pair's records of one row
    constexpr uint32_t kStageData = 2u * kUnitData, kStageRec = 16u * kRecRow;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t n_pair = in_dim >> 9;
    uint8_t* xs_hi = smem;
    uint8_t* xs_lo = smem + in_dim;
    uint8_t* zeros = smem + 2u * (size_t)in_dim;
    float2* xmeta = reinterpret_cast<float2*>(smem + pl.off_xmeta);
    float* red = reinterpret_cast<float*>(smem + pl.off_red);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + pl.off_bar);  // [W][kMaxDepth]
    uint64_t* red_full = full + kMaxWarps * kMaxDepth;
    uint64_t* red_free = red_full + kRedBufs;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(red_free + kRedBufs);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t W = pl.W, D = pl.D;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t tile_lo = (uint32_t)((uint64_t)blockIdx.x * n_tiles / gridDim.x);
    const uint32_t tile_hi = (uint32_t)((uint64_t)(blockIdx.x + 1u) * n_tiles / gridDim.x);
    const uint32_t my_tiles = tile_hi - tile_lo;
    // this warp's pairs of a tile: warp, warp + W, ... below n_pair
    const uint32_t my_pairs = warp < n_pair ? (n_pair - warp + W - 1u) / W : 0u;
    const uint32_t total = my_tiles * my_pairs;

    uint64_t* my_full = full + warp * kMaxDepth;
    uint8_t* my_data = smem + pl.off_data + (size_t)warp * D * kStageData;
    uint8_t* my_rec = smem + pl.off_rec + (size_t)warp * D * kStageRec;

    // (tile, pair) number i of this warp -> stage i % D; issue = arm the barrier, then the copies.
    // Called by the whole (converged) warp: one elected lane issues, so addresses and the
    // tensor-map pointers stay in uniform registers.
    const uint64_t stream_once = tc5::l2_policy_evict_first();   // a plane is read once per launch
    auto issue = [&](uint32_t stage, uint32_t tl, uint32_t pr) {
        uint64_t* bar = my_full + stage;
        tc5::mbar_arrive_expect_tx_elect(bar, kStageData + kStageRec);
        const int32_t row = (int32_t)((tile_lo + tl) * 16u);
#pragma unroll
        for (uint32_t b = 0; b < 2u * F::kDataBoxes; ++b)
            tc5::tma_load_2d_hint_elect(my_data + stage * kStageData + b * kBoxBytes, &dmap, bar,
                                        (int32_t)(pr * 2u * F::kDataBytes + b * 128u), row, stream_once);
        tc5::tma_load_2d_hint_elect(my_rec + stage * kStageRec, &rmap, bar, (int32_t)(pr * kRecRow), row, stream_once);
    };

    // ---- prologue: every warp arms its own barriers and requests its first D stages; only then
    // does the CTA meet (shared barriers of the tile fold) and wait for the previous kernel
    if (lane == 0u) {
        for (uint32_t s = 0; s < D; ++s) tc5::mbar_init(my_full + s, 1u);
        tc5::mbar_fence_init();
    }
    __syncwarp();
    uint32_t i_tl = 0, i_pr = warp, issued = 0;  // issue cursor
    auto issue_next = [&]() {
        issue(issued % D, i_tl, i_pr);
        ++issued;
        i_pr += W;
        if (i_pr >= n_pair) { i_pr = warp; ++i_tl; }
    };
    // the first stage of every warp goes out alone: it is what the first iteration waits for, and
    // it arrives sooner when the chip's first burst is a quarter of the ring
    if (total > 0u) issue_next();
    if (tid == 0u) {
        for (uint32_t b = 0; b < kRedBufs; ++b) {
            tc5::mbar_init(&red_full[b], W);
            tc5::mbar_init(&red_free[b], 1u);
        }
        *abort_flag = 0;
        tc5::mbar_fence_init();
    }
    if (tid < 8u) reinterpret_cast<uint32_t*>(zeros)[tid] = 0u;
    // The CTA meets once, here, where it would wait for the previous kernel anyway: the fold
    // barriers and the zero line are shared, everything after is per warp (invariant plans).
    __syncthreads();
    // Programmatic dependent launch: the next kernel of the stream may start its prologue (its own
    // first requests: weights never depend on this kernel) as soon as this one's CTAs have all started.
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();  // x (and y's previous contents) belong to the previous kernel until here
    uint32_t peer_step = 0u;
    const bool peer_deferred = peers.n != 0u && peers.signal == 2u && blockIdx.x == 0u && tid == 0u;
    if (peer_deferred) peer_step = peer_post_previous(peers);
    const bool invariant = pl.invariant != 0u;
    if (invariant) {
        // A warp only ever meets its own pair's 512 activations: it builds their limbs itself.  The
        // loads of x go out before the rest of the ring is requested, so they do not queue behind it.
        const uint32_t g0 = warp * 64u + lane;   // groups of 8 elements: this lane's two
        float v0[8], v1[8];
        limb_load8(x, xq, xq_scale, g0, v0);
        limb_load8(x, xq, xq_scale, g0 + 32u, v1);
        while (issued < D && issued < total) issue_next();
        limb_store8(v0, g0, xs_hi, xs_lo, xmeta);
        limb_store8(v1, g0 + 32u, xs_hi, xs_lo, xmeta);
        __syncwarp();
    } else {
        const uint32_t groups = in_dim >> 3;
        for (uint32_t grp = tid; grp < groups; grp += W * 32u) {
            float v[8];
            limb_load8(x, xq, xq_scale, grp, v);
            limb_store8(v, grp, xs_hi, xs_lo, xmeta);
        }
        while (issued < D && issued < total) issue_next();
        __syncthreads();
    }
    const tc5::WaitCtx ctx{abort_flag, err};

    const uint32_t g = lane >> 2, t = lane & 3u;
    // B operand of this lane: columns 2b, 2b + 1 are the high and low limb of local block b, so
    // lane (g, t) feeds limb g & 1 of block blk(p, t) when g >> 1 == t, and zeros otherwise.
    const bool role = (g >> 1) == t;
    const uint8_t* my_limb = (g & 1u) ? xs_lo : xs_hi;
    uint32_t vb[2][2][8];  // [unit of the pair][pass]: words 0..3 -> b0 of mma j, words 4..7 -> b1
    float4 xm[2];          // per unit: {step, sum} of blocks blk(0, t) and blk(1, t), the two this lane folds
    auto load_b = [&](uint32_t pr) {
#pragma unroll
        for (uint32_t i = 0; i < 2u; ++i) {
            const uint32_t u = 2u * pr + i;
#pragma unroll
            for (uint32_t p = 0; p < 2u; ++p) {
                const uint8_t* src = role ? my_limb + u * 256u + F::blk(p, t) * 32u : zeros;
                const uint4 a = *reinterpret_cast<const uint4*>(src);
                const uint4 b = *reinterpret_cast<const uint4*>(src + 16u);
                vb[i][p][0] = a.x; vb[i][p][1] = a.y; vb[i][p][2] = a.z; vb[i][p][3] = a.w;
                vb[i][p][4] = b.x; vb[i][p][5] = b.y; vb[i][p][6] = b.z; vb[i][p][7] = b.w;
            }
            const float2 m0 = xmeta[u * 8u + F::blk(0u, t)], m1 = xmeta[u * 8u + F::blk(1u, t)];
            xm[i] = make_float4(m0.x, m0.y, m1.x, m1.y);
        }
    };
    if (invariant && warp < n_pair) load_b(warp);

    // per-lane offsets inside a stage
    const uint32_t o0 = swz(g, 2u * t), o1 = swz(g, 2u * t + 1u);
    const uint32_t rec_g = g * kRecRow, rec8 = 8u * kRecRow;

    // ---- tile fold.  Per tile each warp leaves 16 partial row sums in buffer tl % kRedBufs and
    // arrives on the buffer's barrier (fire and forget).  The tile belongs to warp tl % W, which
    // looks at the barrier once per later iteration and, when all W warps have arrived, adds the
    // partials in warp order, stores y and hands the buffer back; it blocks only before taking on
    // another tile, and at the end.  A buffer is written again (tile tl + kRedBufs) only after
    // its fold.
    constexpr uint32_t kNone = 0xffffffffu;
    uint32_t pend = kNone;  // local index of the tile this warp still has to fold
    bool alive = true;
    auto fold_tile = [&](uint32_t tl_f) {
        const uint32_t rbf = tl_f % kRedBufs;
        const float* rbuf = red + (size_t)rbf * (W * 16u);
        const uint32_t row = (tile_lo + tl_f) * 16u + lane;
        float v = 0.0f;
        if (lane < 16u)
            for (uint32_t w = 0; w < W; ++w) v += rbuf[w * 16u + lane];
        __syncwarp();
        if (lane == 0u) tc5::mbar_arrive(&red_free[rbf]);
        if (lane < 16u && row < out_dim) {
            if (bias) v += bias[row];
            if (peers.n == 0u) {
                y[row] = v;
            } else {
#pragma unroll
                for (uint32_t p = 0; p < 8u; ++p)  // constant indices: the pointers stay in the parameter bank
                    if (p < peers.n) peers.ptr[p][peers.row0 + row] = v;
            }
        }
    };
    auto poll_fold = [&](bool block) {
        if (pend == kNone || !alive) return;
        const uint32_t rbf = pend % kRedBufs, ph = (pend / kRedBufs) & 1u;
        bool done;
        if (block) {
            alive = __all_sync(0xffffffffu, tc5::mbar_wait(&red_full[rbf], ph, ctx, kErrRingFold, rbf));
            done = alive;
        } else {
            done = __all_sync(0xffffffffu, tc5::mbar_try_wait(&red_full[rbf], ph));
        }
        if (done) {
            fold_tile(pend);
            pend = kNone;
        }
    };

    uint32_t stage = 0, phase = 0;       // consume cursor
    uint32_t rb = 0, rb_phase = 0, owner = 0;
    for (uint32_t tl = 0; tl < my_tiles; ++tl) {
        float acc_g = 0.0f, acc_g8 = 0.0f;
        for (uint32_t pr = warp; pr < n_pair; pr += W) {
            if (alive) alive = __all_sync(0xffffffffu, tc5::mbar_wait(my_full + stage, phase, ctx, kErrRingFull, stage));
            if (alive) {
                Stage st[2];
                const uint8_t* sd = my_data + stage * kStageData;
                const uint8_t* sr = my_rec + stage * kStageRec + rec_g;
                F::load_ring(st[0], sd, sr, rec8, o0, o1, t);
                F::load_ring(st[1], sd + kUnitData, sr + F::kRecBytes, rec8, o0, o1, t);
                if (!invariant) load_b(pr);
                // four independent accumulator chains: [unit][pass], {hi, lo} of row g, {hi, lo} of row g + 8
                int c[2][2][4] = {};
#pragma unroll
                for (uint32_t j = 0; j < 4u; ++j) {
#pragma unroll
                    for (uint32_t i = 0; i < 2u; ++i) {
#pragma unroll
                        for (uint32_t p = 0; p < 2u; ++p) {
                            uint32_t a0, a1, a2, a3;
                            F::a_pass(st[i], p, j, a0, a1, a2, a3);
                            if constexpr (F::kUnsignedA) mma_u8s8_nv(c[i][p], a0, a1, a2, a3, vb[i][p][j], vb[i][p][4u + j]);
                            else mma_s8_nv(c[i][p], a0, a1, a2, a3, vb[i][p][j], vb[i][p][4u + j]);
                        }
                    }
                }
#pragma unroll
                for (uint32_t i = 0; i < 2u; ++i) {
                    float f[4];
                    f[0] = (float)(c[i][0][0] * 256 + c[i][0][1]) * xm[i].x;
                    f[1] = (float)((c[i][1][0] * 256 + c[i][1][1]) >> F::kHiShift) * xm[i].z;
                    f[2] = (float)(c[i][0][2] * 256 + c[i][0][3]) * xm[i].x;
                    f[3] = (float)((c[i][1][2] * 256 + c[i][1][3]) >> F::kHiShift) * xm[i].z;
                    F::fold(st[i], f, xm[i].y, xm[i].w, acc_g, acc_g8);
                }
                // Every register the stage's loads filled has been consumed by now, so those loads
                // are complete: the stage can take its next copy.
                __syncwarp();
                if (issued < total) issue_next();
            }
            if (++stage == D) { stage = 0; phase ^= 1u; }
        }
        float a = acc_g, b = acc_g8;
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        b += __shfl_xor_sync(0xffffffffu, b, 1);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        b += __shfl_xor_sync(0xffffffffu, b, 2);
        float* rbuf = red + (size_t)rb * (W * 16u);
        if (alive && tl >= kRedBufs)
            alive = __all_sync(0xffffffffu, tc5::mbar_wait(&red_free[rb], rb_phase ^ 1u, ctx, kErrRingFree, rb));
        if (alive) {
            if (t == 0u) {
                rbuf[warp * 16u + g] = a;
                rbuf[warp * 16u + g + 8u] = b;
            }
            __syncwarp();
            if (lane == 0u) tc5::mbar_arrive(&red_full[rb]);  // release: the partials above are visible to the folding warp
        }
        if (owner == warp) {
            poll_fold(true);   // the previous tile of this warp, if it is still waiting (W tiles ago)
            pend = tl;
        }
        poll_fold(false);
        if (++owner == W) owner = 0;
        if (++rb == kRedBufs) { rb = 0; rb_phase ^= 1u; }
    }
    poll_fold(true);
    if (peers.n != 0u && peers.signal == 1u) {   // uniform over the grid
        __syncthreads();
        if (tid == 0u) peer_signal(peers, err);
    }
    if (peer_deferred) peer_check_previous(peers, peer_step, err);
    if (!alive) {
        // a wait ran out somewhere in the CTA: the copies this warp still has in flight must land
        // before its shared memory can go to another CTA.  At most D are outstanding, one per stage.
        const unsigned long long t0 = tc5::globaltimer_ns();
        for (uint32_t s = 0; s < D && s < issued; ++s) {
            // the last copy into stage s is number n = the largest n < issued with n % D == s
            const uint32_t n = issued - 1u - ((issued - 1u - s) % D);
            while (!tc5::mbar_try_wait(my_full + s, (n / D) & 1u)) {
                if (tc5::globaltimer_ns() - t0 > tc5::kWaitBudgetNs) {
                    if (lane == 0u) tc5::report(err, kErrRingDrain, s);
                    break;
                }
            }
        }
    }
}

template <class F>
bool make_plan(uint32_t in_dim, RingPlan& best) {
    if (in_dim == 0u || (in_dim & 511u) != 0u) return false;  // whole pairs of units
    const uint32_t n_pair = in_dim >> 9;
    if (n_pair < 4u) return false;
    constexpr uint32_t kStage = 2u * F::kDataBoxes * kBoxBytes + 32u * F::kRecBytes;
    double best_cost = 1e30;
    bool found = false;
    for (uint32_t W = kMaxWarps; W >= 4u; --W) {
        RingPlan p{};
        p.W = W;
        const uint32_t rounds = (n_pair + W - 1u) / W;
        p.invariant = (W == n_pair) ? 1u : 0u;
        p.off_xmeta = (2u * in_dim + 32u + 15u) & ~15u;
        p.off_red = p.off_xmeta + (in_dim >> 5) * 8u;
        p.off_bar = p.off_red + kRedBufs * W * 64u;
        p.off_rec = (p.off_bar + (kMaxWarps * kMaxDepth + 2u * kRedBufs) * 8u + 16u + 127u) & ~127u;
        const uint32_t fixed = p.off_rec;
        if (fixed + 1024u + 2u * W * kStage > kSmemMax) continue;
        p.D = (kSmemMax - fixed - 1024u) / (W * kStage);
        if (p.D > kMaxDepth) p.D = kMaxDepth;
        p.off_data = (p.off_rec + W * p.D * 32u * F::kRecBytes + 1023u) & ~1023u;  // swizzled boxes start on 1 KB
        p.smem_bytes = p.off_data + W * p.D * 2u * F::kDataBoxes * kBoxBytes;
        if (p.smem_bytes > kSmemMax) continue;
        double cost = (double)(rounds * W) / (double)n_pair;   // idle warps in a tile's last round
        if (p.D < 3u) cost += 0.04 * (3u - p.D);
        if (W < 8u) cost += 0.03 * (8u - W);
        cost -= 1e-9 * (double)(W * p.D * kStage);            // ties: more bytes in flight
        if (cost < best_cost) {
            best_cost = cost;
            best = p;
            found = true;
        }
    }
    return found;
}

// PDK_GEMV_REGS=1 sends every call to the register-staged kernel (A/B switch, read once).
bool force_regs() {
    static const bool v = [] {
        const char* e = getenv("PDK_GEMV_REGS");
        return e && e[0] == '1';
    }();
    return v;
}

// Tensor maps of the planes a thread used last (weights stay where they are, so a decode loop
// encodes each plane's maps once): [rows][row bytes] uint8, data boxes 128 x 16 swizzled, record
// boxes of a unit pair's records x 16 dense.
struct MapEntry {
    const void *data, *recs;
    uint32_t in_dim, out_dim, rec_box;
    CUtensorMap dmap, rmap;
};
template <class F>
int plane_maps(const void* data, const void* recs, uint32_t in_dim, uint32_t out_dim, const MapEntry** out) {
    constexpr int kEntries = 16;
    thread_local MapEntry cache[kEntries];
    thread_local int next = 0, used = 0;
    for (int i = 0; i < used; ++i) {
        const MapEntry& e = cache[i];
        if (e.data == data && e.recs == recs && e.in_dim == in_dim && e.out_dim == out_dim && e.rec_box == 2u * F::kRecBytes) {
            *out = &e;
            return 0;
        }
    }
    MapEntry& e = cache[next];
    const uint32_t n_unit = in_dim >> 8;
    int rc = pdk_make_tmap_2d(&e.dmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1u, data, (uint64_t)n_unit * F::kDataBytes, out_dim,
                              (uint64_t)n_unit * F::kDataBytes, 128u, 16u);
    if (rc == 0)
        rc = pdk_make_tmap_2d_dense(&e.rmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1u, recs, (uint64_t)n_unit * F::kRecBytes,
                                    out_dim, (uint64_t)n_unit * F::kRecBytes, 2u * F::kRecBytes, 16u);
    if (rc != 0) {
        e.data = nullptr;
        return rc;
    }
    e.data = data; e.recs = recs; e.in_dim = in_dim; e.out_dim = out_dim; e.rec_box = 2u * F::kRecBytes;
    *out = &e;
    next = (next + 1) % kEntries;
    if (used < kEntries) ++used;
    return 0;
}

template <class F>
int launch_ring(const void* data, const void* recs, const float* bias, const float* x, float* y, uint32_t in_dim,
                uint32_t out_dim, cudaStream_t st, const int8_t* xq = nullptr, const float* xq_scale = nullptr,
                const PeerOut* peers = nullptr) {
    if (force_regs() || !pdk_aligned(recs, 16)) return -1;  // tensor maps start on 16 bytes
    RingPlan pl;
    if (!make_plan<F>(in_dim, pl)) return -1;
    const MapEntry* maps = nullptr;
    if (plane_maps<F>(data, recs, in_dim, out_dim, &maps) != 0) return -1;
    auto kern = gemv_ring_kernel<F>;
    static bool attr_set[64] = {false};  // per device, per format (one instance of this function per F)
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    unsigned int* err = pdk_error_word();
    if (err == nullptr) return (int)cudaErrorUnknown;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_tiles) grid = n_tiles;
    PeerOut po{};
    if (peers) po = *peers;
    return pdk_launch_pdl(kern, dim3(grid), dim3(pl.W * 32u), (size_t)pl.smem_bytes, st, maps->dmap, maps->rmap, bias, x, y,
                          in_dim, out_dim, xq, xq_scale, po, pl, err);
}


// ---------------------------------------------------------------------------
// Q8_0 with 2..8 tokens on the same ring: the tokens are the mma's eight columns.
//
// Plans with one unit pair per warp only (W == K / 512, K = 2048 .. 6144): warp w meets the same
// 512 activations of every token in every tile, so its B operand - two int8 limbs of the 15-bit
// block floating point, per (token, 32-block) power-of-two steps - is built once from x and stays
// in 64 registers.  Per 32-weight block: one ldmatrix.x4 takes the 16 rows x 32 int8 out of the
// swizzled box (conflict free: the eight rows of a matrix sit in eight different bank groups),
// one mma per limb gives the integer tile [16 rows][8 tokens], and lane (g, t) folds its four
// entries with d[row][block] * step[token][block] in f32.  Weights leave HBM once for all tokens.
// ---------------------------------------------------------------------------
constexpr uint32_t kBatchRedBufs = 4;

struct BatchPlan {
    uint32_t W, D;
    uint32_t off_steps, off_red, off_bar, off_rec, off_data, smem_bytes;
};

enum : unsigned int { kErrBatchFull = 0x18, kErrBatchFold = 0x19, kErrBatchFree = 0x1a, kErrBatchDrain = 0x1b };

__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(saddr));
}

__global__ void __launch_bounds__(kMaxWarps * 32u, 1)
gemm_ring_q8_kernel(const __grid_constant__ CUtensorMap dmap, const __grid_constant__ CUtensorMap rmap,
                    const float* __restrict__ bias, const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim,
                    uint32_t out_dim, uint32_t batch, const BatchPlan pl, unsigned int* __restrict__ err,
                    const uint32_t last_pass) {
    constexpr uint32_t kUnitData = 2u * kBoxBytes;             // a unit's two boxes (blocks 0..3 | 4..7)
    constexpr uint32_t kRecRow = 2u * Q80::kRecBytes;          // a pair's records of one row
    constexpr uint32_t kStageData = 2u * kUnitData, kStageRec = 16u * kRecRow;
    extern __shared__ __align__(1024) uint8_t smem[];
    float* steps = reinterpret_cast<float*>(smem + pl.off_steps);   // [W][16 blocks][8 tokens]
    float* red = reinterpret_cast<float*>(smem + pl.off_red);       // [kBatchRedBufs][W][16 rows][8 tokens]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + pl.off_bar);
    uint64_t* red_full = full + kMaxWarps * kMaxDepth;
    uint64_t* red_free = red_full + kBatchRedBufs;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(red_free + kBatchRedBufs);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t W = pl.W, D = pl.D;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t tile_lo = (uint32_t)((uint64_t)blockIdx.x * n_tiles / gridDim.x);
    const uint32_t tile_hi = (uint32_t)((uint64_t)(blockIdx.x + 1u) * n_tiles / gridDim.x);
    const uint32_t my_tiles = tile_hi - tile_lo;

    uint64_t* my_full = full + warp * kMaxDepth;
    uint8_t* my_data = smem + pl.off_data + (size_t)warp * D * kStageData;
    uint8_t* my_rec = smem + pl.off_rec + (size_t)warp * D * kStageRec;

    // The call's last pass over the plane loads it evict-first (nothing reads it again); an earlier pass
    // of a call with more than eight tokens leaves what fits in L2 to the pass that follows.
    const uint64_t stream_once = tc5::l2_policy_evict_first();
    auto issue = [&](uint32_t stage, uint32_t tl) {
        uint64_t* bar = my_full + stage;
        tc5::mbar_arrive_expect_tx_elect(bar, kStageData + kStageRec);
        const int32_t row = (int32_t)((tile_lo + tl) * 16u);
        if (last_pass) {
#pragma unroll
            for (uint32_t b = 0; b < 4u; ++b)
                tc5::tma_load_2d_hint_elect(my_data + stage * kStageData + b * kBoxBytes, &dmap, bar,
                                            (int32_t)(warp * 2u * Q80::kDataBytes + b * 128u), row, stream_once);
            tc5::tma_load_2d_hint_elect(my_rec + stage * kStageRec, &rmap, bar, (int32_t)(warp * kRecRow), row, stream_once);
        } else {
#pragma unroll
            for (uint32_t b = 0; b < 4u; ++b)
                tc5::tma_load_2d_elect(my_data + stage * kStageData + b * kBoxBytes, &dmap, bar,
                                       (int32_t)(warp * 2u * Q80::kDataBytes + b * 128u), row);
            tc5::tma_load_2d_elect(my_rec + stage * kStageRec, &rmap, bar, (int32_t)(warp * kRecRow), row);
        }
    };

    if (lane == 0u) {
        for (uint32_t s = 0; s < D; ++s) tc5::mbar_init(my_full + s, 1u);
        tc5::mbar_fence_init();
    }
    __syncwarp();
    uint32_t issued = 0;
    if (my_tiles > 0u) { issue(0u, 0u); issued = 1u; }
    if (tid == 0u) {
        for (uint32_t b = 0; b < kBatchRedBufs; ++b) {
            tc5::mbar_init(&red_full[b], W);
            tc5::mbar_init(&red_free[b], 1u);
        }
        *abort_flag = 0;
        tc5::mbar_fence_init();
    }
    __syncthreads();
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();   // x and y belong to the previous kernel until here

    // ---- B operand: token g, this warp's 16 blocks.  Lane (g, t) holds elements 4t..4t+3 and
    // 16+4t..16+4t+3 of each block, which is exactly its share of the mma's B fragment.
    const uint32_t g = lane >> 2, t = lane & 3u;
    uint32_t bh[16][2], bl[16][2];
    {
        const float* xt = x + (size_t)(g < batch ? g : 0u) * in_dim + warp * 512u + 4u * t;
        float* my_steps = steps + warp * 128u;
#pragma unroll
        for (uint32_t b = 0; b < 16u; ++b) {
            float4 v0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), v1 = v0;
            if (g < batch) {
                v0 = *reinterpret_cast<const float4*>(xt + b * 32u);
                v1 = *reinterpret_cast<const float4*>(xt + b * 32u + 16u);
            }
            float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                               fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            // amax < 2^ex -> step 2^(ex-14): |q| <= 2^14, q = 256 * hi + lo with lo in [-128, 127]
            float step = 1.0f, inv = 0.0f;
            if (amax > 0.0f && amax < 3.0e38f) {
                const int ex = max((int)(__float_as_uint(amax) >> 23) - 126, -110);
                step = __uint_as_float((uint32_t)(ex + 113) << 23);
                inv = __uint_as_float((uint32_t)(141 - ex) << 23);
            }
            const int q0 = __float2int_rn(v0.x * inv), q1 = __float2int_rn(v0.y * inv), q2 = __float2int_rn(v0.z * inv),
                      q3 = __float2int_rn(v0.w * inv), q4 = __float2int_rn(v1.x * inv), q5 = __float2int_rn(v1.y * inv),
                      q6 = __float2int_rn(v1.z * inv), q7 = __float2int_rn(v1.w * inv);
            bl[b][0] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
            bl[b][1] = __byte_perm(__byte_perm(q4, q5, 0x0040), __byte_perm(q6, q7, 0x0040), 0x5410);
            bh[b][0] = __byte_perm(__byte_perm(q0 + 128, q1 + 128, 0x0051), __byte_perm(q2 + 128, q3 + 128, 0x0051), 0x5410);
            bh[b][1] = __byte_perm(__byte_perm(q4 + 128, q5 + 128, 0x0051), __byte_perm(q6 + 128, q7 + 128, 0x0051), 0x5410);
            if (t == 0u) my_steps[b * 8u + g] = step;
        }
        __syncwarp();
    }
    while (issued < D && issued < my_tiles) { issue(issued % D, issued); ++issued; }
    const tc5::WaitCtx ctx{abort_flag, err};

    // ldmatrix row addresses: lane l supplies row (l & 7) + 8 * ((l >> 3) & 1) of k-half (l >> 4);
    // block bb of a unit = chunks 2 * (bb & 3) + k-half of box bb >> 2
    const uint32_t m_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u, m_half = lane >> 4;
    uint32_t a_off[4];
#pragma unroll
    for (uint32_t c = 0; c < 4u; ++c) a_off[c] = swz(m_row, 2u * c + m_half);
    const float* my_steps = steps + warp * 128u + 2u * t;
    const uint32_t rec_g = g * kRecRow, rec8 = 8u * kRecRow;

    constexpr uint32_t kNone = 0xffffffffu;
    uint32_t pend = kNone;
    bool alive = true;
    auto fold_tile = [&](uint32_t tl_f) {
        const uint32_t rbf = tl_f % kBatchRedBufs;
        const float* rbuf = red + (size_t)rbf * (W * 128u);
        // lane -> row lane & 15, tokens 4 * (lane >> 4) .. + 3
        const uint32_t r = lane & 15u, c0 = (lane >> 4) * 4u;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t w = 0; w < W; ++w) {
            const float4 p = *reinterpret_cast<const float4*>(rbuf + w * 128u + r * 8u + c0);
            v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
        }
        __syncwarp();
        if (lane == 0u) tc5::mbar_arrive(&red_free[rbf]);
        const uint32_t row = (tile_lo + tl_f) * 16u + r;
        if (row < out_dim) {
            const float bv = bias ? bias[row] : 0.0f;
#pragma unroll
            for (uint32_t c = 0; c < 4u; ++c)
                if (c0 + c < batch) y[(size_t)(c0 + c) * out_dim + row] = v[c] + bv;
        }
    };
    auto poll_fold = [&](bool block) {
        if (pend == kNone || !alive) return;
        const uint32_t rbf = pend % kBatchRedBufs, ph = (pend / kBatchRedBufs) & 1u;
        bool done;
        if (block) {
            alive = __all_sync(0xffffffffu, tc5::mbar_wait(&red_full[rbf], ph, ctx, kErrBatchFold, rbf));
            done = alive;
        } else {
            done = __all_sync(0xffffffffu, tc5::mbar_try_wait(&red_full[rbf], ph));
        }
        if (done) {
            fold_tile(pend);
            pend = kNone;
        }
    };

    uint32_t stage = 0, phase = 0, rb = 0, rb_phase = 0, owner = 0;
    for (uint32_t tl = 0; tl < my_tiles; ++tl) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // (g, 2t) (g, 2t+1) (g+8, 2t) (g+8, 2t+1)
        if (alive) alive = __all_sync(0xffffffffu, tc5::mbar_wait(my_full + stage, phase, ctx, kErrBatchFull, stage));
        if (alive) {
            const uint32_t sd = tc5::smem_u32(my_data + stage * kStageData);
            const uint8_t* sr = my_rec + stage * kStageRec + rec_g;
#pragma unroll
            for (uint32_t i = 0; i < 2u; ++i) {
                const uint4 dg = *reinterpret_cast<const uint4*>(sr + i * Q80::kRecBytes);
                const uint4 dg8 = *reinterpret_cast<const uint4*>(sr + rec8 + i * Q80::kRecBytes);
#pragma unroll
                for (uint32_t bb = 0; bb < 8u; ++bb) {
                    const uint32_t b = i * 8u + bb;
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(sd + i * kUnitData + (bb >> 2) * kBoxBytes + a_off[bb & 3u], a0, a1, a2, a3);
                    int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
                    mma_s8_nv(ch, a0, a1, a2, a3, bh[b][0], bh[b][1]);
                    mma_s8_nv(cl, a0, a1, a2, a3, bl[b][0], bl[b][1]);
                    const float2 s = *reinterpret_cast<const float2*>(my_steps + b * 8u);
                    const uint32_t wg = word4(dg, bb >> 1), wg8 = word4(dg8, bb >> 1);
                    const __half2 hg = *reinterpret_cast<const __half2*>(&wg), hg8 = *reinterpret_cast<const __half2*>(&wg8);
                    const float d0 = (bb & 1u) ? __high2float(hg) : __low2float(hg);
                    const float d8 = (bb & 1u) ? __high2float(hg8) : __low2float(hg8);
                    acc[0] += (float)(ch[0] * 256 + cl[0]) * (d0 * s.x);
                    acc[1] += (float)(ch[1] * 256 + cl[1]) * (d0 * s.y);
                    acc[2] += (float)(ch[2] * 256 + cl[2]) * (d8 * s.x);
                    acc[3] += (float)(ch[3] * 256 + cl[3]) * (d8 * s.y);
                }
            }
            __syncwarp();
            if (issued < my_tiles) { issue(issued % D, issued); ++issued; }
        }
        if (++stage == D) { stage = 0; phase ^= 1u; }

        float* rbuf = red + (size_t)rb * (W * 128u);
        if (alive && tl >= kBatchRedBufs)
            alive = __all_sync(0xffffffffu, tc5::mbar_wait(&red_free[rb], rb_phase ^ 1u, ctx, kErrBatchFree, rb));
        if (alive) {
            *reinterpret_cast<float2*>(rbuf + warp * 128u + g * 8u + 2u * t) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(rbuf + warp * 128u + (g + 8u) * 8u + 2u * t) = make_float2(acc[2], acc[3]);
            __syncwarp();
            if (lane == 0u) tc5::mbar_arrive(&red_full[rb]);
        }
        if (owner == warp) {
            poll_fold(true);
            pend = tl;
        }
        poll_fold(false);
        if (++owner == W) owner = 0;
        if (++rb == kBatchRedBufs) { rb = 0; rb_phase ^= 1u; }
    }
    poll_fold(true);
    if (!alive) {
        const unsigned long long t0 = tc5::globaltimer_ns();
        for (uint32_t s = 0; s < D && s < issued; ++s) {
            const uint32_t n = issued - 1u - ((issued - 1u - s) % D);
            while (!tc5::mbar_try_wait(my_full + s, (n / D) & 1u)) {
                if (tc5::globaltimer_ns() - t0 > tc5::kWaitBudgetNs) {
                    if (lane == 0u) tc5::report(err, kErrBatchDrain, s);
                    break;
                }
            }
        }
    }
}

bool make_batch_plan(uint32_t in_dim, BatchPlan& p) {
    if (in_dim == 0u || (in_dim & 511u) != 0u) return false;
    const uint32_t W = in_dim >> 9;
    if (W < 4u || W > kMaxWarps) return false;
    constexpr uint32_t kStage = 4u * kBoxBytes + 32u * Q80::kRecBytes;
    p.W = W;
    p.off_steps = 0u;
    p.off_red = W * 512u;
    p.off_bar = p.off_red + kBatchRedBufs * W * 512u;
    p.off_rec = (p.off_bar + (kMaxWarps * kMaxDepth + 2u * kBatchRedBufs) * 8u + 16u + 127u) & ~127u;
    if (p.off_rec + 1024u + 2u * W * kStage > kSmemMax) return false;
    p.D = (kSmemMax - p.off_rec - 1024u) / (W * kStage);
    if (p.D > kMaxDepth) p.D = kMaxDepth;
    p.off_data = (p.off_rec + W * p.D * 32u * Q80::kRecBytes + 1023u) & ~1023u;
    p.smem_bytes = p.off_data + W * p.D * 4u * kBoxBytes;
    return p.smem_bytes <= kSmemMax && p.D >= 2u;
}


}  // namespace

// gemv_i8.cu: the register-staged kernel
int pdk_q4k_gemv_i8_regs(const void*, const void*, const float*, float*, uint32_t, uint32_t, cudaStream_t);
int pdk_q4_0_gemv_i8_regs(const void*, const void*, const float*, float*, uint32_t, uint32_t, cudaStream_t);
int pdk_q5k_gemv_i8_regs(const void*, const void*, const float*, float*, uint32_t, uint32_t, cudaStream_t);
int pdk_q8_0_gemv_i8_regs(const void*, const void*, const float*, const float*, float*, uint32_t, uint32_t, cudaStream_t);
int pdk_q4k_gemv_i8_q8act_regs(const void*, const void*, const int8_t*, const float*, float*, uint32_t, uint32_t,
                               cudaStream_t);
int pdk_q4k_gemv_peers_regs(const void*, const void*, const float*, const gemv_i8::PeerOut*, uint32_t, uint32_t,
                            cudaStream_t);

// Decode GEMV entry points of the int8 tensor path.  Each returns 0 / a cudaError_t, or -1 when the
// shape is outside both kernels' plans (K not a multiple of 256, fewer than four units per row, or
// activations too long for shared memory) and the caller should take another route.  The ring
// kernel takes K >= 2048 (even super-block counts for the formats with 24-byte records); the
// register-staged kernel takes the rest, and Q5_K.
int pdk_q4k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st) {
    const int rc = launch_ring<RQ4K>(data, scales, nullptr, x, y, in_dim, out_dim, st);
    return rc != -1 ? rc : pdk_q4k_gemv_i8_regs(data, scales, x, y, in_dim, out_dim, st);
}

int pdk_q4_0_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                     uint32_t out_dim, cudaStream_t st) {
    const int rc = launch_ring<RQ40>(data, scales, nullptr, x, y, in_dim, out_dim, st);
    return rc != -1 ? rc : pdk_q4_0_gemv_i8_regs(data, scales, x, y, in_dim, out_dim, st);
}

int pdk_q5k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st) {
    return pdk_q5k_gemv_i8_regs(data, scales, x, y, in_dim, out_dim, st);
}

int pdk_q8_0_gemv_i8(const void* data, const void* scale, const float* bias, const float* x, float* y,
                     uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    const int rc = launch_ring<RQ80>(data, scale, bias, x, y, in_dim, out_dim, st);
    return rc != -1 ? rc : pdk_q8_0_gemv_i8_regs(data, scale, bias, x, y, in_dim, out_dim, st);
}

// Q8_0 small batch: x f32 [batch][in_dim], y f32 [batch][out_dim]; tokens in groups of up to eight,
// one weight pass per group.  -1 when the shape is outside the plan (K / 512 warps, 4 .. 12).
int pdk_q8_0_gemm_i8(const void* data, const void* scale, const float* bias, const float* x, float* y, uint32_t in_dim,
                     uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    if (force_regs() || !pdk_aligned(scale, 16)) return -1;
    BatchPlan pl;
    if (!make_batch_plan(in_dim, pl)) return -1;
    const MapEntry* maps = nullptr;
    if (plane_maps<RQ80>(data, scale, in_dim, out_dim, &maps) != 0) return -1;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(gemm_ring_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    unsigned int* err = pdk_error_word();
    if (err == nullptr) return (int)cudaErrorUnknown;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_tiles) grid = n_tiles;
    for (uint32_t t0 = 0; t0 < batch; t0 += 8u) {
        const uint32_t nb = batch - t0 < 8u ? batch - t0 : 8u;
        const int rc = pdk_launch_pdl(gemm_ring_q8_kernel, dim3(grid), dim3(pl.W * 32u), (size_t)pl.smem_bytes, st, maps->dmap,
                                      maps->rmap, bias, x + (size_t)t0 * in_dim, y + (size_t)t0 * out_dim, in_dim, out_dim,
                                      nb, pl, err, t0 + 8u >= batch ? 1u : 0u);
        if (rc != 0) return rc;
    }
    return 0;
}

// Q4_K GEMV on int8 activations (xq int8 [in_dim], one f32 scale per 32): same kernels, the
// activation staging widens q * scale before it builds its limbs.
int pdk_q4k_gemv_i8_q8act(const void* data, const void* scales, const int8_t* xq, const float* xq_scale, float* y,
                          uint32_t in_dim, uint32_t out_dim, cudaStream_t st) {
    const int rc = launch_ring<RQ4K>(data, scales, nullptr, nullptr, y, in_dim, out_dim, st, xq, xq_scale);
    return rc != -1 ? rc : pdk_q4k_gemv_i8_q8act_regs(data, scales, xq, xq_scale, y, in_dim, out_dim, st);
}

namespace {
int shard_launch(const void* data, const void* scales, const void* x, const void* const* y_ptrs, const void* const* flag_ptrs,
                 void* ctr, uint32_t n_ranks, uint32_t rank, uint32_t row0, uint32_t step, uint32_t signal, uint32_t in_dim,
                 uint32_t out_dim, cudaStream_t st) {
    if (out_dim == 0) return 0;
    if (n_ranks == 0 || n_ranks > 8u || y_ptrs == nullptr) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(scales, 8) || !pdk_aligned(x, 16)) return cudaErrorInvalidValue;
    gemv_i8::PeerOut po{};
    for (uint32_t p = 0; p < n_ranks; ++p) {
        if (y_ptrs[p] == nullptr || !pdk_aligned(y_ptrs[p], 4)) return cudaErrorInvalidValue;
        po.ptr[p] = (float*)y_ptrs[p];
    }
    po.n = n_ranks;
    po.row0 = row0;
    if (signal != 0u) {
        if (flag_ptrs == nullptr || ctr == nullptr || rank >= n_ranks || !pdk_aligned(ctr, 4))
            return cudaErrorInvalidValue;
        for (uint32_t p = 0; p < n_ranks; ++p) {
            if (flag_ptrs[p] == nullptr || !pdk_aligned(flag_ptrs[p], 4)) return cudaErrorInvalidValue;
            po.flag[p] = (uint32_t*)flag_ptrs[p];
        }
        po.ctr = (uint32_t*)ctr;
        po.rank = rank;
        po.step = step;
        po.signal = signal;
    }
    int rc = launch_ring<RQ4K>(data, scales, nullptr, (const float*)x, nullptr, in_dim, out_dim, st, nullptr, nullptr, &po);
    if (rc == -1) rc = pdk_q4k_gemv_peers_regs(data, scales, (const float*)x, &po, in_dim, out_dim, st);
    return rc >= 0 ? rc : (int)cudaErrorNotSupported;
}

// One warp: lane p waits until flags[p] has reached the step (wrap-around safe), for at most
// budget_ns; a lane that gives up records kErrFlagWait << 8 | p in the device error word.  The
// step is `step`; or, when that is 0, one more than the count of waits kept in flags[8], which
// the kernel then advances; or, when it is 0x80000000 | r, the value of flags[r].
enum : unsigned int { kErrFlagWait = 0x16 };
__global__ void peer_flags_wait_kernel(uint32_t* flags, uint32_t n_ranks, uint32_t step, unsigned long long budget_ns,
                                       unsigned int* err) {
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();   // ordered after the kernel before it in the stream (this rank's own band)
    const uint32_t p = threadIdx.x;
    const uint32_t target = (step & 0x80000000u) ? flags[step & 7u] : step != 0u ? step : flags[8] + 1u;
    __syncwarp();
    if (step == 0u && p == 0u) flags[8] = target;
    if (p >= n_ranks) return;
    const volatile uint32_t* f = flags + p;
    const unsigned long long t0 = tc5::globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(*f - target) < 0) {
        if ((++spins & 31u) == 0u && tc5::globaltimer_ns() - t0 > budget_ns) {
            tc5::report(err, kErrFlagWait, p);
            return;
        }
    }
    __threadfence_system();   // acquire: the bands stored before the flags are visible to what follows
}
__global__ void peer_flags_post_kernel(const gemv_i8::PeerOut po) {
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();   // the launch this signals, peer stores included, is complete
    if (threadIdx.x != 0u) return;
    const uint32_t step = po.ctr[1];
    if (step == 0u) return;
    for (uint32_t p = 0; p < po.n; ++p) gemv_i8::st_relaxed_sys(po.flag[p] + po.rank, step);
}
}  // namespace

// No counterpart in the reference (its multi-GPU story is one process per GPU, replicas only):
// Q4_K decode GEMV of one rank's row band that writes its band straight into every rank's
// full-length y (y_ptrs[0..n_ranks), device pointers valid on this GPU: its own buffer and the
// peers' buffers mapped over NVLink) at rows row0 .. row0 + out_dim.  The exchange that an
// all-gather would do is the kernel's own stores.  This form signals nothing: the stores are
// complete when the kernel is, and the caller orders consumers after it (stream order locally,
// a barrier across ranks).  n_ranks <= 8.  Returns 801 for shapes outside the GEMV kernels' plans.
PDK_EXPORT int pdk_q4k_gemv_shard(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                                  uint32_t n_ranks, uint32_t row0, uint32_t in_dim, uint32_t out_dim, void* stream) {
    return shard_launch(data, scales, x, y_ptrs, nullptr, nullptr, n_ranks, 0u, row0, 0u, 0u, in_dim, out_dim,
                        (cudaStream_t)stream);
}

// The same with a completion signal, so that a step needs no host barrier: after its band is
// stored everywhere, rank `rank` stores the step number into word `rank` of every rank's flag
// array (flag_ptrs[p] = rank p's array, mapped like y_ptrs; 16 u32 words, zeroed once at set-up:
// words 0..7 the flags, word 8 the count of pdk_peer_flags_wait calls).  ctr = two zeroed u32
// words of this rank's own memory, not shared between streams: the kernel's CTAs count
// themselves out on word 0, word 1 counts the rank's signalled steps.  step != 0 names the step
// (it must grow from call to call); step == 0 takes word 1 plus one, which lets a captured
// launch be replayed.  A consumer of y on rank p runs pdk_peer_flags_wait on its own flag array
// first.  The band is written with plain stores: a rank must not start step s + 1 before its
// consumers of step s are done with y (the wait kernel in the same stream gives that order), or y
// is double buffered.
PDK_EXPORT int pdk_q4k_gemv_shard_sync(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                                       const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank,
                                       uint32_t row0, uint32_t step, uint32_t in_dim, uint32_t out_dim, void* stream) {
    return shard_launch(data, scales, x, y_ptrs, flag_ptrs, ctr, n_ranks, rank, row0, step, 1u, in_dim, out_dim,
                        (cudaStream_t)stream);
}

// The same for a loop that keeps THREE (or more) y buffers in rotation.  All buffers of the loop share
// ONE flag array per rank and one pair of counter words.  Nothing is signalled at the end of the
// kernel (the system-scope fence that takes costs an NVLink round trip per step); instead every launch
// stores, behind its griddepcontrol.wait - when the stream's previous kernel and its peer stores are
// complete - the number of the PREVIOUS launch into the flags, and checks before it ends (at most a
// second; 0x1c << 8 | rank in the error word for a rank that is late) that every rank's previous step has
// arrived here.  What sits between launch s and launch s + 1 in the stream may therefore read step s - 1
// of every rank: a peer can be one launch ahead and already store step s + 1, but its step s + 2 - the
// first to return to the buffer of s - 1 when there are three - cannot start before this rank's launch
// s + 1 has begun.  One launch per step, consecutive steps overlap like single-GPU launches do, and the
// arrival of every step is still observed on the device.  After the last launch pdk_peer_flags_post
// signals it and pdk_peer_flags_wait (step = 0x80000000 | rank) observes it.
PDK_EXPORT int pdk_q4k_gemv_shard_lagged(const void* data, const void* scales, const void* x, const void* const* y_ptrs,
                                         const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank,
                                         uint32_t row0, uint32_t step, uint32_t in_dim, uint32_t out_dim, void* stream) {
    return shard_launch(data, scales, x, y_ptrs, flag_ptrs, ctr, n_ranks, rank, row0, step, 2u, in_dim, out_dim,
                        (cudaStream_t)stream);
}

// Closes a pdk_q4k_gemv_shard_lagged loop: stores the number of the stream's last launch (ctr[1]) into
// word `rank` of every rank's flag array, behind the stream's previous kernel.
PDK_EXPORT int pdk_peer_flags_post(const void* const* flag_ptrs, void* ctr, uint32_t n_ranks, uint32_t rank, void* stream) {
    if (flag_ptrs == nullptr || ctr == nullptr || n_ranks == 0u || n_ranks > 8u || rank >= n_ranks) return cudaErrorInvalidValue;
    gemv_i8::PeerOut po{};
    for (uint32_t p = 0; p < n_ranks; ++p) {
        if (flag_ptrs[p] == nullptr || !pdk_aligned(flag_ptrs[p], 4)) return cudaErrorInvalidValue;
        po.flag[p] = (uint32_t*)flag_ptrs[p];
    }
    po.ctr = (uint32_t*)ctr;
    po.n = n_ranks;
    po.rank = rank;
    return pdk_launch_pdl(peer_flags_post_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, po);
}

// Waits on the device (one small kernel in `stream`) until every one of the n_ranks <= 8 flag
// words of `flags` (this rank's own 16-word flag array) has reached the step: `step`, or, when
// that is 0, one more than the array's count of such waits (word 8), which the kernel advances;
// or, when it is 0x80000000 | r, the step rank r (the caller's own rank) signalled last: every
// rank has then caught up with this rank.
// The wait is bounded: after budget_us microseconds (1 .. 10,000,000) the kernel records
// 0x16 << 8 | rank-that-is-late in the device error word (pdk_device_error) and returns; the
// context stays usable.  What follows in the stream sees every rank's band of that step.
PDK_EXPORT int pdk_peer_flags_wait(void* flags, uint32_t n_ranks, uint32_t step, uint32_t budget_us, void* stream) {
    if (flags == nullptr || n_ranks == 0u || n_ranks > 8u || budget_us == 0u || budget_us > 10000000u ||
        !pdk_aligned(flags, 4))
        return cudaErrorInvalidValue;
    unsigned int* err = pdk_error_word();
    if (err == nullptr) return (int)cudaErrorUnknown;
    return pdk_launch_pdl(peer_flags_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (uint32_t*)flags, n_ranks, step,
                          (unsigned long long)budget_us * 1000ull, err);
}
