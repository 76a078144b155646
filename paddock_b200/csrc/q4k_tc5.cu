// q4k_tc5.cu - Q4_K (and Q4_0) GEMM for 9..32 tokens per launch on the tcgen05 tensor cores (W4A16).
//
// With more than a handful of tokens the per-(block, token) integer fold of q4k_batch_i8.cu
// outgrows the weight stream.  Here the CUDA cores touch each weight once, whatever the token
// count: TMA brings the packed bytes and the scale records of 128 rows into a shared-memory
// ring (six super-block columns in flight per SM), and producer warps - two sets of 8 that take
// the columns in turn - turn the nibbles into f16 weights
//     w = (q - 8) * f16(d * sc) + f16(8 d sc - dmin m)          (two weights per instruction)
// and store them from registers into tensor memory, where tcgen05.mma kind::f16 takes its A
// operand (128 weight rows = 128 lanes, 256 K = 128 columns per stage): the dequantized weights
// never exist in shared memory.  The B operand is the activation tile: a small kernel in front scales each token by a power of two into the f16 range and
// splits it into two f16 terms x = hi + lo (exact for bf16-valued activations, 22 bits
// otherwise), stored as 2 * tokens rows of a library-resident f16 matrix that TMA boxes are
// cut from.  The accumulator [128 rows][hi columns | lo columns] stays in tensor memory over
// the whole K range of a work item; the epilogue adds the two column groups, undoes the token
// scale and adds into y.
//
// A work item is (128-row tile, half of K): twice as many items as tiles keeps 148 SMs evenly
// loaded at 200 tiles.  The two halves of a tile add into y with red.global.add.f32; y is
// zeroed by the kernel in front, and with exactly two addends per element the sum does not
// depend on their order.
//
// What paces it (cycle counters in every role at 16 tokens): the tensor core.  A kind::f16 MMA with the
// A operand in tensor memory takes 64 cycles at M128 K16 however few columns (32) it has, 16 of them per
// column of 128 rows x 256 K: 1030 cycles per column in the issuing warp, 31 k of a CTA's 49 k cycles; the
// producers spend under 1000 cycles on a column and the TMA ring is waited for 13 % of the time.
//
// Precision class: f16-rounded block scales (relative 2^-12, independent per 32-weight block)
// and one f16 rounding per weight; measured rel-L2 against the f64 product of the dequantized
// operands is 3e-4, the condition-relative error 3e-5.
#include <cuda_fp16.h>

#include "tc5.cuh"

namespace {

constexpr uint32_t BM = 128;          // weight rows per work item (MMA M)
constexpr uint32_t kProdWarps = 8;    // dequantizing warps per unit (super-block column of the tile)
// Two sets of producer warps take the units in turn (set 0 the even ones, set 1 the odd ones): a
// producer's chain for a unit - box read, nibble arithmetic, tensor-memory stores, barrier - is
// latency bound, and a second set gives every scheduler four such chains instead of two.
// Warps 0..3 (set 0) also drain the accumulator.
constexpr uint32_t kProdSets = 2;   // one set: 31.6 us at 16 tokens against 29.9
constexpr uint32_t kAllProd = kProdSets * kProdWarps;
constexpr uint32_t kRawWarp = kAllProd, kActWarp = kAllProd + 1, kMmaWarp = kAllProd + 2;
constexpr uint32_t kThreads = (kAllProd + 3) * 32;
constexpr uint32_t kMaxStages = 3;    // operand stages: one Q4_K super-block column (256 K) of 128 rows
// Packed weights wait in shared memory, not in registers: a ring of TMA boxes, each two
// super-block columns of the tile - 2 x [128 rows][128 bytes] (128-byte swizzle, so that the
// 8 rows of a quarter-warp read fall on distinct banks) and [128 rows][48 bytes] of scale
// records.  Three boxes = six columns = 114 KB per SM in flight, independent of the producers.
constexpr uint32_t kRawStages = 3;
constexpr uint32_t kRawData = BM * 128u, kRawRec = BM * 48u;
constexpr uint32_t kRawStageBytes = 2u * kRawData + kRawRec;  // 38912
constexpr uint32_t kMaxK = 16384;

// NC = B columns = 2 * (tokens rounded up to 16 or 32).  BRAW: the activation tiles of two
// super-block columns travel in the weight ring's boxes (everything the tensor core waits for
// then arrives long before it is needed; with the tiles fetched per operand stage, the L2 round
// trip between "stage free" and "stage full" bounded the kernel whatever the producers did).
// The ring then holds 70 KB per box (three boxes: 210 KB): it fits for NC = 32 only, NC = 64 fetches
// per operand stage.
template <uint32_t NC>
struct Cfg {
    static constexpr bool BRAW = NC <= 32u;
    static constexpr uint32_t kBSlab = NC * 128u;
    static constexpr uint32_t kBBytes = 2u * kBSlab;  // per half unit
    static constexpr uint32_t kStages = BRAW ? 3u : 2u;              // A operand stages in tensor memory: one super-block column each
    static constexpr uint32_t kStageBytes = BRAW ? 0u : 2u * kBBytes;  // shared-memory stage: the activation tile, if not in the ring
    static constexpr uint32_t kRawBytes = kRawStageBytes + (BRAW ? 4u * kBBytes : 0u);
    static constexpr uint32_t kFullCount = kProdWarps + (BRAW ? 0u : 1u);
    static constexpr uint32_t kRawEmptyCount = 2u * kProdWarps + (BRAW ? 1u : 0u);   // kProdWarps arrivals per unit of a box
    static constexpr uint32_t kACol0 = 2u * NC;                      // after the two accumulators
    static constexpr uint32_t kACols = 128u;                         // per stage: 256 K as f16 pairs
    static constexpr uint32_t kTmemCols = 512u;                      // 2 NC + kStages * 128 <= 512
    static constexpr uint32_t kIdesc = tc5::idesc_f32acc(0u, 0u, BM, NC);
};

struct Shared {
    uint64_t raw_full[kRawStages];
    uint64_t raw_empty[kRawStages];
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// mbarrier wait that lets the hardware park the thread (up to the hint, in nanoseconds) instead
// of spinning: sixteen producer warps polling a barrier took issue slots from the warps still
// working.  Bounded like tc5::mbar_wait: after the budget the error word is set and false returned.
__device__ __forceinline__ bool mbar_try_wait_park(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc5::smem_u32(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_park(uint64_t* bar, uint32_t parity, const tc5::WaitCtx& ctx, unsigned int code,
                                               unsigned int detail) {
    if (mbar_try_wait_park(bar, parity)) return true;
    const unsigned long long t0 = tc5::globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_park(bar, parity)) {
        if ((++spins & 15u) == 0u) {
            if (*ctx.abort_flag) return false;
            if (tc5::globaltimer_ns() - t0 > tc5::kWaitBudgetNs) {
                *ctx.abort_flag = 1;
                tc5::report(ctx.err, code, detail);
                return false;
            }
        }
    }
    return true;
}

// TMEM -> registers: 32 lanes x 16 columns of 32 bits per warp
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_dup(float v) {
    const __half2 h = __float2half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// ---------------------------------------------------------------- activations -> f16 hi / lo rows
//
// xh f16 [NC][K]: row t = hi term of token t, row NC/2 + t = lo term; tokscale f32 [NC/2] = the
// power of two the token was divided by (0 for unused columns).  One CTA per token column; the
// CTAs past the token columns zero y.
constexpr uint32_t kActThreads = 1024, kZeroCtas = 32;  // kActThreads / 32 == 32: the partial maxima fit one warp
__global__ void __launch_bounds__(kActThreads)
q4k_act_f16_kernel(const float* __restrict__ x, const int8_t* __restrict__ xq, const float* __restrict__ xq_scale,
                   __half* __restrict__ xh, float* __restrict__ tokscale, float* __restrict__ y, uint32_t in_dim,
                   uint32_t out_dim, uint32_t batch, uint32_t half_cols) {
    __shared__ float wmax[kActThreads / 32u];
    const uint32_t tok = blockIdx.x, tid = threadIdx.x;
    pdk_pdl_launch_dependents();
    pdk_pdl_wait();  // the scratch and y may still be in use by the previous kernels in the stream
    if (tok >= half_cols) {
        // y is f32 [batch][out_dim], 4-byte aligned by contract: scalar stores
        const size_t n = (size_t)batch * out_dim;
        for (size_t i = (size_t)(tok - half_cols) * kActThreads + tid; i < n; i += (size_t)kZeroCtas * kActThreads) y[i] = 0.0f;
        return;
    }
    __half* hi = xh + (size_t)tok * in_dim;
    __half* lo = xh + (size_t)(half_cols + tok) * in_dim;
    auto load8 = [&](uint32_t k, float (&v)[8]) {
        const size_t e0 = (size_t)tok * in_dim + k;
        if (xq == nullptr) {
            const float4 a = *reinterpret_cast<const float4*>(x + e0);
            const float4 b = *reinterpret_cast<const float4*>(x + e0 + 4u);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const int2 q = *reinterpret_cast<const int2*>(xq + e0);
            const float s = xq_scale[e0 >> 5];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (float)(int8_t)((i < 4 ? q.x >> (8 * i) : q.y >> (8 * (i - 4))) & 0xff) * s;
        }
    };
    if (tok >= batch) {
        for (uint32_t k = tid * 8u; k < in_dim; k += kActThreads * 8u) {
            *reinterpret_cast<uint4*>(hi + k) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(lo + k) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (tid == 0) tokscale[tok] = 0.0f;
        return;
    }
    // each thread keeps its (at most two) groups of 8 elements in registers across the block-wide maximum
    constexpr uint32_t kGroups = kMaxK / (kActThreads * 8u);
    float v[kGroups][8];
    float amax = 0.0f;
#pragma unroll
    for (uint32_t gi = 0; gi < kGroups; ++gi) {
        const uint32_t k = (gi * kActThreads + tid) * 8u;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[gi][i] = 0.0f;
        if (k < in_dim) load8(k, v[gi]);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[gi][i]));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31u) == 0u) wmax[tid >> 5] = amax;
    __syncthreads();
    amax = wmax[tid & 31u];  // kActThreads / 32 = 32 partial maxima: one per lane
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    // amax < 2^ex  ->  x * 2^(14 - ex) stays below 2^14, inside the f16 range
    float mul = 0.0f, back = 0.0f;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        (void)frexpf(amax, &ex);
        ex = max(-100, min(100, ex));
        mul = ldexpf(1.0f, 14 - ex);
        back = ldexpf(1.0f, ex - 14);
    }
#pragma unroll
    for (uint32_t gi = 0; gi < kGroups; ++gi) {
        const uint32_t k = (gi * kActThreads + tid) * 8u;
        if (k >= in_dim) break;
        uint32_t h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = v[gi][2 * i] * mul, b = v[gi][2 * i + 1] * mul;
            const __half2 hh = __floats2half2_rn(a, b);
            const __half2 ll = __floats2half2_rn(a - __low2float(hh), b - __high2float(hh));
            h[i] = *reinterpret_cast<const uint32_t*>(&hh);
            l[i] = *reinterpret_cast<const uint32_t*>(&ll);
        }
        *reinterpret_cast<uint4*>(hi + k) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(lo + k) = make_uint4(l[0], l[1], l[2], l[3]);
    }
    if (tid == 0) tokscale[tok] = back;
}

// ---------------------------------------------------------------- the GEMM

// 8 registers -> 8 consecutive 32-bit columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A operand from tensor memory (row i of the 128 in lane i, two f16 of consecutive k per
// 32-bit column), B operand from shared memory.
// The sixteen MMAs of one unit (256 K = four 64-element B slabs x four K16 steps) from ONE asm block with
// one election: a_tmem steps by 8 columns per K16 step and 32 per slab, the B descriptor by 32 bytes per
// step and b_slab16 (the slab pitch in 16-byte units) per slab.  One wrapper call per MMA - its own
// elect.sync and predicate set-up - cost the issuing warp about 130 cycles each, 2100 per unit, which was
// what paced the whole kernel; the tensor core needs 16 per M128 N32 K16 step.
__device__ __forceinline__ void mma_f16_ts_unit_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t acc_first, uint64_t b_slab16) {
#define PDK_TS_STEP(J, K, PRED)                                                                      \
    "add.u32 a, %1, " #J "*32+" #K "*8;\n\tmad.lo.u64 b, %5, " #J ", %2;\n\tadd.u64 b, b, " #K "*2;\n\t" \
    "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, " PRED ";\n\t"
#define PDK_TS_SLAB(J, PRED0) PDK_TS_STEP(J, 0, PRED0) PDK_TS_STEP(J, 1, "q") PDK_TS_STEP(J, 2, "q") PDK_TS_STEP(J, 3, "q")
    asm volatile(
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        PDK_TS_SLAB(0, "p") PDK_TS_SLAB(1, "q") PDK_TS_SLAB(2, "q") PDK_TS_SLAB(3, "q") "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc_first), "l"(b_slab16)
        : "memory");
#undef PDK_TS_SLAB
#undef PDK_TS_STEP
}

// The two f16x2 multipliers and offsets of a k-slab (blocks 2G, 2G+1): w = s * (q - 8) + o, the
// high nibble arriving as 16 q.
struct SlabScale {
    uint32_t s_lo, s_hi, o_lo, o_hi;
};
// Q4_K: w = d sc q - dmin m = dsc (q - 8) + (8 dsc - dmin m); the centred nibble halves what the
// scale's f16 rounding costs.  sm = sc[2G] | sc[2G+1] << 8 | m[2G] << 16 | m[2G+1] << 24.
__device__ __forceinline__ SlabScale scale_q4k(uint32_t dd, uint32_t sm) {
    const __half2 dh = *reinterpret_cast<const __half2*>(&dd);
    const float d = __low2float(dh), dmin = __high2float(dh);
    const float dsc_lo = d * (float)(sm & 0xffu), dsc_hi = d * (float)((sm >> 8) & 0xffu);
    SlabScale r;
    r.s_lo = h2_dup(dsc_lo);
    r.s_hi = h2_dup(dsc_hi * 0.0625f);
    r.o_lo = h2_dup(fmaf(8.0f, dsc_lo, -dmin * (float)((sm >> 16) & 0xffu)));
    r.o_hi = h2_dup(fmaf(8.0f, dsc_hi, -dmin * (float)(sm >> 24)));
    return r;
}
// Q4_0 (repacked into the Q4_K nibble convention, kquant_more.cu): w = d[block] (q - 8).
// dpair = {f16 d[2G], f16 d[2G+1]}.
__device__ __forceinline__ SlabScale scale_q4_0(uint32_t dpair) {
    const __half2 dh = *reinterpret_cast<const __half2*>(&dpair);
    SlabScale r;
    r.s_lo = h2_dup(__low2float(dh));
    r.s_hi = h2_dup(__high2float(dh) * 0.0625f);
    r.o_lo = 0u;
    r.o_hi = 0u;
    return r;
}

// 32 weights of one row (16 low nibbles of block 2G, 16 high nibbles of block 2G+1) -> f16 pairs
__device__ __forceinline__ void dequant_regs(const uint4& q, const SlabScale& sc, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
    const uint32_t s_lo = sc.s_lo, s_hi = sc.s_hi, o_lo = sc.o_lo, o_hi = sc.o_hi;
    const uint32_t magic = 0x64086408u;     // f16 1032 twice: (0x6400 | q) - 1032 = q - 8
    const uint32_t magic_hi = 0x64806480u;  // f16 1152 twice: (0x6400 | q << 4) - 1152 = 16 (q - 8)
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t p01 = prmt(w[i], 0x64646464u, 0x4140u);  // bytes {b0, 0x64, b1, 0x64}
        const uint32_t p23 = prmt(w[i], 0x64646464u, 0x4342u);
        lo[2 * i] = h2_fma(h2_sub(p01 & 0x640F640Fu, magic), s_lo, o_lo);
        lo[2 * i + 1] = h2_fma(h2_sub(p23 & 0x640F640Fu, magic), s_lo, o_lo);
        hi[2 * i] = h2_fma(h2_sub(p01 & 0x64F064F0u, magic_hi), s_hi, o_hi);
        hi[2 * i + 1] = h2_fma(h2_sub(p23 & 0x64F064F0u, magic_hi), s_hi, o_hi);
    }
}

template <uint32_t NC, bool Q40>
__global__ void __launch_bounds__(kThreads, 1)
q4k_tc5_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_r, const float* __restrict__ tokscale, float* __restrict__ y,
               uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t ksplit, unsigned int* err_word) {
    using C = Cfg<NC>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    constexpr uint32_t kStages = C::kStages;
    uint8_t* tiles = ring + kRawStages * C::kRawBytes;
    Shared* sh = reinterpret_cast<Shared*>(tiles + kStages * C::kStageBytes);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_unit = in_dim >> 8, upi = n_unit / ksplit;  // units per item (even)
    const uint32_t n_items = ((out_dim + BM - 1u) / BM) * ksplit;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRawStages; ++s) {
            tc5::mbar_init(&sh->raw_full[s], 1);
            tc5::mbar_init(&sh->raw_empty[s], C::kRawEmptyCount);
        }
        for (uint32_t s = 0; s < kStages; ++s) {
            tc5::mbar_init(&sh->full[s], C::kFullCount);  // one arrival per producer warp (+ the activation loader's)
            tc5::mbar_init(&sh->empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            tc5::mbar_init(&sh->tmem_full[b], 1);
            tc5::mbar_init(&sh->tmem_empty[b], 4);
        }
        sh->abort_flag = 0;
        tc5::mbar_fence_init();
        tc5::tma_prefetch_desc(&tmap_x);
        tc5::tma_prefetch_desc(&tmap_w);
        tc5::tma_prefetch_desc(&tmap_r);
    }
    if (warp == kMmaWarp) {
        tc5::tmem_alloc(&sh->tmem_base, C::kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = sh->tmem_base;
    const tc5::WaitCtx ctx{&sh->abort_flag, err_word};
    pdk_pdl_launch_dependents();

    if (warp < kAllProd) {
        // ------------------------------------------------------------ dequantizing producers
        // A thread owns one row of the tile - the tensor-memory lane its warp may write: warp w
        // serves lanes 32 (w % 4).. - and, per unit, half of its 256 K (hf): the four
        // 16-byte chunks 4 hf .. 4 hf + 3 of the row's packed bytes, i.e. k-slabs G = 2 hf, 2 hf + 1.
        // The f16 pairs go straight from registers into the A operand's tensor-memory columns:
        // no shared-memory copy of the dequantized weights, nothing for the tensor core to
        // fetch but the small activation tile, and one barrier round per 128 weights of a row.
        // The 8 lanes of a quarter-warp hold 8 consecutive rows: their 16-byte reads of the
        // swizzled weight box fall on 8 different chunk positions.
        const uint32_t set = warp / kProdWarps, pw = warp % kProdWarps;
        const uint32_t qd = pw & 3u, hf = pw >> 2;
        const uint32_t r_in = qd * 32u + lane, swz = r_in & 7u;
        const uint32_t line_off = (r_in >> 3) * 1024u + swz * 128u;  // the row's 128-byte line in a weight box
        const uint32_t my_items = blockIdx.x < n_items ? (n_items - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
        const uint32_t total = my_items * upi;
        bool ok = true;
        // unit n of this CTA's sequence: box n / 2 (unit n % 2 of it: upi is even, so that is the set), operand
        // stage n % kStages
        for (uint32_t n = set; n < total && ok; n += kProdSets) {
            const uint32_t j = n & 1u, box = n >> 1;
            const uint32_t rs = box % kRawStages, rphase = (box / kRawStages) & 1u;
            const uint32_t stage = n % kStages, phase = (n / kStages) & 1u;
            ok = mbar_wait_park(&sh->raw_full[rs], rphase, ctx, tc5::kErrFullWait, 0x20u + rs);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint8_t* raw = ring + rs * C::kRawBytes;
            uint4 q[4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i)
                q[i] = *reinterpret_cast<const uint4*>(raw + j * kRawData + line_off + (((hf * 4u + i) ^ swz) << 4));
            const uint8_t* rec = raw + 2u * kRawData + r_in * 48u + j * 24u;
            // Q4_K record {f16 d, f16 dmin, sc[8], m[8], pad}: sc / m[4 hf .. 4 hf + 3]; Q4_0 record {f16 d[8], pad}: d[4 hf .. 4 hf + 3]
            const uint32_t dd = *reinterpret_cast<const uint32_t*>(rec + (Q40 ? 8u * hf : 0u));
            const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(rec + 4u + (Q40 ? 8u : 4u) * hf);
            const uint32_t m4 = Q40 ? 0u : *reinterpret_cast<const uint32_t*>(rec + 12u + 4u * hf);
            ok = mbar_wait_park(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, stage);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc5::fence_after_sync();  // the MMAs that read this stage's columns are complete
#pragma unroll
            for (uint32_t g2 = 0; g2 < 2u; ++g2) {
                // slab G = 2 hf + g2: block 2G elements 0..15 | 16..31 | block 2G+1 elements 0..15 | 16..31
                const SlabScale ss = Q40 ? scale_q4_0(g2 == 0u ? dd : sc4)
                                         : scale_q4k(dd, ((sc4 >> (16u * g2)) & 0xffffu) | (((m4 >> (16u * g2)) & 0xffffu) << 16));
                uint32_t lo0[8], hi0[8], lo1[8], hi1[8];
                dequant_regs(q[2u * g2], ss, lo0, hi0);
                dequant_regs(q[2u * g2 + 1u], ss, lo1, hi1);
                const uint32_t ta = tmem_base + ((qd * 32u) << 16) + C::kACol0 + stage * C::kACols + (2u * hf + g2) * 32u;
                tmem_st_32x8(ta, lo0);
                tmem_st_32x8(ta + 8u, lo1);
                tmem_st_32x8(ta + 16u, hi0);
                tmem_st_32x8(ta + 24u, hi1);
            }
            tmem_st_wait();
            tc5::fence_before_sync();  // tensor-memory stores -> ordered before the arrival the MMA warp waits for
            __syncwarp();
            if (lane == 0) {
                tc5::mbar_arrive(&sh->full[stage]);
                tc5::mbar_arrive(&sh->raw_empty[rs]);  // every lane has consumed its bytes of the box
            }
            if (n % upi + kProdSets >= upi && warp < 4u) {
                // ---- set 0 has written its last unit of the item: warps 0..3 drain the item's accumulator
                // (full once set 1's last unit has gone through the tensor core too)
                {
                    const uint32_t iter = n / upi, c_item = blockIdx.x + iter * gridDim.x;
                    const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
                    if (iter == 0u) pdk_pdl_wait();  // tokscale and the zeroed y are the previous kernel's output
                    ok = mbar_wait_park(&sh->tmem_full[buf], aphase, ctx, tc5::kErrTmemFullWait, buf);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc5::fence_after_sync();
                    const uint32_t row = (c_item / ksplit) * BM + warp * 32u + lane;
                    constexpr uint32_t HC = NC / 2u;  // token columns
#pragma unroll 1
                    for (uint32_t t0 = 0; t0 < HC; t0 += 16u) {
                        uint32_t a[16], b[16];
                        tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + buf * NC + t0, a);       // hi terms
                        tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + buf * NC + HC + t0, b);  // lo terms
                        tc5::tmem_ld_wait();
                        if (row < out_dim) {
#pragma unroll
                            for (uint32_t i = 0; i < 16u; ++i) {
                                const uint32_t tok = t0 + i;
                                if (tok < batch)
                                    atomicAdd(y + (size_t)tok * out_dim + row,
                                              (__uint_as_float(a[i]) + __uint_as_float(b[i])) * __ldg(tokscale + tok));
                            }
                        }
                    }
                    tc5::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc5::mbar_arrive(&sh->tmem_empty[buf]);
                }
            }
        }
    } else if (warp == kRawWarp) {
        // ------------------------------------------------------------ packed weights and scale records (TMA)
        // Weights depend on nothing the previous kernel in the stream writes: no wait for it.
        uint32_t rs = 0, rphase = 0;
        bool ok = true, waited = false;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const uint32_t row0 = (item / ksplit) * BM, u0 = (item % ksplit) * upi;
            for (uint32_t u = 0; u < upi; u += 2u) {
                ok = mbar_wait_park(&sh->raw_empty[rs], rphase ^ 1u, ctx, tc5::kErrEmptyWait, 0x20u + rs);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* raw = ring + rs * C::kRawBytes;
                tc5::mbar_arrive_expect_tx_elect(&sh->raw_full[rs], C::kRawBytes);
                tc5::tma_load_2d_elect(raw, &tmap_w, &sh->raw_full[rs], (int32_t)((u0 + u) * 128u), (int32_t)row0);
                tc5::tma_load_2d_elect(raw + kRawData, &tmap_w, &sh->raw_full[rs], (int32_t)((u0 + u + 1u) * 128u), (int32_t)row0);
                tc5::tma_load_2d_elect(raw + 2u * kRawData, &tmap_r, &sh->raw_full[rs], (int32_t)((u0 + u) * 24u), (int32_t)row0);
                if (C::BRAW) {
                    if (!waited) {  // the f16 rows are the previous kernel's output; the weights above are not
                        pdk_pdl_wait();
                        waited = true;
                    }
#pragma unroll
                    for (uint32_t j = 0; j < 8u; ++j)  // 4 half units x 2 k-slabs of 64
                        tc5::tma_load_2d_elect(raw + kRawStageBytes + j * C::kBSlab, &tmap_x, &sh->raw_full[rs],
                                               (int32_t)((u0 + u) * 256u + j * 64u), 0);
                }
                if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
            }
        }
        if (!ok && lane == 0)
            for (int i = 0; i < 64; ++i) __nanosleep(1000);  // copies in flight still land in this CTA's shared memory
    } else if (warp == kActWarp) {
        if (!C::BRAW) {
        // ------------------------------------------------------------ activation tiles (TMA)
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        pdk_pdl_wait();  // the f16 rows are the previous kernel's output
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const uint32_t u0 = (item % ksplit) * upi;
            for (uint32_t u = 0; u < upi; ++u) {
                ok = mbar_wait_park(&sh->empty[stage], phase ^ 1u, ctx, tc5::kErrEmptyWait, 0x10u + stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* b = tiles + stage * C::kStageBytes;
                tc5::mbar_arrive_expect_tx_elect(&sh->full[stage], C::kStageBytes);
#pragma unroll
                for (uint32_t j = 0; j < 4u; ++j)
                    tc5::tma_load_2d_elect(b + j * C::kBSlab, &tmap_x, &sh->full[stage], (int32_t)((u0 + u) * 256u + j * 64u), 0);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0)
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else {
        // ------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        uint32_t stage = 0, phase = 0, iter = 0, rs = 0, rphase = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++iter) {
            const uint32_t buf = iter & 1u, aphase = (iter >> 1) & 1u;
            ok = mbar_wait_park(&sh->tmem_empty[buf], aphase ^ 1u, ctx, tc5::kErrTmemEmptyWait, buf);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc5::fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * NC;
            for (uint32_t u = 0; u < upi; ++u) {
                if (C::BRAW && (u & 1u) == 0u) {  // the activation tiles of this pair of units are in the weight box
                    ok = mbar_wait_park(&sh->raw_full[rs], rphase, ctx, tc5::kErrFullWait, 0x30u + rs);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                ok = mbar_wait_park(&sh->full[stage], phase, ctx, tc5::kErrFullWait, stage);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc5::fence_after_sync();
                const uint32_t a_tmem = tmem_base + C::kACol0 + stage * C::kACols;
                const uint32_t b_addr = C::BRAW ? tc5::smem_u32(ring + rs * C::kRawBytes + kRawStageBytes) + (u & 1u) * 2u * C::kBBytes
                                                : tc5::smem_u32(tiles + stage * C::kStageBytes);
                // 16 f16 of K per instruction: 8 columns of A, 32 bytes of B
                mma_f16_ts_unit_elect(d_tmem, a_tmem, tc5::smem_desc_sw128(b_addr), C::kIdesc, u != 0u, (uint64_t)(C::kBSlab >> 4));
                tc5::mma_commit_elect(&sh->empty[stage]);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                if (C::BRAW && (u & 1u) == 1u) {  // the box's activation tiles have been read
                    tc5::mma_commit_elect(&sh->raw_empty[rs]);
                    if (++rs == kRawStages) { rs = 0; rphase ^= 1u; }
                }
            }
            if (ok) tc5::mma_commit_elect(&sh->tmem_full[buf]);
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Scratch for the f16 activation rows and the token scales: lives in the library (the pack
// allocates nothing at run time), one slice per stream for the first kLanes streams.
constexpr size_t kXhBytes = (size_t)64 * kMaxK * 2u;
constexpr size_t kSliceBytes = kXhBytes + 1024u;
constexpr int kLanes = 2;
__device__ __align__(1024) uint8_t g_q4k_xh[kLanes][kSliceBytes];

PDK_SLICE_TABLE(xh_slice_table, g_q4k_xh, kSliceBytes, kLanes);
uint8_t* xh_slice(cudaStream_t st) { return xh_slice_table.slice(st); }

template <uint32_t NC, bool Q40>
int launch(const void* data, const void* recs, const float* x, const int8_t* xq, const float* xq_scale, float* y,
           uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    using C = Cfg<NC>;
    const uint32_t n_unit = in_dim >> 8;
    // the scale records travel in 48-byte boxes (two super-blocks), 16-byte aligned rows
    if ((in_dim & 255u) != 0u || in_dim > kMaxK || n_unit == 0u || (n_unit & 1u) != 0u || !pdk_aligned(recs, 16)) return -1;
    uint8_t* slice = xh_slice(st);
    if (slice == nullptr) return -1;
    __half* xh = reinterpret_cast<__half*>(slice);
    float* tokscale = reinterpret_cast<float*>(slice + kXhBytes);
    CUtensorMap tx, tw, tr;
    if (int rc = pdk_make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, in_dim, NC, (uint64_t)in_dim * 2u, 64u, NC))
        return rc;
    // rows past out_dim read as zeros (d = 0: zero weights)
    if (int rc = pdk_make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, data, in_dim / 2u, out_dim, in_dim / 2u, 128u, BM))
        return rc;
    if (int rc = pdk_make_tmap_2d_dense(&tr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, recs, (uint64_t)n_unit * 24u, out_dim,
                                        (uint64_t)n_unit * 24u, 48u, BM))
        return rc;
    const size_t smem = (size_t)kRawStages * C::kRawBytes + (size_t)C::kStages * C::kStageBytes + sizeof(Shared) + 1024u;
    auto kern = q4k_tc5_kernel<NC, Q40>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    if (int rc = pdk_launch_pdl(q4k_act_f16_kernel, dim3(NC / 2u + kZeroCtas), dim3(kActThreads), 0, st, x, xq, xq_scale, xh,
                                tokscale, y, in_dim, out_dim, batch, NC / 2u))
        return rc;
    // two K halves per tile when each half is a whole number of record boxes
    const uint32_t ksplit = (n_unit & 3u) == 0u ? 2u : 1u;
    const uint32_t n_items = ((out_dim + BM - 1u) / BM) * ksplit;
    uint32_t grid = (uint32_t)pdk_sm_count();
    if (grid > n_items) grid = n_items;
    return pdk_launch_pdl(kern, dim3(grid), dim3(kThreads), smem, st, tx, tw, tr, (const float*)tokscale, y, in_dim,
                          out_dim, batch, ksplit, pdk_error_word());
}

}  // namespace

// Q4_K GEMM for 1 <= batch <= 32 tokens on the tcgen05 path: y f32 [batch][out_dim].
// Activations are f32 x [batch][in_dim] or (x == nullptr) int8 xq with one f32 scale per 32
// elements.  Returns 0 / a cudaError_t, or -1 when the shape is outside the kernel's plan (K not
// a multiple of 512 or above 16384, scale records not 16-byte aligned, more streams than scratch
// slices) and the caller should
// take another route.  Two launches: the f16 activation rows (which also zeroes y), then the GEMM.
int pdk_q4k_tc5(const void* data, const void* scales, const float* x, const int8_t* xq, const float* xq_scale, float* y,
                uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    if (batch == 0u || batch > 32u) return -1;
    if (batch <= 16u) return launch<32, false>(data, scales, x, xq, xq_scale, y, in_dim, out_dim, batch, st);
    return launch<64, false>(data, scales, x, xq, xq_scale, y, in_dim, out_dim, batch, st);
}

// The same for a repacked Q4_0 plane (f32 activations).
int pdk_q4_0_tc5(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                 uint32_t batch, cudaStream_t st) {
    if (batch == 0u || batch > 32u) return -1;
    if (batch <= 16u) return launch<32, true>(data, scales, x, nullptr, nullptr, y, in_dim, out_dim, batch, st);
    return launch<64, true>(data, scales, x, nullptr, nullptr, y, in_dim, out_dim, batch, st);
}
