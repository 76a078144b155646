// kquant.cu - Q4_K: dequant, repack and the decode GEMV / small-batch GEMM over
// the repacked planes.
//
// Repacked layout (the byte budget the engine allocates: 128 B + 24 B per
// 256-weight super-block; every super-block is self-contained because the
// repack call is only told a super-block count):
//   data   : the 128 nibble bytes verbatim: group G (32 bytes) byte l holds
//            element G*64 + l (low nibble) and element G*64 + 32 + l (high nibble);
//   scales : 24-byte record {f16 d, f16 dmin, u8 sc[8], u8 m[8], 4 pad bytes}
//            with the 6-bit (scale, min) pairs unpacked to bytes.
// Dequant value of element l of sub-block j: (d*sc_j)*q - (dmin*m_j).
//
// The GEMV is HBM-bound (4.5 bits per weight streamed once).  Per-weight f32
// FMAs would make it issue-bound on B200, so the inner product runs on the
// tensor cores without leaving the f32 numeric class: nibbles become the exact
// bf16 integers 128+q (one logic op per pair), activations are split into
// bf16 hi + bf16 lo parts that ride in two columns of the same mma, and the
// per-sub-block scale, the min term and the 128 offset are applied in f32 to
// the 32-element partial sums.
#include <cstdlib>

#include "pdk_common.cuh"

// kquant_more.cu: Q5_K, Q6_K, Q4_0
bool pdk_kq_more_has(uint32_t dtype);
int pdk_kq_more_dequant(const void* src, void* dst, uint64_t n_super, uint32_t dtype, cudaStream_t st);
int pdk_kq_more_repack(const void* src, void* dst_data, void* dst_scales, uint64_t n_super, uint32_t dtype,
                       cudaStream_t st);
int pdk_kq_more_gemm(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, uint32_t dtype, cudaStream_t st);
int pdk_q4k_gemv_i8_q8act(const void* data, const void* scales, const int8_t* xq, const float* xq_scale, float* y,
                          uint32_t in_dim, uint32_t out_dim, cudaStream_t st);
int pdk_q4k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st);
int pdk_q4_0_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                     uint32_t out_dim, cudaStream_t st);
int pdk_q5k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st);
int pdk_iq4xs_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                      cudaStream_t st);  // gemv_i8.cu
int pdk_q6k_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim,
                    uint32_t out_dim, cudaStream_t st);  // gemv_q6k.cu
// q4k_batch_i8.cu: 1..16 tokens, f32 or int8 activations; -1 = shape outside its plan
int pdk_q4k_batch_i8(const void* data, const void* scales, const float* x, const int8_t* xq, const float* xq_scale,
                     float* y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st);
int pdk_q5k_batch_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, cudaStream_t st);
int pdk_q6k_batch_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, cudaStream_t st);
// q4k_tc5.cu: 1..32 tokens on tcgen05 (f16 weights); same operands and return convention
int pdk_q4k_tc5(const void* data, const void* scales, const float* x, const int8_t* xq, const float* xq_scale, float* y,
                uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st);
int pdk_q4_0_tc5(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                 uint32_t batch, cudaStream_t st);

namespace {

// ggml get_scale_min_k4: unpack 6-bit pair j of the 12 packed scale bytes.
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, uint32_t j, uint32_t* sc, uint32_t* m) {
    if (j < 4u) {
        *sc = s[j] & 63u;
        *m = s[j + 4u] & 63u;
    } else {
        *sc = (s[j + 4u] & 0xFu) | ((uint32_t)(s[j - 4u] >> 6) << 4);
        *m = (uint32_t)(s[j + 4u] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

// One warp per super-block; lane l writes element l of each of the 8
// sub-blocks, so every store instruction covers one 128-byte line.
__global__ void q4k_dequant_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, uint64_t n_super) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint8_t* s = src + b * 144u;
    const float d = __half2float(*reinterpret_cast<const __half*>(s));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(s + 2));
    float* y = dst + b * 256u;
#pragma unroll
    for (uint32_t j = 0; j < 8u; ++j) {
        uint32_t sc, m;
        scale_min_k4(s + 4, j, &sc, &m);
        const float dj = __fmul_rn(d, (float)sc), mj = __fmul_rn(dmin, (float)m);
        const uint32_t q = s[16u + (j >> 1) * 32u + lane];
        const uint32_t v = (j & 1u) ? (q >> 4) : (q & 0xFu);
        y[j * 32u + lane] = __fsub_rn(__fmul_rn(dj, (float)v), mj);
    }
}

// One warp per super-block: lane l moves one 4-byte word of the nibble payload
// (the source payload at 144*b + 16 is 4-byte aligned when the plane is);
// lanes 0..7 unpack one (sc, m) pair each into the record.
__global__ void q4k_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst_data,
                                  uint8_t* __restrict__ dst_scales, uint64_t n_super) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint8_t* s = src + b * 144u;
    reinterpret_cast<uint32_t*>(dst_data + b * 128u)[lane] = reinterpret_cast<const uint32_t*>(s + 16)[lane];
    uint8_t* rec = dst_scales + b * 24u;
    if (lane < 8u) {
        uint32_t sc, m;
        scale_min_k4(s + 4, lane, &sc, &m);
        rec[4u + lane] = (uint8_t)sc;
        rec[12u + lane] = (uint8_t)m;
    } else if (lane < 12u) {
        rec[lane - 8u] = s[lane - 8u];  // f16 d, f16 dmin
    } else if (lane < 16u) {
        rec[8u + lane] = 0;             // pad bytes 20..23
    }
}

// ===========================================================================
// Tensor-core streaming GEMV / small-batch GEMM
// ===========================================================================

constexpr uint32_t kTileSlots = 4;                    // 16-row tiles a CTA works on at once
constexpr uint32_t kSlices = 4;                       // K slices per tile (one warp each)
constexpr uint32_t kThreads = kTileSlots * kSlices * 32;

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

struct SbData {   // one super-block of two rows (g and g+8) in registers
    uint2 lo[4];  // row g: bytes 8t..8t+7 of groups 0..3
    uint2 hi[4];  // row g + 8
};
struct SbScale {  // the two rows' 24-byte records (first 20 bytes used)
    uint2 lo[3];
    uint2 hi[3];
};

// Shared-memory plan (dynamic):
//   xs   : bf16 [NCOLS][pitch/2]  activations, permuted per 8 elements as
//          [0,2,1,3,4,6,5,7] so a lane's B fragments for one sub-block are one
//          16-byte read; pitch = 2*K + 64 bytes keeps the 8 columns of an
//          n-tile on distinct banks.
//   xsum : f32 [K/32][NCOLS]      per-sub-block sums of the staged values
//   red  : f32 [2][kTileSlots][kSlices][16][NCOLS]  K-slice partials
//
// NT = number of 8-column n-tiles; SPLIT = columns (2m, 2m+1) carry the bf16
// hi and lo parts of token m (f32-exact activations), else column m = token m
// rounded to bf16.
template <uint32_t NT, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
q4k_mma_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
               const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim, uint32_t out_dim,
               uint32_t batch, uint32_t magic) {
    constexpr uint32_t NCOLS = NT * 8u;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t n_sub = in_dim >> 5, n_super = in_dim >> 8;
    const uint32_t pitch = in_dim * 2u + 64u;
    uint8_t* xs = smem;
    float* xsum = reinterpret_cast<float*>(smem + (size_t)NCOLS * pitch);
    float* red = xsum + (size_t)n_sub * NCOLS;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t slot = warp / kSlices, slice = warp % kSlices;
    const uint32_t n_tiles = (out_dim + 15u) >> 4;
    const uint32_t sb_lo = slice * n_super / kSlices, sb_hi = (slice + 1u) * n_super / kSlices;

    const size_t row_data = (size_t)n_super * 128u, row_rec = (size_t)n_super * 24u;

    auto load_data = [&](SbData& s, const uint8_t* p0, const uint8_t* p1, uint32_t sb) {
        const uint8_t* a = p0 + (size_t)sb * 128u + t * 8u;
        const uint8_t* b = p1 + (size_t)sb * 128u + t * 8u;
#pragma unroll
        for (uint32_t G = 0; G < 4u; ++G) {
            s.lo[G] = pdk_ldg_stream8(a + G * 32u);
            s.hi[G] = pdk_ldg_stream8(b + G * 32u);
        }
    };
    auto load_scale = [&](SbScale& s, const uint8_t* r0, const uint8_t* r1, uint32_t sb) {
        const uint2* a = reinterpret_cast<const uint2*>(r0 + (size_t)sb * 24u);
        const uint2* b = reinterpret_cast<const uint2*>(r1 + (size_t)sb * 24u);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            s.lo[i] = __ldg(a + i);
            s.hi[i] = __ldg(b + i);
        }
    };

    // ---- first tile's weights go in flight before the activations are staged
    uint32_t tile = blockIdx.x * kTileSlots + slot;
    const uint32_t tile_stride = gridDim.x * kTileSlots;
    SbData d0, d1;
    SbScale s0, s1;
    const uint8_t *p0 = data, *p1 = data, *r0 = scales, *r1 = scales;
    auto set_rows = [&](uint32_t tl) {
        const uint32_t ra = min(tl * 16u + g, out_dim - 1u), rb = min(tl * 16u + g + 8u, out_dim - 1u);
        p0 = data + ra * row_data;
        p1 = data + rb * row_data;
        r0 = scales + ra * row_rec;
        r1 = scales + rb * row_rec;
    };
    if (tile < n_tiles) {
        set_rows(tile);
        if (sb_lo < sb_hi) { load_data(d0, p0, p1, sb_lo); load_scale(s0, r0, r1, sb_lo); }
        if (sb_lo + 1u < sb_hi) load_data(d1, p0, p1, sb_lo + 1u);
    }

    // ---- stage activations: one thread per (column, 8 elements)
    {
        const uint32_t groups = in_dim >> 3;  // 8-element groups per column
        const uint32_t used_cols = SPLIT ? 2u * batch : batch;
        for (uint32_t idx = tid; idx < NCOLS * groups; idx += kThreads) {
            const uint32_t col = idx / groups, grp = idx % groups;  // grp = j*4 + t
            float v[8];
            if (col < used_cols) {
                const uint32_t tok = SPLIT ? (col >> 1) : col;
                const float4 a = *reinterpret_cast<const float4*>(x + (size_t)tok * in_dim + grp * 8u);
                const float4 b = *reinterpret_cast<const float4*>(x + (size_t)tok * in_dim + grp * 8u + 4u);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float hi = __bfloat162float(__float2bfloat16_rn(v[i]));
                    if (SPLIT && (col & 1u)) v[i] = __bfloat162float(__float2bfloat16_rn(v[i] - hi));
                    else v[i] = hi;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.0f;
            }
            uint4 w;
            w.x = pack_bf16(v[0], v[2]);
            w.y = pack_bf16(v[1], v[3]);
            w.z = pack_bf16(v[4], v[6]);
            w.w = pack_bf16(v[5], v[7]);
            *reinterpret_cast<uint4*>(xs + (size_t)col * pitch + grp * 16u) = w;
            // the four groups of a sub-block sit in four adjacent lanes
            float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((grp & 3u) == 0u) xsum[(size_t)(grp >> 2) * NCOLS + col] = sum;
        }
    }
    __syncthreads();

    const uint8_t* xs_lane = xs + (size_t)g * pitch + t * 16u;  // column g of each n-tile
    uint32_t iter = 0;
    for (; tile < n_tiles; tile += tile_stride, ++iter) {
        float acc[NT][4];
#pragma unroll
        for (uint32_t n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;

        // one super-block: 8 sub-blocks x (2 mma per n-tile), then the f32 fold
        auto compute = [&](const SbData& dd, const SbScale& ss, uint32_t sb) {
            const __half2 dl = *reinterpret_cast<const __half2*>(&ss.lo[0].x);
            const __half2 dh = *reinterpret_cast<const __half2*>(&ss.hi[0].x);
            const float d_lo = __low2float(dl), m_lo = __high2float(dl);
            const float d_hi = __low2float(dh), m_hi = __high2float(dh);
            // sc[8] = bytes 4..11, m[8] = bytes 12..19 of the record
            const uint32_t sc_lo[2] = {ss.lo[0].y, ss.lo[1].x}, mn_lo[2] = {ss.lo[1].y, ss.lo[2].x};
            const uint32_t sc_hi[2] = {ss.hi[0].y, ss.hi[1].x}, mn_hi[2] = {ss.hi[1].y, ss.hi[2].x};
#pragma unroll
            for (uint32_t G = 0; G < 4u; ++G) {
                // words of rows g / g+8 for group G: (W0, W1) of the 8 bytes
                const uint32_t wl0 = dd.lo[G].x, wl1 = dd.lo[G].y;
                const uint32_t wh0 = dd.hi[G].x, wh1 = dd.hi[G].y;
#pragma unroll
                for (uint32_t h = 0; h < 2u; ++h) {  // h = 0: low nibbles (sub-block 2G), 1: high
                    const uint32_t j = 2u * G + h;
                    const uint32_t sh = h * 4u;
                    const uint32_t M = 0x000F000Fu, O = magic;  // 0x43004300: bf16 128.0 twice
                    const uint32_t a0 = pdk_and_or(wl0 >> sh, M, O), a2 = pdk_and_or(wl0 >> (sh + 8u), M, O);
                    const uint32_t a1 = pdk_and_or(wh0 >> sh, M, O), a3 = pdk_and_or(wh0 >> (sh + 8u), M, O);
                    const uint32_t e0 = pdk_and_or(wl1 >> sh, M, O), e2 = pdk_and_or(wl1 >> (sh + 8u), M, O);
                    const uint32_t e1 = pdk_and_or(wh1 >> sh, M, O), e3 = pdk_and_or(wh1 >> (sh + 8u), M, O);
                    const uint32_t bsh = (j & 3u) * 8u;
                    const float sl = (float)((sc_lo[j >> 2] >> bsh) & 0xffu), ml = (float)((mn_lo[j >> 2] >> bsh) & 0xffu);
                    const float su = (float)((sc_hi[j >> 2] >> bsh) & 0xffu), mu = (float)((mn_hi[j >> 2] >> bsh) & 0xffu);
                    const float dsl = d_lo * sl, dsu = d_hi * su;
                    const float ofl = fmaf(128.0f, dsl, m_lo * ml), ofu = fmaf(128.0f, dsu, m_hi * mu);
                    const uint32_t sub = sb * 8u + j;
#pragma unroll
                    for (uint32_t n = 0; n < NT; ++n) {
                        const uint4 b = *reinterpret_cast<const uint4*>(xs_lane + (size_t)n * 8u * pitch + (size_t)sub * 64u);
                        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        mma_bf16(c, a0, a1, a2, a3, b.x, b.y);
                        mma_bf16(c, e0, e1, e2, e3, b.z, b.w);
                        const float2 xsv = *reinterpret_cast<const float2*>(xsum + (size_t)sub * NCOLS + n * 8u + 2u * t);
                        acc[n][0] += dsl * c[0] - ofl * xsv.x;
                        acc[n][1] += dsl * c[1] - ofl * xsv.y;
                        acc[n][2] += dsu * c[2] - ofu * xsv.x;
                        acc[n][3] += dsu * c[3] - ofu * xsv.y;
                    }
                }
            }
        };

        // software pipeline over the slice: data two super-blocks ahead, records one
        SbData d2;
        for (uint32_t sb = sb_lo; sb < sb_hi; sb += 3u) {
            if (sb + 2u < sb_hi) load_data(d2, p0, p1, sb + 2u);
            if (sb + 1u < sb_hi) load_scale(s1, r0, r1, sb + 1u);
            compute(d0, s0, sb);
            if (sb + 1u >= sb_hi) break;
            if (sb + 3u < sb_hi) load_data(d0, p0, p1, sb + 3u);
            if (sb + 2u < sb_hi) load_scale(s0, r0, r1, sb + 2u);
            compute(d1, s1, sb + 1u);
            if (sb + 2u >= sb_hi) break;
            if (sb + 4u < sb_hi) load_data(d1, p0, p1, sb + 4u);
            if (sb + 3u < sb_hi) load_scale(s1, r0, r1, sb + 3u);
            compute(d2, s0, sb + 2u);
            if (sb + 3u < sb_hi) s0 = s1;
        }

        // next tile's first loads go out before the reduction
        const uint32_t next = tile + tile_stride;
        const uint32_t cur_rows = tile * 16u;
        if (next < n_tiles) {
            set_rows(next);
            if (sb_lo < sb_hi) { load_data(d0, p0, p1, sb_lo); load_scale(s0, r0, r1, sb_lo); }
            if (sb_lo + 1u < sb_hi) load_data(d1, p0, p1, sb_lo + 1u);
        }

        // ---- fold the K slices: [slice][16 rows][NCOLS] per tile slot, two buffers
        float* rbuf = red + ((size_t)(iter & 1u) * kTileSlots + slot) * (kSlices * 16u * NCOLS);
        float* mine = rbuf + (size_t)slice * 16u * NCOLS;
#pragma unroll
        for (uint32_t n = 0; n < NT; ++n) {
            *reinterpret_cast<float2*>(mine + (size_t)g * NCOLS + n * 8u + 2u * t) = make_float2(acc[n][0], acc[n][1]);
            *reinterpret_cast<float2*>(mine + (size_t)(g + 8u) * NCOLS + n * 8u + 2u * t) = make_float2(acc[n][2], acc[n][3]);
        }
        bar_sync(1u + slot, kSlices * 32u);
        const uint32_t sub_tid = slice * 32u + lane;  // 0..127 within the tile slot
        const uint32_t outs = 16u * batch;
        for (uint32_t o = sub_tid; o < outs; o += kSlices * 32u) {
            const uint32_t r = o % 16u, tok = o / 16u;
            float v = 0.0f;
#pragma unroll
            for (uint32_t s = 0; s < kSlices; ++s) {
                const float* pr = rbuf + ((size_t)s * 16u + r) * NCOLS;
                v += SPLIT ? (pr[2u * tok] + pr[2u * tok + 1u]) : pr[tok];
            }
            if (cur_rows + r < out_dim) y[(size_t)tok * out_dim + cur_rows + r] = v;
        }
    }
}

template <uint32_t NT, bool SPLIT>
int launch_mma(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
               uint32_t batch, cudaStream_t st) {
    constexpr uint32_t NCOLS = NT * 8u;
    const size_t smem = (size_t)NCOLS * (in_dim * 2u + 64u) + (size_t)(in_dim >> 5) * NCOLS * 4u +
                        (size_t)2u * kTileSlots * kSlices * 16u * NCOLS * 4u;
    if (smem > 227u * 1024u) return -1;  // caller falls back
    auto kern = q4k_mma_kernel<NT, SPLIT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const uint32_t n_tiles = (out_dim + 15u) / 16u;
    uint32_t grid = (uint32_t)pdk_sm_count();
    const uint32_t need = (n_tiles + kTileSlots - 1u) / kTileSlots;
    if (grid > need) grid = need;
    kern<<<grid, kThreads, smem, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim, out_dim, batch,
                                       0x43004300u);
    return pdk_launch_status();
}

// ===========================================================================
// Plain-load f32 kernel: the route for shapes the tensor-core kernel's shared
// memory plan cannot hold.  A warp owns one output row at a time; lane l reads
// word l of each super-block (a coalesced 128-byte line).
// ===========================================================================
constexpr uint32_t kWarps = 8;

template <uint32_t TOK, uint32_t UNROLL>
__global__ void __launch_bounds__(kWarps * 32)
q4k_gemv_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                const float* __restrict__ x, float* __restrict__ y, uint32_t in_dim, uint32_t out_dim,
                uint32_t batch0) {
    extern __shared__ __align__(16) float xsf[];  // [TOK][in_dim]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float* xg = x + (size_t)batch0 * in_dim;
    for (uint32_t i = tid * 4u; i < TOK * in_dim; i += blockDim.x * 4u)
        *reinterpret_cast<float4*>(xsf + i) = *reinterpret_cast<const float4*>(xg + i);
    __syncthreads();

    const uint32_t n_super = in_dim >> 8;
    // word `lane` of the payload = ggml group G, word w of that group
    const uint32_t G = lane >> 3, w = lane & 7u;
    const uint32_t koff = G * 64u + w * 4u;  // first low-nibble element inside the super-block
    for (uint32_t row = blockIdx.x * kWarps + warp; row < out_dim; row += gridDim.x * kWarps) {
        const uint8_t* drow = data + (size_t)row * n_super * 128u;
        const uint8_t* srow = scales + (size_t)row * n_super * 24u;
        float acc[TOK];
#pragma unroll
        for (uint32_t tk = 0; tk < TOK; ++tk) acc[tk] = 0.0f;
        for (uint32_t sb0 = 0; sb0 < n_super; sb0 += UNROLL) {
            uint32_t q[UNROLL];
            uint32_t dd[UNROLL];
            uint32_t scm[UNROLL];
#pragma unroll
            for (uint32_t u = 0; u < UNROLL; ++u) {
                const uint32_t sb = sb0 + u;
                if (sb < n_super) {
                    q[u] = pdk_ldg_stream4(drow + sb * 128u + lane * 4u);
                    const uint8_t* rec = srow + sb * 24u;
                    dd[u] = *reinterpret_cast<const uint32_t*>(rec);
                    const uint32_t s2 = *reinterpret_cast<const uint16_t*>(rec + 4u + 2u * G);
                    const uint32_t m2 = *reinterpret_cast<const uint16_t*>(rec + 12u + 2u * G);
                    scm[u] = s2 | (m2 << 16);
                } else {
                    q[u] = 0u; dd[u] = 0u; scm[u] = 0u;
                }
            }
#pragma unroll
            for (uint32_t u = 0; u < UNROLL; ++u) {
                const uint32_t sb = sb0 + u;
                if (sb >= n_super) break;
                const __half2 dh = *reinterpret_cast<const __half2*>(&dd[u]);
                const float d = __low2float(dh), dmin = __high2float(dh);
                const float d_lo = d * (float)(scm[u] & 0xffu), d_hi = d * (float)((scm[u] >> 8) & 0xffu);
                const float m_lo = dmin * (float)((scm[u] >> 16) & 0xffu), m_hi = dmin * (float)(scm[u] >> 24);
                const uint32_t k = sb * 256u + koff;
#pragma unroll
                for (uint32_t tk = 0; tk < TOK; ++tk) {
                    const float4 xl = *reinterpret_cast<const float4*>(xsf + tk * in_dim + k);
                    const float4 xh = *reinterpret_cast<const float4*>(xsf + tk * in_dim + k + 32u);
                    float sl = (float)(q[u] & 0xFu) * xl.x;
                    sl = fmaf((float)((q[u] >> 8) & 0xFu), xl.y, sl);
                    sl = fmaf((float)((q[u] >> 16) & 0xFu), xl.z, sl);
                    sl = fmaf((float)((q[u] >> 24) & 0xFu), xl.w, sl);
                    float sh = (float)((q[u] >> 4) & 0xFu) * xh.x;
                    sh = fmaf((float)((q[u] >> 12) & 0xFu), xh.y, sh);
                    sh = fmaf((float)((q[u] >> 20) & 0xFu), xh.z, sh);
                    sh = fmaf((float)(q[u] >> 28), xh.w, sh);
                    const float xsl = (xl.x + xl.y) + (xl.z + xl.w);
                    const float xsh = (xh.x + xh.y) + (xh.z + xh.w);
                    acc[tk] += (d_lo * sl - m_lo * xsl) + (d_hi * sh - m_hi * xsh);
                }
            }
        }
#pragma unroll
        for (uint32_t tk = 0; tk < TOK; ++tk) {
            const float v = pdk_warp_sum(acc[tk]);
            if (lane == 0) y[(size_t)(batch0 + tk) * out_dim + row] = v;
        }
    }
}

template <uint32_t TOK>
int launch_plain(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                 uint32_t batch0, cudaStream_t st) {
    const size_t smem = (size_t)TOK * in_dim * sizeof(float);
    auto kern = q4k_gemv_kernel<TOK, 10>;
    if (smem > 48u * 1024u) {
        if (smem > 200u * 1024u) return cudaErrorNotSupported;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)(kWarps * 32u), smem) != cudaSuccess ||
        per_sm < 1)
        per_sm = 1;
    uint32_t grid = (uint32_t)pdk_sm_count() * (uint32_t)per_sm;
    const uint32_t need = (out_dim + kWarps - 1u) / kWarps;
    if (grid > need) grid = need;
    kern<<<grid, kWarps * 32u, smem, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim, out_dim, batch0);
    return pdk_launch_status();
}

int plain_batch(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                uint32_t batch, cudaStream_t st) {
    uint32_t b = 0;
    for (; b + 4u <= batch; b += 4u)
        if (int rc = launch_plain<4>(data, scales, x, y, in_dim, out_dim, b, st)) return rc;
    for (; b + 2u <= batch; b += 2u)
        if (int rc = launch_plain<2>(data, scales, x, y, in_dim, out_dim, b, st)) return rc;
    for (; b < batch; ++b)
        if (int rc = launch_plain<1>(data, scales, x, y, in_dim, out_dim, b, st)) return rc;
    return 0;
}

// PDK_Q4K_PLAIN=1 forces the plain-load kernel (A/B switch, read once).
bool force_plain() {
    static const bool v = [] {
        const char* e = getenv("PDK_Q4K_PLAIN");
        return e && e[0] == '1';
    }();
    return v;
}

// PDK_Q4K_BATCH_BF16=1 keeps the bf16 tensor-core kernel for 2..16 tokens (A/B switch, read once).
bool force_bf16_batch() {
    static const bool v = [] {
        const char* e = getenv("PDK_Q4K_BATCH_BF16");
        return e && e[0] == '1';
    }();
    return v;
}

// From how many tokens on the tcgen05 kernel takes a call (PDK_Q4K_TC5_MIN, read once; 0 = never).
uint32_t tc5_min_tokens() {
    static const uint32_t v = [] {
        const char* e = getenv("PDK_Q4K_TC5_MIN");
        return e ? (uint32_t)atoi(e) : 9u;
    }();
    return v;
}

// 2 <= tokens on the tensor paths: up to 32 tokens per launch on tcgen05 from tc5_min_tokens() on,
// up to 16 on the int8 path below that.  Activations f32 (x) or int8 with per-32 scales (xq, xs).
// Returns the number of tokens done (all of them unless a shape is outside both plans), or
// -(cudaError_t) - 1 on a launch error.
int small_batch(const void* data, const void* scales, const float* x, const int8_t* xq, const float* xs, float* y,
                uint32_t in_dim, uint32_t out_dim, uint32_t batch, cudaStream_t st) {
    uint32_t b = 0;
    while (b < batch) {
        const uint32_t left = batch - b;
        const float* xb = x ? x + (size_t)b * in_dim : nullptr;
        const int8_t* qb = xq ? xq + (size_t)b * in_dim : nullptr;
        const float* sb = xs ? xs + (size_t)b * (in_dim >> 5) : nullptr;
        float* yb = y + (size_t)b * out_dim;
        uint32_t take = 0;
        int rc = -1;
        if (tc5_min_tokens() != 0u && left >= tc5_min_tokens()) {
            take = left < 32u ? left : 32u;
            rc = pdk_q4k_tc5(data, scales, xb, qb, sb, yb, in_dim, out_dim, take, st);
        }
        if (rc == -1) {
            take = left < 16u ? left : 16u;
            rc = pdk_q4k_batch_i8(data, scales, xb, qb, sb, yb, in_dim, out_dim, take, st);
        }
        if (rc == -1) break;
        if (rc != 0) return -rc - 1;
        b += take;
    }
    return (int)b;
}

int gemm_any(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
             uint32_t batch, cudaStream_t st) {
    if (!force_plain() && batch == 1u) {
        const int rc = pdk_q4k_gemv_i8(data, scales, x, y, in_dim, out_dim, st);
        if (rc != -1) return rc;
    }
    if (!force_plain() && !force_bf16_batch()) {
        const int done = small_batch(data, scales, x, nullptr, nullptr, y, in_dim, out_dim, batch, st);
        if (done < 0) return -done - 1;
        if ((uint32_t)done == batch) return 0;
        // outside both plans: the bf16 kernel or the plain route take what is left
        x += (size_t)done * in_dim;
        y += (size_t)done * out_dim;
        batch -= (uint32_t)done;
    }
    if (!force_plain()) {
        uint32_t b = 0;
        int rc = 0;
        while (b < batch && rc == 0) {
            const uint32_t left = batch - b;
            const float* xb = x + (size_t)b * in_dim;
            float* yb = y + (size_t)b * out_dim;
            uint32_t take;
            if (left <= 4u) { take = left; rc = launch_mma<1, true>(data, scales, xb, yb, in_dim, out_dim, take, st); }
            else if (left <= 8u) { take = left; rc = launch_mma<1, false>(data, scales, xb, yb, in_dim, out_dim, take, st); }
            else { take = left < 16u ? left : 16u; rc = launch_mma<2, false>(data, scales, xb, yb, in_dim, out_dim, take, st); }
            if (rc == -1) break;  // shared-memory plan does not fit: plain route for the rest
            b += take;
        }
        if (rc > 0) return rc;
        if (b == batch) return 0;
        return plain_batch(data, scales, x + (size_t)b * in_dim, y + (size_t)b * out_dim, in_dim, out_dim, batch - b, st);
    }
    return plain_batch(data, scales, x, y, in_dim, out_dim, batch, st);
}

// Q4_0 / Q5_K / Q6_K decode GEMV on the integer tensor path; -1 = shape outside the kernels' plan
int more_gemv_i8(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                 uint32_t dtype, cudaStream_t st) {
    if (dtype == PDK_KQ_Q4_0) return pdk_q4_0_gemv_i8(data, scales, x, y, in_dim, out_dim, st);
    if (dtype == PDK_KQ_Q5K) return pdk_q5k_gemv_i8(data, scales, x, y, in_dim, out_dim, st);
    if (dtype == PDK_KQ_Q6K) return pdk_q6k_gemv_i8(data, scales, x, y, in_dim, out_dim, st);
    if (dtype == PDK_KQ_IQ4XS) return pdk_iq4xs_gemv_i8(data, scales, x, y, in_dim, out_dim, st);
    return -1;
}

int check_gemv(const void* data, const void* scales, const void* x, const void* y, uint32_t in_dim, uint32_t dtype) {
    if (dtype != PDK_KQ_Q4K && !pdk_kq_more_has(dtype))
        return cudaErrorInvalidValue;
    if (in_dim == 0u || (in_dim & 255u) != 0u) return cudaErrorInvalidValue;
    if (!pdk_aligned(data, 16) || !pdk_aligned(scales, 8) || !pdk_aligned(x, 16) || !pdk_aligned(y, 4))
        return cudaErrorInvalidValue;
    return 0;
}

}  // namespace

PDK_EXPORT int pd_kquant_dequant(const void* src, void* dst, uint64_t n_super, uint32_t dtype, void* stream) {
    if (n_super == 0) return 0;
    if (pdk_kq_more_has(dtype)) return pdk_kq_more_dequant(src, dst, n_super, dtype, (cudaStream_t)stream);
    if (dtype != PDK_KQ_Q4K) return cudaErrorInvalidValue;
    if (!pdk_aligned(src, 2) || !pdk_aligned(dst, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    q4k_dequant_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (float*)dst, n_super);
    return pdk_launch_status();
}

PDK_EXPORT int pd_kquant_repack(const void* src, void* dst_data, void* dst_scales, uint64_t n_super, uint32_t dtype,
                                void* stream) {
    if (n_super == 0) return 0;
    if (pdk_kq_more_has(dtype))
        return pdk_kq_more_repack(src, dst_data, dst_scales, n_super, dtype, (cudaStream_t)stream);
    if (dtype != PDK_KQ_Q4K) return cudaErrorInvalidValue;
    if (!pdk_aligned(src, 4) || !pdk_aligned(dst_data, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    q4k_repack_kernel<<<(uint32_t)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst_data, (uint8_t*)dst_scales, n_super);
    return pdk_launch_status();
}

PDK_EXPORT int pd_kquant_gemv(const void* data, const void* scales, const void* x, void* y, uint32_t in_dim,
                              uint32_t out_dim, uint32_t dtype, void* stream) {
    if (out_dim == 0) return 0;
    if (int rc = check_gemv(data, scales, x, y, in_dim, dtype)) return rc;
    if (dtype != PDK_KQ_Q4K && !force_plain() && pdk_aligned(data, 16)) {
        const int rc = more_gemv_i8(data, scales, (const float*)x, (float*)y, in_dim, out_dim, dtype, (cudaStream_t)stream);
        if (rc != -1) return rc;
    }
    if (dtype != PDK_KQ_Q4K)
        return pdk_kq_more_gemm(data, scales, (const float*)x, (float*)y, in_dim, out_dim, 1u, dtype, (cudaStream_t)stream);
    return gemm_any(data, scales, (const float*)x, (float*)y, in_dim, out_dim, 1u, (cudaStream_t)stream);
}

PDK_EXPORT int pdk_kquant_gemm_f32(const void* data, const void* scales, const void* x, void* y, uint32_t in_dim,
                                   uint32_t out_dim, uint32_t batch, uint32_t dtype, void* stream) {
    if (out_dim == 0 || batch == 0) return 0;
    if (batch > 64u) return cudaErrorInvalidValue;
    if (int rc = check_gemv(data, scales, x, y, in_dim, dtype)) return rc;
    if (dtype == PDK_KQ_Q4_0 && batch >= 4u && !force_plain() && tc5_min_tokens() != 0u) {
        // Q4_0 shares Q4_K's nibble planes: from four tokens on the tcgen05 kernel (32 us per 32 tokens at K=5120,
        // N=25600) beats one 17 us decode GEMV per token
        uint32_t b = 0;
        int rc = 0;
        while (b < batch && rc == 0) {
            const uint32_t take = batch - b < 32u ? batch - b : 32u;
            rc = pdk_q4_0_tc5(data, scales, (const float*)x + (size_t)b * in_dim, (float*)y + (size_t)b * out_dim, in_dim,
                              out_dim, take, (cudaStream_t)stream);
            if (rc == 0) b += take;
        }
        if (rc > 0) return rc;
        if (b == batch) return 0;
        // -1: the shape is outside the kernel's plan, or this stream has no scratch slice (both hold for
        // the whole call, so b is 0 here unless slices were released meanwhile): the routes below
        // take what is left
        x = (const float*)x + (size_t)b * in_dim;
        y = (float*)y + (size_t)b * out_dim;
        batch -= b;
    }
    if ((dtype == PDK_KQ_Q5K || dtype == PDK_KQ_Q6K) && batch >= 2u && !force_plain() && pdk_aligned(data, 16)) {
        // Q5_K: Q4_K's integer batch kernel with the fifth bit ORed into the codes; Q6_K: its sibling with one
        // product per 16-weight block.  16 tokens per weight pass
        uint32_t b = 0;
        int rc = 0;
        while (b < batch && rc == 0) {
            const uint32_t take = batch - b < 16u ? batch - b : 16u;
            rc = (dtype == PDK_KQ_Q5K ? pdk_q5k_batch_i8 : pdk_q6k_batch_i8)(
                data, scales, (const float*)x + (size_t)b * in_dim, (float*)y + (size_t)b * out_dim, in_dim, out_dim, take,
                (cudaStream_t)stream);
            if (rc == 0) b += take;
        }
        if (rc > 0) return rc;
        if (b == batch) return 0;
        x = (const float*)x + (size_t)b * in_dim;   // -1: outside the kernel's plan, the routes below take what is left
        y = (float*)y + (size_t)b * out_dim;
        batch -= b;
    }
    if (dtype != PDK_KQ_Q4K && !force_plain() && pdk_aligned(data, 16)) {
        // Q4_0 below four tokens (and Q5_K / Q6_K outside the batch kernels' plan) have no batch kernel on the tensor path yet: one decode GEMV per token
        // (17-25 us each at K=5120 N=25600, the later ones partly from L2) beats the plain f32
        // kernel's 165 us per four tokens
        int rc = 0;
        for (uint32_t b = 0; b < batch && rc == 0; ++b)
            rc = more_gemv_i8(data, scales, (const float*)x + (size_t)b * in_dim, (float*)y + (size_t)b * out_dim, in_dim,
                              out_dim, dtype, (cudaStream_t)stream);
        if (rc != -1) return rc;  // -1 comes from the first call (the plan depends on the shape alone): nothing is done yet
    }
    if (dtype != PDK_KQ_Q4K)
        return pdk_kq_more_gemm(data, scales, (const float*)x, (float*)y, in_dim, out_dim, batch, dtype,
                                (cudaStream_t)stream);
    return gemm_any(data, scales, (const float*)x, (float*)y, in_dim, out_dim, batch, (cudaStream_t)stream);
}

// ---------------------------------------------------------------- int8 activation operands (W4A8 slots)
namespace {

// One warp per 32-element block: scale = amax / 127, q = RN(x / scale) clamped to +-127;
// optionally the two per-16 sums of q as f32 (packs/cuda/src/attn/decode.cuh:2981-3004, 3041-3068).
__global__ void quantize_q8_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale,
                                   float* __restrict__ sums, uint32_t n_blocks) {
    const uint32_t b = blockIdx.x * 8u + (threadIdx.x >> 5), d = threadIdx.x & 31u;
    if (b >= n_blocks) return;
    const float v = x[(size_t)b * 32u + d];
    float a = fabsf(v);
#pragma unroll
    for (uint32_t s = 16; s > 0; s >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, s));
    const float scl = a * (1.0f / 127.0f);
    if (d == 0) scale[b] = scl;
    const float inv = scl > 0.0f ? 1.0f / scl : 0.0f;
    int qi = __float2int_rn(v * inv);
    qi = qi < -127 ? -127 : (qi > 127 ? 127 : qi);
    q[(size_t)b * 32u + d] = (int8_t)qi;
    if (sums != nullptr) {
        int s16 = qi;
#pragma unroll
        for (uint32_t s = 8; s > 0; s >>= 1) s16 += __shfl_xor_sync(0xffffffffu, s16, s);
        if ((d & 15u) == 0u) sums[(size_t)b * 2u + (d >> 4)] = (float)s16;
    }
}

// x[i] = q[i] * scale[i / 32]: the f32 activations the batch kernels take
__global__ void q8_act_widen_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, float* __restrict__ x,
                                    uint64_t n4) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
    const float s = scale[i >> 3];
    reinterpret_cast<float4*>(x)[i] = make_float4((float)(int8_t)(w & 0xff) * s, (float)(int8_t)((w >> 8) & 0xff) * s,
                                                  (float)(int8_t)((w >> 16) & 0xff) * s, (float)(int8_t)(w >> 24) * s);
}

int w4a8_gemm(const void* data, const void* scales, const void* xq, const void* xs, void* part, void* y,
              uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t dtype, cudaStream_t st) {
    if (out_dim == 0 || batch == 0) return 0;
    if (batch > 64u) return cudaErrorInvalidValue;
    if (int rc = check_gemv(data, scales, xq, y, in_dim, dtype)) return rc;
    if (dtype != PDK_KQ_Q4K) return cudaErrorNotSupported;
    if (batch == 1u) {
        const int rc = pdk_q4k_gemv_i8_q8act(data, scales, (const int8_t*)xq, (const float*)xs, (float*)y, in_dim, out_dim, st);
        if (rc >= 0) return rc;
    }
    if (!force_plain() && !force_bf16_batch() && pdk_aligned(xq, 8)) {
        const int done = small_batch(data, scales, nullptr, (const int8_t*)xq, (const float*)xs, (float*)y, in_dim,
                                     out_dim, batch, st);
        if (done < 0) return -done - 1;
        if ((uint32_t)done == batch) return 0;
        // outside both plans, or no scratch slice for this stream: the widening route takes what is left
        xq = (const int8_t*)xq + (size_t)done * in_dim;
        xs = (const float*)xs + (size_t)done * (in_dim >> 5);
        y = (float*)y + (size_t)done * out_dim;
        batch -= (uint32_t)done;
    }
    // the batch kernels take f32 activations: widen q * scale into the caller's partial
    // buffer (>= 8 * out_dim * batch floats by the slot's contract)
    if (part == nullptr || !pdk_aligned(part, 16) || !pdk_aligned(xq, 4) || (uint64_t)in_dim > 8ull * out_dim)
        return cudaErrorInvalidValue;
    const uint64_t n4 = (uint64_t)batch * in_dim / 4u;
    q8_act_widen_kernel<<<(uint32_t)((n4 + 255u) / 256u), 256, 0, st>>>((const int8_t*)xq, (const float*)xs, (float*)part, n4);
    return gemm_any(data, scales, (const float*)part, (float*)y, in_dim, out_dim, batch, st);
}

}  // namespace

// slot 18, packs/cuda/src/gemm/f32_qkv.cuh:283-292
PDK_EXPORT int pd_quantize_q8(const void* x, void* q, void* scale, uint32_t n, void* stream) {
    const uint32_t n_blocks = n >> 5;
    if (n_blocks == 0) return 0;
    quantize_q8_kernel<<<(n_blocks + 7u) / 8u, 256, 0, (cudaStream_t)stream>>>((const float*)x, (int8_t*)q, (float*)scale,
                                                                               nullptr, n_blocks);
    return pdk_launch_status();
}

// slot 218, packs/cuda/src/gemm/f32_qkv.cuh:304-311: also the per-16 sums of q (f32 [n/16])
PDK_EXPORT int pd_quantize_q8_sums(const void* x, void* q, void* scale, void* sums, uint32_t n, void* stream) {
    const uint32_t n_blocks = n >> 5;
    if (n_blocks == 0) return 0;
    if (sums == nullptr) return cudaErrorInvalidValue;
    quantize_q8_kernel<<<(n_blocks + 7u) / 8u, 256, 0, (cudaStream_t)stream>>>((const float*)x, (int8_t*)q, (float*)scale,
                                                                               (float*)sums, n_blocks);
    return pdk_launch_status();
}

// slot 217, packs/cuda/src/quant/kquant_w4a8.cuh:1266-1330: decode GEMV on int8 activations.
// xsums (the min term's per-16 sums) is accepted and not needed: the kernel rebuilds its
// own sums from q * scale.  Shapes outside the GEMV kernel's plan answer "not supported"
// (there is no scratch argument to widen the activations into).
PDK_EXPORT int pd_kquant_gemv_w4a8(const void* data, const void* scales, const void* xq, const void* xs,
                                   const void* xsums, void* y, uint32_t in_dim, uint32_t out_dim, uint32_t dtype,
                                   void* stream) {
    (void)xsums;
    if (out_dim == 0) return 0;
    if (int rc = check_gemv(data, scales, xq, y, in_dim, dtype)) return rc;
    if (dtype != PDK_KQ_Q4K) return cudaErrorNotSupported;
    const int rc = pdk_q4k_gemv_i8_q8act(data, scales, (const int8_t*)xq, (const float*)xs, (float*)y, in_dim, out_dim,
                                         (cudaStream_t)stream);
    return rc >= 0 ? rc : (int)cudaErrorNotSupported;
}

// slot 212, packs/cuda/src/quant/kquant_w4a8.cuh:2364-2430: batch <= 64, y f32 [batch][out_dim];
// `part` (>= 8 * out_dim * batch floats) is used as scratch for the widened activations.
PDK_EXPORT int pd_kquant_gemm_mma_ks(const void* data, const void* scales, const void* xq, const void* xs,
                                     const void* xsums, void* part, void* y, uint32_t in_dim, uint32_t out_dim,
                                     uint32_t batch, uint32_t dtype, void* stream) {
    (void)xsums;
    return w4a8_gemm(data, scales, xq, xs, part, y, in_dim, out_dim, batch, dtype, (cudaStream_t)stream);
}

// slot 837, packs/cuda/src/quant/kquant_w4a8_sb.cuh:300-353: same contract as slot 212
PDK_EXPORT int pd_kquant_gemm_w4a8_sb(const void* data, const void* scales, const void* xq, const void* xs,
                                      const void* xsums, void* part, void* y, uint32_t in_dim, uint32_t out_dim,
                                      uint32_t batch, uint32_t dtype, void* stream) {
    (void)xsums;
    return w4a8_gemm(data, scales, xq, xs, part, y, in_dim, out_dim, batch, dtype, (cudaStream_t)stream);
}
