// kquant_more.cu - the other resident formats behind the k-quant slots: Q5_K, Q6_K and
// Q4_0 (packs/cuda/src/quant/kquant.cuh:37-80 for the layouts, :144-250 dequant, :255-345
// repack, :372-653 GEMV).  Dequant and repack are bit- and byte-exact.  The GEMM here is a
// plain f32 kernel (one warp per output row, lane l takes element l of each 32-element
// sub-block so every load instruction covers whole lines): it serves more than one token and
// the shapes the tensor-core decode kernels (gemv_i8.cu, gemv_q6k.cu) decline.
//
// Repacked planes (the reference's byte budgets):
//   Q5_K  data 160 B/sb = qs[128] then qh[32];  record 24 B {f16 d, f16 dmin, u8 sc[8], u8 m[8], pad4}
//   Q6_K  data 192 B/sb = ql[128] then qh[64];  record 24 B {f16 d, pad2, i8 sc[16], pad4}
//   Q4_0  data 128 B/sb, nibbles permuted into the Q4_K convention (group g byte l = block 2g
//         weight l low | block 2g+1 weight l high);  record 24 B {f16 d[8], pad8}
//   IQ4_XS data 128 B/sb = qs verbatim (sub-block ib byte j = weight j low | weight 16 + j high, each a
//         code-book index);  record 24 B {f16 d, pad2, i8 ls - 32 [8], pad12}
#include "pdk_common.cuh"

namespace {

__device__ __forceinline__ void scale_min_k4(const uint8_t* s, uint32_t j, uint32_t* sc, uint32_t* m) {
    if (j < 4u) {
        *sc = s[j] & 63u;
        *m = s[j + 4u] & 63u;
    } else {
        *sc = (uint32_t)(s[j + 4u] & 0xFu) | ((uint32_t)(s[j - 4u] >> 6) << 4);
        *m = (uint32_t)(s[j + 4u] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}
// ggml's 16-entry non-linear 4-bit code book (IQ4_NL / IQ4_XS), eight signed bytes per word
__device__ __forceinline__ int iq4nl(uint32_t index) {
    const uint64_t lo = 0xF6EADDCFBFAD9881ull;   // -127 -104 -83 -65 -49 -35 -22 -10
    const uint64_t hi = 0x7159453526190D01ull;   //    1   13  25  38  53  69  89 113
    return (int)(int8_t)(((index & 8u) ? hi : lo) >> ((index & 7u) * 8u));
}
__device__ __forceinline__ float f16_at(const uint8_t* p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// ---------------------------------------------------------------- dequant of the raw ggml blocks
// One warp per 256 weights; lane l writes element l of each 32-element run.
__global__ void kq_dequant_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, uint64_t n_super,
                                  uint32_t dtype) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t l = threadIdx.x & 31u;
    float* y = dst + b * 256u;
    if (dtype == PDK_KQ_Q5K) {
        const uint8_t* s = src + b * 176u;
        const float d = f16_at(s), dmin = f16_at(s + 2);
        const uint32_t hbits = s[16u + l];
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            uint32_t sc, m;
            scale_min_k4(s + 4, j, &sc, &m);
            const float dj = __fmul_rn(d, (float)sc), mj = __fmul_rn(dmin, (float)m);
            const uint32_t q = s[48u + (j >> 1) * 32u + l];
            const uint32_t v = ((j & 1u) ? (q >> 4) : (q & 0xFu)) + (((hbits >> j) & 1u) << 4);
            y[j * 32u + l] = __fsub_rn(__fmul_rn(dj, (float)v), mj);
        }
    } else if (dtype == PDK_KQ_Q6K) {
        const uint8_t* s = src + b * 210u;
        const float d = f16_at(s + 208);
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
            const uint32_t qlo = s[nh * 64u + l], qlh = s[nh * 64u + 32u + l], h = s[128u + nh * 32u + l];
            const int q[4] = {(int)((qlo & 0xFu) | ((h & 3u) << 4)) - 32, (int)((qlh & 0xFu) | (((h >> 2) & 3u) << 4)) - 32,
                              (int)((qlo >> 4) | (((h >> 4) & 3u) << 4)) - 32, (int)((qlh >> 4) | (((h >> 6) & 3u) << 4)) - 32};
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r) {
                const float ds = __fmul_rn(d, (float)(int8_t)s[192u + nh * 8u + r * 2u + (l >> 4)]);
                y[nh * 128u + r * 32u + l] = __fmul_rn(ds, (float)q[r]);
            }
        }
    } else if (dtype == PDK_KQ_IQ4XS) {
        const uint8_t* s = src + b * 136u;
        const float d = f16_at(s);
        const uint32_t sh = (uint32_t)s[2] | ((uint32_t)s[3] << 8);
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const int ls = (int)(((s[4u + (j >> 1)] >> (4u * (j & 1u))) & 0xFu) | (((sh >> (2u * j)) & 3u) << 4)) - 32;
            const uint32_t q = s[8u + j * 16u + (l & 15u)];
            y[j * 32u + l] = __fmul_rn(__fmul_rn(d, (float)ls), (float)iq4nl(l < 16u ? (q & 0xFu) : (q >> 4)));
        }
    } else {  // Q4_0: eight 18-byte blocks
        const uint8_t* s = src + b * 144u;
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint8_t* blk = s + j * 18u;
            const uint32_t q = blk[2u + (l & 15u)];
            const int v = (int)((l < 16u) ? (q & 0xFu) : (q >> 4)) - 8;
            y[j * 32u + l] = __fmul_rn(f16_at(blk), (float)v);
        }
    }
}

// ---------------------------------------------------------------- repack
__global__ void kq_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst_data,
                                 uint8_t* __restrict__ dst_scales, uint64_t n_super, uint32_t dtype) {
    const uint64_t b = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_super) return;
    const uint32_t l = threadIdx.x & 31u;
    uint8_t* rec = dst_scales + b * 24u;
    if (dtype == PDK_KQ_Q5K) {
        const uint8_t* s = src + b * 176u;
        uint8_t* d = dst_data + b * 160u;
        for (uint32_t i = l; i < 128u; i += 32u) d[i] = s[48u + i];
        d[128u + l] = s[16u + l];
        if (l < 8u) {
            uint32_t sc, m;
            scale_min_k4(s + 4, l, &sc, &m);
            rec[4u + l] = (uint8_t)sc;
            rec[12u + l] = (uint8_t)m;
        } else if (l < 12u) {
            rec[l - 8u] = s[l - 8u];
        } else if (l < 16u) {
            rec[8u + l] = 0;
        }
    } else if (dtype == PDK_KQ_Q6K) {
        const uint8_t* s = src + b * 210u;
        uint8_t* d = dst_data + b * 192u;
        for (uint32_t i = l; i < 192u; i += 32u) d[i] = s[i];
        if (l < 16u) rec[4u + l] = s[192u + l];
        if (l == 16u) { rec[0] = s[208]; rec[1] = s[209]; rec[2] = 0; rec[3] = 0; }
        if (l >= 20u && l < 24u) rec[l] = 0;
    } else if (dtype == PDK_KQ_IQ4XS) {
        const uint8_t* s = src + b * 136u;
        uint8_t* d = dst_data + b * 128u;
        for (uint32_t i = l; i < 128u; i += 32u) d[i] = s[8u + i];
        if (l < 8u) {
            const uint32_t sh = (uint32_t)s[2] | ((uint32_t)s[3] << 8);
            const int ls = (int)(((s[4u + (l >> 1)] >> (4u * (l & 1u))) & 0xFu) | (((sh >> (2u * l)) & 3u) << 4)) - 32;
            rec[4u + l] = (uint8_t)(int8_t)ls;
        } else if (l < 10u) {
            rec[l - 8u] = s[l - 8u];
        } else if (l < 12u) {
            rec[l - 8u] = 0;
        } else if (l < 24u) {
            rec[l] = 0;
        }
    } else {  // Q4_0
        const uint8_t* s = src + b * 144u;
        uint8_t* d = dst_data + b * 128u;
#pragma unroll
        for (uint32_t g = 0; g < 4u; ++g) {
            const uint8_t* a = s + (2u * g) * 18u + 2u;
            const uint8_t* c = s + (2u * g + 1u) * 18u + 2u;
            const uint32_t lo = l < 16u ? (a[l] & 0xFu) : (uint32_t)(a[l - 16u] >> 4);
            const uint32_t hi = l < 16u ? (c[l] & 0xFu) : (uint32_t)(c[l - 16u] >> 4);
            d[g * 32u + l] = (uint8_t)(lo | (hi << 4));
        }
        if (l < 8u) { rec[2u * l] = s[l * 18u]; rec[2u * l + 1u] = s[l * 18u + 1u]; }
        if (l >= 16u && l < 24u) rec[l] = 0;
    }
}

// ---------------------------------------------------------------- GEMV / small-batch GEMM, f32
// The eight values lane l holds of one repacked super-block: element j*32 + l, j = 0..7.
__device__ __forceinline__ void decode8(uint32_t dtype, const uint8_t* d, const uint8_t* rec, uint32_t l, float (&w)[8]) {
    if (dtype == PDK_KQ_Q5K) {
        const float dd = f16_at(rec), dmin = f16_at(rec + 2);
        const uint32_t hbits = d[128u + l];
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t q = d[(j >> 1) * 32u + l];
            const uint32_t v = ((j & 1u) ? (q >> 4) : (q & 0xFu)) + (((hbits >> j) & 1u) << 4);
            w[j] = __fsub_rn(__fmul_rn(__fmul_rn(dd, (float)rec[4u + j]), (float)v), __fmul_rn(dmin, (float)rec[12u + j]));
        }
    } else if (dtype == PDK_KQ_Q6K) {
        const float dd = f16_at(rec);
#pragma unroll
        for (uint32_t nh = 0; nh < 2u; ++nh) {
            const uint32_t qlo = d[nh * 64u + l], qlh = d[nh * 64u + 32u + l], h = d[128u + nh * 32u + l];
            const int q[4] = {(int)((qlo & 0xFu) | ((h & 3u) << 4)) - 32, (int)((qlh & 0xFu) | (((h >> 2) & 3u) << 4)) - 32,
                              (int)((qlo >> 4) | (((h >> 4) & 3u) << 4)) - 32, (int)((qlh >> 4) | (((h >> 6) & 3u) << 4)) - 32};
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r)
                w[nh * 4u + r] = __fmul_rn(__fmul_rn(dd, (float)(int8_t)rec[4u + nh * 8u + r * 2u + (l >> 4)]), (float)q[r]);
        }
    } else if (dtype == PDK_KQ_IQ4XS) {
        const float dd = f16_at(rec);
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t q = d[j * 16u + (l & 15u)];
            w[j] = __fmul_rn(__fmul_rn(dd, (float)(int8_t)rec[4u + j]), (float)iq4nl(l < 16u ? (q & 0xFu) : (q >> 4)));
        }
    } else {  // Q4_0 in the Q4_K nibble convention, eight independent f16 scales
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            const uint32_t q = d[(j >> 1) * 32u + l];
            const int v = (int)((j & 1u) ? (q >> 4) : (q & 0xFu)) - 8;
            w[j] = __fmul_rn(f16_at(rec + 2u * j), (float)v);
        }
    }
}

template <uint32_t TB>  // tokens per pass
__global__ void __launch_bounds__(256)
kq_gemm_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ recs, const float* __restrict__ x,
               float* __restrict__ y, uint32_t in_dim, uint32_t out_dim, uint32_t batch, uint32_t dtype, uint32_t datab) {
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5), l = threadIdx.x & 31u;
    if (row >= out_dim) return;
    const uint32_t n_super = in_dim >> 8;
    const uint8_t* drow = data + (size_t)row * n_super * datab;
    const uint8_t* rrow = recs + (size_t)row * n_super * 24u;
    for (uint32_t t0 = 0; t0 < batch; t0 += TB) {
        float acc[TB];
#pragma unroll
        for (uint32_t t = 0; t < TB; ++t) acc[t] = 0.0f;
        for (uint32_t sb = 0; sb < n_super; ++sb) {
            float w[8];
            decode8(dtype, drow + (size_t)sb * datab, rrow + (size_t)sb * 24u, l, w);
#pragma unroll
            for (uint32_t t = 0; t < TB; ++t) {
                if (t0 + t >= batch) break;
                const float* xr = x + (size_t)(t0 + t) * in_dim + sb * 256u + l;
#pragma unroll
                for (uint32_t j = 0; j < 8u; ++j) acc[t] = fmaf(w[j], xr[j * 32u], acc[t]);
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < TB; ++t) {
            if (t0 + t >= batch) break;
            const float s = pdk_warp_sum(acc[t]);
            if (l == 0) y[(size_t)(t0 + t) * out_dim + row] = s;
        }
    }
}

uint32_t data_bytes(uint32_t dtype) { return dtype == PDK_KQ_Q5K ? 160u : dtype == PDK_KQ_Q6K ? 192u : 128u; }

}  // namespace

bool pdk_kq_more_has(uint32_t dtype) {
    return dtype == PDK_KQ_Q5K || dtype == PDK_KQ_Q6K || dtype == PDK_KQ_Q4_0 || dtype == PDK_KQ_IQ4XS;
}

int pdk_kq_more_dequant(const void* src, void* dst, uint64_t n_super, uint32_t dtype, cudaStream_t st) {
    if (!pdk_aligned(dst, 4)) return cudaErrorInvalidValue;
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    kq_dequant_kernel<<<(uint32_t)blocks, 256, 0, st>>>((const uint8_t*)src, (float*)dst, n_super, dtype);
    return pdk_launch_status();
}

int pdk_kq_more_repack(const void* src, void* dst_data, void* dst_scales, uint64_t n_super, uint32_t dtype,
                       cudaStream_t st) {
    const uint64_t blocks = (n_super + 7u) / 8u;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    kq_repack_kernel<<<(uint32_t)blocks, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst_data, (uint8_t*)dst_scales,
                                                       n_super, dtype);
    return pdk_launch_status();
}

int pdk_kq_more_gemm(const void* data, const void* scales, const float* x, float* y, uint32_t in_dim, uint32_t out_dim,
                     uint32_t batch, uint32_t dtype, cudaStream_t st) {
    if (in_dim == 0u || (in_dim & 255u) != 0u) return cudaErrorInvalidValue;
    const uint32_t grid = (out_dim + 7u) / 8u;
    if (batch == 1u)
        kq_gemm_kernel<1><<<grid, 256, 0, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim, out_dim, batch,
                                                dtype, data_bytes(dtype));
    else
        kq_gemm_kernel<4><<<grid, 256, 0, st>>>((const uint8_t*)data, (const uint8_t*)scales, x, y, in_dim, out_dim, batch,
                                                dtype, data_bytes(dtype));
    return pdk_launch_status();
}
