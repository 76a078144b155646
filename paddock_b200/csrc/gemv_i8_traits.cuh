// gemv_i8_traits.cuh - format traits shared by the decode GEMV kernels on the int8 tensor path
// (gemv_i8.cu: operands prefetched into registers; gemv_ring.cu: operands staged in a
// shared-memory ring by bulk copies).
//
// A "unit" is 256 weights of one row (a Q4_K / Q5_K super-block, eight Q4_0 or Q8_0 blocks).
// Lane (g, t) of a warp holds rows g and g + 8 of a 16-row tile and owns blocks 2t and 2t+1 of
// the unit.  `load<kShared>` fills a Stage from the unit's data / record bytes of the two rows:
// streaming global loads (kShared = false) or plain loads from a staged copy (kShared = true).
#pragma once
#include "pdk_common.cuh"

namespace gemv_i8 {

template <bool kShared>
__device__ __forceinline__ uint4 ld16(const void* p) {
    if constexpr (kShared) return *reinterpret_cast<const uint4*>(p);
    else return pdk_ldg_stream16(p);
}
template <bool kShared>
__device__ __forceinline__ uint2 ld8(const void* p) {
    if constexpr (kShared) return *reinterpret_cast<const uint2*>(p);
    else return pdk_ldg_stream8(p);
}
template <bool kShared>
__device__ __forceinline__ uint32_t ld4(const void* p) {
    if constexpr (kShared) return *reinterpret_cast<const uint32_t*>(p);
    else return __ldg(reinterpret_cast<const uint32_t*>(p));
}
template <bool kShared>
__device__ __forceinline__ uint32_t ld2(const void* p) {
    if constexpr (kShared) return (uint32_t)*reinterpret_cast<const uint16_t*>(p);
    else return (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p));
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with unsigned A bytes (codes 0..255 against signed activation limbs).
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Non-volatile forms: the compiler may interleave independent accumulator chains.
__device__ __forceinline__ void mma_s8_nv(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8_nv(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------
// Format traits.  A "unit" is 256 weights of one row (a Q4_K super-block, or
// eight Q8_0 blocks).  Lane t owns blocks 2t and 2t+1 of the unit.
// ---------------------------------------------------------------------------
struct Q4K {
    static constexpr uint32_t kDepth = 3;
    static constexpr uint32_t kDataBytes = 128;  // per row per unit
    static constexpr uint32_t kRecBytes = 24;
    static constexpr bool kSplitBlock = false;   // a 32-byte lane run holds two blocks side by side (low / high nibbles, or halves)
    struct Stage {
        uint4 q[4];      // row g: bytes 0..15 / 16..31 of ggml group t; row g+8 likewise
        uint32_t dd[2];  // {f16 d, f16 dmin} of the two rows
        uint32_t sm[2];  // sc[2t] | sc[2t+1]<<8 | m[2t]<<16 | m[2t+1]<<24
    };
    template <bool kShared>
    __device__ static __forceinline__ void load(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                                const uint8_t* r1, uint32_t t) {
        s.q[0] = ld16<kShared>(d0 + t * 32u);
        s.q[1] = ld16<kShared>(d0 + t * 32u + 16u);
        s.q[2] = ld16<kShared>(d1 + t * 32u);
        s.q[3] = ld16<kShared>(d1 + t * 32u + 16u);
        s.dd[0] = ld4<kShared>(r0);
        s.dd[1] = ld4<kShared>(r1);
        s.sm[0] = ld2<kShared>(r0 + 4u + 2u * t) |
                  (ld2<kShared>(r0 + 12u + 2u * t) << 16);
        s.sm[1] = ld2<kShared>(r1 + 4u + 2u * t) |
                  (ld2<kShared>(r1 + 12u + 2u * t) << 16);
    }
    // A registers of mma i (i = 0..7): word i of the lane's 32 bytes, low nibbles
    // (block 2t) in k-slots 4t..4t+3, high nibbles (block 2t+1) in slots 16+4t..
    __device__ static __forceinline__ void a_regs(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint4& lo = s.q[i >> 2];
        const uint4& hi = s.q[2u + (i >> 2)];
        const uint32_t wl = (i & 3u) == 0u ? lo.x : (i & 3u) == 1u ? lo.y : (i & 3u) == 2u ? lo.z : lo.w;
        const uint32_t wh = (i & 3u) == 0u ? hi.x : (i & 3u) == 1u ? hi.y : (i & 3u) == 2u ? hi.z : hi.w;
        a0 = wl & 0x0F0F0F0Fu;
        a1 = wh & 0x0F0F0F0Fu;
        a2 = (wl >> 4) & 0x0F0F0F0Fu;
        a3 = (wh >> 4) & 0x0F0F0F0Fu;
    }
    // The ring kernel's form: codes stay where they are in the byte.  a0 / a1 = low nibbles, a2 / a3 =
    // the high nibbles left in place (16 x code, an unsigned byte), so a word costs two ANDs per
    // row instead of two ANDs and two shifts; the sums of blocks 2t+1 come out 16 times too large
    // and are shifted back (exactly: every product is a multiple of 16) before the f32 conversion.
    static constexpr bool kUnsignedA = true;
    static constexpr int kHiShift = 4;
    __device__ static __forceinline__ void a_frag(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint4& lo = s.q[i >> 2];
        const uint4& hi = s.q[2u + (i >> 2)];
        const uint32_t wl = (i & 3u) == 0u ? lo.x : (i & 3u) == 1u ? lo.y : (i & 3u) == 2u ? lo.z : lo.w;
        const uint32_t wh = (i & 3u) == 0u ? hi.x : (i & 3u) == 1u ? hi.y : (i & 3u) == 2u ? hi.z : hi.w;
        a0 = wl & 0x0F0F0F0Fu;
        a1 = wh & 0x0F0F0F0Fu;
        a2 = wl & 0xF0F0F0F0u;
        a3 = wh & 0xF0F0F0F0u;
    }
    // f[0..1]: row g blocks 2t, 2t+1 (already times the activation step); f[2..3]: row g+8.
    // X0, X1: the blocks' activation sums.
    __device__ static __forceinline__ void fold(const Stage& s, const float (&f)[4], float X0, float X1,
                                                float& acc_g, float& acc_g8) {
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[0]);
            const float s0 = (float)(s.sm[0] & 0xffu), s1 = (float)((s.sm[0] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[0] >> 16) & 0xffu), m1 = (float)(s.sm[0] >> 24);
            acc_g += __low2float(dh) * (s0 * f[0] + s1 * f[1]) - __high2float(dh) * (m0 * X0 + m1 * X1);
        }
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[1]);
            const float s0 = (float)(s.sm[1] & 0xffu), s1 = (float)((s.sm[1] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[1] >> 16) & 0xffu), m1 = (float)(s.sm[1] >> 24);
            acc_g8 += __low2float(dh) * (s0 * f[2] + s1 * f[3]) - __high2float(dh) * (m0 * X0 + m1 * X1);
        }
    }
};

// Q5_K repacked (kquant_more.cu): 128 bytes of low nibbles in the Q4_K convention, then 32 bytes
// of high bits (bit j of byte l = bit 4 of element l of block j); the record is Q4_K's.
struct Q5K {
    static constexpr uint32_t kDepth = 2;
    static constexpr uint32_t kDataBytes = 160;
    static constexpr uint32_t kRecBytes = 24;
    static constexpr bool kSplitBlock = false;   // a 32-byte lane run holds two blocks side by side (low / high nibbles, or halves)
    struct Stage {
        uint4 q[4];      // as Q4K
        uint2 hb[2];     // high-bit bytes 8t..8t+7 of row g / row g+8 (the other lanes of the row hold the rest)
        uint32_t dd[2];
        uint32_t sm[2];
    };
    template <bool kShared>
    __device__ static __forceinline__ void load(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                                const uint8_t* r1, uint32_t t) {
        s.q[0] = ld16<kShared>(d0 + t * 32u);
        s.q[1] = ld16<kShared>(d0 + t * 32u + 16u);
        s.q[2] = ld16<kShared>(d1 + t * 32u);
        s.q[3] = ld16<kShared>(d1 + t * 32u + 16u);
        s.hb[0] = ld8<kShared>(d0 + 128u + t * 8u);
        s.hb[1] = ld8<kShared>(d1 + 128u + t * 8u);
        s.dd[0] = ld4<kShared>(r0);
        s.dd[1] = ld4<kShared>(r1);
        s.sm[0] = ld2<kShared>(r0 + 4u + 2u * t) |
                  (ld2<kShared>(r0 + 12u + 2u * t) << 16);
        s.sm[1] = ld2<kShared>(r1 + 4u + 2u * t) |
                  (ld2<kShared>(r1 + 12u + 2u * t) << 16);
    }
    __device__ static __forceinline__ uint32_t word(const uint4& v, uint32_t i) {
        return i == 0u ? v.x : i == 1u ? v.y : i == 2u ? v.z : v.w;
    }
    // mma i: nibbles of word i as in Q4K, plus bit 2t (block 2t) / 2t+1 (block 2t+1) of the
    // high-bit bytes 4i..4i+3 - held by lane i/2 of the row's four - as bit 4 of each code
    __device__ static __forceinline__ void a_regs(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint32_t lane = threadIdx.x & 31u, t2 = 2u * (lane & 3u), src = (lane & 28u) | (i >> 1);
        const uint32_t wl = word(s.q[i >> 2], i & 3u), wh = word(s.q[2u + (i >> 2)], i & 3u);
        const uint32_t hl = (__shfl_sync(0xffffffffu, (i & 1u) ? s.hb[0].y : s.hb[0].x, src) >> t2) << 4;
        const uint32_t hh = (__shfl_sync(0xffffffffu, (i & 1u) ? s.hb[1].y : s.hb[1].x, src) >> t2) << 4;
        a0 = (wl & 0x0F0F0F0Fu) | (hl & 0x10101010u);
        a1 = (wh & 0x0F0F0F0Fu) | (hh & 0x10101010u);
        a2 = ((wl >> 4) & 0x0F0F0F0Fu) | ((hl >> 1) & 0x10101010u);
        a3 = ((wh >> 4) & 0x0F0F0F0Fu) | ((hh >> 1) & 0x10101010u);
    }
    static constexpr bool kUnsignedA = true;
    static constexpr int kHiShift = 0;
    __device__ static __forceinline__ void a_frag(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        a_regs(s, i, a0, a1, a2, a3);
    }
    __device__ static __forceinline__ void fold(const Stage& s, const float (&f)[4], float X0, float X1,
                                                float& acc_g, float& acc_g8) {
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[0]);
            const float s0 = (float)(s.sm[0] & 0xffu), s1 = (float)((s.sm[0] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[0] >> 16) & 0xffu), m1 = (float)(s.sm[0] >> 24);
            acc_g += __low2float(dh) * (s0 * f[0] + s1 * f[1]) - __high2float(dh) * (m0 * X0 + m1 * X1);
        }
        {
            const __half2 dh = *reinterpret_cast<const __half2*>(&s.dd[1]);
            const float s0 = (float)(s.sm[1] & 0xffu), s1 = (float)((s.sm[1] >> 8) & 0xffu);
            const float m0 = (float)((s.sm[1] >> 16) & 0xffu), m1 = (float)(s.sm[1] >> 24);
            acc_g8 += __low2float(dh) * (s0 * f[2] + s1 * f[3]) - __high2float(dh) * (m0 * X0 + m1 * X1);
        }
    }
};

// Q4_0 repacked (kquant_more.cu): the data plane is in the Q4_K nibble convention, the record
// holds eight f16 block scales; w = d (q - 8), so the activation sums carry the -8.
struct Q40 {
    static constexpr uint32_t kDepth = 3;
    static constexpr uint32_t kDataBytes = 128;
    static constexpr uint32_t kRecBytes = 24;
    static constexpr bool kSplitBlock = false;   // a 32-byte lane run holds two blocks side by side (low / high nibbles, or halves)
    struct Stage {
        uint4 q[4];
        uint32_t dd[2];  // {f16 d[2t], f16 d[2t+1]} of the two rows
    };
    template <bool kShared>
    __device__ static __forceinline__ void load(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                                const uint8_t* r1, uint32_t t) {
        s.q[0] = ld16<kShared>(d0 + t * 32u);
        s.q[1] = ld16<kShared>(d0 + t * 32u + 16u);
        s.q[2] = ld16<kShared>(d1 + t * 32u);
        s.q[3] = ld16<kShared>(d1 + t * 32u + 16u);
        s.dd[0] = ld4<kShared>(r0 + 4u * t);
        s.dd[1] = ld4<kShared>(r1 + 4u * t);
    }
    __device__ static __forceinline__ void a_regs(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint4& lo = s.q[i >> 2];
        const uint4& hi = s.q[2u + (i >> 2)];
        const uint32_t wl = (i & 3u) == 0u ? lo.x : (i & 3u) == 1u ? lo.y : (i & 3u) == 2u ? lo.z : lo.w;
        const uint32_t wh = (i & 3u) == 0u ? hi.x : (i & 3u) == 1u ? hi.y : (i & 3u) == 2u ? hi.z : hi.w;
        a0 = wl & 0x0F0F0F0Fu;
        a1 = wh & 0x0F0F0F0Fu;
        a2 = (wl >> 4) & 0x0F0F0F0Fu;
        a3 = (wh >> 4) & 0x0F0F0F0Fu;
    }
    // The ring kernel's form: codes stay where they are in the byte.  a0 / a1 = low nibbles, a2 / a3 =
    // the high nibbles left in place (16 x code, an unsigned byte), so a word costs two ANDs per
    // row instead of two ANDs and two shifts; the sums of blocks 2t+1 come out 16 times too large
    // and are shifted back (exactly: every product is a multiple of 16) before the f32 conversion.
    static constexpr bool kUnsignedA = true;
    static constexpr int kHiShift = 4;
    __device__ static __forceinline__ void a_frag(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        const uint4& lo = s.q[i >> 2];
        const uint4& hi = s.q[2u + (i >> 2)];
        const uint32_t wl = (i & 3u) == 0u ? lo.x : (i & 3u) == 1u ? lo.y : (i & 3u) == 2u ? lo.z : lo.w;
        const uint32_t wh = (i & 3u) == 0u ? hi.x : (i & 3u) == 1u ? hi.y : (i & 3u) == 2u ? hi.z : hi.w;
        a0 = wl & 0x0F0F0F0Fu;
        a1 = wh & 0x0F0F0F0Fu;
        a2 = wl & 0xF0F0F0F0u;
        a3 = wh & 0xF0F0F0F0u;
    }
    __device__ static __forceinline__ void fold(const Stage& s, const float (&f)[4], float X0, float X1,
                                                float& acc_g, float& acc_g8) {
        const __half2 d0 = *reinterpret_cast<const __half2*>(&s.dd[0]);
        const __half2 d1 = *reinterpret_cast<const __half2*>(&s.dd[1]);
        const float o0 = -8.0f * X0, o1 = -8.0f * X1;
        acc_g += __low2float(d0) * (f[0] + o0) + __high2float(d0) * (f[1] + o1);
        acc_g8 += __low2float(d1) * (f[2] + o0) + __high2float(d1) * (f[3] + o1);
    }
};

struct Q80 {
    static constexpr uint32_t kDepth = 2;
    static constexpr uint32_t kDataBytes = 256;  // 8 blocks of 32 int8
    static constexpr uint32_t kRecBytes = 16;    // 8 f16 scales
    static constexpr bool kSplitBlock = false;   // a 32-byte lane run holds two blocks side by side (low / high nibbles, or halves)
    struct Stage {
        uint4 q[8];      // row g: blocks 2t, 2t+1 (64 bytes); row g+8 likewise
        uint32_t dd[2];  // {f16 d[2t], f16 d[2t+1]} of the two rows
    };
    template <bool kShared>
    __device__ static __forceinline__ void load(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                                const uint8_t* r1, uint32_t t) {
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i) {
            s.q[i] = ld16<kShared>(d0 + t * 64u + i * 16u);
            s.q[4u + i] = ld16<kShared>(d1 + t * 64u + i * 16u);
        }
        s.dd[0] = ld4<kShared>(r0 + 4u * t);
        s.dd[1] = ld4<kShared>(r1 + 4u * t);
    }
    __device__ static __forceinline__ uint32_t word(const uint4& v, uint32_t i) {
        return i == 0u ? v.x : i == 1u ? v.y : i == 2u ? v.z : v.w;
    }
    // mma i: word i of block 2t in slots 4t..4t+3, word i of block 2t+1 in slots 16+4t..
    __device__ static __forceinline__ void a_regs(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        a0 = word(s.q[i >> 2], i & 3u);
        a2 = word(s.q[2u + (i >> 2)], i & 3u);
        a1 = word(s.q[4u + (i >> 2)], i & 3u);
        a3 = word(s.q[6u + (i >> 2)], i & 3u);
    }
    static constexpr bool kUnsignedA = false;
    static constexpr int kHiShift = 0;
    __device__ static __forceinline__ void a_frag(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        a_regs(s, i, a0, a1, a2, a3);
    }
    __device__ static __forceinline__ void fold(const Stage& s, const float (&f)[4], float, float, float& acc_g,
                                                float& acc_g8) {
        const __half2 d0 = *reinterpret_cast<const __half2*>(&s.dd[0]);
        const __half2 d1 = *reinterpret_cast<const __half2*>(&s.dd[1]);
        acc_g += __low2float(d0) * f[0] + __high2float(d0) * f[1];
        acc_g8 += __low2float(d1) * f[2] + __high2float(d1) * f[3];
    }
};

// IQ4_XS repacked (kquant_more.cu): qs verbatim - per 32-weight block 16 bytes, byte j = code of
// element j (low nibble) and of element 16 + j (high nibble) - and a 24-byte record {f16 d, pad2,
// i8 ls - 32 [8], pad12}; w = d * (ls - 32) * book[code] with ggml's 16-entry signed code book.
// Lane t's 32 bytes of a row are blocks 2t (words 0..3) and 2t+1 (words 4..7), so mma i feeds ONE block:
// both halves of its k-slots (low nibbles = elements 4(i&3).., high nibbles = elements 16 + 4(i&3)..)
// belong to block 2t + i/4, and the kernel's B operand follows (kSplitBlock).  The codes become book
// values with byte permutes: per 16 bits of codes one permute over each half of the book, one that
// picks per byte by the code's top bit; two more put a word's low-nibble and high-nibble values in
// separate registers.
struct IQ4XS {
    static constexpr uint32_t kDepth = 2;
    static constexpr uint32_t kDataBytes = 128;
    static constexpr uint32_t kRecBytes = 24;
    static constexpr bool kSplitBlock = true;
    struct Stage {
        uint4 q[4];      // row g: bytes [32t, 32t+32); row g+8 likewise
        uint32_t d[2];   // f16 d of the two rows (low half)
        uint32_t ls[2];  // i8 ls' of blocks 2t, 2t+1 of the two rows (low two bytes)
    };
    template <bool kShared>
    __device__ static __forceinline__ void load(Stage& s, const uint8_t* d0, const uint8_t* d1, const uint8_t* r0,
                                                const uint8_t* r1, uint32_t t) {
        s.q[0] = ld16<kShared>(d0 + t * 32u);
        s.q[1] = ld16<kShared>(d0 + t * 32u + 16u);
        s.q[2] = ld16<kShared>(d1 + t * 32u);
        s.q[3] = ld16<kShared>(d1 + t * 32u + 16u);
        s.d[0] = ld2<kShared>(r0);
        s.d[1] = ld2<kShared>(r1);
        s.ls[0] = ld2<kShared>(r0 + 4u + 2u * t);
        s.ls[1] = ld2<kShared>(r1 + 4u + 2u * t);
    }
    __device__ static __forceinline__ uint32_t word(const uint4& v, uint32_t i) {
        return i == 0u ? v.x : i == 1u ? v.y : i == 2u ? v.z : v.w;
    }
    // four book values for the four codes in the low 16 bits of c (code j in bits 4j..4j+3 -> byte j)
    __device__ static __forceinline__ uint32_t book4(uint32_t c) {
        const uint32_t sel = c & 0x7777u;
        const uint32_t low = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);    // -127 -104 -83 -65 | -49 -35 -22 -10
        const uint32_t high = __byte_perm(0x26190D01u, 0x71594535u, sel);   //    1   13  25  38 |  53  69  89 113
        return __byte_perm(low, high, 0x3210u | ((c & 0x8888u) >> 1));
    }
    // a word of eight codes -> the values of its four low nibbles and of its four high nibbles
    __device__ static __forceinline__ void book8(uint32_t w, uint32_t& lo, uint32_t& hi) {
        const uint32_t r0 = book4(w), r1 = book4(w >> 16);   // codes (n0 n1 n2 n3), (n4 n5 n6 n7): low / high nibble alternate
        lo = __byte_perm(r0, r1, 0x6420u);
        hi = __byte_perm(r0, r1, 0x7531u);
    }
    __device__ static __forceinline__ void a_regs(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        book8(word(s.q[i >> 2], i & 3u), a0, a2);
        book8(word(s.q[2u + (i >> 2)], i & 3u), a1, a3);
    }
    static constexpr bool kUnsignedA = false;
    static constexpr int kHiShift = 0;
    __device__ static __forceinline__ void a_frag(const Stage& s, uint32_t i, uint32_t& a0, uint32_t& a1,
                                                  uint32_t& a2, uint32_t& a3) {
        a_regs(s, i, a0, a1, a2, a3);
    }
    __device__ static __forceinline__ void fold(const Stage& s, const float (&f)[4], float, float, float& acc_g,
                                                float& acc_g8) {
        const float d_g = __half2float(__ushort_as_half((unsigned short)s.d[0]));
        const float d_g8 = __half2float(__ushort_as_half((unsigned short)s.d[1]));
        acc_g += d_g * ((float)(int8_t)(s.ls[0] & 0xffu) * f[0] + (float)(int8_t)((s.ls[0] >> 8) & 0xffu) * f[1]);
        acc_g8 += d_g8 * ((float)(int8_t)(s.ls[1] & 0xffu) * f[2] + (float)(int8_t)((s.ls[1] >> 8) & 0xffu) * f[3]);
    }
};

// Row-sharded output: when n > 0 the kernel stores row r of its band at ptr[p][row0 + r] for
// every p < n - the full-length y of each rank, peer memory over NVLink included - instead of
// y[r].  Plain peer stores.  With signal == 0 the caller orders the stores itself.
// signal == 1: the kernel also tells every rank when its band is complete: its CTAs count
// themselves out on ctr[0] (this rank's memory, zero between launches) and the last one stores the
// step number into flag[p][rank] of every rank p, where a consumer waits for it
// (pdk_peer_flags_wait).  The step number is `step`, or, when that is 0, one more than the rank's
// own count ctr[1], which the kernel then advances - so that a captured launch can be replayed.
// signal == 2 (deferred): nothing is signalled at the end.  Instead thread 0 of CTA 0 stores, at
// the START of the launch and behind griddepcontrol.wait - when the previous kernel of the stream,
// peer stores included, is complete - the number of the PREVIOUS launch into the flags (one flag
// array and one counter shared by all y buffers of the loop, three or more), and checks before it
// leaves that every rank's previous step has arrived here.
struct PeerOut {
    float* ptr[8];
    uint32_t* flag[8];
    uint32_t* ctr;
    uint32_t n, row0, rank, step, signal;
};

// peer_signal: called by one thread of each CTA after a CTA-wide barrier that follows the CTA's last
// store (signal == 1).
//
// Cost: the system-scope fence waits until the peers have acknowledged this GPU's outstanding stores,
// one NVLink round trip at the end of the kernel, behind which the next kernel of the stream waits:
// 3.5 - 4 us per step at two GPUs (a second fence behind the flag stores cost another 2.4 us).  The
// deferred form pays none of it: stream order already puts the previous kernel's stores before the
// flag, and the step's arrival is observed one launch later.  acq_rel fences, not the sequentially
// consistent ones __threadfence*() give.
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void peer_signal(const PeerOut& po, unsigned int* err = nullptr) {
    if (po.n == 0u || po.signal != 1u) return;
    // Release at GPU scope: this CTA's stores (seen through the barrier) before the count.  Only the
    // last CTA pays for a system-scope fence - it has observed every other CTA's count, so its
    // fence covers their stores too (causality order is cumulative) - instead of every CTA waiting
    // for its own peer stores to be acknowledged over NVLink before it may even count itself out.
    fence_acq_rel_gpu();
    const uint32_t prev = atomicAdd(po.ctr, 1u);
    if (prev != gridDim.x - 1u) return;
    fence_acq_rel_gpu();                               // acquire: the other CTAs' stores
    po.ctr[0] = 0u;                                    // the next launch on this stream counts from zero
    uint32_t step = po.step;
    if (step == 0u) {
        step = po.ctr[1] + 1u;
        po.ctr[1] = step;
    }
    fence_acq_rel_sys();                               // every CTA's stores before the flags
#pragma unroll
    for (uint32_t p = 0; p < 8u; ++p)
        if (p < po.n) st_relaxed_sys(po.flag[p] + po.rank, step);
}


__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// signal == 2, thread 0 of CTA 0, behind griddepcontrol.wait: counts this launch and tells every rank
// that the previous launch's band is in place.  Returns this launch's number.
__device__ __forceinline__ uint32_t peer_post_previous(const PeerOut& po) {
    uint32_t step = po.step;
    if (step == 0u) step = po.ctr[1] + 1u;
    po.ctr[1] = step;
    if (step > 1u) {
#pragma unroll
        for (uint32_t p = 0; p < 8u; ++p)
            if (p < po.n) st_relaxed_sys(po.flag[p] + po.rank, step - 1u);
    }
    return step;
}
// signal == 2, the same thread before it leaves: every rank's previous step (flags >= step - 1) has
// arrived here, or - after a second - 0x1c << 8 | rank of a late one goes into the error word.
__device__ __forceinline__ void peer_check_previous(const PeerOut& po, uint32_t step, unsigned int* err) {
    if (step <= 1u || po.rank >= po.n) return;
    const uint32_t* mine = po.flag[po.rank];
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (uint32_t q = 0; q < po.n; ++q) {
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(mine + q) - (step - 1u)) < 0) {
            if ((++spins & 31u) != 0u) continue;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
            if (t1 - t0 > 1000000000ull) {
                if (err != nullptr) atomicOr(err, (0x1cu << 8) | q);
                break;
            }
        }
    }
}

// Activations -> block floating point limbs: per 32-element block a power-of-two step and 15-bit
// integers kept as two int8 limbs, v = 256 * hi + lo (xs_hi, xs_lo: int8 [in_dim]), and
// xmeta[block] = {step, step * sum of the block's integers}.  x f32 [in_dim], or int8 xq with one
// f32 scale per 32.  A thread handles groups of 8 elements; the 4 lanes of a block agree on the
// step through two shuffles, so whole warps must call with consecutive groups.
//
// limb_load8: the group's 8 values; limb_store8: their limbs and the block's meta entry.
__device__ __forceinline__ void limb_load8(const float* __restrict__ x, const int8_t* __restrict__ xq,
                                           const float* __restrict__ xq_scale, uint32_t grp, float (&v)[8]) {
    if (xq == nullptr) {
        const float4 a = *reinterpret_cast<const float4*>(x + grp * 8u);
        const float4 b = *reinterpret_cast<const float4*>(x + grp * 8u + 4u);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        // int8 activations with one f32 scale per 32 (the W4A8 slots' operands)
        const int2 q = *reinterpret_cast<const int2*>(xq + grp * 8u);
        const float s = xq_scale[grp >> 2];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)(int8_t)((i < 4 ? q.x >> (8 * i) : q.y >> (8 * (i - 4))) & 0xff) * s;
    }
}
__device__ __forceinline__ void limb_store8(const float (&v)[8], uint32_t grp, uint8_t* xs_hi, uint8_t* xs_lo,
                                            float2* xmeta) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // amax < 2^ex  ->  step 2^(ex-14) keeps |v| <= 2^14 (no clamp needed: |x| <= amax; an infinite or
    // NaN block gets inv = 0 and all-zero limbs)
    float step = 1.0f, inv = 0.0f;
    if (amax > 0.0f && amax < 3.0e38f) {
        // frexp's exponent from the bits (denormals land on the clamp), powers of two built in place
        const int ex = max((int)(__float_as_uint(amax) >> 23) - 126, -110);
        step = __uint_as_float((uint32_t)(ex + 113) << 23);
        inv = __uint_as_float((uint32_t)(141 - ex) << 23);
    }
    // lo limb = the integer's low byte (two's complement), hi limb = byte 1 of (q + 128): then
    // q = 256 * hi + lo with lo in [-128, 127]; four of each are gathered with byte permutes
    int q[8], r[8], isum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = __float2int_rn(v[i] * inv);
        r[i] = q[i] + 128;
        isum += q[i];
    }
    uint2 lo, hi;
    lo.x = __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
    lo.y = __byte_perm(__byte_perm(q[4], q[5], 0x0040), __byte_perm(q[6], q[7], 0x0040), 0x5410);
    hi.x = __byte_perm(__byte_perm(r[0], r[1], 0x0051), __byte_perm(r[2], r[3], 0x0051), 0x5410);
    hi.y = __byte_perm(__byte_perm(r[4], r[5], 0x0051), __byte_perm(r[6], r[7], 0x0051), 0x5410);
    *reinterpret_cast<uint2*>(xs_hi + (size_t)grp * 8u) = hi;
    *reinterpret_cast<uint2*>(xs_lo + (size_t)grp * 8u) = lo;
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    if ((grp & 3u) == 0u) xmeta[grp >> 2] = make_float2(step, step * (float)isum);
}

// All of x by `nthreads` threads of a CTA (whole warps), plus the 32-byte zero line.
__device__ __forceinline__ void act_limbs(const float* __restrict__ x, const int8_t* __restrict__ xq,
                                          const float* __restrict__ xq_scale, uint32_t in_dim, uint8_t* xs_hi,
                                          uint8_t* xs_lo, uint8_t* zeros, float2* xmeta, uint32_t tid,
                                          uint32_t nthreads) {
    const uint32_t groups = in_dim >> 3;
    for (uint32_t grp = tid; grp < groups; grp += nthreads) {
        float v[8];
        limb_load8(x, xq, xq_scale, grp, v);
        limb_store8(v, grp, xs_hi, xs_lo, xmeta);
    }
    if (tid < 8u) reinterpret_cast<uint32_t*>(zeros)[tid] = 0u;
}

}  // namespace gemv_i8
