// moe_route.cuh - the top-k router of one token as a warp routine, shared by the routing kernel
// (moe_route.cu) and the fused decode-width front of the tensor-core MoE path (moe_tc5.cu).
#pragma once
#include "pdk_common.cuh"

namespace moe_route {

// One warp per token, up to 512 experts (16 per lane), k <= 16.  The selection rule - largest
// logit + bias first, equal values to the lower expert index - is folded into one unsigned
// 64-bit sort key per expert: the float's bits mapped so that unsigned order equals float order
// in the high word, the complemented expert index in the low word.  A round is then a plain
// 64-bit maximum over the warp; the winner's lane marks its slot as taken in a bit mask.
// Key 0 stands for "no expert" (every real key has a non-zero high word).
__device__ __forceinline__ uint64_t topk_key(float value, uint32_t expert) {
    const uint32_t bits = __float_as_uint(value + 0.0f);                    // -0 joins +0, as float compare has it
    const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return ((uint64_t)ordered << 32) | (uint64_t)(0xffffffffu - expert);
}
__device__ __forceinline__ float topk_key_value(uint64_t key) {
    const uint32_t ordered = (uint32_t)(key >> 32);
    return __uint_as_float((ordered & 0x80000000u) ? (ordered & 0x7fffffffu) : ~ordered);
}

// One warp routes one token: idx[r] / w[r] (r < k) receive the r-th pick and its softmax weight.
__device__ __forceinline__ void topk_warp(const float* __restrict__ scores, const float* __restrict__ bias,
                                          uint32_t n_expert, uint32_t k, uint32_t lane, uint32_t* idx, float* w) {
    uint64_t key[16];
#pragma unroll
    for (uint32_t j = 0; j < 16u; ++j) {
        const uint32_t expert = 32u * j + lane;
        key[j] = expert < n_expert ? topk_key(scores[expert] + (bias ? bias[expert] : 0.0f), expert) : 0ull;
    }
    uint32_t taken = 0;      // bit j: this lane's j-th expert has been selected
    float picked = 0.0f;     // lane r keeps the value of the r-th pick
    for (uint32_t round = 0; round < k; ++round) {
        uint64_t top = 0ull;
#pragma unroll
        for (uint32_t j = 0; j < 16u; ++j)
            if (!((taken >> j) & 1u) && key[j] > top) top = key[j];
#pragma unroll
        for (uint32_t step = 1; step < 32u; step <<= 1) {
            const uint64_t other = __shfl_xor_sync(0xffffffffu, top, step);
            top = other > top ? other : top;
        }
        const uint32_t expert = 0xffffffffu - (uint32_t)top;
        if ((expert & 31u) == lane) taken |= 1u << (expert >> 5);
        if (lane == round) picked = topk_key_value(top);
        if (lane == 0) idx[round] = expert;
    }
    // softmax over the k picks; lane 0 holds the largest, the sum runs in pick order as a scalar walk would
    const float peak = __shfl_sync(0xffffffffu, picked, 0);
    const float e = lane < k ? __expf(picked - peak) : 0.0f;
    float sum = 0.0f;
    for (uint32_t r = 0; r < k; ++r) sum += __shfl_sync(0xffffffffu, e, r);
    if (lane < k) w[lane] = e / sum;
}

}  // namespace moe_route
