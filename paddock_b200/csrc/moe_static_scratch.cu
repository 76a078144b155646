// moe_static_scratch.cu - the MoE down projection + slot combine for callers that
// cannot allocate device memory.
//
// pdk_mxfp4_moe_down needs a per-(token, slot) partial buffer between the expert
// GEMM and the fixed-order combine.  Normally the caller allocates it.  Some
// callers cannot: code that runs where cudaMalloc is off limits (a latency-
// critical serving loop that must never take the allocator's lock or trigger an
// implicit device synchronization, a plug-in that is handed pointers by a host
// it may not ask for more memory, a process whose memory budget is fixed at
// start-up).  For them this file keeps the partial buffer in a file-scope
// __device__ array that lives in the library image: every GPU that loads the
// library holds kStaticPartFloats * 4 bytes (1 MiB) for it until the process
// exits, and the entry point below allocates nothing.
#include <cstdio>

#include "pdk_common.cuh"

// 64 (token, slot) pairs of 4096 channels, e.g. 16 tokens x top-4 x embd 4096
constexpr size_t kStaticPartFloats = 64u * 4096u;
static __device__ __align__(256) float g_static_part[kStaticPartFloats];

static thread_local char t_refusal[160] = "";

// Device address of g_static_part on the current device.  In host code the name
// g_static_part is only a handle for the runtime, not a device address, so it is
// resolved with cudaGetSymbolAddress once per device, with that device current.
static float* static_part_ptr(int* rc) {
    static float* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
    if (dev < 0 || dev >= 64) { *rc = cudaErrorInvalidDevice; return nullptr; }
    if (!cached[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_part);
        if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
        cached[dev] = p;
    }
    *rc = 0;
    return cached[dev];
}

// Largest rows * n_active * embd the static buffer holds.
PDK_EXPORT uint64_t pdk_static_part_capacity(void) { return (uint64_t)kStaticPartFloats; }

// Reason of the last refusal of pdk_mxfp4_moe_down_combine_static on this thread ("" if none).
PDK_EXPORT const char* pdk_static_last_refusal(void) { return t_refusal; }

// residual[t] += sum over slots of topk_w * (W_down h + bias): pdk_mxfp4_moe_down
// followed by pd_moe_slot_combine, with the partial buffer in the library's
// static device array instead of caller memory.
//  - Allocates nothing (no cudaMalloc / cudaFree, no allocating library call).
//  - rows * n_active * embd must not exceed pdk_static_part_capacity(); a larger
//    request is refused with cudaErrorInvalidValue and pdk_static_last_refusal()
//    says why.
//  - The first call on a device resolves the array's device address
//    (cudaGetSymbolAddress).  Make that first call outside any stream capture.
//  - Every call on a device shares the one array and finds the previous call's
//    contents in it; the region a call uses is cleared first.  Two calls that
//    overlap on the GPU (different streams, no ordering between them) race on
//    it: serialize them.
PDK_EXPORT int pdk_mxfp4_moe_down_combine_static(const void* down_data, const void* down_scale,
                                                 const void* down_bias, const void* sorted_row,
                                                 const void* sorted_slot, const void* block_expert,
                                                 const void* topk_w, const void* hq, const void* hscale,
                                                 void* residual, uint32_t ff, uint32_t embd, uint32_t n_active,
                                                 uint32_t rows, uint32_t bm, uint32_t max_blocks, void* stream) {
    t_refusal[0] = 0;
    if (rows == 0 || embd == 0 || n_active == 0 || max_blocks == 0) return 0;
    // three 32-bit factors can pass 2^64: compare stepwise, so a wrapped product never slips through
    const uint64_t pairs = (uint64_t)rows * n_active;
    const uint64_t need = pairs <= kStaticPartFloats ? pairs * embd : ~0ull;
    if (need > kStaticPartFloats) {
        snprintf(t_refusal, sizeof(t_refusal),
                 "rows*n_active*embd = %llu floats exceeds the static partial buffer of %llu floats",
                 (unsigned long long)need, (unsigned long long)kStaticPartFloats);
        return cudaErrorInvalidValue;
    }
    int rc = 0;
    float* part = static_part_ptr(&rc);
    if (!part) {
        snprintf(t_refusal, sizeof(t_refusal), "cudaGetSymbolAddress for the static partial buffer failed (%d)", rc);
        return rc;
    }
    cudaError_t e = cudaMemsetAsync(part, 0, need * sizeof(float), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    rc = pdk_mxfp4_moe_down(down_data, down_scale, down_bias, sorted_row, sorted_slot, block_expert, topk_w, hq,
                            hscale, part, ff, embd, n_active, bm, max_blocks, stream);
    if (rc != 0) return rc;
    return pd_moe_slot_combine(part, residual, embd, n_active, rows, stream);
}
