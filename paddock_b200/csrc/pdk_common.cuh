// pdk_common.cuh - helpers shared by every translation unit of the pack.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/paddock_pack.h"

#define PDK_EXPORT extern "C" __attribute__((visibility("default")))

// 0 or the raw cudaError_t of the launch just issued (the reference's
// launchers return the same, packs/cuda/src/gemm/f32_qkv.cuh:7).
static inline int pdk_launch_status() { return (int)cudaGetLastError(); }

static inline bool pdk_aligned(const void* p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Number of SMs of the current device, read once per process per device.
int pdk_sm_count();

// Programmatic dependent launch (the reference chains its decode kernels the
// same way, packs/cuda/src/abi.cuh:4560-4590): the kernel may start while its
// predecessor in the stream drains.  Kernels launched through this call
// griddepcontrol.launch_dependents early and griddepcontrol.wait before they
// touch anything the predecessor may still read or write.  PDK_NO_PDL=1 (read
// once) launches them as ordinary kernels.
#include <cstdlib>
static inline bool pdk_pdl_enabled() {
    static const bool v = [] {
        const char* e = getenv("PDK_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return v;
}
template <class... KArgs, class... Args>
static inline int pdk_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdk_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    return e == cudaSuccess ? pdk_launch_status() : (int)e;
}
__device__ __forceinline__ void pdk_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdk_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float pdk_warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// 16-byte streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 pdk_ldg_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
// (a & m) | o in one LOP3.  `o` must live in a register: callers pass a value
// that comes in as a kernel argument so it is not folded into a second immediate.
__device__ __forceinline__ uint32_t pdk_and_or(uint32_t a, uint32_t m, uint32_t o) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(m), "r"(o));
    return d;
}

// ---------------------------------------------------------------------------
// Library-resident scratch, one slice per (device, stream).
//
// A few launchers keep per-call scratch in `static __device__` arrays (the pack allocates
// nothing).  Calls on different streams can overlap on the GPU, so every (device, stream) pair
// that makes such a call gets a slice of its own, up to the array's lane count per device;
// further streams get nullptr and the caller takes its scratch-free route.  The table is shared
// by host threads (a mutex guards it), the array's device address is resolved per device, and
// pdk_stream_release() gives the slices of a stream that is about to be destroyed back.
// ---------------------------------------------------------------------------
struct PdkSliceTable {
    static constexpr int kMaxDev = 64, kMaxLanes = 4;
    void* (*resolve)();        // device address of the array on the current device, or nullptr
    size_t slice_bytes;
    int lanes;                 // <= kMaxLanes
    uint8_t* base[kMaxDev];
    cudaStream_t owner[kMaxDev][kMaxLanes];
    bool used[kMaxDev][kMaxLanes];
    PdkSliceTable* next;       // registry walked by pdk_stream_release
    PdkSliceTable(void* (*r)(), size_t bytes, int n);
    uint8_t* slice(cudaStream_t st);
};
#define PDK_SLICE_TABLE(name, symbol, bytes, n)                                             \
    static void* name##_resolve() {                                                         \
        void* p = nullptr;                                                                  \
        return cudaGetSymbolAddress(&p, symbol) == cudaSuccess ? p : nullptr;               \
    }                                                                                       \
    static PdkSliceTable name(name##_resolve, bytes, n)

__device__ __forceinline__ uint2 pdk_ldg_stream8(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t pdk_ldg_stream4(const void* p) {
    uint32_t r;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
