// tc5.cuh - sm_100a building blocks shared by the tcgen05 GEMMs: mbarriers with
// bounded waits, TMA tensor maps and loads, tensor-memory allocation, UMMA
// descriptors, MMA issue / commit and TMEM loads.
//
// Every wait in here is bounded: a wait that has not succeeded after
// kWaitBudgetNs records a code in the device error word and returns false, and
// the kernels built on it then leave their loops, free their tensor memory and
// exit.  Nothing spins forever and nothing traps.
#pragma once
#include <cuda.h>

#include "pdk_common.cuh"

// Device error word: 0 = no error.  Kernels OR in (code << 8 | detail); the host
// reads it through pdk_device_error().  Launchers pass its device address
// (pdk_error_word(), resolved once per device) to the kernels.
unsigned int* pdk_error_word();

namespace tc5 {

constexpr unsigned long long kWaitBudgetNs = 1000000000ull;  // 1 s per wait

enum ErrCode : unsigned int {
    kErrFullWait = 1,      // MMA warp: TMA data never arrived
    kErrEmptyWait = 2,     // producer: smem stage never released
    kErrTmemFullWait = 3,  // epilogue: accumulator never completed
    kErrTmemEmptyWait = 4, // MMA warp: accumulator never drained
    kErrTestWait = 5       // self-test: a barrier nothing arrives on
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

struct WaitCtx {
    volatile int* abort_flag;  // shared-memory flag: one role gave up, the others leave too
    unsigned int* err;         // device error word
};

__device__ __forceinline__ void report(unsigned int* err, unsigned int code, unsigned int detail) {
    atomicOr(err, (code << 8) | (detail & 0xffu));
}

// ---- mbarrier --------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: true when the phase completed; false after the budget (the
// caller must then abandon its loop).  `abort_flag` lets the other roles of the
// CTA leave early once one of them has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, unsigned int code,
                                          unsigned int detail, unsigned long long budget_ns = kWaitBudgetNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u) {
            if (*ctx.abort_flag) return false;
            if (globaltimer_ns() - t0 > budget_ns) {
                *ctx.abort_flag = 1;
                report(ctx.err, code, detail);
                return false;
            }
        }
    }
    return true;
}

// ---- TMA -------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 2-D tiled load: x = innermost (byte) coordinate, y = row.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t x,
                                            int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// ---- issue from a converged warp ---------------------------------------------
// The *_elect forms are called by all 32 lanes of a converged warp; elect.sync
// picks one lane (the same one every time) to issue.  Keeping the issuing warp
// converged lets addresses and descriptors live in uniform registers: issued
// from inside an `if (lane == 0)` branch, every tcgen05 / TMA instruction cost
// about 60 cycles of issue time.
#define TC5_ELECT "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
__device__ __forceinline__ void mbar_arrive_expect_tx_elect(uint64_t* bar, uint32_t bytes) {
    asm volatile(TC5_ELECT "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d_elect(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t x,
                                                  int32_t y) {
    asm volatile(TC5_ELECT
                 "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
                 "[%2];\n\t}" ::"r"(smem_u32(smem_dst)),
                 "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// The same with an L2 eviction-priority hint (a createpolicy value): evict_first for planes that are
// streamed once per launch.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint_elect(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t x,
                                                       int32_t y, uint64_t policy) {
    asm volatile(TC5_ELECT
                 "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], "
                 "[%1, {%3, %4}], [%2], %5;\n\t}" ::"r"(smem_u32(smem_dst)),
                 "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void bulk_load_elect(void* smem_dst, const void* gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(TC5_ELECT
                 "@e cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 2-D tiled store of a dense (unswizzled) shared-memory box; rows / columns past the tensor's
// extent are clipped by the hardware.  One thread issues; tma_store_wait_read() before the box
// is overwritten.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(m),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// all but the newest store have read their boxes (two boxes written in turn)
__device__ __forceinline__ void tma_store_wait_read1() {
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tensor memory -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- descriptors ---------------------------------------------------------------
// Shared-memory operand descriptor, K-major tile with 128-byte rows written by
// a SWIZZLE_128B tensor map: start address and offsets in 16-byte units,
// stride between 8-row groups 1024 bytes, descriptor version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)1u << 16) | ((uint64_t)64u << 32) | ((uint64_t)1u << 46) |
           ((uint64_t)2u << 61);
}
// Instruction descriptor for kind::f8f6f4 / kind::f16: D = f32, both operands
// K-major.  fmt: f8f6f4 0 = e4m3, 1 = e5m2, 5 = e2m1; f16 kind 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t idesc_f32acc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA issue (one thread) ------------------------------------------------------
__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every MMA this thread has issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_f8f6f4_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(TC5_ELECT
                 ".reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Four MMAs over the four 32-byte K steps of one 128-byte swizzled row, issued by the lane one
// elect.sync picks, the descriptors stepped inside the asm block: 3 + 4 * 3 instructions per
// group.  A loop of single-MMA wrappers, each with its own election and predicate set-up, costs
// the issuing warp more than the 128 cycles the tensor core needs per M128 N256 MMA.
// acc_first: whether the first of the four accumulates (the other three always do).
#define TC5_MMA_X4(KIND_STR)                                                                  \
    asm volatile(                                                                             \
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 a, b;\n\t"                                     \
        "elect.sync _|e, 0xffffffff;\n\t"                                                     \
        "setp.ne.b32 p, %4, 0;\n\t"                                                           \
        "setp.eq.b32 q, 0, 0;\n\t"                                                            \
        "@e tcgen05.mma.cta_group::1.kind::" KIND_STR " [%0], %1, %2, %3, p;\n\t"             \
        "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"                                          \
        "@e tcgen05.mma.cta_group::1.kind::" KIND_STR " [%0], a, b, %3, q;\n\t"               \
        "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"                                          \
        "@e tcgen05.mma.cta_group::1.kind::" KIND_STR " [%0], a, b, %3, q;\n\t"               \
        "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"                                          \
        "@e tcgen05.mma.cta_group::1.kind::" KIND_STR " [%0], a, b, %3, q;\n\t}" ::"r"(d_tmem), \
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first)                                  \
        : "memory")
__device__ __forceinline__ void mma_f8f6f4_x4_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t acc_first) {
    TC5_MMA_X4("f8f6f4");
}
__device__ __forceinline__ void mma_f16_x4_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t acc_first) {
    TC5_MMA_X4("f16");
}
__device__ __forceinline__ void mma_commit_elect(uint64_t* bar) {
    asm volatile(TC5_ELECT "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// ---- TMEM -> registers: 32 lanes x 32 columns of 32 bits per warp ------------------
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- pairs of CTAs (tcgen05 cta_group::2) -----------------------------------------
// Two CTAs of a cluster drive one MMA: the leader (cluster rank 0) issues, each CTA's tensor core
// reads A and its half of B from its own shared memory and the other half of B from its partner's.
namespace pair {
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;   // a shared::cluster address with the pair's rank bit cleared: the leader's copy

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// one full warp of each CTA of the pair, the same warp index in both
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose bytes are counted on the leader's barrier
__device__ __forceinline__ void tma_load_2d_pair_elect(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t x, int32_t y) {
    asm volatile(TC5_ELECT
                 "@e cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];\n\t}" ::"r"(smem_u32(smem_dst)),
                 "l"(m), "r"(smem_u32(bar) & kPeerMask), "r"(x), "r"(y)
                 : "memory");
}
// four MMAs over the four 32-byte K steps of a stage, both CTAs' tensor cores
__device__ __forceinline__ void mma_f8f6f4_x4_pair_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                         uint32_t acc_first) {
    asm volatile(
        "{\n\t.reg .pred e, p, q;\n\t.reg .b64 a, b;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t"
        "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t"
        "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], a, b, %3, q;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first)
        : "memory");
}
// arrive on the barrier at this offset in BOTH CTAs once the MMAs issued so far are complete
__device__ __forceinline__ void mma_commit_pair_elect(uint64_t* bar) {
    asm volatile(TC5_ELECT
                 ".reg .b16 mask;\n\tmov.b16 mask, 3;\n\t"
                 "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], mask;\n\t}" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
// arrive on the leader's copy of a barrier (for the leader: its own)
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask) : "memory");
}

}  // namespace pair

}  // namespace tc5

// Host: 2-D byte/element tensor map with 128-byte-swizzled boxes.
//   inner  = innermost extent in elements, rows = outer extent,
//   pitch  = bytes between rows (multiple of 16), box = {inner elements, rows}.
// Returns 0 or a cudaError_t.
int pdk_make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                     uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows);
// The same without swizzle (dense boxes, for stores): box_inner up to 256 elements.
int pdk_make_tmap_2d_dense(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                           uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows);
