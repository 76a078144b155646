// exports.cu - the two symbols a kernel pack exports, and the slot table.
#include "pdk_common.cuh"

static_assert(sizeof(PdkPackInfo) == 36, "PackInfo layout");
static_assert(sizeof(PdkKernelTableV1) == PDK_TABLE_BYTES, "KernelTableV1 is 8 + 953 * 8 bytes");

int pdk_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- per-(device, stream) scratch slices (pdk_common.cuh)
#include <mutex>
namespace {
std::mutex g_slice_mu;
PdkSliceTable* g_slice_tables = nullptr;
}  // namespace

PdkSliceTable::PdkSliceTable(void* (*r)(), size_t bytes, int n)
    : resolve(r), slice_bytes(bytes), lanes(n < kMaxLanes ? n : kMaxLanes), base{}, owner{}, used{}, next(nullptr) {
    std::lock_guard<std::mutex> lock(g_slice_mu);
    next = g_slice_tables;
    g_slice_tables = this;
}

uint8_t* PdkSliceTable::slice(cudaStream_t st) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lock(g_slice_mu);
    if (base[dev] == nullptr) {
        base[dev] = (uint8_t*)resolve();
        if (base[dev] == nullptr) return nullptr;
    }
    int free_lane = -1;
    for (int i = 0; i < lanes; ++i) {
        if (used[dev][i] && owner[dev][i] == st) return base[dev] + (size_t)i * slice_bytes;
        if (!used[dev][i] && free_lane < 0) free_lane = i;
    }
    if (free_lane < 0) return nullptr;
    used[dev][free_lane] = true;
    owner[dev][free_lane] = st;
    return base[dev] + (size_t)free_lane * slice_bytes;
}

// No counterpart in the reference.  The small-batch k-quant GEMMs, the NVFP4 W4A16 GEMV and the
// prefill-width NVFP4 GEMM keep per-call scratch in the library, one slice per (device, stream),
// two streams per device.  A caller that destroys a stream calls this first (current device =
// the stream's) so that a later stream can take the slices over; the stream must be idle.
PDK_EXPORT void pdk_stream_release(void* stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PdkSliceTable::kMaxDev) return;
    std::lock_guard<std::mutex> lock(g_slice_mu);
    for (PdkSliceTable* t = g_slice_tables; t != nullptr; t = t->next)
        for (int i = 0; i < t->lanes; ++i)
            if (t->used[dev][i] && t->owner[dev][i] == (cudaStream_t)stream) t->used[dev][i] = false;
}

static const PdkPackInfo g_info = {
    PDK_PACK_MAGIC, PDK_PACK_ABI_VERSION, {'c', 'u', 'd', 'a', '-', 's', 'm', '1', '0', '0', 'a', 0, 0, 0, 0, 0},
    {0u, 1u, 0u}};

static PdkKernelTableV1 g_table;

// Every kernel of this library is built for sm_100a alone, and such code loads only on a device
// of compute capability 10.0 exactly (a 10.3 or 12.x die rejects it at the first launch).  So the
// table is resolved against the device, as packs/cuda/src/exports.cuh:2118-2400 does for its
// block-scale families: any other capability gets an empty table and the engine reports every
// operator as missing at load time instead of failing at the first call.
static void fill_table_for(PdkKernelTableV1& g_table, int cc_major, int cc_minor) {
    memset(&g_table, 0, sizeof(g_table));
    g_table.size = PDK_TABLE_BYTES;
    g_table.reserved = 0;
    if (cc_major != 10 || cc_minor != 0) return;
#define PDK_SET(name) g_table.slot[PDK_SLOT_##name] = (void*)&pd_##name
    PDK_SET(mxfp4_dequant_f32);
    PDK_SET(q8_0_dequant_f32);
    PDK_SET(add_inplace_f32);
    PDK_SET(mxfp4_repack);
    PDK_SET(q8_0_repack);
    PDK_SET(q8_0_gemv_repacked);
    PDK_SET(q8_0_gemm_repacked);
    PDK_SET(kquant_dequant);
    PDK_SET(kquant_repack);
    PDK_SET(kquant_gemv);
    PDK_SET(quantize_e4m3_row);
    PDK_SET(f8row_gemm);
    PDK_SET(bf16_to_f8row);
    PDK_SET(f8row_gemm_tc5x);
    PDK_SET(quantize_nvf4);
    PDK_SET(add_rmsnorm_quant_nvf4_batch);
    PDK_SET(add_rmsnorm_nvf4_batch);
    PDK_SET(quantize_nvf4_swiglu);
    PDK_SET(swiglu_fused_nvf4);
    PDK_SET(swiglu_quant_e4m3_row);
    PDK_SET(rmsnorm_quant_e4m3_row);
    PDK_SET(add_rmsnorm_scaled_quant_e4m3_row);
    PDK_SET(nvf4_dequant);
    PDK_SET(nvf4_gemv);
    PDK_SET(nvf4_gemm_tc5w);
    PDK_SET(nvf4_tc5_tile_scales);
    PDK_SET(moe_topk_batch);
    PDK_SET(moe_align);
    PDK_SET(moe_align_bm);
    PDK_SET(moe_slot_combine);
    PDK_SET(quantize_q8);
    PDK_SET(quantize_q8_sums);
    PDK_SET(kquant_gemv_w4a8);
    PDK_SET(kquant_gemm_mma_ks);
    PDK_SET(kquant_gemm_w4a8_sb);
    PDK_SET(mxfp4_gu_interleave);
    PDK_SET(mxfp4_moe_gate_up_mmq);
    PDK_SET(mxfp4_moe_down_mmq);
    PDK_SET(mxfp4_moe_gate_up_dp4a_b);
    PDK_SET(mxfp4_moe_down_dp4a_b);
#undef PDK_SET
}

// Resolution uses the device that is current at the first fetch (the engine binds its device
// before it loads a pack, loader.rs:253-283).  Without a device to ask (no driver, no GPU) the
// table is left as built: nothing can launch there anyway and every launcher returns the error.
static void fill_table() {
    int dev = 0, major = 10, minor = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        int a = 0, b = 0;
        if (cudaDeviceGetAttribute(&a, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&b, cudaDevAttrComputeCapabilityMinor, dev) == cudaSuccess) {
            major = a;
            minor = b;
        }
    }
    (void)cudaGetLastError();
    fill_table_for(g_table, major, minor);
}

PDK_EXPORT const PdkPackInfo* paddock_pack_info(void) { return &g_info; }

PDK_EXPORT const PdkKernelTableV1* paddock_pack_kernels_v1(void) {
    static const bool once = (fill_table(), true);
    (void)once;
    return &g_table;
}

// Diagnostics: the table as it would be resolved on a device of the given compute capability,
// written to caller storage of PDK_TABLE_BYTES bytes.
PDK_EXPORT int pdk_kernels_for_cc(int cc_major, int cc_minor, PdkKernelTableV1* out) {
    if (out == nullptr) return 1;
    fill_table_for(*out, cc_major, cc_minor);
    return 0;
}
