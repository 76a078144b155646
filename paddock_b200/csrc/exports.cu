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

static const PdkPackInfo g_info = {
    PDK_PACK_MAGIC, PDK_PACK_ABI_VERSION, {'c', 'u', 'd', 'a', '-', 's', 'm', '1', '0', '0', 'a', 0, 0, 0, 0, 0},
    {0u, 1u, 0u}};

static PdkKernelTableV1 g_table;

static void fill_table() {
    g_table.size = PDK_TABLE_BYTES;
    g_table.reserved = 0;
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
#undef PDK_SET
}

PDK_EXPORT const PdkPackInfo* paddock_pack_info(void) { return &g_info; }

PDK_EXPORT const PdkKernelTableV1* paddock_pack_kernels_v1(void) {
    static const bool once = (fill_table(), true);
    (void)once;
    return &g_table;
}
