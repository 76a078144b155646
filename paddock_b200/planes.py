"""Device planes and operator calls, named after the reference's operator API
(crates/paddock-engine/src/gpu: types.rs plane structs, upload.rs / kquant.rs /
q8_gemm.rs wrappers).  Buffers are torch tensors (torch is the allocator and
stream owner here, as cudarc is for the reference); every compute call goes
through the C ABI of libpaddock_b200.so on the current torch stream.
"""
from dataclasses import dataclass

import torch

from .pack import KernelPack

GGML_Q8_0 = 8
GGML_Q4_K = 12


def _stream():
    return torch.cuda.current_stream().cuda_stream


@dataclass
class RepackedQ8:
    """types.rs:482-487: int8 data [out][in] + f16 scale [out][in/32]; dims = (in, out)."""
    data: torch.Tensor
    scale: torch.Tensor
    dims: tuple


@dataclass
class RepackedKQ:
    """types.rs:268-281: k-quant data + 24-byte scale records; dims = (in, out)."""
    data: torch.Tensor
    scales: torch.Tensor
    dims: tuple
    ty: int


class GpuExecutor:
    """The subset of crates/paddock-engine/src/gpu/mod.rs:143-252 that drives the
    quantized linear layer.  Method names and argument meaning follow the Rust
    wrappers; a NULL slot raises MissingOp, a refused launch raises LaunchError."""

    def __init__(self, pack=None, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("paddock_b200 needs a CUDA device: there is no CPU path")
        self.pack = pack or KernelPack.load()
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)

    # -- upload / repack (gpu/upload.rs:305-353, gpu/kquant.rs:284-374) --------
    def upload_raw(self, host_bytes):
        """Raw GGUF tensor bytes (a pinned or pageable uint8 tensor) -> device."""
        return host_bytes.to(self.device, non_blocking=True)

    def repack_q8_blocks(self, raw_dev, in_dim, out_dim):
        n_blocks = in_dim * out_dim // 32
        data = torch.empty(n_blocks * 32, dtype=torch.int8, device=self.device)
        scale = torch.empty(n_blocks, dtype=torch.float16, device=self.device)
        self.pack.call("q8_0_repack", raw_dev, data, scale, n_blocks, stream=_stream())
        return RepackedQ8(data, scale, (in_dim, out_dim))

    def repack_kquant_raw(self, raw_dev, in_dim, out_dim, ty=GGML_Q4_K):
        n_super = in_dim * out_dim // 256
        data = torch.empty(n_super * 128, dtype=torch.uint8, device=self.device)
        scales = torch.empty(n_super * 24, dtype=torch.uint8, device=self.device)
        self.pack.call("kquant_repack", raw_dev, data, scales, n_super, ty, stream=_stream())
        return RepackedKQ(data, scales, (in_dim, out_dim), ty)

    # -- linear calls (gpu/q8_gemm.rs:11-47, gpu/kquant.rs:499-528) --------------
    def q8_0_gemv_repacked(self, w, bias, x, y):
        self.pack.call("q8_0_gemv_repacked", w.data, w.scale, bias, x, y, w.dims[0], w.dims[1], stream=_stream())

    def q8_0_gemm_repacked(self, w, bias, x, y, batch):
        self.pack.call("q8_0_gemm_repacked", w.data, w.scale, bias, x, y, w.dims[0], w.dims[1], batch,
                       stream=_stream())

    def kquant_gemv(self, w, x, y):
        self.pack.call("kquant_gemv", w.data, w.scales, x, y, w.dims[0], w.dims[1], w.ty, stream=_stream())

    def kquant_gemm_f32(self, w, x, y, batch):
        self.pack.call("pdk_kquant_gemm_f32", w.data, w.scales, x, y, w.dims[0], w.dims[1], batch, w.ty,
                       stream=_stream())


@dataclass
class RepackedMxfp4:
    """types.rs:111-127: 16-byte nibble blocks + 1-byte E8M0 scales."""
    data: torch.Tensor
    scale: torch.Tensor


@dataclass
class MoeMxfp4Planes:
    """One MoE layer's expert planes (gate / up: [expert][ff][embd], down: [expert][embd][ff])
    and optional f32 biases ([expert][ff] / [expert][embd])."""
    gate: RepackedMxfp4
    up: RepackedMxfp4
    down: RepackedMxfp4
    n_expert: int
    embd: int
    ff: int
    gate_bias: torch.Tensor = None
    up_bias: torch.Tensor = None
    down_bias: torch.Tensor = None
    tc5: dict = None  # per plane name: (tiled UE4M3 scale records, meta) from prepare_tc5()


def prepare_tc5(ex, planes):
    """Load-time step of the tensor-core expert path: tile each plane's E8M0 scales into UE4M3
    scale records (pdk_mxfp4_tc5_tile_scales).  Costs 1/8 of the scale plane's bytes again."""
    if planes.tc5 is not None:
        return planes
    out = {}
    for name, rows, k in (("gate", planes.ff, planes.embd), ("up", planes.ff, planes.embd),
                          ("down", planes.embd, planes.ff)):
        n_bytes = planes.n_expert * ((rows + 127) // 128) * ((k + 255) // 256) * 2048
        tiled = torch.empty(n_bytes, dtype=torch.uint8, device=ex.device)
        meta = torch.zeros(2, dtype=torch.int32, device=ex.device)
        ex.pack.call("pdk_mxfp4_tc5_tile_scales", getattr(planes, name).scale, tiled, meta, rows, k, planes.n_expert,
                     stream=_stream())
        out[name] = (tiled, meta)
    planes.tc5 = out
    return planes


def repack_mxfp4(ex, raw_dev):
    """gpu/moe_mxfp4.rs:908-936: raw 17-byte blocks -> data + scale planes."""
    n_blocks = raw_dev.numel() // 17
    data = torch.empty(n_blocks * 16, dtype=torch.uint8, device=ex.device)
    scale = torch.empty(n_blocks, dtype=torch.uint8, device=ex.device)
    ex.pack.call("mxfp4_repack", raw_dev, data, scale, n_blocks, stream=_stream())
    return RepackedMxfp4(data, scale)


class MoeWorkspace:
    """Buffers of one MoE block call, sized for `tokens` tokens (allocated once, reused)."""

    def __init__(self, ex, planes, tokens, n_active, bm):
        dev, f32, u32 = ex.device, torch.float32, torch.int32
        pairs = tokens * n_active
        self.bm, self.tokens, self.n_active = bm, tokens, n_active
        self.max_blocks = min(pairs, pairs // bm + planes.n_expert)
        nb = self.max_blocks * bm
        self.idx = torch.empty(pairs, dtype=u32, device=dev)
        self.w = torch.empty(pairs, dtype=f32, device=dev)
        self.sorted_row = torch.empty(nb, dtype=u32, device=dev)
        self.sorted_slot = torch.empty(nb, dtype=u32, device=dev)
        self.block_expert = torch.empty(self.max_blocks, dtype=u32, device=dev)
        self.xq = torch.empty(tokens * planes.embd * 2, dtype=torch.uint8, device=dev)
        self.xscale = torch.empty(tokens, dtype=f32, device=dev)
        self.h = torch.zeros(nb * planes.ff, dtype=f32, device=dev)
        self.hq = torch.empty(nb * planes.ff * 2, dtype=torch.uint8, device=dev)
        self.hscale = torch.empty(nb, dtype=f32, device=dev)
        self.part = torch.empty(pairs * planes.embd, dtype=f32, device=dev)
        # tensor-core path: four NVFP4 term rows per block position, raw gate / up outputs
        self.x4q = torch.empty(nb * 4 * planes.embd // 2, dtype=torch.uint8, device=dev)
        self.x4s = torch.zeros(self.max_blocks * ((planes.embd + 255) // 256) * 2048, dtype=torch.uint8, device=dev)
        self.x4step = torch.empty(nb, dtype=f32, device=dev)
        self.h4q = torch.empty(nb * 4 * planes.ff // 2, dtype=torch.uint8, device=dev)
        self.h4s = torch.zeros(self.max_blocks * ((planes.ff + 255) // 256) * 2048, dtype=torch.uint8, device=dev)
        self.h4step = torch.empty(nb, dtype=f32, device=dev)
        self.g_raw = torch.empty(nb * planes.ff, dtype=f32, device=dev)
        self.u_raw = torch.empty(nb * planes.ff, dtype=f32, device=dev)


def moe_mxfp4_experts(ex, planes, ws, x, rows, alpha=1.702, limit=7.0):
    """align -> activation step -> gate|up + SwiGLU -> activation step -> down for `rows` token rows whose
    expert choices and routing weights are already in ws.idx / ws.w ([rows][ws.n_active]); leaves the
    weighted per-(row, slot) outputs in ws.part.  Five launches."""
    st = _stream()
    c = ex.pack.call
    k, bm = ws.n_active, ws.bm
    max_blocks = min(ws.max_blocks, min(rows * k, rows * k // bm + planes.n_expert))
    c("moe_align_bm", ws.idx, ws.sorted_row, ws.sorted_slot, ws.block_expert, rows, k, planes.n_expert, bm,
      max_blocks, stream=st)
    c("pdk_moe_prep_act", x, ws.xq, ws.xscale, planes.embd, rows, stream=st)
    c("pdk_mxfp4_moe_gate_up", planes.gate.data, planes.gate.scale, planes.gate_bias, planes.up.data,
      planes.up.scale, planes.up_bias, ws.sorted_row, ws.block_expert, ws.xq, ws.xscale, ws.h, planes.embd,
      planes.ff, bm, max_blocks, alpha, limit, stream=st)
    c("pdk_moe_prep_act", ws.h, ws.hq, ws.hscale, planes.ff, max_blocks * bm, stream=st)
    c("pdk_mxfp4_moe_down", planes.down.data, planes.down.scale, planes.down_bias, ws.sorted_row, ws.sorted_slot,
      ws.block_expert, ws.w, ws.hq, ws.hscale, ws.part, planes.ff, planes.embd, k, bm, max_blocks, stream=st)
    return 5


def moe_mxfp4_experts_tc5(ex, planes, ws, x, rows, alpha=1.702, limit=7.0, route=None):
    """moe_mxfp4_experts on the block-scaled tensor-core path (planes prepared with prepare_tc5):
    align -> term rows of x -> gate and up GEMM -> SwiGLU + term rows of h -> down GEMM scattered
    into ws.part.  Five launches; with route = (router_logits, router_bias) at decode widths the
    top-k, the alignment and the first preparation are one launch (four in all)."""
    st = _stream()
    c = ex.pack.call
    k, bm, t = ws.n_active, ws.bm, planes.tc5
    max_blocks = min(ws.max_blocks, min(rows * k, rows * k // bm + planes.n_expert))
    if route is not None:
        c("pdk_moe_route_prep_f4", route[0], route[1], x, ws.idx, ws.w, ws.sorted_row, ws.sorted_slot, ws.block_expert,
          ws.x4q, ws.x4s, ws.x4step, planes.n_expert, k, rows, planes.embd, bm, max_blocks, stream=st)
    else:
        c("moe_align_bm", ws.idx, ws.sorted_row, ws.sorted_slot, ws.block_expert, rows, k, planes.n_expert, bm,
          max_blocks, stream=st)
        c("pdk_moe_prep_act_f4", x, None, ws.sorted_row, ws.block_expert, ws.x4q, ws.x4s, ws.x4step, planes.embd, bm,
          max_blocks, 0, alpha, limit, stream=st)
    c("pdk_mxfp4_moe_gemm_tc5", planes.gate.data, t["gate"][0], t["gate"][1], planes.gate_bias, ws.g_raw,
      planes.up.data, t["up"][0], t["up"][1], planes.up_bias, ws.u_raw, ws.x4q, ws.x4s, ws.x4step,
      ws.block_expert, ws.sorted_row, None, None, planes.embd, planes.ff, planes.n_expert, bm, max_blocks, k, 0,
      stream=st)
    c("pdk_moe_prep_act_f4", ws.g_raw, ws.u_raw, ws.sorted_row, ws.block_expert, ws.h4q, ws.h4s, ws.h4step, planes.ff, bm,
      max_blocks, 1, alpha, limit, stream=st)
    c("pdk_mxfp4_moe_gemm_tc5", planes.down.data, t["down"][0], t["down"][1], planes.down_bias, ws.part,
      None, None, None, None, None, ws.h4q, ws.h4s, ws.h4step, ws.block_expert, ws.sorted_row, ws.sorted_slot,
      ws.w, planes.ff, planes.embd, planes.n_expert, bm, max_blocks, k, 1, stream=st)
    return 5


def moe_mxfp4_forward(ex, planes, ws, x, router_logits, out, alpha=1.702, limit=7.0, router_bias=None):
    """The MoE block the way crates/paddock-engine/src/gpu_model/gpt_oss.rs:2279-2521 walks it:
    top-k -> align -> activation step -> gate|up + SwiGLU -> activation step -> down -> combine.
    x f32[tokens][embd], router_logits f32[tokens][n_expert], out f32[tokens][embd] (accumulated into)."""
    st = _stream()
    c = ex.pack.call
    T, k = ws.tokens, ws.n_active
    if planes.tc5 is not None and T <= 8 and T * k <= 32 and planes.n_expert <= 512 and ws.max_blocks <= 32:
        # decode widths: routing, alignment and the first activation preparation in one launch
        moe_mxfp4_experts_tc5(ex, planes, ws, x, T, alpha, limit, route=(router_logits, router_bias))
        c("moe_slot_combine", ws.part, out, planes.embd, k, T, stream=st)
        return 5
    c("moe_topk_batch", router_logits, router_bias, planes.n_expert, k, ws.idx, ws.w, T, stream=st)
    if planes.tc5 is not None:
        moe_mxfp4_experts_tc5(ex, planes, ws, x, T, alpha, limit)
    else:
        moe_mxfp4_experts(ex, planes, ws, x, T, alpha, limit)
    c("moe_slot_combine", ws.part, out, planes.embd, k, T, stream=st)
    return 7  # launches


# ---- NVFP4 expert planes (gpu/types.rs:176-226, Row order) on the same grouped GEMM

@dataclass
class Nvf4MoePlane:
    data: torch.Tensor      # u8 [n_expert*rows][in_dim/2]
    scale: torch.Tensor     # e4m3 [n_expert*rows][in_dim/16]
    scale2: torch.Tensor    # f32 [n_expert]
    n_expert: int
    rows: int
    in_dim: int
    tiled: torch.Tensor = None


def nvf4_moe_prepare(ex, plane):
    """Load-time: tile the plane's per-16 scales into scale records (pdk_nvf4_moe_tile_scales)."""
    if plane.tiled is None:
        n = plane.n_expert * ((plane.rows + 127) // 128) * ((plane.in_dim + 255) // 256) * 2048
        plane.tiled = torch.empty(n, dtype=torch.uint8, device=ex.device)
        ex.pack.call("pdk_nvf4_moe_tile_scales", plane.scale, plane.tiled, plane.rows, plane.in_dim, plane.n_expert,
                     stream=_stream())
    return plane


def moe_nvf4_forward(ex, gate, up, down, ws, x, router_logits, out, gated=True, alpha=1.0, limit=float("inf"),
                     up_add=0.0, router_bias=None):
    """NVFP4 MoE block: top-k -> align -> term rows -> up (and gate) GEMM -> activation + term rows -> down
    GEMM -> combine.  gated: silu-gated unit (plain SwiGLU by default); else relu(up x)^2 (gate ignored).
    ws is a MoeWorkspace built for an object with n_expert / embd / ff attributes."""
    st = _stream()
    c = ex.pack.call
    T, k, bm = ws.tokens, ws.n_active, ws.bm
    n_expert, embd, ff = up.n_expert, up.in_dim, up.rows
    c("moe_topk_batch", router_logits, router_bias, n_expert, k, ws.idx, ws.w, T, stream=st)
    max_blocks = min(ws.max_blocks, min(T * k, T * k // bm + n_expert))
    c("moe_align_bm", ws.idx, ws.sorted_row, ws.sorted_slot, ws.block_expert, T, k, n_expert, bm, max_blocks, stream=st)
    c("pdk_moe_prep_act_f4n", x, None, ws.sorted_row, ws.block_expert, ws.x4q, ws.x4s, ws.x4step, embd, bm, max_blocks, 0,
      alpha, limit, up_add, stream=st)
    if gated:
        c("pdk_nvf4_moe_gemm_tc5", gate.data, gate.tiled, gate.scale2, None, ws.g_raw, up.data, up.tiled, up.scale2, None,
          ws.u_raw, ws.x4q, ws.x4s, ws.x4step, ws.block_expert, ws.sorted_row, None, None, embd, ff, n_expert, bm,
          max_blocks, k, 0, stream=st)
        c("pdk_moe_prep_act_f4n", ws.g_raw, ws.u_raw, ws.sorted_row, ws.block_expert, ws.h4q, ws.h4s, ws.h4step, ff, bm,
          max_blocks, 1, alpha, limit, up_add, stream=st)
    else:
        c("pdk_nvf4_moe_gemm_tc5", up.data, up.tiled, up.scale2, None, ws.u_raw, None, None, None, None, None, ws.x4q,
          ws.x4s, ws.x4step, ws.block_expert, ws.sorted_row, None, None, embd, ff, n_expert, bm, max_blocks, k, 0,
          stream=st)
        c("pdk_moe_prep_act_f4n", ws.u_raw, None, ws.sorted_row, ws.block_expert, ws.h4q, ws.h4s, ws.h4step, ff, bm,
          max_blocks, 2, alpha, limit, up_add, stream=st)
    c("pdk_nvf4_moe_gemm_tc5", down.data, down.tiled, down.scale2, None, ws.part, None, None, None, None, None, ws.h4q,
      ws.h4s, ws.h4step, ws.block_expert, ws.sorted_row, ws.sorted_slot, ws.w, ff, embd, n_expert, bm, max_blocks, k, 1,
      stream=st)
    c("moe_slot_combine", ws.part, out, embd, k, T, stream=st)
    return 7
