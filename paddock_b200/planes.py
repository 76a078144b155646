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
