"""ctypes front end of libpaddock_exec.so (include/paddock_exec.h): the C++ operator layer
above the kernel-pack table - executor, resident planes, upload / repack / launch wrappers named
after crates/paddock-engine/src/gpu (GpuExecutor, QuantW, RepackedQ8, RepackedKQ, F8RowPlane,
Nvf4Plane, QuantTensor).  Weight bytes are host memory (numpy arrays or mapped tensors),
activations and outputs are device pointers (ints, or anything with data_ptr())."""
import ctypes as C
import os

import numpy as np

from . import formats as F

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ERRORS = ["Ok", "MissingOp", "NoKernel", "Unsupported", "Driver", "Launch", "Pack", "Format"]
PLANE_KINDS = ["Raw", "Q8", "Kq", "F8Row", "Nvf4", "Mxfp4"]
NVF4_LAYOUTS = ["Row", "Tiled", "Frag"]


class GpuError(RuntimeError):
    """gpu/error.rs: kind is one of ERRORS."""

    def __init__(self, kind, message):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


class PlaneInfo(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("ggml_type", C.c_uint32), ("in_dim", C.c_uint64), ("out_dim", C.c_uint64),
                ("bytes", C.c_uint64), ("data", C.c_void_p), ("scale", C.c_void_p), ("scale_tc5", C.c_void_p),
                ("scale2", C.c_float), ("layout", C.c_uint32)]


def lib_path():
    return os.path.join(_HERE, "libpaddock_exec.so")


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(lib_path())
        _LIB.pdx_stream.restype = C.c_void_p
        _LIB.pdx_last_error.restype = C.c_char_p
        _LIB.pdx_staging_bytes.restype = C.c_uint64
    return _LIB


def _ptr(a):
    if a is None:
        return None
    if hasattr(a, "data_ptr"):
        return C.c_void_p(a.data_ptr())
    return C.c_void_p(int(a))


def _host(a):
    """(pointer, byte length, keep-alive) of host bytes."""
    arr = np.ascontiguousarray(a if isinstance(a, np.ndarray) else np.frombuffer(a, np.uint8))
    return C.c_void_p(arr.ctypes.data), arr.nbytes, arr


class Plane:
    """A resident weight (QuantW / QuantTensor / F8RowPlane / Nvf4Plane); freed with its executor
    or by free()."""

    def __init__(self, ex, handle):
        self._ex, self._h = ex, handle

    def info(self):
        out = PlaneInfo()
        _lib().pdx_plane_info(self._h, C.byref(out))
        return out

    @property
    def kind(self):
        return PLANE_KINDS[self.info().kind]

    @property
    def dims(self):
        i = self.info()
        return (i.in_dim, i.out_dim)

    def bytes(self):
        return self.info().bytes

    def free(self):
        if self._h and self._ex._h:
            _lib().pdx_plane_free(self._ex._h, self._h)
        self._h = None


class GpuExecutor:
    """gpu/mod.rs:143-252 for the quantized linear layer: pack + stream + staging buffer."""

    def __init__(self, pack_path=None, device=0):
        self._h = None
        h, err = C.c_void_p(), C.create_string_buffer(512)
        rc = _lib().pdx_open(pack_path.encode() if pack_path else None, C.c_int(device), C.byref(h), err, C.c_size_t(512))
        if rc != 0:
            raise GpuError(ERRORS[rc], err.value.decode(errors="replace"))
        self._h = h
        self._planes = []

    def close(self):
        if self._h:
            for p in self._planes:
                p.free()
            _lib().pdx_close(self._h)
            self._h = None

    __del__ = close

    def _check(self, rc):
        if rc != 0:
            raise GpuError(ERRORS[rc], _lib().pdx_last_error(self._h).decode(errors="replace"))

    def _plane(self, fn, *args):
        h = C.c_void_p()
        self._check(fn(self._h, *args, C.byref(h)))
        p = Plane(self, h)
        self._planes.append(p)
        return p

    @property
    def stream(self):
        return _lib().pdx_stream(self._h)

    def synchronize(self):
        self._check(_lib().pdx_synchronize(self._h))

    def has(self, slot_name):
        return bool(_lib().pdx_has(self._h, slot_name.encode()))

    def staging_bytes(self):
        return _lib().pdx_staging_bytes(self._h)

    def release_staging(self):
        _lib().pdx_release_staging(self._h)

    # ---- loaders ------------------------------------------------------------------------------
    def upload_raw(self, mapped, name):
        return self._plane(_lib().pdx_upload_raw, mapped._h, name.encode())

    def load_quantw(self, mapped, name):
        return self._plane(_lib().pdx_load_quantw, mapped._h, name.encode())

    def repack_q8_blocks(self, raw, in_dim, out_dim):
        p, n, keep = _host(raw)
        return self._plane(_lib().pdx_repack_q8_blocks, p, C.c_uint64(n), C.c_uint64(in_dim), C.c_uint64(out_dim))

    def repack_kquant_raw(self, raw, in_dim, out_dim, ggml_type):
        p, n, keep = _host(raw)
        return self._plane(_lib().pdx_repack_kquant_raw, p, C.c_uint64(n), C.c_uint64(in_dim), C.c_uint64(out_dim),
                           C.c_uint32(ggml_type))

    def repack_kquant_bands(self, mapped, name, n_bands):
        hs = (C.c_void_p * n_bands)()
        self._check(_lib().pdx_repack_kquant_bands(self._h, mapped._h, name.encode(), C.c_uint32(n_bands), hs))
        out = [Plane(self, C.c_void_p(h)) for h in hs]
        self._planes += out
        return out

    def repack_kquant_concat(self, mapped, names):
        arr = (C.c_char_p * len(names))(*[n.encode() for n in names])
        return self._plane(_lib().pdx_repack_kquant_concat, mapped._h, arr, C.c_uint32(len(names)))

    def repack_mxfp4(self, raw, in_dim, rows):
        p, n, keep = _host(raw)
        return self._plane(_lib().pdx_repack_mxfp4, p, C.c_uint64(n), C.c_uint64(in_dim), C.c_uint64(rows))

    def bf16_to_f8row(self, bf16_bits, in_dim, out_dim):
        p, n, keep = _host(bf16_bits)
        assert n == in_dim * out_dim * 2
        return self._plane(_lib().pdx_bf16_to_f8row, p, C.c_uint64(in_dim), C.c_uint64(out_dim))

    def f8row_upload(self, e4m3, row_scales, in_dim, out_dim):
        p, n, keep = _host(e4m3)
        s = np.ascontiguousarray(row_scales, np.float32)
        assert n == in_dim * out_dim and s.size == out_dim
        return self._plane(_lib().pdx_f8row_upload, p, s.ctypes.data_as(C.POINTER(C.c_float)), C.c_uint64(in_dim),
                           C.c_uint64(out_dim))

    def nvf4_upload(self, packed, scales, scale2, out_dim, in_dim):
        p, n, keep = _host(packed)
        s, sn, keep2 = _host(scales)
        return self._plane(_lib().pdx_nvf4_upload, p, C.c_uint64(n), s, C.c_uint64(sn), C.c_float(scale2),
                           C.c_uint64(out_dim), C.c_uint64(in_dim))

    # ---- launches -----------------------------------------------------------------------------
    def dequant_rows(self, plane, row0, rows, out):
        self._check(_lib().pdx_dequant_rows(self._h, plane._h, C.c_uint64(row0), C.c_uint64(rows), _ptr(out)))

    def quantw_gemv(self, w, bias, x, y):
        self._check(_lib().pdx_quantw_gemv(self._h, w._h, _ptr(bias), _ptr(x), _ptr(y)))

    def quantw_gemm(self, w, bias, x, y, batch):
        self._check(_lib().pdx_quantw_gemm(self._h, w._h, _ptr(bias), _ptr(x), _ptr(y), C.c_uint32(batch)))

    def quantize_e4m3_row(self, x, q, rscale, n_dim, batch):
        self._check(_lib().pdx_quantize_e4m3_row(self._h, _ptr(x), _ptr(q), _ptr(rscale), C.c_uint32(n_dim),
                                                 C.c_uint32(batch)))

    def swiglu_quant_e4m3_row(self, gate, up, q, rs, n_ff, batch):
        """-> True when the pack ran the fused kernel (gpu/fp8.rs:469-497)."""
        fused = C.c_int()
        self._check(_lib().pdx_swiglu_quant_e4m3_row(self._h, _ptr(gate), _ptr(up), _ptr(q), _ptr(rs), C.c_uint32(n_ff),
                                                     C.c_uint32(batch), C.byref(fused)))
        return bool(fused.value)

    def rmsnorm_quant_e4m3_row(self, x, w, xn, q, rs, n, eps, batch):
        fused = C.c_int()
        self._check(_lib().pdx_rmsnorm_quant_e4m3_row(self._h, _ptr(x), _ptr(w), _ptr(xn), _ptr(q), _ptr(rs), C.c_uint32(n),
                                                      C.c_float(eps), C.c_uint32(batch), C.byref(fused)))
        return bool(fused.value)

    def add_rmsnorm_scaled_quant_e4m3_row(self, x, proj, w, xn, q, rs, n, eps, pscale, batch):
        fused = C.c_int()
        self._check(_lib().pdx_add_rmsnorm_scaled_quant_e4m3_row(self._h, _ptr(x), _ptr(proj), _ptr(w), _ptr(xn), _ptr(q),
                                                                 _ptr(rs), C.c_uint32(n), C.c_float(eps), C.c_float(pscale),
                                                                 C.c_uint32(batch), C.byref(fused)))
        return bool(fused.value)

    def f8row_gemm(self, w, xq, xrs, y, batch):
        self._check(_lib().pdx_f8row_gemm(self._h, w._h, _ptr(xq), _ptr(xrs), _ptr(y), C.c_uint32(batch)))

    def quantize_nvf4(self, x, q, scale, n):
        self._check(_lib().pdx_quantize_nvf4(self._h, _ptr(x), _ptr(q), _ptr(scale), C.c_uint32(n)))

    def nvf4_gemm_f4(self, w, xq, xs, y, bias, batch):
        self._check(_lib().pdx_nvf4_gemm_f4(self._h, w._h, _ptr(xq), _ptr(xs), _ptr(y), _ptr(bias), C.c_uint32(batch)))

    def nvf4_gemv(self, w, bias, x, y):
        self._check(_lib().pdx_nvf4_gemv(self._h, w._h, _ptr(bias), _ptr(x), _ptr(y)))


__all__ = ["GpuExecutor", "GpuError", "Plane", "PlaneInfo", "ERRORS", "PLANE_KINDS", "NVF4_LAYOUTS", "lib_path", "F"]
