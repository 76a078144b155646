"""numpy front end of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the ``cpu_baseline`` / ``--impl reference`` legs of bench.py as the checker
or the timed CPU baseline.  The product package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build():
    """Compile oracle.c into liboracle.so (gcc + OpenMP)."""
    subprocess.check_call(["make", "-s", "-C", _HERE])


def _load():
    src = os.path.join(_HERE, "oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        build()
    return C.CDLL(_SO)


_lib = _load()

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def _sig(name, res, *args):
    f = getattr(_lib, name)
    f.restype = res
    f.argtypes = list(args)
    return f


_f16_to_f32 = _sig("orc_f16_to_f32", C.c_float, C.c_uint16)
_f32_to_f16 = _sig("orc_f32_to_f16", C.c_uint16, C.c_float)
_e8m0 = _sig("orc_e8m0_half_to_f32", C.c_float, C.c_uint8)
_e2m1 = _sig("orc_e2m1_to_f32", C.c_float, C.c_uint8)
_e4m3 = _sig("orc_e4m3_to_f32", C.c_float, C.c_uint8)
_to_e4m3 = _sig("orc_f32_to_e4m3", C.c_uint8, C.c_float)
_e2m1_rn = _sig("orc_e2m1_rn", C.c_uint8, C.c_float)
_dq_mxfp4 = _sig("orc_dequant_mxfp4", C.c_int, _u8p, C.c_size_t, _f32p, C.c_size_t)
_dq_q8 = _sig("orc_dequant_q8_0", C.c_int, _u8p, C.c_size_t, _f32p, C.c_size_t)
_dq_q4k = _sig("orc_dequant_q4_k", C.c_int, _u8p, C.c_size_t, _f32p, C.c_size_t)
_dq_kq = {name: _sig(f"orc_dequant_{name}", C.c_int, _u8p, C.c_size_t, _f32p, C.c_size_t)
          for name in ("q5_k", "q6_k", "q4_0", "iq4_xs")}
_dq_nvfp4 = _sig("orc_dequant_nvfp4", None, _u8p, _u8p, C.c_float, _f32p, C.c_uint32, C.c_uint32)
_dq_fp8 = _sig("orc_dequant_fp8_channel", None, _u8p, _f32p, _f32p, C.c_uint32, C.c_uint32)
_q_q8 = _sig("orc_quantize_q8_0", None, _f32p, C.c_size_t, _u8p)
_q_q4k = _sig("orc_quantize_q4_k", None, _f32p, C.c_size_t, _u8p)
_q_fp8 = _sig("orc_quantize_fp8_absmax", None, _f32p, C.c_uint32, C.c_uint32, _u8p, _f32p)
_q_e4m3row = _sig("orc_quantize_e4m3_row_pow2", None, _f32p, C.c_uint32, C.c_uint32, _u8p, _f32p)
_q_nvf4 = _sig("orc_quantize_nvf4_global", None, _f32p, C.c_size_t, C.c_float, _u8p, _u8p)
_q_mxfp4 = _sig("orc_quantize_mxfp4", None, _f32p, C.c_size_t, _u8p)
_q_q8act = _sig("orc_quantize_q8_act", None, _f32p, C.c_size_t, _i8p, _f32p, C.c_void_p)
_rp_q8 = _sig("orc_repack_q8_0", None, _u8p, C.c_uint64, _i8p, _u16p)
_rp_mxfp4 = _sig("orc_repack_mxfp4", None, _u8p, C.c_uint64, _u8p, _u8p)
_matvec = _sig("orc_matvec_f32", None, _f32p, _f32p, _f32p, C.c_uint32, C.c_uint32)
_matmul = _sig("orc_matmul_f64", None, _f32p, _f32p, _f32p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32)
_topk = _sig("orc_moe_topk", None, _f32p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, _u32p, _f32p)
_swiglu = _sig("orc_swiglu_oai", None, _f32p, _f32p, C.c_size_t, C.c_float, C.c_float)
_moe = _sig("orc_moe_mxfp4_layer", None, _u8p, _u8p, _u8p, C.c_void_p, C.c_void_p, C.c_void_p, _f32p,
            _u32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float)
_fill = _sig("orc_fill_normal", None, _f32p, C.c_size_t, C.c_uint64, C.c_float)
num_threads = _sig("orc_num_threads", C.c_int)
set_num_threads = _sig("orc_set_num_threads", None, C.c_int)


class DequantError(ValueError):
    """Mirror of reference/mod.rs DequantError (BadInputLen / BadOutputLen)."""


def f16_to_f32(h): return _f16_to_f32(int(h))
def f32_to_f16(f): return _f32_to_f16(float(f))
def e8m0_half_to_f32(e): return _e8m0(int(e))
def e2m1_to_f32(c): return _e2m1(int(c))
def e4m3_to_f32(b): return _e4m3(int(b))
def f32_to_e4m3(f): return _to_e4m3(float(f))
def e2m1_rn(f): return _e2m1_rn(float(f))


def _u8(a):
    return np.ascontiguousarray(np.frombuffer(bytes(a), np.uint8) if isinstance(a, (bytes, bytearray)) else a,
                                dtype=np.uint8)


def _check(rc, kind):
    if rc == -1:
        raise DequantError(f"input length is not a whole number of {kind} blocks")
    if rc == -2:
        raise DequantError("output length != expected elements")


def dequant_mxfp4(data, out=None):
    data = _u8(data)
    if out is None:
        out = np.empty(data.size // 17 * 32, np.float32)
    _check(_dq_mxfp4(data, data.size, out, out.size), "mxfp4")
    return out


def dequant_q8_0(data, out=None):
    data = _u8(data)
    if out is None:
        out = np.empty(data.size // 34 * 32, np.float32)
    _check(_dq_q8(data, data.size, out, out.size), "q8_0")
    return out


KQUANT_LAYOUT = {"q4_k": (144, 256), "q5_k": (176, 256), "q6_k": (210, 256), "q4_0": (18, 32), "iq4_xs": (136, 256)}  # (bytes, elements)


def dequant_kquant(name, data):
    """q5_k / q6_k / q4_0 / iq4_xs (crates/paddock-engine/tests/gpu_kquant_parity.rs:39-128)."""
    data = _u8(data)
    nbytes, elems = KQUANT_LAYOUT[name]
    out = np.empty(data.size // nbytes * elems, np.float32)
    _check(_dq_kq[name](data, data.size, out, out.size), name)
    return out


def dequant_q4_k(data, out=None):
    data = _u8(data)
    if out is None:
        out = np.empty(data.size // 144 * 256, np.float32)
    _check(_dq_q4k(data, data.size, out, out.size), "q4_k")
    return out


def dequant_nvfp4(data, scale, scale2, in_dim, out_dim):
    out = np.empty((out_dim, in_dim), np.float32)
    _dq_nvfp4(_u8(data).reshape(-1), _u8(scale).reshape(-1), float(scale2), out.reshape(-1), in_dim, out_dim)
    return out


def dequant_fp8_channel(w, scale, in_dim, out_dim):
    out = np.empty((out_dim, in_dim), np.float32)
    _dq_fp8(_u8(w).reshape(-1), np.ascontiguousarray(scale, np.float32), out.reshape(-1), in_dim, out_dim)
    return out


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def quantize_q8_0(w):
    w = _f32(w)
    out = np.empty(w.size // 32 * 34, np.uint8)
    _q_q8(w, w.size, out)
    return out


def quantize_q4_k(w):
    w = _f32(w)
    out = np.empty(w.size // 256 * 144, np.uint8)
    _q_q4k(w, w.size, out)
    return out


def quantize_fp8_absmax(w, rows, k):
    q = np.empty((rows, k), np.uint8)
    s = np.empty(rows, np.float32)
    _q_fp8(_f32(w), rows, k, q.reshape(-1), s)
    return q, s


def quantize_e4m3_row_pow2(x, rows, k):
    q = np.empty((rows, k), np.uint8)
    s = np.empty(rows, np.float32)
    _q_e4m3row(_f32(x), rows, k, q.reshape(-1), s)
    return q, s


def quantize_nvf4(x, scale2=1.0):
    x = _f32(x)
    q = np.empty(x.size // 2, np.uint8)
    s = np.empty(x.size // 16, np.uint8)
    _q_nvf4(x, x.size, float(scale2), q, s)
    return q, s


def add_rmsnorm(x, proj, w, eps):
    """Residual add + RMSNorm of each row, the arithmetic of packs/cuda/src/quant/nvf4.cuh:455-543:
    v = x + proj in f32; f32 squares accumulated in f64; inv = 1 / sqrtf((float)(sum / n) + eps);
    out = (v * inv) * w in f32.  x, proj f32 [rows][n] (proj may be None), w f32 [n].
    Returns (v, out)."""
    x = np.asarray(x, np.float32)
    v = x if proj is None else (x + np.asarray(proj, np.float32)).astype(np.float32)
    n = v.shape[-1]
    total = (v * v).astype(np.float32).astype(np.float64).sum(axis=-1)
    mean = (total / float(n)).astype(np.float32) + np.float32(eps)
    inv = (np.float32(1.0) / np.sqrt(mean.astype(np.float32))).astype(np.float32)
    out = ((v * inv[..., None]).astype(np.float32) * np.asarray(w, np.float32)).astype(np.float32)
    return v, out


def rmsnorm_scaled_add(x, proj, w, eps, pscale=1.0):
    """The arithmetic in front of the e4m3 row quantizer (packs/cuda/src/gemm/dense_f8_decode.cuh:4357-4530):
    v = fmaf(pscale, proj, x) in f32 (proj None: v = x); f32 squares, mean in f64 here (the reference sums
    in double-float or f32, which agrees to an ulp of the sum); inv = 1 / sqrtf(mean + eps); xn = (v * inv) * w.
    Returns (v, xn)."""
    x = np.asarray(x, np.float32)
    if proj is None:
        v = x
    else:   # one rounding: the product of two f32 is exact in f64
        v = (x.astype(np.float64) + np.float64(np.float32(pscale)) * np.asarray(proj, np.float32).astype(np.float64)).astype(np.float32)
    n = v.shape[-1]
    total = (v * v).astype(np.float32).astype(np.float64).sum(axis=-1)
    mean = (total / float(n)).astype(np.float32) + np.float32(eps)
    inv = (np.float32(1.0) / np.sqrt(mean.astype(np.float32))).astype(np.float32)
    xn = ((v * inv[..., None]).astype(np.float32) * np.asarray(w, np.float32)).astype(np.float32)
    return v, xn


def swiglu_silu(gate, up):
    """h = (g / (1 + expf(-g))) * u in f32 (packs/cuda/src/exports.cuh:404-412); numpy's f32 exp may differ
    from the device's by an ulp."""
    g = np.asarray(gate, np.float32)
    one = np.float32(1.0)
    return ((g / (one + np.exp(-g).astype(np.float32))).astype(np.float32) * np.asarray(up, np.float32)).astype(np.float32)


def quantize_mxfp4(w):
    w = _f32(w)
    out = np.empty(w.size // 32 * 17, np.uint8)
    _q_mxfp4(w, w.size, out)
    return out


def quantize_q8_act(x, with_sums=True):
    x = _f32(x)
    q = np.empty(x.size, np.int8)
    s = np.empty(x.size // 32, np.float32)
    sums = np.empty(x.size // 16, np.float32) if with_sums else None
    _q_q8act(x, x.size, q, s, sums.ctypes.data if with_sums else None)
    return q, s, sums


def repack_q8_0(src):
    src = _u8(src)
    n = src.size // 34
    data = np.empty(n * 32, np.int8)
    scale = np.empty(n, np.uint16)
    _rp_q8(src, n, data, scale)
    return data, scale


def repack_mxfp4(src):
    src = _u8(src)
    n = src.size // 17
    data = np.empty(n * 16, np.uint8)
    scale = np.empty(n, np.uint8)
    _rp_mxfp4(src, n, data, scale)
    return data, scale


def matvec_f32(w, x, in_dim, out_dim):
    y = np.empty(out_dim, np.float32)
    _matvec(_f32(w), _f32(x), y, in_dim, out_dim)
    return y


def matmul_f64(w, x, in_dim, out_dim, batch, with_abs=False):
    """y[batch][out_dim] (f64 accumulate) and optionally sum_k |w x|."""
    y = np.empty((batch, out_dim), np.float32)
    ab = np.empty((batch, out_dim), np.float32) if with_abs else None
    _matmul(_f32(w), _f32(x), y.reshape(-1), ab.ctypes.data if with_abs else None, in_dim, out_dim, batch)
    return (y, ab) if with_abs else y


def moe_topk(logits, n_expert, k, bias=None):
    logits = _f32(logits)
    batch = logits.size // n_expert
    idx = np.empty((batch, k), np.uint32)
    w = np.empty((batch, k), np.float32)
    b = None if bias is None else _f32(bias)
    _topk(logits, None if b is None else b.ctypes.data, n_expert, k, batch, idx.reshape(-1), w.reshape(-1))
    return idx, w


def swiglu_oai(gate, up, alpha=1.702, limit=7.0):
    g = _f32(gate).copy()
    _swiglu(g, _f32(up), g.size, alpha, limit)
    return g


def moe_mxfp4_layer(gate, up, down, x, topk_idx, topk_w, tokens, n_active, embd, ff,
                    gate_b=None, up_b=None, down_b=None, alpha=1.702, limit=7.0):
    out = np.empty((tokens, embd), np.float32)
    keep = [None if b is None else _f32(b) for b in (gate_b, up_b, down_b)]
    ptrs = [None if b is None else b.ctypes.data for b in keep]
    _moe(_u8(gate).reshape(-1), _u8(up).reshape(-1), _u8(down).reshape(-1), ptrs[0], ptrs[1], ptrs[2],
         _f32(x), np.ascontiguousarray(topk_idx, np.uint32).reshape(-1), _f32(topk_w), out.reshape(-1),
         tokens, n_active, embd, ff, alpha, limit)
    return out


def fill_normal(n, seed, sigma=1.0):
    out = np.empty(n, np.float32)
    _fill(out, n, seed, sigma)
    return out


def bf16_round(x):
    """Round f32 to the nearest bf16 (RNE) and widen back to f32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return r.astype(np.uint32).view(np.float32)
