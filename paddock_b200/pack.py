"""Kernel-pack loader: the Python twin of crates/paddock-kernels/src/loader.rs.

``KernelPack.load(path)`` dlopens a pack, resolves ``paddock_pack_info`` and
``paddock_pack_kernels_v1``, and applies the reference loader's checks in the
same order with the same error kinds (loader.rs:44-63, 140-283): null
descriptor, magic, ABI version, table size, then a min(size, sizeof) copy into
a zeroed table so entries a pack does not fill read as missing.
"""
import ctypes as C
import os
import re

PACK_MAGIC = 0x504B4450
PACK_ABI_VERSION = 2
TABLE_SLOTS = 953
TABLE_BYTES = 8 + 8 * TABLE_SLOTS

_PKG = os.path.dirname(os.path.abspath(__file__))


def lib_path():
    return os.path.join(_PKG, "libpaddock_b200.so")


def header_path():
    return os.path.join(os.path.dirname(_PKG), "include", "paddock_pack.h")


def _parse_slots():
    """Slot name -> index, read from the PdkSlot enum of include/paddock_pack.h."""
    with open(header_path()) as f:
        text = f.read()
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"PDK_SLOT_(\w+)\s*=\s*(\d+)", text)}


SLOTS = _parse_slots()


class PackError(Exception):
    """Base of the loader's error kinds (loader.rs:44-63)."""


class Open(PackError):
    pass


class NotAPack(PackError):
    pass


class BadDescriptor(PackError):
    pass


class BadMagic(PackError):
    pass


class AbiMismatch(PackError):
    def __init__(self, path, found, expected):
        super().__init__(f"{path} was built for pack ABI {found}, this engine expects {expected}")
        self.found, self.expected = found, expected


class NoKernelTable(PackError):
    pass


class BadKernelTable(PackError):
    pass


class MissingOp(PackError):
    """A slot the pack leaves NULL (crates/paddock-engine/src/gpu/error.rs:36-40)."""


class LaunchError(RuntimeError):
    """Non-zero launcher status (gpu/error.rs:106-128 maps it to GpuError::Launch)."""

    def __init__(self, name, status):
        super().__init__(f"kernel launcher {name} returned CUDA error {status}")
        self.status = status


class PackInfo(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("abi_version", C.c_uint32), ("arch", C.c_uint8 * 16),
                ("pack_version", C.c_uint32 * 3)]

    def arch_str(self):
        raw = bytes(self.arch)
        return raw.split(b"\0", 1)[0].decode("ascii")


# ctypes argument kinds by launcher; 'p' device pointer, 'u' u32, 'U' u64, 'f' f32.
# The stream argument is appended by call().
_SIGS = {
    "mxfp4_dequant_f32": "ppU", "q8_0_dequant_f32": "ppU", "add_inplace_f32": "ppu",
    "mxfp4_repack": "pppU", "q8_0_repack": "pppU",
    "q8_0_gemv_repacked": "pppppuu", "q8_0_gemm_repacked": "pppppuuu",
    "quantize_e4m3_row": "pppuu", "bf16_to_f8row": "pppuu",
    "f8row_gemm": "pppppuuu", "f8row_gemm_tc5x": "pppppuuu",
    "swiglu_quant_e4m3_row": "ppppuu", "rmsnorm_quant_e4m3_row": "pppppufu",
    "add_rmsnorm_scaled_quant_e4m3_row": "ppppppuffu",
    "quantize_nvf4": "pppu", "add_rmsnorm_quant_nvf4_batch": "ppppppufu", "add_rmsnorm_nvf4_batch": "ppppppufu",
    "quantize_nvf4_swiglu": "ppppu", "swiglu_fused_nvf4": "pppuu", "nvf4_dequant": "ppfpuu", "nvf4_gemv": "pppppfuu",
    "nvf4_tc5_tile_scales": "ppuu", "nvf4_gemm_tc5w": "ppppppfuuupU",
    "moe_topk_batch": "ppuuppu", "moe_align": "ppppuuuu", "moe_align_bm": "ppppuuuuu", "moe_slot_combine": "ppuuu",
    "kquant_dequant": "ppUu", "kquant_repack": "pppUu", "kquant_gemv": "ppppuuu",
    "quantize_q8": "pppu", "quantize_q8_sums": "ppppu", "kquant_gemv_w4a8": "ppppppuuu",
    "kquant_gemm_mma_ks": "pppppppuuuu", "kquant_gemm_w4a8_sb": "pppppppuuuu",
    "mxfp4_gu_interleave": "pppuU", "mxfp4_moe_gate_up_mmq": "pppppppppppp" + "uuu" + "fff",
    "mxfp4_moe_down_mmq": "pppppppppp" + "uuuu", "mxfp4_moe_gate_up_dp4a_b": "pppppppppp" + "uuuu" + "ff",
    "mxfp4_moe_down_dp4a_b": "pppppppp" + "uuuu",
}
_EXTRA_SIGS = {
    "pdk_kquant_gemm_f32": "ppppuuuu",
    "pdk_f8row_gemm_bf16": "pppppuuu",
    "pdk_nvf4_gemm_bf16": "ppppppfuuu",
    "pdk_moe_prep_act": "pppuu",
    "pdk_mxfp4_moe_gate_up": "pppppppppppuuuuff",
    "pdk_mxfp4_moe_down": "ppppppppppuuuuu",
    "pdk_mxfp4_moe_down_combine_static": "ppppppppppuuuuuu",
    "pdk_q4k_gemv_shard": "ppppuuuu",
    "pdk_q4k_gemv_shard_sync": "ppppppuuuuuu",
    "pdk_q4k_gemv_shard_lagged": "ppppppuuuuuu",
    "pdk_peer_flags_wait": "puuu",
    "pdk_peer_flags_post": "ppuu",
    "pdk_selftest_bounded_wait": "up",
    "pdk_tc5_issue_probe": "uup",
    "pdk_mxfp4_tc5_tile_scales": "pppuuu",
    "pdk_moe_prep_act_f4": "pppppppuuuuff",
    "pdk_moe_route_prep_f4": "p" * 11 + "u" * 6,
    "pdk_mxfp4_moe_gemm_tc5": "p" * 17 + "u" * 7,
    "pdk_nvf4_moe_tile_scales": "ppuuu",
    "pdk_moe_prep_act_f4n": "pppppppuuuufff",
    "pdk_nvf4_moe_gemm_tc5": "p" * 17 + "u" * 7,
}
_KIND = {"p": C.c_void_p, "u": C.c_uint32, "U": C.c_uint64, "f": C.c_float}


def _proto(sig):
    return C.CFUNCTYPE(C.c_int, *[_KIND[c] for c in sig], C.c_void_p)


class KernelPack:
    def __init__(self, lib, info, table, origin):
        self._lib, self.info, self._table, self.origin = lib, info, table, origin
        self._fns = {}

    @classmethod
    def load(cls, path=None):
        path = path or lib_path()
        try:
            lib = C.CDLL(path)
        except OSError as e:
            raise Open(f"failed to open kernel pack {path}: {e}") from e
        try:
            info_fn = lib.paddock_pack_info
        except AttributeError:
            raise NotAPack(f"{path} is not a Paddock kernel pack (missing paddock_pack_info symbol)")
        info_fn.restype = C.POINTER(PackInfo)
        ptr = info_fn()
        if not ptr:
            raise BadDescriptor(f"{path} returned a null/invalid descriptor")
        info = PackInfo.from_buffer_copy(ptr.contents)
        if info.magic != PACK_MAGIC:
            raise BadMagic(f"{path} has wrong magic - not a pack or corrupted download")
        if info.abi_version != PACK_ABI_VERSION:
            raise AbiMismatch(path, info.abi_version, PACK_ABI_VERSION)
        try:
            table_fn = lib.paddock_pack_kernels_v1
        except AttributeError:
            raise NoKernelTable(f"{path} exports no kernel table (missing paddock_pack_kernels_v1)")
        table_fn.restype = C.c_void_p
        tptr = table_fn()
        if not tptr:
            raise BadKernelTable(f"{path} kernel table is null or truncated (size 0)")
        declared = C.c_uint32.from_address(tptr).value
        if declared < 8:
            raise BadKernelTable(f"{path} kernel table is null or truncated (size {declared})")
        table = (C.c_uint8 * TABLE_BYTES)()
        C.memmove(table, tptr, min(declared, TABLE_BYTES))
        return cls(lib, info, table, path)

    # -- table access -------------------------------------------------------
    def table_size(self):
        return C.c_uint32.from_buffer(self._table, 0).value

    def slot_ptr(self, idx):
        return C.c_uint64.from_buffer(self._table, 8 + 8 * idx).value

    def has(self, name):
        return name in SLOTS and self.slot_ptr(SLOTS[name]) != 0

    def fn(self, name):
        """Function pointer of a table slot, typed; MissingOp when NULL."""
        if name not in self._fns:
            if name not in SLOTS or name not in _SIGS:
                raise MissingOp(name)
            addr = self.slot_ptr(SLOTS[name])
            if addr == 0:
                raise MissingOp(name)
            self._fns[name] = _proto(_SIGS[name])(addr)
        return self._fns[name]

    def fn_at(self, idx, sig):
        """Slot `idx` with signature string `sig` (for slots this package does not name, e.g. when
        timing another pack)."""
        addr = self.slot_ptr(idx)
        if addr == 0:
            raise MissingOp(f"slot {idx}")
        return _proto(sig)(addr)

    def extra(self, symbol):
        """A named export that has no table slot."""
        if symbol not in self._fns:
            f = getattr(self._lib, symbol)
            f.restype = C.c_int
            f.argtypes = [_KIND[c] for c in _EXTRA_SIGS[symbol]] + [C.c_void_p]
            self._fns[symbol] = f
        return self._fns[symbol]

    def device_error(self):
        """Read and clear the device error word (0 = no timed-out wait)."""
        f = self._lib.pdk_device_error
        f.restype = C.c_uint
        return f()

    def call(self, name, *args, stream=0):
        """Launch slot `name` (or a named extra) and raise LaunchError on a
        non-zero status.  Pointer arguments may be ints or torch tensors."""
        f = self.extra(name) if name in _EXTRA_SIGS else self.fn(name)
        rc = f(*[_arg(a) for a in args], stream)
        if rc != 0:
            raise LaunchError(name, rc)

    def bind(self, name, *args, stream=0):
        """A zero-argument callable that launches `name` with these arguments (converted once): for
        loops where the per-call argument marshalling would rival a short kernel's run time.  The
        tensors behind the pointers must outlive it; it raises LaunchError like call()."""
        f = self.extra(name) if name in _EXTRA_SIGS else self.fn(name)
        conv = tuple(_arg(a) for a in args) + (stream,)

        def launch():
            rc = f(*conv)
            if rc != 0:
                raise LaunchError(name, rc)
        launch.keep = args
        return launch

    def status(self, name, *args, stream=0):
        """Like call() but returns the raw status instead of raising."""
        f = self.extra(name) if name in _EXTRA_SIGS else self.fn(name)
        return f(*[_arg(a) for a in args], stream)


def _arg(a):
    if a is None:
        return None
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    return a
