"""ctypes front end of libpaddock_host.so (include/paddock_host.h): the weight
format table, the GGUF and safetensors readers and the quantized checkpoint
views.  Names follow crates/paddock-models (GgmlType, MappedGguf,
ShardedSafetensors, nvfp4_view, fp8_channel_view, gguf_nvfp4::repack_rows)."""
import ctypes as C
import os

import numpy as np

_LIB = C.CDLL(os.path.join(os.path.dirname(os.path.abspath(__file__)), "libpaddock_host.so"))
_ERR = 256

GGUF_ERRORS = ["Ok", "BadMagic", "UnsupportedVersion", "Truncated", "CountTooLarge", "BadUtf8", "UnknownValueType",
               "ArrayTooDeep", "BadAlignment", "BadTensor", "DuplicateTensor", "Io", "NotFound"]
MAP_ERRORS = ["Ok", "Io", "Parse", "NoSuchTensor", "OutOfRange", "Unsizable", "NotFirstSplit", "SplitNameMismatch",
              "ShardMismatch", "MissingSplitKey", "TensorCountMismatch", "DuplicateAcrossShards", "TooManySplits"]
ST_DTYPES = ["F8_E4M3", "BF16", "F16", "F32", "I64", "U8", "U32", "OTHER"]


class FormatError(ValueError):
    def __init__(self, kind, message):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


def block_layout(raw_type):
    """(elements, bytes) per block, or None for an unknown layout (ggml_type.rs:146-190)."""
    e, b = C.c_uint32(), C.c_uint32()
    return (e.value, b.value) if _LIB.pdk_ggml_block_layout(C.c_uint32(raw_type), C.byref(e), C.byref(b)) else None


def byte_size(raw_type, n_elements):
    """Bytes of n_elements in a type, or None (unknown layout / partial block) (ggml_type.rs:192-203)."""
    out = C.c_uint64()
    return out.value if _LIB.pdk_ggml_byte_size(C.c_uint32(raw_type), C.c_uint64(n_elements), C.byref(out)) else None


def _view(ptr, nbytes, owner):
    """Zero-copy uint8 view of mapped bytes; the view keeps `owner` (and so the mapping) alive."""
    if not nbytes:
        return np.empty(0, np.uint8)
    buf = (C.c_uint8 * nbytes).from_address(ptr.value)
    buf._owner = owner
    return np.frombuffer(buf, np.uint8)


class Gguf:
    """MappedGguf (mapped.rs:176,343): open / parse, then zero-copy tensor bytes."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def _finish(cls, rc, h, err):
        if rc != 0:
            raise FormatError(GGUF_ERRORS[rc], err.value.decode(errors="replace"))
        return cls(h)

    @classmethod
    def open(cls, path):
        h, err = C.c_void_p(), C.create_string_buffer(_ERR)
        return cls._finish(_LIB.pdk_gguf_open(path.encode(), C.byref(h), err, _ERR), h, err)

    @classmethod
    def parse(cls, data):
        h, err = C.c_void_p(), C.create_string_buffer(_ERR)
        return cls._finish(_LIB.pdk_gguf_parse(bytes(data), C.c_size_t(len(data)), C.byref(h), err, _ERR), h, err)

    def close(self):
        if self._h:
            _LIB.pdk_gguf_close(self._h)
            self._h = None

    __del__ = close

    @property
    def version(self):
        _LIB.pdk_gguf_version.restype = C.c_uint32
        return _LIB.pdk_gguf_version(self._h)

    @property
    def alignment(self):
        _LIB.pdk_gguf_alignment.restype = C.c_uint64
        return _LIB.pdk_gguf_alignment(self._h)

    @property
    def data_offset(self):
        _LIB.pdk_gguf_data_offset.restype = C.c_uint64
        return _LIB.pdk_gguf_data_offset(self._h)

    def tensors(self):
        _LIB.pdk_gguf_tensor_count.restype = C.c_uint64
        out = []
        for i in range(_LIB.pdk_gguf_tensor_count(self._h)):
            name, nd, dims = C.c_char_p(), C.c_uint32(), (C.c_uint64 * 8)()
            ty, off, nb = C.c_uint32(), C.c_uint64(), C.c_uint64()
            _LIB.pdk_gguf_tensor_at(self._h, C.c_uint64(i), C.byref(name), C.byref(nd), dims, C.byref(ty),
                                    C.byref(off), C.byref(nb))
            out.append((name.value.decode(), list(dims[:nd.value]), ty.value, off.value, nb.value))
        return out

    def tensor_bytes(self, name):
        """(numpy uint8 view, raw type, dims) of a tensor; dims[0] is the row length."""
        ptr, nb, ty, nd, dims = C.c_void_p(), C.c_uint64(), C.c_uint32(), C.c_uint32(), (C.c_uint64 * 8)()
        rc = _LIB.pdk_gguf_tensor_bytes(self._h, name.encode(), C.byref(ptr), C.byref(nb), C.byref(ty), C.byref(nd), dims)
        if rc != 0:
            raise FormatError(GGUF_ERRORS[rc], name)
        return _view(ptr, nb.value, self), ty.value, list(dims[:nd.value])

    def meta_u64(self, key):
        v = C.c_uint64()
        return v.value if _LIB.pdk_gguf_meta_u64(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key):
        v = C.c_char_p()
        return v.value.decode() if _LIB.pdk_gguf_meta_str(self._h, key.encode(), C.byref(v)) == 0 else None


def parse_split_name(path):
    """split.rs:37-62: ("<prefix>", no_1based, count) of a "<prefix>-00002-of-00003.gguf" name, else None."""
    prefix, no, count = C.create_string_buffer(4096), C.c_uint32(), C.c_uint32()
    if _LIB.pdk_split_name_parse(str(path).encode(), prefix, C.c_size_t(4096), C.byref(no), C.byref(count)) != 0:
        return None
    return prefix.value.decode(), no.value, count.value


class MappedGguf:
    """mapped.rs:176-345: one GGUF file or a split family opened through its first shard; tensors
    resolve to the shard that holds them, metadata comes from the first shard."""

    def __init__(self, path):
        self._h = None
        h, err = C.c_void_p(), C.create_string_buffer(_ERR)
        rc = _LIB.pdk_gguf_family_open(str(path).encode(), C.byref(h), err, _ERR)
        if rc != 0:
            raise FormatError(MAP_ERRORS[rc], err.value.decode(errors="replace"))
        self._h = h
        for fn in ("shard_count", "tensor_count", "total_len"):
            getattr(_LIB, "pdk_gguf_family_" + fn).restype = C.c_uint64
        _LIB.pdk_gguf_family_shard.restype = C.c_void_p
        _LIB.pdk_gguf_family_shard_path.restype = C.c_char_p

    def close(self):
        if self._h:
            _LIB.pdk_gguf_family_close(self._h)
            self._h = None

    __del__ = close

    def shard_count(self):
        return _LIB.pdk_gguf_family_shard_count(self._h)

    def tensor_count(self):
        return _LIB.pdk_gguf_family_tensor_count(self._h)

    def total_len(self):
        return _LIB.pdk_gguf_family_total_len(self._h)

    def shard_path(self, shard):
        return _LIB.pdk_gguf_family_shard_path(self._h, C.c_uint64(shard)).decode()

    def meta_u64(self, key):
        v = C.c_uint64()
        first = C.c_void_p(_LIB.pdk_gguf_family_shard(self._h, C.c_uint64(0)))
        return v.value if _LIB.pdk_gguf_meta_u64(first, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key):
        v = C.c_char_p()
        first = C.c_void_p(_LIB.pdk_gguf_family_shard(self._h, C.c_uint64(0)))
        return v.value.decode() if _LIB.pdk_gguf_meta_str(first, key.encode(), C.byref(v)) == 0 else None

    def tensor_infos(self):
        """(name, dims, raw type, bytes, shard) of every tensor, shards in family order."""
        out = []
        for i in range(self.tensor_count()):
            name, nd, dims = C.c_char_p(), C.c_uint32(), (C.c_uint64 * 8)()
            ty, nb, shard = C.c_uint32(), C.c_uint64(), C.c_uint32()
            _LIB.pdk_gguf_family_tensor_at(self._h, C.c_uint64(i), C.byref(name), C.byref(nd), dims, C.byref(ty),
                                           C.byref(nb), C.byref(shard))
            out.append((name.value.decode(), list(dims[:nd.value]), ty.value, nb.value, shard.value))
        return out

    def tensor_bytes(self, name):
        """(numpy uint8 view into the holding shard's mapping, raw type, dims, shard)."""
        ptr, nb, ty, nd, dims = C.c_void_p(), C.c_uint64(), C.c_uint32(), C.c_uint32(), (C.c_uint64 * 8)()
        shard = C.c_uint32()
        rc = _LIB.pdk_gguf_family_tensor_bytes(self._h, name.encode(), C.byref(ptr), C.byref(nb), C.byref(ty),
                                               C.byref(nd), dims, C.byref(shard))
        if rc != 0:
            raise FormatError(MAP_ERRORS[rc], name)
        return _view(ptr, nb.value, self), ty.value, list(dims[:nd.value]), shard.value


class Safetensors:
    """ShardedSafetensors (safetensors.rs:336-420): a file or a sharded directory."""

    def __init__(self, path):
        self._h = None
        h, err = C.c_void_p(), C.create_string_buffer(_ERR)
        rc = _LIB.pdk_st_open(path.encode(), C.byref(h), err, _ERR)
        if rc != 0:
            raise FormatError(["Ok", "Io", "Header", "NotFound"][rc], err.value.decode(errors="replace"))
        self._h = h

    def close(self):
        if self._h:
            _LIB.pdk_st_close(self._h)
            self._h = None

    __del__ = close

    def __len__(self):
        _LIB.pdk_st_tensor_count.restype = C.c_uint64
        return _LIB.pdk_st_tensor_count(self._h)

    def bytes(self, name):
        """(dtype name, shape, numpy uint8 view) or None when absent."""
        dt, nd, shape, ptr, nb = C.c_uint32(), C.c_uint32(), (C.c_uint64 * 8)(), C.c_void_p(), C.c_uint64()
        if _LIB.pdk_st_tensor(self._h, name.encode(), C.byref(dt), C.byref(nd), shape, C.byref(ptr), C.byref(nb)) != 0:
            return None
        return ST_DTYPES[dt.value], list(shape[:nd.value]), _view(ptr, nb.value, self)

    def nvfp4_view(self, prefix):
        """modelopt.rs:168-238 -> dict(packed, scales, scale2, n, k)."""
        p, s, s2, n, k = C.c_void_p(), C.c_void_p(), C.c_float(), C.c_uint64(), C.c_uint64()
        err = C.create_string_buffer(_ERR)
        if _LIB.pdk_st_nvfp4_view(self._h, prefix.encode(), C.byref(p), C.byref(s), C.byref(s2), C.byref(n),
                                  C.byref(k), err, _ERR) != 0:
            raise FormatError("Header", err.value.decode(errors="replace"))
        return dict(packed=_view(p, n.value * k.value // 2, self).reshape(n.value, -1),
                    scales=_view(s, n.value * k.value // 16, self).reshape(n.value, -1), scale2=np.float32(s2.value),
                    n=n.value, k=k.value)

    def fp8_channel_view(self, prefix):
        """modelopt.rs:291-342 -> dict(weight, scales, n, k)."""
        w, sc, n, k = C.c_void_p(), C.POINTER(C.c_float)(), C.c_uint64(), C.c_uint64()
        err = C.create_string_buffer(_ERR)
        if _LIB.pdk_st_fp8_channel_view(self._h, prefix.encode(), C.byref(w), C.byref(sc), C.byref(n), C.byref(k),
                                        err, _ERR) != 0:
            raise FormatError("Header", err.value.decode(errors="replace"))
        return dict(weight=_view(w, n.value * k.value, self).reshape(n.value, k.value),
                    scales=np.ctypeslib.as_array(sc, shape=(n.value,)).copy(), n=n.value, k=k.value)


def nvfp4_gguf_repack_rows(src, rows, in_dim):
    """gguf_nvfp4.rs:34-83 -> (codes [rows, in/2], scales [rows, in/16], nan_scales)."""
    src = np.ascontiguousarray(src, np.uint8)
    codes = np.zeros(rows * in_dim // 2, np.uint8)
    scales = np.zeros(rows * in_dim // 16, np.uint8)
    nans, err = C.c_uint64(), C.create_string_buffer(_ERR)
    rc = _LIB.pdk_nvfp4_gguf_repack_rows(src.ctypes.data_as(C.c_void_p), C.c_uint64(src.size), C.c_uint64(rows),
                                         C.c_uint64(in_dim), codes.ctypes.data_as(C.c_void_p),
                                         scales.ctypes.data_as(C.c_void_p), C.byref(nans), err, _ERR)
    if rc != 0:
        raise FormatError("Repack", err.value.decode(errors="replace"))
    return codes.reshape(rows, -1), scales.reshape(rows, -1), nans.value
