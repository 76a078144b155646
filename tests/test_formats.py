"""Host-side formats (include/paddock_host.h): weight-format table, GGUF and
safetensors readers on well-formed and hostile files, quantized checkpoint
views and the GGUF-NVFP4 row repack.  Replays the reference's own unit tests
where it has them (ggml_type.rs:208-257, gguf_nvfp4.rs:115-157, modelopt.rs:443-460)."""
import json
import struct

import numpy as np
import pytest

import oracle
from paddock_b200 import formats as F


# ---- ggml_type.rs:208-257 ---------------------------------------------------
def test_block_layouts_and_sizing():
    assert F.byte_size(39, 2880) == 1530                    # mxfp4_sizing_matches_gpt_oss_expectations
    assert F.byte_size(143, 17408 * 5120) == 19_496_960     # prism_ternary_sizing...
    assert F.byte_size(142, 17408 * 5120) == 23_674_880
    assert F.byte_size(143, 128) == 28 and F.byte_size(142, 128) == 34
    assert F.block_layout(99) is None and F.byte_size(99, 64) is None   # unknown_types_are_carried_not_dropped
    assert F.byte_size(12, 100) is None                     # partial_blocks_are_rejected
    assert F.block_layout(8) == (32, 34) and F.block_layout(12) == (256, 144)
    assert F.block_layout(39) == (32, 17) and F.block_layout(40) == (64, 36) and F.block_layout(30) == (1, 2)
    # plane sizes of the benchmark shapes
    assert F.byte_size(8, 17408 * 5120) == 94_699_520
    assert F.byte_size(12, 25600 * 5120) == 73_728_000


# ---- GGUF writer for tests (the counterpart of paddock-models/src/testutil.rs) --
def gstr(s):
    b = s.encode() if isinstance(s, str) else s
    return struct.pack("<Q", len(b)) + b


def build_gguf(tensors, kv=(), version=3, alignment=None, magic=b"GGUF", n_tensors=None, pad_data=True):
    """tensors: list of (name, dims, raw_type, payload bytes)."""
    kv = list(kv)
    if alignment is not None:
        kv.append(("general.alignment", 4, struct.pack("<I", alignment)))
    align = alignment or 32
    head = magic + struct.pack("<IQQ", version, len(tensors) if n_tensors is None else n_tensors, len(kv))
    for key, ty, payload in kv:
        head += gstr(key) + struct.pack("<I", ty) + payload
    infos, data = b"", b""
    for name, dims, ty, payload in tensors:
        off = len(data)
        infos += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ty, off)
        data += payload
        if pad_data:
            data += b"\0" * (-len(data) % align)
    head += infos
    head += b"\0" * (-len(head) % align)
    return head + data


def q8_payload(rows, k, seed):
    return oracle.quantize_q8_0(oracle.fill_normal(rows * k, seed, 0.02)).tobytes()


def test_gguf_round_trip(tmp_path):
    p0, p1 = q8_payload(4, 64, 1), oracle.quantize_q4_k(oracle.fill_normal(2 * 256, 2, 0.02)).tobytes()
    kv = [("general.architecture", 8, gstr("gpt-oss")), ("gpt-oss.block_count", 4, struct.pack("<I", 24)),
          ("tokenizer.tokens", 9, struct.pack("<IQ", 8, 2) + gstr("a") + gstr("bc"))]
    blob = build_gguf([("blk.0.ffn_up.weight", [64, 4], 8, p0), ("blk.0.ffn_down.weight", [256, 2], 12, p1)], kv)
    path = tmp_path / "m.gguf"
    path.write_bytes(blob)
    for g in (F.Gguf.open(str(path)), F.Gguf.parse(blob)):
        assert g.version == 3 and g.alignment == 32 and g.data_offset % 32 == 0
        assert g.meta_str("general.architecture") == "gpt-oss" and g.meta_u64("gpt-oss.block_count") == 24
        assert g.meta_u64("missing") is None
        names = [t[0] for t in g.tensors()]
        assert names == ["blk.0.ffn_up.weight", "blk.0.ffn_down.weight"]
        data, ty, dims = g.tensor_bytes("blk.0.ffn_up.weight")
        assert ty == 8 and dims == [64, 4] and data.tobytes() == p0
        data, ty, dims = g.tensor_bytes("blk.0.ffn_down.weight")
        assert ty == 12 and dims == [256, 2] and data.tobytes() == p1
        with pytest.raises(F.FormatError):
            g.tensor_bytes("nope")
        g.close()


@pytest.mark.parametrize("blob,kind", [
    (b"GGML" + bytes(28), "BadMagic"),
    (build_gguf([], version=1), "UnsupportedVersion"),
    (build_gguf([], version=4), "UnsupportedVersion"),
    (build_gguf([("t", [64, 4], 8, q8_payload(4, 64, 3))])[:40], "Truncated"),
    (build_gguf([], n_tensors=1 << 40), "CountTooLarge"),
    (b"GGUF" + struct.pack("<IQQ", 3, 0, 1 << 30), "CountTooLarge"),
    (build_gguf([], kv=[("k", 8, struct.pack("<Q", 1 << 40))]), "CountTooLarge"),
    (build_gguf([], kv=[("k", 8, struct.pack("<Q", 2) + b"\xff\xfe")]), "BadUtf8"),
    (build_gguf([], kv=[("k", 77, b"")]), "UnknownValueType"),
    (build_gguf([], kv=[("k", 9, (struct.pack("<IQ", 9, 1)) * 5 + struct.pack("<IQ", 4, 0))]), "ArrayTooDeep"),
    (build_gguf([], alignment=24), "BadAlignment"),
    (build_gguf([("t", [64] * 9, 8, b"")]), "BadTensor"),
    (build_gguf([("t", [64, 4], 8, q8_payload(4, 64, 3)), ("t", [64, 4], 8, q8_payload(4, 64, 4))]), "DuplicateTensor"),
    (build_gguf([("t", [64, 400], 8, q8_payload(4, 64, 3))]), "BadTensor"),               # extends past end of file
    (build_gguf([("a", [32], 8, bytes(34)), ("b", [32], 8, bytes(34))], pad_data=False), "BadTensor"),  # misaligned offset
])
def test_gguf_hostile_files_are_refused(blob, kind):
    with pytest.raises(F.FormatError) as e:
        F.Gguf.parse(blob)
    assert e.value.kind == kind


def test_gguf_unsizable_tensor_only_needs_offset_in_range():
    blob = build_gguf([("odd", [100], 12, bytes(64))])         # Q4_K with 100 elements: no byte size
    g = F.Gguf.parse(blob)
    assert g.tensors()[0][4] == 0
    with pytest.raises(F.FormatError):
        g.tensor_bytes("odd")


# ---- safetensors ---------------------------------------------------------------
def build_st(tensors, extra=None):
    """tensors: {name: (dtype, shape, bytes)}."""
    header, data = {}, b""
    for name, (dt, shape, payload) in tensors.items():
        header[name] = {"dtype": dt, "shape": shape, "data_offsets": [len(data), len(data) + len(payload)]}
        data += payload
    header["__metadata__"] = {"format": "pt"}
    if extra:
        header.update(extra)
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


def test_safetensors_file_and_sharded_dir(tmp_path):
    a = np.arange(24, dtype=np.float32)
    b = np.arange(16, dtype=np.uint8)
    (tmp_path / "one.safetensors").write_bytes(build_st({"x": ("F32", [4, 6], a.tobytes()), "y": ("U8", [16], b.tobytes())}))
    st = F.Safetensors(str(tmp_path / "one.safetensors"))
    assert len(st) == 2
    dt, shape, data = st.bytes("x")
    assert dt == "F32" and shape == [4, 6] and data.tobytes() == a.tobytes()
    assert st.bytes("zz") is None
    d = tmp_path / "model"
    d.mkdir()
    (d / "s1.safetensors").write_bytes(build_st({"x": ("F32", [4, 6], a.tobytes())}))
    (d / "s2.safetensors").write_bytes(build_st({"y": ("U8", [16], b.tobytes())}))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    sh = F.Safetensors(str(d))
    assert len(sh) == 2 and sh.bytes("y")[2].tobytes() == b.tobytes()


@pytest.mark.parametrize("blob", [
    b"\x01\x02",                                                      # shorter than the length prefix
    struct.pack("<Q", 1 << 40) + b"{}",                               # header length exceeds file
    struct.pack("<Q", 5) + b"[1,2]",                                  # not an object
    struct.pack("<Q", 7) + b'{"a": }',                                # bad JSON
    build_st({}, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 64]}}),      # offsets past the data
    build_st({"t": ("F32", [3], bytes(8))}),                          # shape x dtype != bytes
    build_st({}, {"t": {"shape": [2], "data_offsets": [0, 0]}}),      # missing dtype
])
def test_safetensors_hostile_headers_are_refused(tmp_path, blob):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(blob)
    with pytest.raises(F.FormatError):
        F.Safetensors(str(p))


def test_sharded_index_may_not_leave_the_directory(tmp_path):
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../evil.safetensors"}}))
    with pytest.raises(F.FormatError):
        F.Safetensors(str(tmp_path))


# ---- quantized views ---------------------------------------------------------------
def test_nvfp4_view_both_dialects_and_dequant(tmp_path):
    n, k = 8, 64
    w = oracle.fill_normal(n * k, 21, 0.02)
    scale2 = np.float32(np.abs(w).max() / (6 * 448))
    q, s = oracle.quantize_nvf4(w, scale2)
    modelopt = {"l.weight": ("U8", [n, k // 2], q.tobytes()), "l.weight_scale": ("F8_E4M3", [n, k // 16], s.tobytes()),
                "l.weight_scale_2": ("F32", [], scale2.tobytes())}
    llmc = {"l.weight_packed": ("U8", [n, k // 2], q.tobytes()), "l.weight_scale": ("F8_E4M3", [n, k // 16], s.tobytes()),
            "l.weight_global_scale": ("F32", [1], np.float32(1.0 / scale2).tobytes())}
    for i, tensors in enumerate((modelopt, llmc)):
        p = tmp_path / f"m{i}.safetensors"
        p.write_bytes(build_st(tensors))
        v = F.Safetensors(str(p)).nvfp4_view("l")
        assert (v["n"], v["k"]) == (n, k)
        assert np.array_equal(v["packed"].reshape(-1), q) and np.array_equal(v["scales"].reshape(-1), s)
        assert np.isclose(v["scale2"], scale2, rtol=1e-6)
        deq = oracle.dequant_nvfp4(v["packed"], v["scales"], v["scale2"], k, n)
        assert np.linalg.norm(deq.reshape(-1) - w) / np.linalg.norm(w) < 0.2
    bad = dict(modelopt)
    bad["l.weight_scale"] = ("F8_E4M3", [n, 3], s.tobytes()[:n * 3])
    p = tmp_path / "bad.safetensors"
    p.write_bytes(build_st(bad))
    with pytest.raises(F.FormatError):
        F.Safetensors(str(p)).nvfp4_view("l")
    neg = dict(llmc)
    neg["l.weight_global_scale"] = ("F32", [1], np.float32(-1.0).tobytes())
    p.write_bytes(build_st(neg))
    with pytest.raises(F.FormatError):
        F.Safetensors(str(p)).nvfp4_view("l")


def test_fp8_channel_view_reads_both_exports(tmp_path):
    # modelopt.rs:443-460 fp8_row_scales_read_both_exports
    n, k = 2, 16
    w = bytes(range(n * k))
    bf = bytes([0x80, 0x3f, 0x00, 0x40])                               # bf16 1.0, 2.0
    p = tmp_path / "c.safetensors"
    p.write_bytes(build_st({"l.weight": ("F8_E4M3", [n, k], w), "l.weight_scale": ("BF16", [n, 1], bf)}))
    v = F.Safetensors(str(p)).fp8_channel_view("l")
    assert v["scales"].tolist() == [1.0, 2.0] and v["weight"].tobytes() == w
    s = np.float32(0.0031415927)
    p.write_bytes(build_st({"l.weight": ("F8_E4M3", [n, k], w), "l.weight_scale": ("F32", [], s.tobytes())}))
    v = F.Safetensors(str(p)).fp8_channel_view("l")
    assert v["scales"].view(np.uint32).tolist() == [s.view(np.uint32)] * 2
    p.write_bytes(build_st({"l.weight": ("F8_E4M3", [n, k], w), "l.weight_scale": ("BF16", [3, 1], bf + bf[:2])}))
    with pytest.raises(F.FormatError):
        F.Safetensors(str(p)).fp8_channel_view("l")


# ---- gguf_nvfp4.rs:115-157 ------------------------------------------------------------
def ggml_nvfp4_value(blk, e):
    s, m = e // 16, e % 16
    byte = blk[4 + s * 8 + (m % 8)]
    code = byte & 0x0F if m < 8 else byte >> 4
    d = 0.0 if blk[s] == 0x7F else oracle.e4m3_to_f32(blk[s])
    return np.float32(oracle.e2m1_to_f32(code)) * np.float32(d)


def test_nvfp4_gguf_repack_every_element_keeps_its_value():
    rows, in_dim = 3, 128
    seed, src = 0x2545F491, bytearray()
    for _ in range(rows * in_dim // 64):
        for i in range(36):
            seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
            src.append(((seed >> 24) & 0x7E) if i < 4 else (seed >> 24) & 0xFF)
    src[1] = 0x7F
    codes, scales, nans = F.nvfp4_gguf_repack_rows(np.frombuffer(bytes(src), np.uint8), rows, in_dim)
    assert nans == 1
    for r in range(rows):
        for e in range(in_dim):
            blk = src[(r * in_dim + e) // 64 * 36:][:36]
            want = ggml_nvfp4_value(blk, e % 64)
            byte = codes[r, e // 2]
            code = byte & 0x0F if e % 2 == 0 else byte >> 4
            got = np.float32(oracle.e2m1_to_f32(int(code))) * np.float32(oracle.e4m3_to_f32(int(scales[r, e // 16])))
            assert got.view(np.uint32) == np.float32(want).view(np.uint32), (r, e)


def test_nvfp4_gguf_repack_refuses_signed_scale_and_short_tensor():
    blk = np.zeros(36, np.uint8)
    blk[2] = 0x81
    for src, rows, k in ((blk, 1, 64), (np.zeros(35, np.uint8), 1, 64), (np.zeros(36, np.uint8), 1, 32)):
        with pytest.raises(F.FormatError):
            F.nvfp4_gguf_repack_rows(src, rows, k)


# ---- split families (split.rs:64-100, mapped.rs tests) ------------------------------------------
def test_split_names_parse_strictly():
    assert F.parse_split_name("/m/gpt-oss-120b-mxfp4-00001-of-00003.gguf") == ("/m/gpt-oss-120b-mxfp4", 1, 3)
    for name in ["model.gguf", "model-1-of-3.gguf", "model-00000-of-00003.gguf", "model-00004-of-00003.gguf",
                 "model-00001-of-00000.gguf", "-00001-of-00002.gguf", "model-00001-of-00003.notgguf",
                 "model-abcde-of-00003.gguf"]:
        assert F.parse_split_name(name) is None, name


def u16kv(key, v):
    return (key, 2, struct.pack("<H", v))


def i32kv(key, v):
    return (key, 5, struct.pack("<i", v))


def write_family(tmp_path, n_shards, total=None, stem="fam", **over):
    """n_shards files of one Q8_0 tensor each; `over` patches single shards' metadata."""
    payloads = []
    for s in range(n_shards):
        p = q8_payload(2, 64, 50 + s)
        payloads.append(p)
        kv = [u16kv("split.no", over.get("no", {}).get(s, s)), u16kv("split.count", over.get("count", {}).get(s, n_shards))]
        if s in over.get("drop_no", ()):
            kv = kv[1:]
        if s == 0:
            kv.append(("general.architecture", 8, gstr("llama")))
            if total is not False:
                kv.append(i32kv("split.tensors.count", n_shards if total is None else total))
        name = over.get("names", {}).get(s, f"blk.{s}.w")
        (tmp_path / f"{stem}-{s + 1:05d}-of-{n_shards:05d}.gguf").write_bytes(build_gguf([(name, [64, 2], 8, p)], kv))
    return str(tmp_path / f"{stem}-00001-of-{n_shards:05d}.gguf"), payloads


def test_split_family_resolves_each_tensor_to_its_shard(tmp_path):
    first, payloads = write_family(tmp_path, 3)
    m = F.MappedGguf(first)
    assert m.shard_count() == 3 and m.tensor_count() == 3
    assert m.meta_str("general.architecture") == "llama" and m.meta_u64("split.count") == 3
    assert [(t[0], t[4]) for t in m.tensor_infos()] == [("blk.0.w", 0), ("blk.1.w", 1), ("blk.2.w", 2)]
    for s in range(3):
        data, ty, dims, shard = m.tensor_bytes(f"blk.{s}.w")
        assert (ty, dims, shard) == (8, [64, 2], s) and data.tobytes() == payloads[s]
        assert m.shard_path(s).endswith(f"fam-{s + 1:05d}-of-00003.gguf")
    import os
    assert m.total_len() == sum(os.path.getsize(m.shard_path(s)) for s in range(3))
    with pytest.raises(F.FormatError) as e:
        m.tensor_bytes("blk.9.w")
    assert e.value.kind == "NoSuchTensor"
    m.close()


def test_single_file_keeps_its_behaviour(tmp_path):
    p = q8_payload(2, 64, 7)
    path = tmp_path / "plain.gguf"
    path.write_bytes(build_gguf([("w", [64, 2], 8, p)], [u16kv("split.count", 1)]))
    m = F.MappedGguf(str(path))
    assert m.shard_count() == 1 and m.tensor_bytes("w")[0].tobytes() == p


def test_split_family_errors_are_load_errors(tmp_path):
    def kind(path):
        with pytest.raises(F.FormatError) as e:
            F.MappedGguf(path)
        return e.value.kind

    d = lambda n: (tmp_path / n).mkdir() or tmp_path / n
    first, _ = write_family(d("a"), 3)
    assert kind(first.replace("00001-of", "00002-of")) == "NotFirstSplit"      # opened through the second shard
    import os
    os.remove(first.replace("00001-of", "00003-of"))
    assert kind(first) == "Io"                                                  # a sibling is missing
    first, _ = write_family(d("b"), 2, no={1: 0})
    assert kind(first) == "ShardMismatch"                                       # a copy of shard 1 in shard 2's place
    first, _ = write_family(d("c"), 2, count={1: 3})
    assert kind(first) == "ShardMismatch"
    first, _ = write_family(d("d"), 2, drop_no=(1,))
    assert kind(first) == "MissingSplitKey"
    first, _ = write_family(d("e"), 2, total=5)
    assert kind(first) == "TensorCountMismatch"
    first, _ = write_family(d("f"), 2, total=False)
    assert kind(first) == "MissingSplitKey"
    first, _ = write_family(d("g"), 2, names={1: "blk.0.w"})
    assert kind(first) == "DuplicateAcrossShards"
    # metadata says split, the name does not follow the convention
    odd = d("h") / "model.gguf"
    odd.write_bytes(build_gguf([("w", [64, 2], 8, q8_payload(2, 64, 1))],
                               [u16kv("split.no", 0), u16kv("split.count", 2), i32kv("split.tensors.count", 2)]))
    assert kind(str(odd)) == "SplitNameMismatch"
    big = d("i") / "m-00001-of-04000.gguf"
    big.write_bytes(build_gguf([], [u16kv("split.no", 0), u16kv("split.count", 4000)]))
    assert kind(str(big)) == "TooManySplits"
