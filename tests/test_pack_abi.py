"""CPU-side checks of the drop-in boundary: the library loads, exports every
symbol include/paddock_pack.h declares, and passes / fails the reference
loader's validation (crates/paddock-kernels/src/loader.rs) the way a pack must."""
import ctypes as C
import os
import re
import subprocess

import pytest

import paddock_b200 as pb
from paddock_b200 import pack as packmod


def declared_functions():
    text = open(pb.header_path()).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(pd_\w+|pdk_\w+|paddock_pack_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(pb.lib_path())
    names = declared_functions()
    assert "paddock_pack_info" in names and "paddock_pack_kernels_v1" in names
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in paddock_pack.h but not exported"


def test_pack_info_matches_abi(pack):
    # abi.rs:8-28: magic "PDKP", abi 2, NUL-terminated ASCII arch tag
    assert pack.info.magic == 0x504B4450
    assert pack.info.abi_version == 2
    assert pack.info.arch_str() == "cuda-sm100a"
    assert C.sizeof(packmod.PackInfo) == 36


def test_kernel_table_shape(pack):
    # abi.rs:12805-12812: 8-byte header + 953 pointers = 7632 bytes
    assert pack.table_size() == 7632 == packmod.TABLE_BYTES
    filled = {i for i in range(packmod.TABLE_SLOTS) if pack.slot_ptr(i)}
    assert filled == set(pb.SLOTS.values())
    # the engine's preflight launches add_inplace_f32 (gpu/mod.rs:507-528)
    assert pack.has("add_inplace_f32")


def test_table_slots_point_at_the_named_exports(pack):
    lib = C.CDLL(pb.lib_path())
    for name, idx in pb.SLOTS.items():
        addr = C.cast(getattr(lib, "pd_" + name), C.c_void_p).value
        assert pack.slot_ptr(idx) == addr, name


def test_missing_slot_is_reported_not_called(pack):
    with pytest.raises(pb.MissingOp):
        pack.fn("rmsnorm_f32")


# ---- loader failure paths (loader.rs:163-194, 253-283) on hostile packs ----

FAKE = r"""
#include <stdint.h>
typedef struct { uint32_t magic, abi; uint8_t arch[16]; uint32_t ver[3]; } Info;
static Info info = { MAGIC, ABI, "fake", {0,0,0} };
static struct { uint32_t size, reserved; void* slot[4]; } table = { TSIZE, 0, {0} };
#if HAVE_INFO
const Info* paddock_pack_info(void) { return NULL_INFO ? 0 : &info; }
#endif
#if HAVE_TABLE
const void* paddock_pack_kernels_v1(void) { return NULL_TABLE ? 0 : &table; }
#endif
"""


def build_fake(tmp_path, name, **defs):
    d = dict(MAGIC="0x504b4450u", ABI="2u", TSIZE="40u", HAVE_INFO="1", HAVE_TABLE="1", NULL_INFO="0",
             NULL_TABLE="0")
    d.update(defs)
    src = tmp_path / f"{name}.c"
    src.write_text(FAKE)
    out = tmp_path / f"lib{name}.so"
    cmd = ["gcc", "-shared", "-fPIC", "-o", str(out), str(src)] + [f"-D{k}={v}" for k, v in d.items()]
    subprocess.check_call(cmd)
    return str(out)


def test_loader_rejects_non_library():
    with pytest.raises(pb.Open):
        pb.KernelPack.load("/definitely/not/a/pack.so")


def test_loader_rejects_library_without_symbols(tmp_path):
    with pytest.raises(pb.NotAPack):
        pb.KernelPack.load(build_fake(tmp_path, "nosym", HAVE_INFO="0"))


def test_loader_rejects_null_descriptor(tmp_path):
    with pytest.raises(pb.BadDescriptor):
        pb.KernelPack.load(build_fake(tmp_path, "nullinfo", NULL_INFO="1"))


def test_loader_rejects_bad_magic(tmp_path):
    with pytest.raises(pb.BadMagic):
        pb.KernelPack.load(build_fake(tmp_path, "magic", MAGIC="0x12345678u"))


def test_loader_rejects_abi_mismatch(tmp_path):
    with pytest.raises(pb.AbiMismatch) as e:
        pb.KernelPack.load(build_fake(tmp_path, "abi", ABI="3u"))
    assert e.value.found == 3 and e.value.expected == 2


def test_loader_rejects_missing_or_truncated_table(tmp_path):
    with pytest.raises(pb.NoKernelTable):
        pb.KernelPack.load(build_fake(tmp_path, "notable", HAVE_TABLE="0"))
    with pytest.raises(pb.BadKernelTable):
        pb.KernelPack.load(build_fake(tmp_path, "nulltable", NULL_TABLE="1"))
    with pytest.raises(pb.BadKernelTable):
        pb.KernelPack.load(build_fake(tmp_path, "short", TSIZE="4u"))


def test_loader_min_copies_a_shorter_table(tmp_path):
    # append-only growth contract: a pack that predates later slots reads as NULL there
    p = pb.KernelPack.load(build_fake(tmp_path, "old", TSIZE="40u"))
    assert p.table_size() == 40
    assert all(p.slot_ptr(i) == 0 for i in range(packmod.TABLE_SLOTS))
    with pytest.raises(pb.MissingOp):
        p.fn("q8_0_gemv_repacked")


def test_slot_indices_and_argument_counts_match_the_reference_table():
    """Every PDK_SLOT_* index of the header is the index of the member of that name in the
    reference's KernelTableV1 (tests/golden/kernel_table_v1.json, generated from
    packs/cuda/src/abi.cuh by tests/golden/gen_kernel_table.py), and every served slot is bound
    here with as many arguments as the reference declares."""
    import json
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kernel_table_v1.json")
    members = json.load(open(golden))["members"]
    assert len(members) == packmod.TABLE_SLOTS
    by_name = {name: (idx, args) for idx, name, args in members}
    assert [m[0] for m in members] == list(range(len(members)))
    assert len(packmod.SLOTS) >= 34
    for name, idx in packmod.SLOTS.items():
        assert name in by_name, name
        assert by_name[name][0] == idx, (name, idx, by_name[name][0])
        if name in packmod._SIGS:
            n_ref = len([a for a in by_name[name][1].split(",") if a.strip()])
            assert len(packmod._SIGS[name]) + 1 == n_ref, (name, packmod._SIGS[name], by_name[name][1])   # + the stream


def test_table_is_resolved_against_the_device_capability():
    """packs/cuda/src/exports.cuh:2118-2400 NULLs what the running die cannot execute; sm_100a
    code loads on compute capability 10.0 only, so any other device gets an empty table."""
    lib = C.CDLL(pb.lib_path())
    buf = (C.c_uint8 * packmod.TABLE_BYTES)()
    fn = lib.pdk_kernels_for_cc
    fn.argtypes = [C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int

    def filled(major, minor):
        assert fn(major, minor, C.addressof(buf)) == 0
        words = (C.c_uint64 * (packmod.TABLE_BYTES // 8)).from_buffer(buf)
        assert words[0] & 0xffffffff == packmod.TABLE_BYTES
        return sum(1 for i in range(packmod.TABLE_SLOTS) if words[1 + i])

    assert filled(10, 0) == len(packmod.SLOTS)
    for cc in [(9, 0), (10, 3), (12, 0), (12, 1), (8, 9)]:
        assert filled(*cc) == 0
    assert fn(10, 0, None) == 1
