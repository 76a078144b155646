"""Bit-exact parity of the dequant / repack kernels against the CPU oracle
(the pattern of crates/paddock-engine/tests/pack_parity.rs:14-118)."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import dev, host
from test_oracle_kat import pack_parity_mxfp4_bytes, pack_parity_q8_bytes

pytestmark = pytest.mark.gpu


def run_dequant(pack, name, raw, n_units, n_out, *extra):
    d_in = dev(np.frombuffer(raw, np.uint8) if isinstance(raw, bytes) else raw)
    d_out = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    pack.call(name, d_in, d_out, n_units, *extra)
    torch.cuda.synchronize()
    return d_out.cpu().numpy()


def test_pack_parity_vectors_bit_exact(pack):
    # tests/pack_parity.rs: 3 MXFP4 blocks (normal, 0.5, denormal scale) + 1 Q8_0 block
    raw = pack_parity_mxfp4_bytes()
    got = run_dequant(pack, "mxfp4_dequant_f32", raw, 3, 96)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_mxfp4(raw).view(np.uint32))
    raw8 = pack_parity_q8_bytes()
    got8 = run_dequant(pack, "q8_0_dequant_f32", raw8, 1, 32)
    assert np.array_equal(got8.view(np.uint32), oracle.dequant_q8_0(raw8).view(np.uint32))


def test_mxfp4_every_scale_byte_and_nibble(pack):
    blocks = bytearray()
    for e in range(256):
        blocks.append(e)
        blocks.extend(((e + j) * 0x11 + j) & 0xFF for j in range(16))
    raw = bytes(blocks)
    got = run_dequant(pack, "mxfp4_dequant_f32", raw, 256, 256 * 32)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_mxfp4(raw).view(np.uint32))


@pytest.mark.parametrize("n_blocks", [1, 7, 160, 5120 * 17408 // 32 // 64])
def test_q8_0_dequant_and_repack(pack, n_blocks):
    w = oracle.fill_normal(n_blocks * 32, 101 + n_blocks, 0.02)
    raw = oracle.quantize_q8_0(w)
    got = run_dequant(pack, "q8_0_dequant_f32", raw, n_blocks, n_blocks * 32)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_q8_0(raw).view(np.uint32))
    d_src = dev(raw)
    d_data = torch.zeros(n_blocks * 32, dtype=torch.int8, device="cuda")
    d_scale = torch.zeros(n_blocks, dtype=torch.float16, device="cuda")
    pack.call("q8_0_repack", d_src, d_data, d_scale, n_blocks)
    torch.cuda.synchronize()
    want_data, want_scale = oracle.repack_q8_0(raw)
    assert np.array_equal(host(d_data, np.int8), want_data)
    assert np.array_equal(host(d_scale, np.uint16), want_scale)


@pytest.mark.parametrize("n_blocks", [1, 90, 2880 * 2880 // 32])
def test_mxfp4_dequant_and_repack(pack, n_blocks):
    w = oracle.fill_normal(n_blocks * 32, 201 + n_blocks, 0.02)
    raw = oracle.quantize_mxfp4(w)
    got = run_dequant(pack, "mxfp4_dequant_f32", raw, n_blocks, n_blocks * 32)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_mxfp4(raw).view(np.uint32))
    d_src = dev(raw)
    d_data = torch.zeros(n_blocks * 16, dtype=torch.uint8, device="cuda")
    d_scale = torch.zeros(n_blocks, dtype=torch.uint8, device="cuda")
    pack.call("mxfp4_repack", d_src, d_data, d_scale, n_blocks)
    torch.cuda.synchronize()
    want_data, want_scale = oracle.repack_mxfp4(raw)
    assert np.array_equal(host(d_data, np.uint8), want_data)
    assert np.array_equal(host(d_scale, np.uint8), want_scale)


@pytest.mark.parametrize("n_super", [1, 20, 20 * 257])
def test_q4_k_dequant_bit_exact(pack, n_super):
    w = oracle.fill_normal(n_super * 256, 301 + n_super, 0.02)
    raw = oracle.quantize_q4_k(w)
    got = run_dequant(pack, "kquant_dequant", raw, n_super, n_super * 256, 12)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_q4_k(raw).view(np.uint32))


def test_q4_k_dequant_random_bytes_bit_exact(pack):
    # every 6-bit scale/min packing path, not only what the quantizer emits
    rng = np.random.default_rng(5)
    n_super = 64
    raw = rng.integers(0, 256, n_super * 144, dtype=np.uint8)
    hdr = np.frombuffer(np.array([0.013, 0.021], np.float16).tobytes(), np.uint8)
    for b in range(n_super):
        raw[b * 144:b * 144 + 4] = hdr
    got = run_dequant(pack, "kquant_dequant", raw, n_super, n_super * 256, 12)
    assert np.array_equal(got.view(np.uint32), oracle.dequant_q4_k(raw).view(np.uint32))


def test_q4_k_repack_layout(pack):
    """packs/cuda/src/quant/kquant.cuh:37-54: nibbles verbatim + 24-byte record."""
    n_super = 40
    raw = oracle.quantize_q4_k(oracle.fill_normal(n_super * 256, 77, 0.02))
    d_data = torch.zeros(n_super * 128, dtype=torch.uint8, device="cuda")
    d_sc = torch.full((n_super * 24,), 0xAA, dtype=torch.uint8, device="cuda")
    pack.call("kquant_repack", dev(raw), d_data, d_sc, n_super, 12)
    torch.cuda.synchronize()
    data, rec = host(d_data, np.uint8).reshape(n_super, 128), host(d_sc, np.uint8).reshape(n_super, 24)
    src = raw.reshape(n_super, 144)
    assert np.array_equal(data, src[:, 16:])
    assert np.array_equal(rec[:, 0:4], src[:, 0:4])
    assert not rec[:, 20:24].any()
    for b in range(n_super):
        for j in range(8):
            s = src[b, 4:16]
            if j < 4:
                sc, m = s[j] & 63, s[j + 4] & 63
            else:
                sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)
                m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
            assert rec[b, 4 + j] == sc and rec[b, 12 + j] == m


def test_empty_inputs_are_accepted(pack):
    for name, extra in (("q8_0_dequant_f32", ()), ("mxfp4_dequant_f32", ()), ("kquant_dequant", (12,))):
        pack.call(name, 0, 0, 0, *extra)
    pack.call("q8_0_repack", 0, 0, 0, 0)
    pack.call("mxfp4_repack", 0, 0, 0, 0)
    pack.call("kquant_repack", 0, 0, 0, 0, 12)


def test_unknown_kquant_dtype_is_refused(pack):
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    assert pack.status("kquant_dequant", buf, buf, 1, 99) == 1      # cudaErrorInvalidValue
    assert pack.status("kquant_dequant", buf, buf, 1, 16) == 1      # IQ2_XXS: no kernel class in this pack


def test_add_inplace(pack):
    a = torch.arange(1000, dtype=torch.float32, device="cuda")
    b = torch.ones(1000, dtype=torch.float32, device="cuda")
    pack.call("add_inplace_f32", a, b, 1000)
    torch.cuda.synchronize()
    assert torch.equal(a.cpu(), torch.arange(1000, dtype=torch.float32) + 1)
