"""Pins the CPU oracle to the known-answer vectors the reference's own tests
hold for this path.  Each test names the reference test it replays."""
import math
import struct

import numpy as np
import pytest

import oracle


def bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def from_bits(u):
    return struct.unpack("<f", struct.pack("<I", u))[0]


# crates/paddock-kernels/src/reference/mod.rs:121-128 e8m0_half_matches_known_points
def test_e8m0_half_known_points():
    assert oracle.e8m0_half_to_f32(128) == 1.0
    assert oracle.e8m0_half_to_f32(127) == 0.5
    assert oracle.e8m0_half_to_f32(129) == 2.0
    assert bits(oracle.e8m0_half_to_f32(0)) == 0x00200000
    assert bits(oracle.e8m0_half_to_f32(1)) == 0x00400000


def test_e8m0_half_all_codes_are_powers_of_two():
    for e in range(256):
        assert oracle.e8m0_half_to_f32(e) == math.ldexp(1.0, e - 128)


# reference/mod.rs:131-147 mxfp4_dequant_hand_computed_block
def test_mxfp4_hand_block():
    block = bytearray(17)
    block[0], block[1], block[2] = 128, 0x51, 0x9F
    out = oracle.dequant_mxfp4(block)
    assert out[0] == 1.0 and out[16] == 6.0
    assert out[1] == -12.0 and out[17] == -1.0
    assert out[2] == 0.0


# reference/mod.rs:150-157 mxfp4_scale_applies
def test_mxfp4_scale_applies():
    block = bytearray(17)
    block[0], block[1] = 129, 0x07
    assert oracle.dequant_mxfp4(block)[0] == 24.0


# reference/mod.rs:160-168 q8_0_dequant_hand_computed_block
def test_q8_0_hand_block():
    block = bytearray(34)
    block[0:2] = struct.pack("<e", 0.5)
    block[2] = 100
    block[3] = (-100) & 0xFF
    out = oracle.dequant_q8_0(block)
    assert out[0] == 50.0 and out[1] == -50.0


# reference/mod.rs:171-175 length_mismatches_are_errors
def test_length_mismatches_are_errors():
    out = np.zeros(32, np.float32)
    with pytest.raises(oracle.DequantError):
        oracle.dequant_mxfp4(bytes(16), out)
    with pytest.raises(oracle.DequantError):
        oracle.dequant_mxfp4(bytes(17), out[:31])
    with pytest.raises(oracle.DequantError):
        oracle.dequant_q8_0(bytes(33), out)


def pack_parity_mxfp4_bytes():
    """crates/paddock-engine/tests/pack_parity.rs:33-37: three blocks exercising
    the scale paths (normal, 0.5, denormal)."""
    buf = bytearray()
    for e, fill in ((128, 0x10), (127, 0xFF), (1, 0x73)):
        buf.append(e)
        buf.extend((fill + j * 0x11) & 0xFF for j in range(16))
    return bytes(buf)


def pack_parity_q8_bytes():
    """tests/pack_parity.rs:80-81: one block, scale 0.5, values spanning int8."""
    return struct.pack("<e", 0.5) + bytes(((j * 8 - 128) & 0xFF) for j in range(32))


def test_pack_parity_vectors_against_independent_formula():
    fp4 = [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]
    data = pack_parity_mxfp4_bytes()
    got = oracle.dequant_mxfp4(data)
    for b in range(3):
        blk = data[b * 17:(b + 1) * 17]
        d = math.ldexp(1.0, blk[0] - 128)
        for j in range(16):
            assert bits(got[b * 32 + j]) == bits(np.float32(fp4[blk[1 + j] & 15] * d))
            assert bits(got[b * 32 + j + 16]) == bits(np.float32(fp4[blk[1 + j] >> 4] * d))
    got8 = oracle.dequant_q8_0(pack_parity_q8_bytes())
    for j in range(32):
        assert got8[j] == (j * 8 - 128) * 0.5


# crates/paddock-models/src/modelopt.rs:431-441 e2m1_covers_all_sixteen_codes
def test_e2m1_all_sixteen_codes():
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    for code, w in enumerate(want):
        assert bits(oracle.e2m1_to_f32(code)) == bits(w), hex(code)


# modelopt.rs:462-472 e4m3_decode_spots
def test_e4m3_decode_spots():
    assert bits(oracle.e4m3_to_f32(0x00)) == bits(0.0)
    assert bits(oracle.e4m3_to_f32(0x80)) == bits(-0.0)
    assert oracle.e4m3_to_f32(0x38) == 1.0
    assert oracle.e4m3_to_f32(0x39) == 1.125
    assert oracle.e4m3_to_f32(0x7e) == 448.0
    assert oracle.e4m3_to_f32(0x01) == 2.0 ** -9
    assert oracle.e4m3_to_f32(0xc0) == -2.0
    assert math.isnan(oracle.e4m3_to_f32(0x7f))
    assert math.isnan(oracle.e4m3_to_f32(0xff))


def test_e4m3_encode_round_trips_and_rounds_to_nearest_even():
    finite = [c for c in range(256) if (c & 0x7f) != 0x7f]
    for c in finite:
        v = oracle.e4m3_to_f32(c)
        if v == 0.0:
            continue
        assert oracle.f32_to_e4m3(v) == c
    # ties: midway between neighbours goes to the even mantissa
    for c in range(0x01, 0x7e):
        lo, hi = oracle.e4m3_to_f32(c), oracle.e4m3_to_f32(c + 1)
        mid = (lo + hi) / 2
        want = c if (c & 1) == 0 else c + 1
        assert oracle.f32_to_e4m3(mid) == want, hex(c)
    assert oracle.f32_to_e4m3(1e9) == 0x7e          # saturate to finite
    assert oracle.f32_to_e4m3(-1e9) == 0xfe
    assert oracle.f32_to_e4m3(460.0) == 0x7e
    assert oracle.f32_to_e4m3(2.0 ** -11) == 0x00   # half the smallest subnormal: tie to even


# packs/cuda/src/quant/e2m1.cuh:12-26: grid and tie rules
def test_e2m1_rn_ties():
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i, g in enumerate(grid):
        assert oracle.e2m1_rn(g) == i
        assert oracle.e2m1_rn(-g) == (i | 8 if g else 0)
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6}
    for v, code in ties.items():
        assert oracle.e2m1_rn(v) == code
    assert oracle.e2m1_rn(100.0) == 7


# crates/paddock-engine/tests/gpu_kquant_parity.rs:27-36 scale_min_k4, checked
# against a bit-level restatement of ggml's 12-byte packing.
def test_q4_k_dequant_against_python_restatement():
    rng = np.random.default_rng(7)
    n_super = 6
    raw = rng.integers(0, 256, n_super * 144, dtype=np.uint8)
    for b in range(n_super):          # keep d/dmin finite f16
        raw[b * 144:b * 144 + 4] = np.frombuffer(struct.pack("<ee", 0.01 * (b + 1), 0.02 * (b + 1)), np.uint8)
    got = oracle.dequant_q4_k(raw)
    want = np.zeros(n_super * 256, np.float32)
    for b in range(n_super):
        s = raw[b * 144:(b + 1) * 144]
        d, dmin = (np.float32(v) for v in struct.unpack("<ee", bytes(s[0:4])))
        sc12, qs = s[4:16], s[16:144]
        for j in range(8):
            if j < 4:
                sc, m = sc12[j] & 63, sc12[j + 4] & 63
            else:
                sc = (sc12[j + 4] & 0xF) | ((sc12[j - 4] >> 6) << 4)
                m = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4)
            dj = np.float32(d * np.float32(sc))
            mj = np.float32(dmin * np.float32(m))
            for l in range(32):
                q = qs[(j >> 1) * 32 + l]
                v = (q >> 4) if (j & 1) else (q & 0xF)
                want[b * 256 + j * 32 + l] = np.float32(dj * np.float32(v)) - mj
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# crates/paddock-engine/src/gpu_model/laguna/dflash.rs:233-253
def test_q8_0_quantizer_round_trip():
    w = oracle.fill_normal(32 * 64, 11, 0.02)
    blocks = oracle.quantize_q8_0(w)
    assert blocks.size == 64 * 34
    deq = oracle.dequant_q8_0(blocks)
    amax = np.abs(w.reshape(64, 32)).max(axis=1)
    err = np.abs(deq - w).reshape(64, 32).max(axis=1)
    assert np.all(err <= amax / 127.0 * 0.5 + amax * 2.0 ** -10)
    q = blocks.reshape(64, 34)[:, 2:].view(np.int8)
    assert np.abs(q.astype(np.int32)).max() == 127


def test_q4_k_quantizer_round_trip():
    w = oracle.fill_normal(256 * 40, 12, 0.02)
    blocks = oracle.quantize_q4_k(w)
    deq = oracle.dequant_q4_k(blocks)
    rel = np.linalg.norm(deq - w) / np.linalg.norm(w)
    assert rel < 0.12


def test_mxfp4_quantizer_scale_rule():
    # packs/cuda/src/gemm/dense_fp4_w8.cuh:39-46: smallest e with amax/2^e <= 6
    w = np.zeros(32, np.float32)
    w[3] = 6.0
    blk = oracle.quantize_mxfp4(w)
    assert blk[0] == 127 and oracle.dequant_mxfp4(blk)[3] == 6.0
    w[3] = 6.5
    blk = oracle.quantize_mxfp4(w)
    assert blk[0] == 128
    w = oracle.fill_normal(32 * 50, 13, 0.02)
    deq = oracle.dequant_mxfp4(oracle.quantize_mxfp4(w))
    assert np.linalg.norm(deq - w) / np.linalg.norm(w) < 0.15


def test_nvf4_quantizer_matches_scale_rules():
    # packs/cuda/src/quant/e2m1.cuh:30-41
    x = np.zeros(32, np.float32)
    x[0] = 6.0          # amax/6 = 1.0 -> scale byte 0x38
    x[16] = 1e-6        # tiny: scale rounds to 0 -> floor to the smallest subnormal
    q, s = oracle.quantize_nvf4(x)
    assert s[0] == 0x38 and (q[0] & 0xF) == 7
    assert s[1] == 0x01
    z, sz = oracle.quantize_nvf4(np.zeros(16, np.float32))
    assert sz[0] == 0 and not z.any()


def test_quantize_e4m3_row_pow2_bound():
    # packs/cuda/src/gemm/dense_f8_decode.cuh:3213-3219: amax/2^e <= 448
    x = oracle.fill_normal(4 * 512, 14, 1.0).reshape(4, 512)
    x[1] *= 448.0
    q, s = oracle.quantize_e4m3_row_pow2(x, 4, 512)
    for r in range(4):
        amax = np.abs(x[r]).max()
        assert amax / s[r] <= 448.0 and amax / s[r] > 224.0
        assert math.log2(s[r]).is_integer()
    deq = oracle.dequant_fp8_channel(q, s, 512, 4)
    assert np.linalg.norm(deq - x) / np.linalg.norm(x) < 0.04


def test_topk_ties_go_to_lowest_index():
    # packs/cuda/src/attn/decode.cuh:1410-1425
    logits = np.array([[1.0, 3.0, 3.0, 0.0, 3.0, -1.0, 2.0, 2.0]], np.float32)
    idx, w = oracle.moe_topk(logits, 8, 4)
    assert idx.tolist() == [[1, 2, 4, 6]]
    e = np.exp(np.array([3, 3, 3, 2], np.float32) - 3)
    assert np.allclose(w[0], e / e.sum(), rtol=1e-6)


def test_swiglu_oai_reference_points():
    # crates/paddock-kernels/src/reference/ops.rs:27-36
    g = np.array([10.0, -3.0, 0.5], np.float32)
    u = np.array([9.0, -9.0, 0.25], np.float32)
    out = oracle.swiglu_oai(g, u)
    want = []
    for a, b in zip(g, u):
        x = min(a, 7.0)
        y = max(-7.0, min(b, 7.0))
        want.append(x / (1.0 + math.exp(-1.702 * x)) * (y + 1.0))
    assert np.allclose(out, want, rtol=1e-6)


def test_matvec_is_ascending_k_f32():
    # crates/paddock-engine/src/reference/tensor.rs:39-54
    w = oracle.fill_normal(3 * 64, 15, 1.0)
    x = oracle.fill_normal(64, 16, 1.0)
    y = oracle.matvec_f32(w, x, 64, 3)
    for o in range(3):
        acc = np.float32(0)
        for k in range(64):
            acc = np.float32(acc + np.float32(w[o * 64 + k] * x[k]))
        assert bits(y[o]) == bits(acc)


def test_fill_normal_is_thread_count_independent_and_normal():
    a = oracle.fill_normal(100001, 5, 2.0)
    b = oracle.fill_normal(100001, 5, 2.0)
    assert np.array_equal(a, b)
    assert abs(a.mean()) < 0.03 and abs(a.std() - 2.0) < 0.03


def test_add_rmsnorm_hand_values():
    """The fused producer's norm (packs/cuda/src/quant/nvf4.cuh:455-543) on values worked by hand:
    a row of 32 with 3 and 4 in front has mean square 25/32; eps = 0."""
    import numpy as np
    x = np.zeros((1, 32), np.float32)
    x[0, 0], x[0, 1] = 1.0, 4.0
    proj = np.zeros((1, 32), np.float32)
    proj[0, 0] = 2.0
    w = np.full(32, 2.0, np.float32)
    v, out = oracle.add_rmsnorm(x, proj, w, 0.0)
    assert v[0, 0] == 3.0 and v[0, 1] == 4.0
    inv = np.float32(1.0) / np.sqrt(np.float32(25.0 / 32.0))
    assert out[0, 0] == np.float32(np.float32(3.0) * inv) * np.float32(2.0)
    assert abs(float(out[0, 1]) - 8.0 / (25.0 / 32.0) ** 0.5) < 1e-6
    assert not out[0, 2:].any()
    v2, out2 = oracle.add_rmsnorm(x, None, w, 0.0)
    assert v2[0, 0] == 1.0 and abs(float(out2[0, 1]) - 8.0 / (17.0 / 32.0) ** 0.5) < 1e-6


def test_iq4_xs_dequant_against_a_scalar_walk():
    """IQ4_XS (gpu_kquant_parity.rs:19-21, 96-115): 136-byte super-blocks, 6-bit sub-block scales split
    over scales_l / scales_h, ggml's 16-entry code book; the C restatement against a plain Python walk."""
    book = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]
    rng = np.random.default_rng(77)
    raw = rng.integers(0, 256, (3, 136), dtype=np.uint8)
    raw[:, 0:2] = np.array([0.0123, -0.5, 1.0 / 1024], np.float16).view(np.uint8).reshape(3, 2)
    got = oracle.dequant_kquant("iq4_xs", raw.reshape(-1)).reshape(3, 256)
    for b in range(3):
        s = raw[b]
        d = np.frombuffer(s[0:2].tobytes(), np.float16)[0].astype(np.float32)
        sh = int(s[2]) | int(s[3]) << 8
        for ib in range(8):
            ls = (((int(s[4 + ib // 2]) >> (4 * (ib & 1))) & 15) | (((sh >> (2 * ib)) & 3) << 4)) - 32
            dl = np.float32(d * np.float32(ls))
            for j in range(16):
                q = int(s[8 + ib * 16 + j])
                assert got[b, ib * 32 + j] == np.float32(dl * np.float32(book[q & 15]))
                assert got[b, ib * 32 + 16 + j] == np.float32(dl * np.float32(book[q >> 4]))
    with pytest.raises(Exception):
        oracle.dequant_kquant("iq4_xs", raw.reshape(-1)[:100])
