"""Cross-check against the reference's own CUDA pack, slot by slot.

`oracle/build_ref.sh` compiles the reference's `packs/cuda/pack.cu` into
`oracle/_ref/pd-cuda-ref.so` (test infrastructure, never shipped).  Both
libraries are opened through the same loader and the same table offsets
(crates/paddock-kernels/src/loader.rs:140-283) and given identical device
operands: dequant / repack / quantizer outputs must be byte-identical, GEMV and
GEMM outputs agree within the stated tolerance.  A slot the reference build
leaves NULL or answers "not supported" for on this device is skipped with that
reason.  The whole module is skipped when the reference library was not built.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, dev, dev_f32, rel_l2
from paddock_b200 import KernelPack
from paddock_b200.pack import LaunchError, MissingOp

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.abspath(oracle.__file__)), "_ref", "pd-cuda-ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("reference pack not built (oracle/build_ref.sh)")
    return KernelPack.load(REF_SO)


def run_both(pack, ref, name, make_args, n_out):
    """Call slot `name` of both packs on operands from make_args(); returns the
    last n_out tensors each call wrote, as numpy byte arrays."""
    outs = []
    for p in (pack, ref):
        args, written = make_args()
        try:
            p.call(name, *args)
        except MissingOp:
            assert p is ref
            pytest.skip(f"reference pack has no {name} on this build")
        except LaunchError as e:
            assert p is ref, e
            pytest.skip(f"reference {name} declined: {e}")
        torch.cuda.synchronize()
        outs.append([w.cpu().numpy().view(np.uint8).copy() for w in written[:n_out]])
    return outs


def assert_bytes_equal(outs):
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def test_reference_pack_descriptor(ref):
    assert ref.info.magic == 0x504B4450 and ref.info.abi_version == 2
    assert ref.table_size() == 7632


def test_mxfp4_and_q8_0_dequant(pack, ref):
    rng = np.random.default_rng(11)
    raw = rng.integers(0, 256, 4096 * 17, dtype=np.uint8)
    raw[::17] = rng.integers(0, 255, 4096, dtype=np.uint8)

    def mk():
        out = torch.zeros(4096 * 32, dtype=torch.float32, device="cuda")
        return (dev(raw), out, 4096), [out]
    assert_bytes_equal(run_both(pack, ref, "mxfp4_dequant_f32", mk, 1))
    q8 = oracle.quantize_q8_0(oracle.fill_normal(4096 * 32, 12, 0.02))

    def mk8():
        out = torch.zeros(4096 * 32, dtype=torch.float32, device="cuda")
        return (dev(q8), out, 4096), [out]
    assert_bytes_equal(run_both(pack, ref, "q8_0_dequant_f32", mk8, 1))


def test_q8_0_and_mxfp4_repack(pack, ref):
    nb = 5120 // 32 * 64
    q8 = oracle.quantize_q8_0(oracle.fill_normal(nb * 32, 13, 0.02))

    def mk():
        d = torch.zeros(nb * 32, dtype=torch.uint8, device="cuda")
        s = torch.zeros(nb * 2, dtype=torch.uint8, device="cuda")
        return (dev(q8), d, s, nb), [d, s]
    assert_bytes_equal(run_both(pack, ref, "q8_0_repack", mk, 2))
    mx = oracle.quantize_mxfp4(oracle.fill_normal(nb * 32, 14, 0.02))

    def mkm():
        d = torch.zeros(nb * 16, dtype=torch.uint8, device="cuda")
        s = torch.zeros(nb, dtype=torch.uint8, device="cuda")
        return (dev(mx), d, s, nb), [d, s]
    assert_bytes_equal(run_both(pack, ref, "mxfp4_repack", mkm, 2))


def q4k_planes(pack, n, k, seed):
    from paddock_b200 import synth
    raw = synth.quantize_q4_k(torch.from_numpy(oracle.fill_normal(n * k, seed, 0.02))).numpy()
    return raw, n * k // 256


def test_q4k_dequant_repack_gemv(pack, ref):
    k, n = 5120, 512
    raw, ns = q4k_planes(pack, n, k, 15)

    def mkd():
        out = torch.zeros(n * k, dtype=torch.float32, device="cuda")
        return (dev(raw), out, ns, 12), [out]
    assert_bytes_equal(run_both(pack, ref, "kquant_dequant", mkd, 1))

    def mkr():
        d = torch.zeros(ns * 128, dtype=torch.uint8, device="cuda")
        s = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
        return (dev(raw), d, s, ns, 12), [d, s]
    planes = run_both(pack, ref, "kquant_repack", mkr, 2)
    assert_bytes_equal(planes)
    x = oracle.bf16_round(oracle.fill_normal(k, 16, 1.0))

    def mkg():
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        return (dev(planes[0][0]), dev(planes[0][1]), dev_f32(x), y, k, n, 12), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "kquant_gemv", mkg, 1))
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL


def test_q8_0_gemv_and_gemm(pack, ref):
    k, n = 5120, 768
    q8 = oracle.quantize_q8_0(oracle.fill_normal(n * k, 17, 0.02))
    nb = n * k // 32
    d = torch.zeros(nb * 32, dtype=torch.uint8, device="cuda")
    s = torch.zeros(nb * 2, dtype=torch.uint8, device="cuda")
    pack.call("q8_0_repack", dev(q8), d, s, nb)
    x = oracle.bf16_round(oracle.fill_normal(4 * k, 18, 1.0))
    bias = oracle.fill_normal(n, 19, 0.1)

    def mkv():
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        return (d, s, dev_f32(bias), dev_f32(x[:k]), y, k, n), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "q8_0_gemv_repacked", mkv, 1))
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL

    def mkm():
        y = torch.zeros(4 * n, dtype=torch.float32, device="cuda")
        return (d, s, None, dev_f32(x), y, k, n, 4), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "q8_0_gemm_repacked", mkm, 1))
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL


def test_moe_routing_and_combine(pack, ref):
    tokens, n_expert, k, bm = 70, 128, 4, 32
    logits = oracle.fill_normal(tokens * n_expert, 20, 1.0)
    logits[5] = logits[9]                       # a tie: lowest index wins

    def mkt():
        i = torch.zeros(tokens * k, dtype=torch.int32, device="cuda")
        w = torch.zeros(tokens * k, dtype=torch.float32, device="cuda")
        return (dev_f32(logits), None, n_expert, k, i, w, tokens), [i, w]
    ours, theirs = run_both(pack, ref, "moe_topk_batch", mkt, 2)
    assert np.array_equal(ours[0], theirs[0])
    assert np.allclose(ours[1].view(np.float32), theirs[1].view(np.float32), rtol=2e-6, atol=0)
    idx = ours[0].view(np.uint32)
    max_blocks = (tokens * k + n_expert * (bm - 1)) // bm + 1

    def mka():
        r = torch.full((max_blocks * bm,), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
        sl = torch.full((max_blocks * bm,), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
        be = torch.full((max_blocks,), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
        return (dev(idx), r, sl, be, tokens, k, n_expert, max_blocks), [be, r, sl]
    ours, theirs = run_both(pack, ref, "moe_align", mka, 3)
    be_o, be_t = ours[0].view(np.uint32), theirs[0].view(np.uint32)
    assert np.array_equal(be_o, be_t)
    # the same (row, slot) pairs in every block; order inside a block is the implementation's
    ro, so = ours[1].view(np.uint32).reshape(-1, bm), ours[2].view(np.uint32).reshape(-1, bm)
    rt, st = theirs[1].view(np.uint32).reshape(-1, bm), theirs[2].view(np.uint32).reshape(-1, bm)
    for b in range(max_blocks):
        a = sorted(zip(ro[b].tolist(), so[b].tolist()))
        c = sorted(zip(rt[b].tolist(), st[b].tolist()))
        live_a = [p for p in a if p[0] < tokens]
        live_c = [p for p in c if p[0] < tokens]
        assert live_a == live_c, b

    part = oracle.fill_normal(tokens * k * 64, 21, 1.0)
    res = oracle.fill_normal(tokens * 64, 22, 1.0)

    def mkc():
        r = dev_f32(res)
        return (dev_f32(part), r, 64, k, tokens), [r]
    assert_bytes_equal(run_both(pack, ref, "moe_slot_combine", mkc, 1))


def test_nvf4_quantize_dequant_tile_gemv(pack, ref):
    n_el = 64 * 5120
    x = oracle.fill_normal(n_el, 23, 1.0)
    x[:16] = 0.0

    def mkq():
        q = torch.zeros(n_el // 2, dtype=torch.uint8, device="cuda")
        s = torch.zeros(n_el // 16, dtype=torch.uint8, device="cuda")
        return (dev_f32(x), q, s, n_el), [q, s]
    assert_bytes_equal(run_both(pack, ref, "quantize_nvf4", mkq, 2))

    n, k = 300, 1024
    rng = np.random.default_rng(24)
    q = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = rng.integers(0, 0x7F, (n, k // 16), dtype=np.uint8)

    def mkd():
        y = torch.zeros(n * k, dtype=torch.float32, device="cuda")
        return (dev(q), dev(s), 0.0173, y, k, n), [y]
    assert_bytes_equal(run_both(pack, ref, "nvf4_dequant", mkd, 1))

    def mkt():
        t = torch.zeros(((n + 127) // 128) * (k // 256) * 2048, dtype=torch.uint8, device="cuda")
        return (dev(s), t, k, n), [t]
    assert_bytes_equal(run_both(pack, ref, "nvf4_tc5_tile_scales", mkt, 1))

    s_small = rng.integers(0x28, 0x48, (n, k // 16), dtype=np.uint8)
    xv = oracle.bf16_round(oracle.fill_normal(k, 25, 1.0))

    def mkg():
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        return (dev(q), dev(s_small), None, dev_f32(xv), y, 0.0173, k, n), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "nvf4_gemv", mkg, 1))
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL


def test_fp8_row_quantizers(pack, ref):
    k, rows = 5120, 96
    x = oracle.fill_normal(rows * k, 26, 1.0)
    x[:k] = 0.0

    def mkq():
        q = torch.zeros(rows * k, dtype=torch.uint8, device="cuda")
        s = torch.zeros(rows, dtype=torch.float32, device="cuda")
        return (dev_f32(x), q, s, k, rows), [q, s]
    assert_bytes_equal(run_both(pack, ref, "quantize_e4m3_row", mkq, 2))
    w = torch.from_numpy(oracle.fill_normal(rows * k, 27, 0.02)).to(torch.bfloat16)

    def mkw():
        q = torch.zeros(rows * k, dtype=torch.uint8, device="cuda")
        s = torch.zeros(rows, dtype=torch.float32, device="cuda")
        return (w.cuda(), q, s, k, rows), [q, s]
    assert_bytes_equal(run_both(pack, ref, "bf16_to_f8row", mkw, 2))


def test_q8_activation_quantizers_and_w4a8_gemv(pack, ref):
    n_el = 8 * 5120
    x = oracle.fill_normal(n_el, 28, 1.0)
    x[:32] = 0.0

    def mkq():
        q = torch.zeros(n_el, dtype=torch.int8, device="cuda")
        s = torch.zeros(n_el // 32, dtype=torch.float32, device="cuda")
        sums = torch.zeros(n_el // 16, dtype=torch.float32, device="cuda")
        return (dev_f32(x), q, s, sums, n_el), [q, s, sums]
    outs = run_both(pack, ref, "quantize_q8_sums", mkq, 3)
    assert_bytes_equal(outs)

    k, n = 5120, 512
    raw, ns = q4k_planes(pack, n, k, 29)
    d = torch.zeros(ns * 128, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
    pack.call("kquant_repack", dev(raw), d, sc, ns, 12)
    q = outs[0][0][:k]
    s = outs[0][1][: k // 32 * 4]
    sums = outs[0][2][: k // 16 * 4]

    def mkg():
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        return (d, sc, dev(q), dev(s), dev(sums), y, k, n, 12), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "kquant_gemv_w4a8", mkg, 1))
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL


@pytest.mark.parametrize("name,dtype,datab", [("q5_k", 13, 160), ("q6_k", 14, 192), ("q4_0", 2, 128), ("iq4_xs", 23, 128)])
def test_more_kquants_against_reference_pack(pack, ref, name, dtype, datab):
    from test_gpu_gemv import raw_kquant
    k, n = 1024, 64
    ns = n * k // 256
    raw = raw_kquant(name, ns, 30 + dtype)

    def mkd():
        out = torch.zeros(ns * 256, dtype=torch.float32, device="cuda")
        return (dev(raw), out, ns, dtype), [out]
    assert_bytes_equal(run_both(pack, ref, "kquant_dequant", mkd, 1))

    def mkr():
        d = torch.zeros(ns * datab, dtype=torch.uint8, device="cuda")
        s = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
        return (dev(raw), d, s, ns, dtype), [d, s]
    planes = run_both(pack, ref, "kquant_repack", mkr, 2)
    assert_bytes_equal(planes)
    x = oracle.bf16_round(oracle.fill_normal(k, 31, 1.0))

    def mkg():
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        return (dev(planes[0][0]), dev(planes[0][1]), dev_f32(x), y, k, n, dtype), [y]
    ours, theirs = (o[0].view(np.float32) for o in run_both(pack, ref, "kquant_gemv", mkg, 1))
    # Q5_K and Q4_0 run the integer tensor-core GEMV (15-bit block-floating activations), as Q4_K does
    assert rel_l2(ours, theirs.astype(np.float64)) < 1e-4 < TOL


def test_add_rmsnorm_quant_nvf4_against_reference_pack(pack, ref):
    """Slot 436 on both packs: the summed rows are identical, the normed rows agree to an ulp of the
    norm scale, and the scale bytes differ, if at all, only where that ulp crosses a rounding tie."""
    n, batch, eps = 5120, 4, 1e-6
    x = oracle.fill_normal(batch * n, 5200, 1.5)
    proj = oracle.fill_normal(batch * n, 5201, 0.5)
    w = (1.0 + 0.1 * oracle.fill_normal(n, 5202, 1.0)).astype(np.float32)

    def mk():
        dx = dev_f32(x)
        out = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
        q = torch.zeros(batch * n // 2, dtype=torch.uint8, device="cuda")
        s = torch.zeros(batch * n // 16, dtype=torch.uint8, device="cuda")
        return (dx, dev_f32(proj), dev_f32(w), out, q, s, n, eps, batch), [dx, out, s, q]
    ours, theirs = run_both(pack, ref, "add_rmsnorm_quant_nvf4_batch", mk, 4)
    assert np.array_equal(ours[0], theirs[0])
    assert np.allclose(ours[1].view(np.float32), theirs[1].view(np.float32), rtol=4e-7, atol=0)
    assert np.mean(ours[2] != theirs[2]) < 1e-3
    assert np.mean(ours[3] != theirs[3]) < 1e-3


def test_e4m3_producers_against_reference_pack(pack, ref):
    """Slots 511 / 512 / 513 on both packs: SwiGLU + quantizer byte-identical; the norm forms write the
    same summed rows, normed rows that agree to an ulp of the norm scale, the same row scales and
    codes that differ, if at all, only where that ulp crosses a rounding tie."""
    n, batch, eps = 5120, 6, 1e-6
    g = oracle.fill_normal(batch * n, 5300, 2.0)
    u = oracle.fill_normal(batch * n, 5301, 1.0)

    def mk_sw():
        q = torch.zeros(batch * n, dtype=torch.uint8, device="cuda")
        s = torch.zeros(batch, dtype=torch.float32, device="cuda")
        return (dev_f32(g), dev_f32(u), q, s, n, batch), [q, s]
    assert_bytes_equal(run_both(pack, ref, "swiglu_quant_e4m3_row", mk_sw, 2))
    w = (1.0 + 0.1 * oracle.fill_normal(n, 5302, 1.0)).astype(np.float32)

    def mk_norm(residual):
        def mk():
            dx = dev_f32(g)
            xn = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
            q = torch.zeros(batch * n, dtype=torch.uint8, device="cuda")
            s = torch.zeros(batch, dtype=torch.float32, device="cuda")
            if residual:
                return (dx, dev_f32(u), dev_f32(w), xn, q, s, n, eps, 0.5, batch), [dx, xn, s, q]
            return (dx, dev_f32(w), xn, q, s, n, eps, batch), [dx, xn, s, q]
        return mk
    for name, residual in (("rmsnorm_quant_e4m3_row", False), ("add_rmsnorm_scaled_quant_e4m3_row", True)):
        ours, theirs = run_both(pack, ref, name, mk_norm(residual), 4)
        assert np.array_equal(ours[0], theirs[0])
        assert np.allclose(ours[1].view(np.float32), theirs[1].view(np.float32), rtol=4e-7, atol=0)
        assert np.array_equal(ours[2], theirs[2])
        assert np.mean(ours[3] != theirs[3]) < 1e-3


def test_nvf4_swiglu_quantizers_against_reference_pack(pack, ref):
    """Slots 120 and 516 on both packs: byte-identical planes."""
    rows, ff = 5, 2880
    g = oracle.fill_normal(rows * ff, 5400, 2.0)
    u = oracle.fill_normal(rows * ff, 5401, 1.0)

    def mk():
        q = torch.zeros(rows * ff // 2, dtype=torch.uint8, device="cuda")
        s = torch.zeros(rows * ff // 16, dtype=torch.uint8, device="cuda")
        return (dev_f32(g), dev_f32(u), q, s, rows * ff), [q, s]
    assert_bytes_equal(run_both(pack, ref, "quantize_nvf4_swiglu", mk, 2))
    fused = np.concatenate([g.reshape(rows, ff), u.reshape(rows, ff)], axis=1).reshape(-1)

    def mkf():
        q = torch.zeros(rows * ff // 2, dtype=torch.uint8, device="cuda")
        s = torch.zeros(rows * ff // 16, dtype=torch.uint8, device="cuda")
        return (dev_f32(fused), q, s, ff, rows), [q, s]
    assert_bytes_equal(run_both(pack, ref, "swiglu_fused_nvf4", mkf, 2))


def _moe_slot_chain(p, raw, x, idx, w, tokens, n_expert, k, embd, ff, decode):
    """The engine's MoE chain through pack `p`'s own slots (its own fused gate|up plane);
    decode: the unsorted pair 92 / 93, else align -> 88 -> 89 -> combine."""
    i32, f32, i8 = torch.int32, torch.float32, torch.int8
    z = lambda n, dt: torch.zeros(n, dtype=dt, device="cuda")
    planes = {}
    for name in ("gate", "up", "down"):
        nb = raw[name].size // 17
        data, scale = z(nb * 16, torch.uint8), z(nb, torch.uint8)
        p.call("mxfp4_repack", dev(raw[name]), data, scale, nb)
        planes[name] = (data, scale)
    n_kb = embd // 32
    fused = z(n_expert * ff * ((n_kb + 3) // 4) * 128, torch.uint8)
    p.call("mxfp4_gu_interleave", planes["gate"][0], planes["up"][0], fused, n_kb, n_expert * ff)
    d_idx, d_w = dev(idx.astype(np.uint32)).view(i32), dev_f32(w.reshape(-1))
    zb_ff, zb_embd = z(n_expert * ff, f32), z(n_expert * embd, f32)
    xq, xs = z(tokens * embd, i8), z(tokens * embd // 32, f32)
    dummy = z(16, torch.uint8)
    out = z(tokens * embd, f32)
    pairs = tokens * k
    p.call("quantize_q8", dev_f32(x), xq, xs, tokens * embd)
    if decode:
        h, hq, hs = z(pairs * ff, f32), z(pairs * ff, i8), z(pairs * ff // 32, f32)
        p.call("mxfp4_moe_gate_up_dp4a_b", fused, planes["gate"][1], zb_ff, dummy, planes["up"][1], zb_ff, d_idx, xq, xs, h,
               embd, ff, k, tokens, 1.702, 7.0)
        p.call("quantize_q8", h, hq, hs, pairs * ff)
        p.call("mxfp4_moe_down_dp4a_b", planes["down"][0], planes["down"][1], zb_embd, d_idx, d_w, hq, hs, out, ff, embd, k,
               tokens)
    else:
        bm = 32
        max_blocks = (pairs + n_expert * (bm - 1) + bm - 1) // bm
        nb = max_blocks * bm
        s_row, s_slot, b_exp = z(nb, i32), z(nb, i32), z(max_blocks, i32)
        fq, fs, part = z(nb * ff, i8), z(nb * ff // 32, f32), z(pairs * max(ff, embd), f32)
        p.call("moe_align", d_idx, s_row, s_slot, b_exp, tokens, k, n_expert, max_blocks)
        p.call("mxfp4_moe_gate_up_mmq", fused, planes["gate"][1], zb_ff, dummy, planes["up"][1], zb_ff, s_row, b_exp, xq, xs,
               fq, fs, embd, ff, max_blocks, 1.702, 7.0, 1.0)
        p.call("mxfp4_moe_down_mmq", planes["down"][0], planes["down"][1], zb_embd, s_row, s_slot, b_exp, d_w, fq, fs, part,
               ff, embd, k, max_blocks)
        p.call("moe_slot_combine", part, out, embd, k, tokens)
    torch.cuda.synchronize()
    return out.cpu().numpy().reshape(tokens, embd)


@pytest.mark.parametrize("tokens,decode", [(40, False), (3, True)])
def test_mxfp4_moe_slot_chain_against_reference(pack, ref, tokens, decode):
    """Slots 155 / 88 / 89 / 91 (and the decode pair 92 / 93) of both packs on the same raw planes,
    tokens and routing: the same int8 activation class, so the blocks agree far inside the
    activation quantization's own error (about 1e-2 of the result)."""
    n_expert, k, embd, ff = 16, 4, 2880, 2880
    raw = {n: oracle.quantize_mxfp4(oracle.fill_normal(n_expert * ff * embd, 1500 + i, 0.02))
           for i, n in enumerate(("gate", "up", "down"))}
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 1510, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, 1511, 1.0)
    idx, w = oracle.moe_topk(logits, n_expert, k)
    try:
        theirs = _moe_slot_chain(ref, raw, x, idx, w, tokens, n_expert, k, embd, ff, decode)
    except MissingOp as e:
        pytest.skip(f"reference pack: {e}")
    ours = _moe_slot_chain(pack, raw, x, idx, w, tokens, n_expert, k, embd, ff, decode)
    assert pack.device_error() == 0
    assert np.isfinite(ours).all()
    assert rel_l2(ours, theirs.astype(np.float64)) < 5e-3 < TOL
