"""MXFP4 MoE (128 experts, top-4, 2880 / 2880 in the benchmark): router and alignment against the oracle /
their invariants, then the whole block (top-k -> align -> gate|up + SwiGLU ->
down -> combine) within 1e-2 of the oracle's f64 walk over dequantized experts."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, dev, dev_f32, rel_l2
from paddock_b200 import planes as P

pytestmark = pytest.mark.gpu
PAD = 0xFFFFFFFF


@pytest.mark.parametrize("tokens,n_expert,k", [(1, 128, 4), (64, 128, 4), (33, 8, 2), (5, 512, 10)])
def test_topk_matches_oracle(pack, tokens, n_expert, k):
    logits = oracle.fill_normal(tokens * n_expert, 700 + tokens, 1.0)
    logits[:n_expert // 2] = np.round(logits[:n_expert // 2])       # force ties in token 0
    bias = oracle.fill_normal(n_expert, 701, 0.5)
    idx_ref, w_ref = oracle.moe_topk(logits, n_expert, k, bias)
    d_idx = torch.zeros(tokens * k, dtype=torch.int32, device="cuda")
    d_w = torch.zeros(tokens * k, dtype=torch.float32, device="cuda")
    pack.call("moe_topk_batch", dev_f32(logits), dev_f32(bias), n_expert, k, d_idx, d_w, tokens)
    torch.cuda.synchronize()
    assert np.array_equal(d_idx.cpu().numpy().view(np.uint32).reshape(tokens, k), idx_ref)
    assert np.allclose(d_w.cpu().numpy().reshape(tokens, k), w_ref, rtol=2e-6, atol=0)


@pytest.mark.parametrize("tokens,n_expert,k,bm", [(1, 128, 4, 8), (64, 128, 4, 8), (200, 16, 4, 32), (1024, 128, 4, 32),
                                                    (1500, 8, 2, 32), (60, 2048, 2, 8)])   # many chunks; the scan kernel (experts > 1500)
def test_align_is_a_stable_grouping(pack, tokens, n_expert, k, bm):
    rng = np.random.default_rng(tokens)
    idx = np.stack([rng.permutation(n_expert)[:k] for _ in range(tokens)]).astype(np.uint32)
    pairs = tokens * k
    max_blocks = min(pairs, pairs // bm + n_expert)
    d_row = torch.full((max_blocks * bm,), 7, dtype=torch.int32, device="cuda")
    d_slot = torch.full((max_blocks * bm,), 7, dtype=torch.int32, device="cuda")
    d_be = torch.full((max_blocks,), 7, dtype=torch.int32, device="cuda")
    name, args = ("moe_align", ()) if bm == 32 else ("moe_align_bm", (bm,))
    pack.call(name, dev(idx), d_row, d_slot, d_be, tokens, k, n_expert, *args, max_blocks)
    torch.cuda.synchronize()
    row = d_row.cpu().numpy().view(np.uint32).reshape(max_blocks, bm)
    slot = d_slot.cpu().numpy().view(np.uint32).reshape(max_blocks, bm)
    be = d_be.cpu().numpy().view(np.uint32)
    used = be != PAD
    assert not used[np.argmin(used):].any() if not used.all() else True     # used blocks come first
    assert list(be[used]) == sorted(be[used])                                # experts ascending
    seen = []
    for b in np.nonzero(used)[0]:
        valid = row[b] != PAD
        assert valid[:valid.sum()].all()                                     # padding only at a block's tail
        for r, s in zip(row[b][valid], slot[b][valid]):
            assert idx[r, s] == be[b]
            seen.append(int(r) * k + int(s))
    assert sorted(seen) == list(range(pairs))                                # every pair exactly once
    for e in range(n_expert):                                                # ascending pair order inside an expert
        mine = [p for p in seen if idx[p // k, p % k] == e]
        assert mine == sorted(mine)


def make_layer(n_expert, embd, ff, seed, with_bias):
    def plane(rows, cols, sd):
        raw = oracle.quantize_mxfp4(oracle.fill_normal(n_expert * rows * cols, sd, 0.02))
        return raw
    raw = {"gate": plane(ff, embd, seed), "up": plane(ff, embd, seed + 1), "down": plane(embd, ff, seed + 2)}
    bias = {}
    if with_bias:
        bias = {"gate": oracle.fill_normal(n_expert * ff, seed + 3, 0.02),
                "up": oracle.fill_normal(n_expert * ff, seed + 4, 0.02),
                "down": oracle.fill_normal(n_expert * embd, seed + 5, 0.02)}
    return raw, bias


@pytest.mark.parametrize("tokens,n_expert,k,embd,ff,bm,with_bias", [
    (1, 8, 2, 64, 96, 8, True),
    (5, 8, 2, 128, 160, 8, False),
    (40, 8, 4, 128, 64, 32, True),
    (70, 4, 2, 256, 256, 32, False),
    (3, 16, 4, 2880, 2880, 8, True),      # the benchmark geometry, a few tokens
    (48, 16, 4, 2880, 2880, 32, False),
])
def test_moe_block_matches_oracle(pack, tokens, n_expert, k, embd, ff, bm, with_bias):
    ex = P.GpuExecutor(pack)
    raw, bias = make_layer(n_expert, embd, ff, 800 + tokens + ff, with_bias)
    planes = P.MoeMxfp4Planes(P.repack_mxfp4(ex, dev(raw["gate"])), P.repack_mxfp4(ex, dev(raw["up"])),
                              P.repack_mxfp4(ex, dev(raw["down"])), n_expert, embd, ff,
                              *(dev_f32(bias[n]) if with_bias else None for n in ("gate", "up", "down")))
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 810, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, 811, 1.0)
    ws = P.MoeWorkspace(ex, planes, tokens, k, bm)
    out = torch.zeros(tokens * embd, dtype=torch.float32, device="cuda")
    P.moe_mxfp4_forward(ex, planes, ws, dev_f32(x), dev_f32(logits), out)
    torch.cuda.synchronize()
    idx, w = oracle.moe_topk(logits, n_expert, k)
    ref = oracle.moe_mxfp4_layer(raw["gate"], raw["up"], raw["down"], x, idx, w, tokens, k, embd, ff,
                                 bias.get("gate"), bias.get("up"), bias.get("down"))
    y = out.cpu().numpy().reshape(tokens, embd)
    assert np.isfinite(y).all()
    assert rel_l2(y, ref) < 2e-3 < TOL
    assert np.max(np.abs(y - ref)) < 1e-2 * np.max(np.abs(ref))


@pytest.mark.parametrize("tokens,n_expert,k,embd,ff,bm,with_bias", [
    (9, 8, 2, 128, 192, 8, True),
    (40, 8, 4, 128, 64, 32, True),
    (70, 4, 2, 256, 256, 32, False),
    (3, 16, 4, 2880, 2880, 8, True),      # the benchmark geometry: K = 11 slabs + a quarter
    (48, 16, 4, 2880, 2880, 32, False),
])
def test_moe_block_tensor_core_path_matches_oracle(pack, tokens, n_expert, k, embd, ff, bm, with_bias):
    """The same block through the block-scaled tcgen05 expert GEMMs (four NVFP4 activation terms)."""
    ex = P.GpuExecutor(pack)
    raw, bias = make_layer(n_expert, embd, ff, 900 + tokens + ff, with_bias)
    planes = P.MoeMxfp4Planes(P.repack_mxfp4(ex, dev(raw["gate"])), P.repack_mxfp4(ex, dev(raw["up"])),
                              P.repack_mxfp4(ex, dev(raw["down"])), n_expert, embd, ff,
                              *(dev_f32(bias[n]) if with_bias else None for n in ("gate", "up", "down")))
    P.prepare_tc5(ex, planes)
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 910, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, 911, 1.0)
    ws = P.MoeWorkspace(ex, planes, tokens, k, bm)
    out = torch.zeros(tokens * embd, dtype=torch.float32, device="cuda")
    P.moe_mxfp4_forward(ex, planes, ws, dev_f32(x), dev_f32(logits), out)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    idx, w = oracle.moe_topk(logits, n_expert, k)
    ref = oracle.moe_mxfp4_layer(raw["gate"], raw["up"], raw["down"], x, idx, w, tokens, k, embd, ff,
                                 bias.get("gate"), bias.get("up"), bias.get("down"))
    y = out.cpu().numpy().reshape(tokens, embd)
    assert np.isfinite(y).all()
    assert rel_l2(y, ref) < 2e-3 < TOL
    assert np.max(np.abs(y - ref)) < 1e-2 * np.max(np.abs(ref))


@pytest.mark.parametrize("tokens,n_expert,k,embd,bm", [
    (1, 128, 4, 2880, 8),      # one decode token of the benchmark layer
    (8, 128, 4, 2880, 8),      # the widest the fused front takes (32 pairs)
    (3, 16, 4, 2880, 8),
    (5, 8, 2, 512, 8),
    (2, 512, 8, 256, 32),
])
def test_route_and_prepare_in_one_launch_equals_the_three_calls(pack, tokens, n_expert, k, embd, bm):
    """pdk_moe_route_prep_f4 leaves the tables and the term rows of moe_topk_batch + moe_align_bm +
    pdk_moe_prep_act_f4, byte for byte (routing weights bit for bit)."""
    ex = P.GpuExecutor(pack)
    c = ex.pack.call
    pairs = tokens * k
    max_blocks = min(pairs, pairs // bm + n_expert)
    nb = max_blocks * bm
    x = dev_f32(oracle.bf16_round(oracle.fill_normal(tokens * embd, 1310 + tokens, 1.0)))
    logits = dev_f32(oracle.fill_normal(tokens * n_expert, 1311 + tokens, 1.0))
    rbias = dev_f32(oracle.fill_normal(n_expert, 1312, 0.1))

    def buffers():
        i32, u8, f32 = torch.int32, torch.uint8, torch.float32
        return dict(idx=torch.full((pairs,), -1, dtype=i32, device="cuda"), w=torch.zeros(pairs, dtype=f32, device="cuda"),
                    row=torch.full((nb,), -7, dtype=i32, device="cuda"), slot=torch.full((nb,), -7, dtype=i32, device="cuda"),
                    blk=torch.full((max_blocks,), -7, dtype=i32, device="cuda"),
                    q=torch.zeros(nb * 4 * embd // 2, dtype=u8, device="cuda"),
                    s=torch.zeros(max_blocks * ((embd + 255) // 256) * 2048, dtype=u8, device="cuda"),
                    step=torch.zeros(nb, dtype=f32, device="cuda"))
    for bias in (None, rbias):
        a, b = buffers(), buffers()
        c("moe_topk_batch", logits, bias, n_expert, k, a["idx"], a["w"], tokens)
        c("moe_align_bm", a["idx"], a["row"], a["slot"], a["blk"], tokens, k, n_expert, bm, max_blocks)
        c("pdk_moe_prep_act_f4", x, None, a["row"], a["blk"], a["q"], a["s"], a["step"], embd, bm, max_blocks, 0, 1.702, 7.0)
        c("pdk_moe_route_prep_f4", logits, bias, x, b["idx"], b["w"], b["row"], b["slot"], b["blk"], b["q"], b["s"],
          b["step"], n_expert, k, tokens, embd, bm, max_blocks)
        torch.cuda.synchronize()
        assert pack.device_error() == 0
        # positions of unused blocks: the alignment call leaves their row and slot entries unwritten
        used = (a["blk"] != -1).repeat_interleave(bm)
        for name in a:
            ta, tb = a[name], b[name]
            if name in ("row", "slot"):
                ta, tb = ta[used], tb[used]
            assert torch.equal(ta.view(torch.uint8), tb.view(torch.uint8)), name


def test_route_and_prepare_refuses_what_it_cannot_hold(pack):
    """More than 8 rows, more than 32 pairs, more than 512 experts, more than 32 blocks, a block size other than
    8 or 32, a row length that is not whole 32-element blocks: cudaErrorInvalidValue, nothing launched."""
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    args = lambda n_expert, k, rows, dim, bm, max_blocks: (buf, None, buf, buf, buf, buf, buf, buf, buf, buf, buf,
                                                           n_expert, k, rows, dim, bm, max_blocks)
    assert pack.status("pdk_moe_route_prep_f4", *args(128, 4, 1, 2880, 8, 4)) == 0
    for bad in [(128, 4, 9, 2880, 8, 36), (128, 8, 5, 2880, 8, 32), (513, 4, 1, 2880, 8, 4), (128, 4, 8, 2880, 8, 33),
                (128, 4, 1, 2880, 16, 4), (128, 4, 1, 2880 + 16, 8, 4), (4, 5, 1, 2880, 8, 4), (128, 0, 1, 2880, 8, 4)]:
        assert pack.status("pdk_moe_route_prep_f4", *args(*bad)) == 1, bad
    torch.cuda.synchronize()
    assert pack.device_error() == 0


def test_slot_combine_fixed_order(pack):
    rows, k, embd = 7, 4, 64
    part = oracle.fill_normal(rows * k * embd, 820, 1.0)
    res = oracle.fill_normal(rows * embd, 821, 1.0)
    d_res = dev_f32(res)
    pack.call("moe_slot_combine", dev_f32(part), d_res, embd, k, rows)
    torch.cuda.synchronize()
    p = part.reshape(rows, k, embd)
    acc = np.zeros((rows, embd), np.float32)
    for s in range(k):
        acc = acc + p[:, s]
    want = res.reshape(rows, embd) + acc
    assert np.array_equal(d_res.cpu().numpy().reshape(rows, embd), want)


# ---- NVFP4 expert planes on the same grouped tensor-core GEMM

def nvf4_expert_plane(ex, n_expert, rows, cols, seed):
    """Per expert: N(0, 0.02) weights, scale2 = absmax / (6 * 448), NVFP4 blocks (the ModelOpt recipe)."""
    data, scale, scale2, deq = [], [], [], []
    for e in range(n_expert):
        w = oracle.fill_normal(rows * cols, seed + e, 0.02)
        s2 = np.float32(np.abs(w).max() / (6.0 * 448.0))
        q, s = oracle.quantize_nvf4(w, float(s2))
        data.append(q); scale.append(s); scale2.append(s2)
        deq.append(oracle.dequant_nvfp4(q.reshape(rows, cols // 2), s.reshape(rows, cols // 16), s2, cols, rows))
    plane = P.Nvf4MoePlane(dev(np.concatenate(data)), dev(np.concatenate(scale)), dev_f32(np.array(scale2, np.float32)),
                           n_expert, rows, cols)
    return P.nvf4_moe_prepare(ex, plane), np.stack(deq).astype(np.float64)


@pytest.mark.parametrize("tokens,n_expert,k,embd,ff,bm,gated", [
    (9, 8, 2, 128, 192, 8, True),
    (40, 8, 4, 256, 128, 32, True),
    (21, 4, 2, 1344, 320, 8, False),        # K = 5 slabs and a quarter, relu^2 experts
])
def test_nvf4_moe_block_matches_f64(pack, tokens, n_expert, k, embd, ff, bm, gated):
    ex = P.GpuExecutor(pack)
    gate, wg = nvf4_expert_plane(ex, n_expert, ff, embd, 1000)
    up, wu = nvf4_expert_plane(ex, n_expert, ff, embd, 2000)
    down, wd = nvf4_expert_plane(ex, n_expert, embd, ff, 3000)
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 4000, 1.0)).reshape(tokens, embd)
    logits = oracle.fill_normal(tokens * n_expert, 4001, 1.0)

    class Shape:
        pass
    shape = Shape()
    shape.n_expert, shape.embd, shape.ff = n_expert, embd, ff
    ws = P.MoeWorkspace(ex, shape, tokens, k, bm)
    out = torch.zeros(tokens * embd, dtype=torch.float32, device="cuda")
    P.moe_nvf4_forward(ex, gate, up, down, ws, dev_f32(x), dev_f32(logits), out, gated=gated)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    idx, w = oracle.moe_topk(logits, n_expert, k)
    idx, w = idx.reshape(tokens, k), w.reshape(tokens, k)
    ref = np.zeros((tokens, embd))
    for t in range(tokens):
        for s in range(k):
            e = idx[t, s]
            u = wu[e] @ x[t].astype(np.float64)
            if gated:
                g = wg[e] @ x[t].astype(np.float64)
                h = g / (1.0 + np.exp(-g)) * u
            else:
                h = np.maximum(u, 0.0) ** 2
            ref[t] += w[t, s] * (wd[e] @ h)
    y = out.cpu().numpy().reshape(tokens, embd)
    assert np.isfinite(y).all()
    assert rel_l2(y, ref) < 2e-3 < TOL


# ---- the reference's own MoE slots (155 / 88 / 89 and the decode pair 92 / 93): int8 activations

def _q8_roundtrip(v):
    """What pd_quantize_q8 keeps of a vector: per 32, d = amax / 127, q = round(v / d)."""
    q, s, _ = oracle.quantize_q8_act(np.ascontiguousarray(v, np.float32).reshape(-1), with_sums=False)
    return (q.astype(np.float32).reshape(-1, 32) * s[:, None]).reshape(np.shape(v)).astype(np.float64)


def _slot_layer_ref(raw, x, idx, w, tokens, k, embd, ff, n_expert, quantized):
    """f64 walk of the block over dequantized experts; quantized: activations pass through int8 where
    the slot chain passes them (x before gate|up, h before down)."""
    deq = {n: oracle.dequant_mxfp4(raw[n]).astype(np.float64) for n in raw}
    wg, wu = deq["gate"].reshape(n_expert, ff, embd), deq["up"].reshape(n_expert, ff, embd)
    wd = deq["down"].reshape(n_expert, embd, ff)
    xx = _q8_roundtrip(x.reshape(tokens, embd)) if quantized else x.reshape(tokens, embd).astype(np.float64)
    out = np.zeros((tokens, embd))
    for t in range(tokens):
        for s in range(k):
            e = idx[t, s]
            g, u = wg[e] @ xx[t], wu[e] @ xx[t]
            xg, yu = np.minimum(g, 7.0), np.clip(u, -7.0, 7.0)
            h = xg / (1.0 + np.exp(-1.702 * xg)) * (yu + 1.0)
            if quantized:
                h = _q8_roundtrip(h)
            out[t] += w[t, s] * (wd[e] @ h)
    return out


def _fused_planes(pack, raw, n_expert, embd, ff):
    ex = P.GpuExecutor(pack)
    g, u, d = (P.repack_mxfp4(ex, dev(raw[n])) for n in ("gate", "up", "down"))
    n_kb = embd // 32
    fused = torch.zeros(n_expert * ff * ((n_kb + 3) // 4) * 128, dtype=torch.uint8, device="cuda")
    pack.call("mxfp4_gu_interleave", g.data, u.data, fused, n_kb, n_expert * ff)
    return fused, g.scale, u.scale, d


@pytest.mark.parametrize("tokens,n_expert,k,embd,ff", [(9, 8, 2, 128, 160), (70, 4, 2, 256, 256), (40, 16, 4, 2880, 2880)])
def test_moe_reference_slots_sorted_chain(pack, tokens, n_expert, k, embd, ff):
    """quantize_q8 -> moe_align -> gate_up_mmq (88) -> down_mmq (89) -> slot_combine, the chain
    crates/paddock-engine/src/gpu_model/gpt_oss.rs:2393-2440 runs above 8 tokens, on the plane slot 155 fused."""
    raw, _ = make_layer(n_expert, embd, ff, 1300 + tokens + ff, False)
    fused, gs, us, down = _fused_planes(pack, raw, n_expert, embd, ff)
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 1310, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, 1311, 1.0)
    idx, w = oracle.moe_topk(logits, n_expert, k)
    pairs, bm = tokens * k, 32
    max_blocks = (pairs + n_expert * (bm - 1) + bm - 1) // bm
    nb = max_blocks * bm
    i32, f32 = torch.int32, torch.float32
    d_idx, d_w = dev(idx.astype(np.uint32)).view(i32), dev_f32(w.reshape(-1))
    s_row, s_slot = torch.zeros(nb, dtype=i32, device="cuda"), torch.zeros(nb, dtype=i32, device="cuda")
    b_exp = torch.zeros(max_blocks, dtype=i32, device="cuda")
    xq, xs = torch.zeros(tokens * embd, dtype=torch.int8, device="cuda"), torch.zeros(tokens * embd // 32, dtype=f32, device="cuda")
    fq, fs = torch.zeros(nb * ff, dtype=torch.int8, device="cuda"), torch.zeros(nb * ff // 32, dtype=f32, device="cuda")
    part = torch.zeros(pairs * embd, dtype=f32, device="cuda")
    out = torch.zeros(tokens * embd, dtype=f32, device="cuda")
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    pack.call("moe_align", d_idx, s_row, s_slot, b_exp, tokens, k, n_expert, max_blocks)
    pack.call("quantize_q8", dev_f32(x), xq, xs, tokens * embd)
    pack.call("mxfp4_moe_gate_up_mmq", fused, gs, None, dummy, us, None, s_row, b_exp, xq, xs, fq, fs, embd, ff, max_blocks,
              1.702, 7.0, 1.0)
    pack.call("mxfp4_moe_down_mmq", down.data, down.scale, None, s_row, s_slot, b_exp, d_w, fq, fs, part, ff, embd, k,
              max_blocks)
    pack.call("moe_slot_combine", part, out, embd, k, tokens)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    y = out.cpu().numpy().reshape(tokens, embd)
    assert np.isfinite(y).all()
    same_class = _slot_layer_ref(raw, x, idx, w, tokens, k, embd, ff, n_expert, True)
    exact = _slot_layer_ref(raw, x, idx, w, tokens, k, embd, ff, n_expert, False)
    assert rel_l2(y, same_class) < 5e-3                 # the same int8 activations: what is left is f16 staging and rounding ties
    assert rel_l2(y, exact) < 3e-2                      # the int8 activation class against the unquantized walk


@pytest.mark.parametrize("tokens,n_expert,k,embd,ff", [(1, 8, 2, 128, 160), (3, 16, 4, 2880, 2880), (8, 4, 2, 256, 96)])
def test_moe_reference_slots_decode_pair(pack, tokens, n_expert, k, embd, ff):
    """quantize_q8 -> gate_up_dp4a_b (92) -> quantize_q8 -> down_dp4a_b (93): the unsorted chain of
    gpt_oss.rs:2441-2480 for up to 8 tokens; the result accumulates into the residual."""
    raw, _ = make_layer(n_expert, embd, ff, 1400 + tokens + ff, False)
    fused, gs, us, down = _fused_planes(pack, raw, n_expert, embd, ff)
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, 1410, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, 1411, 1.0)
    idx, w = oracle.moe_topk(logits, n_expert, k)
    pairs = tokens * k
    f32 = torch.float32
    d_idx, d_w = dev(idx.astype(np.uint32)).view(torch.int32), dev_f32(w.reshape(-1))
    xq, xs = torch.zeros(tokens * embd, dtype=torch.int8, device="cuda"), torch.zeros(tokens * embd // 32, dtype=f32, device="cuda")
    h = torch.zeros(pairs * ff, dtype=f32, device="cuda")
    hq, hs = torch.zeros(pairs * ff, dtype=torch.int8, device="cuda"), torch.zeros(pairs * ff // 32, dtype=f32, device="cuda")
    res0 = oracle.fill_normal(tokens * embd, 1412, 1.0)
    res = dev_f32(res0)
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    pack.call("quantize_q8", dev_f32(x), xq, xs, tokens * embd)
    pack.call("mxfp4_moe_gate_up_dp4a_b", fused, gs, None, dummy, us, None, d_idx, xq, xs, h, embd, ff, k, tokens, 1.702, 7.0)
    pack.call("quantize_q8", h, hq, hs, pairs * ff)
    pack.call("mxfp4_moe_down_dp4a_b", down.data, down.scale, None, d_idx, d_w, hq, hs, res, ff, embd, k, tokens)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    y = res.cpu().numpy().reshape(tokens, embd) - res0.reshape(tokens, embd)
    same_class = _slot_layer_ref(raw, x, idx, w, tokens, k, embd, ff, n_expert, True)
    assert rel_l2(y, same_class) < 5e-3
    assert pack.status("mxfp4_moe_down_dp4a_b", down.data, down.scale, None, d_idx, d_w, hq, hs, res, ff, 1 << 20, k,
                       tokens) == 801                   # per-pair rows beyond the scratch slice
