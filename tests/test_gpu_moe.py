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
