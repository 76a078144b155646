"""Parity at the full benchmark shapes, through the C ABI.

The other GPU test files check every output of small cases against the oracle.  Tile walks, grid
sizing, ring wrap-around, scale re-tiling and block tables behave differently at full size, so this
file runs each benchmark shape once at full size and checks

  * a few hundred sampled outputs against the oracle's f64 products of the dequantized operands
    (the gates of the small cases: max |err| / sum|w x| and rel-L2, both far below the stated 1e-2),
  * every output against a plain f32 torch matmul of the same dequantized operands (a second,
    looser opinion whose only job is to notice a tile that was skipped or written twice),
  * that the device error word stayed zero (no bounded wait ran out).

Shapes: Q8_0 GEMV K=5120 N=17408; Q4_K K=5120 N=25600 at 1 / 4 / 16 tokens; FP8 GEMM 4096 tokens,
K=5120, N=5120 / 17408 / 27648 (f32 and bf16 outputs); NVFP4 GEMM K=5120 N=17408 at 1 / 8 / 64 /
512 / 8192 tokens; MXFP4 MoE block with 128 experts, top-4, 2880 / 2880, 1 / 64 / 1024 tokens on
both expert paths.  Inputs are seeded draws with the distributions the benchmark uses.
"""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, bf16_activations, cond_err, dev, dev_f32, rel_l2, seed_for
from paddock_b200 import planes as P

pytestmark = pytest.mark.gpu


def sample(rng, n, count):
    """`count` distinct indices below n, always including the first and the last."""
    count = min(count, n)
    idx = rng.choice(n, size=count, replace=False)
    idx[0], idx[-1] = 0, n - 1
    return np.unique(idx)


def check_sampled(y, w_rows, x_rows, rows, toks, k, tol_cond, tol_l2):
    """y [tokens][n] from the GPU; w_rows f32 [len(rows)][k], x_rows f32 [len(toks)][k] dequantized."""
    ref, ab = oracle.matmul_f64(w_rows, x_rows, k, len(rows), len(toks), with_abs=True)
    got = y[np.ix_(toks, rows)]
    assert np.isfinite(got).all()
    assert cond_err(got, ref, ab) < tol_cond < TOL
    assert rel_l2(got, ref) < tol_l2 < TOL


def check_all(y_dev, w_dev, x_dev, tol):
    """y_dev [m][n] against x_dev [m][k] @ w_dev [n][k]^T in f32 on the device (TF32 off)."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = x_dev @ w_dev.t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert torch.isfinite(y_dev).all()
    err = float((y_dev.float() - ref).norm() / ref.norm())
    assert err < tol
    # no tile skipped or written twice: the largest single deviation stays small too
    worst = float((y_dev.float() - ref).abs().max() / ref.abs().max())
    assert worst < 40 * tol


# ---------------------------------------------------------------------------------- Q8_0, Q4_K

def test_q8_0_gemv_full(pack):
    k, n = 5120, 17408
    w = oracle.fill_normal(n * k, seed_for(1, 0), 0.02)
    x = bf16_activations(k, seed_for(1, 1))
    raw = oracle.quantize_q8_0(w)
    nb = n * k // 32
    d_data = torch.zeros(nb * 32, dtype=torch.int8, device="cuda")
    d_scale = torch.zeros(nb, dtype=torch.float16, device="cuda")
    pack.call("q8_0_repack", dev(raw), d_data, d_scale, nb)
    d_y = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    d_x = dev_f32(x)
    pack.call("q8_0_gemv_repacked", d_data, d_scale, None, d_x, d_y, k, n)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    rows = sample(np.random.default_rng(1), n, 384)
    raw_rows = raw.reshape(n, k // 32 * 34)[rows]
    check_sampled(d_y.cpu().numpy()[None, :], oracle.dequant_q8_0(raw_rows).reshape(len(rows), k), x[None, :], rows,
                  np.array([0]), k, 1e-5, 1e-4)
    w_dev = d_data.view(n, k // 32, 32).float() * d_scale.view(n, k // 32, 1).float()
    check_all(d_y.view(1, n), w_dev.view(n, k), d_x.view(1, k), 1e-4)


@pytest.fixture(scope="module")
def q4k_full(pack):
    k, n = 5120, 25600
    w = oracle.fill_normal(n * k, seed_for(2, 0), 0.02)
    raw = oracle.quantize_q4_k(w)
    ns = n * k // 256
    d_data = torch.zeros(ns * 128, dtype=torch.uint8, device="cuda")
    d_sc = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
    d_raw = dev(raw)
    pack.call("kquant_repack", d_raw, d_data, d_sc, ns, 12)
    w_dev = torch.zeros(n * k, dtype=torch.float32, device="cuda")
    pack.call("kquant_dequant", d_raw, w_dev, ns, 12)
    torch.cuda.synchronize()
    return k, n, raw.reshape(n, k // 256 * 144), d_data, d_sc, w_dev.view(n, k)


@pytest.mark.parametrize("batch", [1, 4, 16])
def test_q4_k_full(pack, q4k_full, batch):
    k, n, raw, d_data, d_sc, w_dev = q4k_full
    x = bf16_activations(batch * k, seed_for(2, 100 + batch))
    d_x = dev_f32(x)
    d_y = torch.full((batch * n,), float("nan"), dtype=torch.float32, device="cuda")
    if batch == 1:
        pack.call("kquant_gemv", d_data, d_sc, d_x, d_y, k, n, 12)
    else:
        pack.call("pdk_kquant_gemm_f32", d_data, d_sc, d_x, d_y, k, n, batch, 12)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    rows = sample(np.random.default_rng(2 + batch), n, 256)
    toks = np.arange(batch)
    tight = batch <= 8          # integer tensor path; from 9 tokens on the f16-weight tcgen05 path
    check_sampled(d_y.cpu().numpy().reshape(batch, n), oracle.dequant_q4_k(raw[rows]).reshape(len(rows), k),
                  x.reshape(batch, k), rows, toks, k, 1e-5 if tight else 1e-4, 1e-4 if tight else 1e-3)
    check_all(d_y.view(batch, n), w_dev, d_x.view(batch, k), 1e-4 if tight else 1e-3)


# ---------------------------------------------------------------------------------- FP8 E4M3

@pytest.fixture(scope="module")
def fp8_tokens():
    m, k = 4096, 5120
    x = oracle.bf16_round(oracle.fill_normal(m * k, seed_for(3, 1), 1.0))
    xq, xs = oracle.quantize_fp8_absmax(x, m, k)
    d_xq, d_xs = dev(xq), dev_f32(xs)
    x_dev = d_xq.view(torch.float8_e4m3fn).view(m, k).float() * d_xs.view(m, 1)
    return m, k, xq, xs, d_xq, d_xs, x_dev


@pytest.mark.parametrize("n", [5120, 17408, 27648])
def test_f8row_gemm_full(pack, fp8_tokens, n):
    m, k, xq, xs, d_xq, d_xs, x_dev = fp8_tokens
    w = oracle.fill_normal(n * k, seed_for(3, n), 0.02)
    wq, ws = oracle.quantize_fp8_absmax(w, n, k)
    del w
    d_wq, d_ws = dev(wq), dev_f32(ws)
    w_dev = d_wq.view(torch.float8_e4m3fn).view(n, k).float() * d_ws.view(n, 1)
    rng = np.random.default_rng(n)
    rows, toks = sample(rng, n, 48), sample(rng, m, 12)
    wd = oracle.dequant_fp8_channel(wq[rows], ws[rows], k, len(rows))
    xd = oracle.dequant_fp8_channel(xq[toks], xs[toks], k, len(toks))
    for out, name in (("f32", "f8row_gemm"), ("bf16", "pdk_f8row_gemm_bf16")):
        d_y = torch.full((m * n,), float("nan"), dtype=torch.float32 if out == "f32" else torch.bfloat16, device="cuda")
        pack.call(name, d_wq, d_ws, d_xq, d_xs, d_y, k, n, m)
        torch.cuda.synchronize()
        assert pack.device_error() == 0
        y = d_y.view(m, n)[torch.from_numpy(toks).cuda()][:, torch.from_numpy(rows).cuda()].float().cpu().numpy()
        ref, ab = oracle.matmul_f64(wd, xd, k, len(rows), len(toks), with_abs=True)
        if out == "f32":
            assert cond_err(y, ref, ab) < 1e-5 < TOL
            assert rel_l2(y, ref) < 1e-5
        else:
            assert rel_l2(y, ref) < 4e-3 < TOL          # bf16 rounding of the output
        check_all(d_y.view(m, n), w_dev, x_dev, 3e-5 if out == "f32" else 4e-3)
        del d_y


# ---------------------------------------------------------------------------------- NVFP4

@pytest.fixture(scope="module")
def nvf4_full(pack):
    k, n = 5120, 17408
    w = oracle.fill_normal(n * k, seed_for(4, 0), 0.02)
    scale2 = float(np.abs(w).max() / (6.0 * 448.0))
    q, s = oracle.quantize_nvf4(w, scale2)
    q, s = q.reshape(n, k // 2), s.reshape(n, k // 16)
    d_q = dev(q)
    d_tiled = torch.zeros(((n + 127) // 128) * (k // 256) * 2048, dtype=torch.uint8, device="cuda")
    pack.call("nvf4_tc5_tile_scales", dev(s), d_tiled, k, n)
    w_dev = torch.zeros(n * k, dtype=torch.float32, device="cuda")
    pack.call("nvf4_dequant", d_q, dev(s), scale2, w_dev, k, n)
    torch.cuda.synchronize()
    return k, n, q, s, np.float32(scale2), d_q, d_tiled, w_dev.view(n, k)


@pytest.mark.parametrize("m", [1, 8, 64, 512, 8192])
def test_nvf4_gemm_full(pack, nvf4_full, m):
    k, n, q, s, scale2, d_q, d_tiled, w_dev = nvf4_full
    x = oracle.bf16_round(oracle.fill_normal(m * k, seed_for(4, 10 + m), 1.0))
    d_x = dev_f32(x)
    d_xq = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
    d_xs = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    pack.call("quantize_nvf4", d_x, d_xq, d_xs, m * k)
    torch.cuda.synchronize()
    # activations as the GEMM sees them: the quantizer's planes (bit-exact against the oracle in the
    # small cases), dequantized on the device for the full check and by the oracle for the samples
    x_dev = torch.zeros(m * k, dtype=torch.float32, device="cuda")
    pack.call("nvf4_dequant", d_xq, d_xs, 1.0, x_dev, k, m)
    rng = np.random.default_rng(m)
    rows, toks = sample(rng, n, 48), sample(rng, m, 12)
    xq, xs = d_xq.cpu().numpy().reshape(m, k // 2), d_xs.cpu().numpy().reshape(m, k // 16)
    wd = oracle.dequant_nvfp4(q[rows], s[rows], scale2, k, len(rows))
    xd = oracle.dequant_nvfp4(xq[toks], xs[toks], 1.0, k, len(toks))
    ref, ab = oracle.matmul_f64(wd, xd, k, len(rows), len(toks), with_abs=True)
    sel = lambda t: t.view(m, n)[torch.from_numpy(toks).cuda()][:, torch.from_numpy(rows).cuda()].float().cpu().numpy()
    d_y = torch.full((m * n,), float("nan"), dtype=torch.float32, device="cuda")
    pack.call("nvf4_gemm_tc5w", d_q, d_tiled, None, d_xq, d_xs, d_y, float(scale2), k, n, m, None, 0)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    assert cond_err(sel(d_y), ref, ab) < 1e-5 < TOL
    assert rel_l2(sel(d_y), ref) < 1e-4
    check_all(d_y.view(m, n), w_dev, x_dev.view(m, k), 1e-4)
    del d_y
    d_yb = torch.full((m * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    pack.call("pdk_nvf4_gemm_bf16", d_q, d_tiled, None, d_xq, d_xs, d_yb, float(scale2), k, n, m)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    assert rel_l2(sel(d_yb), ref) < 4e-3 < TOL
    check_all(d_yb.view(m, n), w_dev, x_dev.view(m, k), 4e-3)


# ---------------------------------------------------------------------------------- MXFP4 MoE

N_EXPERT, TOP_K, EMBD, FF = 128, 4, 2880, 2880


@pytest.fixture(scope="module")
def moe_full(pack):
    """128 experts of N(0, 0.02) weights quantized to MXFP4 by the oracle, one expert at a time."""
    ex = P.GpuExecutor(pack)
    per = FF * EMBD // 32 * 17
    raw = {name: np.empty(N_EXPERT * per, np.uint8) for name in ("gate", "up", "down")}
    for i, name in enumerate(("gate", "up", "down")):
        for e in range(N_EXPERT):
            raw[name][e * per:(e + 1) * per] = oracle.quantize_mxfp4(
                oracle.fill_normal(FF * EMBD, seed_for(5, 1000 * i + e), 0.02))
    planes = P.MoeMxfp4Planes(P.repack_mxfp4(ex, dev(raw["gate"])), P.repack_mxfp4(ex, dev(raw["up"])),
                              P.repack_mxfp4(ex, dev(raw["down"])), N_EXPERT, EMBD, FF)
    torch.cuda.synchronize()
    return ex, raw, per, planes


@pytest.mark.parametrize("path", ["tc5", "mma"])
@pytest.mark.parametrize("tokens", [1, 64, 1024])
def test_moe_block_full(pack, moe_full, tokens, path):
    ex, raw, per, planes = moe_full
    if path == "tc5":
        P.prepare_tc5(ex, planes)
    saved, planes.tc5 = planes.tc5, (planes.tc5 if path == "tc5" else None)
    try:
        bm = 8 if tokens * TOP_K <= 1024 else 32
        x = oracle.bf16_round(oracle.fill_normal(tokens * EMBD, seed_for(5, 7000 + tokens), 1.0))
        logits = oracle.fill_normal(tokens * N_EXPERT, seed_for(5, 8000 + tokens), 1.0)
        ws = P.MoeWorkspace(ex, planes, tokens, TOP_K, bm)
        out = torch.zeros(tokens * EMBD, dtype=torch.float32, device="cuda")
        P.moe_mxfp4_forward(ex, planes, ws, dev_f32(x), dev_f32(logits), out)
        torch.cuda.synchronize()
        assert pack.device_error() == 0
    finally:
        planes.tc5 = saved
    idx, w = oracle.moe_topk(logits, N_EXPERT, TOP_K)
    assert np.array_equal(ws.idx.cpu().numpy().view(np.uint32).reshape(tokens, TOP_K), idx)   # routing of every token
    y = out.cpu().numpy().reshape(tokens, EMBD)
    assert np.isfinite(y).all()
    # the oracle's block for a sample of tokens, over the experts those tokens use (renumbered)
    toks = sample(np.random.default_rng(tokens), tokens, 20)
    used, inv = np.unique(idx[toks], return_inverse=True)
    sub = {name: np.concatenate([raw[name][e * per:(e + 1) * per] for e in used]) for name in raw}
    ref = oracle.moe_mxfp4_layer(sub["gate"], sub["up"], sub["down"], x.reshape(tokens, EMBD)[toks],
                                 inv.reshape(len(toks), TOP_K).astype(np.uint32), w[toks], len(toks), TOP_K, EMBD, FF)
    assert rel_l2(y[toks], ref) < 2e-3 < TOL
    assert np.max(np.abs(y[toks] - ref)) < 1e-2 * np.max(np.abs(ref))
    # tokens outside the sample: the same scale, nothing left at zero
    rms = np.sqrt((y.astype(np.float64) ** 2).mean(axis=1))
    assert rms.min() > 0.2 * np.median(rms) and rms.max() < 5.0 * np.median(rms)
