"""NVFP4 path (K=5120, N=17408 in the benchmark): quantizer and dequant bit-exact against the
oracle, W4A16 GEMV and the block-scaled tcgen05 W4A4 GEMM within 1e-2 of an
f64 matmul of the dequantized operands."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, cond_err, dev, dev_f32, rel_l2

pytestmark = pytest.mark.gpu


def nvf4_weights(n, k, seed):
    """The benchmark recipe: per-tensor scale2 = absmax / (6 * 448), e4m3 block scales, e2m1 elements."""
    w = oracle.fill_normal(n * k, seed, 0.02)
    scale2 = float(np.abs(w).max() / (6.0 * 448.0))
    q, s = oracle.quantize_nvf4(w, scale2)
    return q.reshape(n, k // 2), s.reshape(n, k // 16), np.float32(scale2)


@pytest.mark.parametrize("n", [32, 5120, 64 * 5120])
def test_quantize_nvf4_bit_exact(pack, n):
    x = oracle.fill_normal(n, 600 + n, 1.0)
    x[:16] = 0.0
    x[16:32] *= 1e-6
    q_ref, s_ref = oracle.quantize_nvf4(x)
    d_q = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(n // 16, dtype=torch.uint8, device="cuda")
    pack.call("quantize_nvf4", dev_f32(x), d_q, d_s, n)
    torch.cuda.synchronize()
    assert np.array_equal(d_s.cpu().numpy(), s_ref)
    assert np.array_equal(d_q.cpu().numpy(), q_ref)


def test_nvf4_dequant_bit_exact_all_codes(pack):
    n, k = 16, 512
    rng = np.random.default_rng(3)
    q = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = rng.integers(0, 0x7F, (n, k // 16), dtype=np.uint8)   # finite e4m3 scale bytes
    scale2 = np.float32(0.0173)
    d_y = torch.zeros(n * k, dtype=torch.float32, device="cuda")
    pack.call("nvf4_dequant", dev(q), dev(s), float(scale2), d_y, k, n)
    torch.cuda.synchronize()
    ref = oracle.dequant_nvfp4(q, s, scale2, k, n)
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), ref.reshape(-1).view(np.uint32))


@pytest.mark.parametrize("k,n", [(32, 3), (1024, 77), (5120, 512)])
def test_nvf4_gemv_w4a16(pack, k, n):
    q, s, scale2 = nvf4_weights(n, k, 610 + n)
    x = oracle.bf16_round(oracle.fill_normal(k, 611, 1.0))
    bias = oracle.fill_normal(n, 612, 0.1)
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("nvf4_gemv", dev(q), dev(s), dev_f32(bias), dev_f32(x), d_y, float(scale2), k, n)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_nvfp4(q, s, scale2, k, n), x, k, n, 1, with_abs=True)
    y = d_y.cpu().numpy() - bias
    assert cond_err(y, ref[0], ab[0]) < 1e-5 < TOL


def tile_scales_ref(s, n, k):
    """byte l*16 + c*4 + b of cell j of record (rt, kb) = scale[rt*128 + c*32 + l][kb*16 + j*4 + b]"""
    n_rt, n_kb = (n + 127) // 128, k // 256
    pad = np.zeros((n_rt * 128, k // 16), np.uint8)
    pad[:n] = s
    t = pad.reshape(n_rt, 4, 32, n_kb, 4, 4)          # rt, c, l, kb, j, b
    return np.ascontiguousarray(t.transpose(0, 3, 4, 2, 1, 5)).reshape(-1)   # rt, kb, j, l, c, b


def test_tile_scales_layout(pack):
    n, k = 300, 1024
    s = np.random.default_rng(9).integers(0, 256, (n, k // 16), dtype=np.uint8)
    want = tile_scales_ref(s, n, k)
    d_t = torch.full((want.size,), 0xAA, dtype=torch.uint8, device="cuda")
    pack.call("nvf4_tc5_tile_scales", dev(s), d_t, k, n)
    torch.cuda.synchronize()
    assert np.array_equal(d_t.cpu().numpy(), want)


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (8, 128, 512), (64, 384, 5120), (33, 256, 1280), (128, 128, 256), (130, 200, 768),
                                   (512, 1024, 5120),
                                   # enough 256-row x 128-token tiles for every pair of SMs: the cta_group::2
                                   # kernel, whole tiles and ragged ones (odd count of 128-row tiles, odd slabs)
                                   (1024, 2560, 512), (1000, 2440, 768), (200, 9600, 256)])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_nvf4_gemm_w4a4(pack, m, n, k, out):
    check_nvf4_gemm_w4a4(pack, m, n, k, out)


@pytest.mark.parametrize("m,n,k", [(1024, 2560, 512), (1000, 2440, 768), (200, 9600, 256), (300, 2560, 1280), (257, 2304, 256)])
@pytest.mark.parametrize("out", ["f32", "bf16"])
@pytest.mark.parametrize("tile", [128, 256])
def test_nvf4_gemm_w4a4_pair_kernel_forms(pack, monkeypatch, m, n, k, out, tile):
    """Both token-tile widths of the pair kernel on the same shapes (whole and ragged tiles; an odd
    count of 128-token scale records)."""
    monkeypatch.setenv("PDK_NVF4_PAIR_BN", str(tile))
    check_nvf4_gemm_w4a4(pack, m, n, k, out)


def check_nvf4_gemm_w4a4(pack, m, n, k, out):
    q, s, scale2 = nvf4_weights(n, k, 620 + n + m)
    x = oracle.bf16_round(oracle.fill_normal(m * k, 621 + m, 1.0))
    d_x = dev_f32(x)
    d_xq = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
    d_xs = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    pack.call("quantize_nvf4", d_x, d_xq, d_xs, m * k)
    d_tiled = torch.zeros(((n + 127) // 128) * (k // 256) * 2048, dtype=torch.uint8, device="cuda")
    pack.call("nvf4_tc5_tile_scales", dev(s), d_tiled, k, n)
    bias = oracle.fill_normal(n, 622, 0.1)
    if out == "f32":
        d_y = torch.full((m * n,), float("nan"), dtype=torch.float32, device="cuda")
        pack.call("nvf4_gemm_tc5w", dev(q), d_tiled, dev_f32(bias), d_xq, d_xs, d_y, float(scale2), k, n, m, None, 0)
    else:
        d_y = torch.full((m * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
        pack.call("pdk_nvf4_gemm_bf16", dev(q), d_tiled, dev_f32(bias), d_xq, d_xs, d_y, float(scale2), k, n, m)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    xq, xs = oracle.quantize_nvf4(x)
    wd = oracle.dequant_nvfp4(q, s, scale2, k, n)
    xd = oracle.dequant_nvfp4(xq.reshape(m, k // 2), xs.reshape(m, k // 16), 1.0, k, m)
    ref, ab = oracle.matmul_f64(wd, xd, k, n, m, with_abs=True)
    y = d_y.float().cpu().numpy().reshape(m, n) - bias[None, :]
    assert np.isfinite(y).all()
    if out == "f32":
        assert cond_err(y, ref, ab) < 1e-5 < TOL
        assert rel_l2(y, ref) < 1e-4
    else:
        assert rel_l2(y, ref) < 2e-2   # bf16 rounding of acc + bias with |bias| >> |acc|


@pytest.mark.parametrize("n,batch,residual", [(5120, 3, True), (2880 + 32, 1, True), (64, 5, False), (17408, 2, True)])
def test_add_rmsnorm_quant_nvf4_batch(pack, n, batch, residual):
    """Slot 436: the summed row is written back bit-exactly, the normed row matches the oracle's
    arithmetic to an ulp of the scale, and the NVFP4 planes are exactly the quantizer's output on
    the normed row the kernel wrote."""
    x = oracle.fill_normal(batch * n, 4100 + n, 1.5).reshape(batch, n)
    proj = oracle.fill_normal(batch * n, 4101 + n, 0.5).reshape(batch, n) if residual else None
    w = (1.0 + 0.1 * oracle.fill_normal(n, 4102, 1.0)).astype(np.float32)
    x[0, :16] = 0.0
    if residual:
        proj[0, :16] = 0.0                       # an all-zero 16-block: scale byte 0
    eps = 1e-6
    v_ref, out_ref = oracle.add_rmsnorm(x, proj, w, eps)
    d_x = dev_f32(x.reshape(-1))
    d_out = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    d_q = torch.zeros(batch * n // 2, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(batch * n // 16, dtype=torch.uint8, device="cuda")
    pack.call("add_rmsnorm_quant_nvf4_batch", d_x, dev_f32(proj.reshape(-1)) if residual else None, dev_f32(w), d_out, d_q,
              d_s, n, eps, batch)
    torch.cuda.synchronize()
    assert np.array_equal(d_x.cpu().numpy().view(np.uint32), v_ref.reshape(-1).view(np.uint32))
    out = d_out.cpu().numpy().reshape(batch, n)
    assert np.allclose(out, out_ref, rtol=4e-7, atol=0)
    for b in range(batch):
        q_ref, s_ref = oracle.quantize_nvf4(out[b])
        assert np.array_equal(d_q.cpu().numpy().reshape(batch, -1)[b], q_ref)
        assert np.array_equal(d_s.cpu().numpy().reshape(batch, -1)[b], s_ref)
    assert d_s.cpu().numpy()[0] == 0


def test_add_rmsnorm_quant_nvf4_refuses_bad_shapes(pack):
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    assert pack.status("add_rmsnorm_quant_nvf4_batch", buf, None, buf, buf, buf, buf, 48, 1e-6, 1) == 1
    assert pack.status("add_rmsnorm_quant_nvf4_batch", buf, None, buf, buf, buf, buf, 0, 1e-6, 1) == 0


@pytest.mark.parametrize("rows,ff", [(1, 32), (3, 2880), (40, 17408)])
def test_swiglu_in_front_of_the_nvf4_quantizer(pack, rows, ff):
    """Slots 120 (two planes) and 516 (fused gate | up rows): the same planes, and the quantizer's
    output on silu(gate) * up (numpy's f32 exp may be an ulp off the device's: codes equal or one
    step apart on a handful of elements, scale bytes likewise)."""
    g = oracle.fill_normal(rows * ff, 4300 + ff, 2.0).reshape(rows, ff)
    u = oracle.fill_normal(rows * ff, 4301 + ff, 1.0).reshape(rows, ff)
    h = oracle.swiglu_silu(g, u)
    q_ref, s_ref = oracle.quantize_nvf4(h.reshape(-1))
    outs = []
    for fused in (False, True):
        d_q = torch.zeros(rows * ff // 2, dtype=torch.uint8, device="cuda")
        d_s = torch.zeros(rows * ff // 16, dtype=torch.uint8, device="cuda")
        if fused:
            pack.call("swiglu_fused_nvf4", dev_f32(np.concatenate([g, u], axis=1).reshape(-1)), d_q, d_s, ff, rows)
        else:
            pack.call("quantize_nvf4_swiglu", dev_f32(g.reshape(-1)), dev_f32(u.reshape(-1)), d_q, d_s, rows * ff)
        torch.cuda.synchronize()
        outs.append((d_q.cpu().numpy(), d_s.cpu().numpy()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert np.mean(outs[0][1] != s_ref.reshape(-1)) < 2e-3
    assert np.mean(outs[0][0] != q_ref.reshape(-1)) < 5e-3
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert pack.status("quantize_nvf4_swiglu", buf, buf, buf, buf, 48) == 1
    assert pack.status("swiglu_fused_nvf4", buf, buf, buf, 48, 2) == 1


def test_add_rmsnorm_nvf4_batch_is_slot_436_with_a_residual(pack):
    n, batch, eps = 5120, 3, 1e-6
    x = oracle.fill_normal(batch * n, 4400, 1.5)
    proj = oracle.fill_normal(batch * n, 4401, 0.5)
    w = (1.0 + 0.1 * oracle.fill_normal(n, 4402, 1.0)).astype(np.float32)
    res = []
    for name in ("add_rmsnorm_quant_nvf4_batch", "add_rmsnorm_nvf4_batch"):
        d_x, d_out = dev_f32(x), torch.zeros(batch * n, dtype=torch.float32, device="cuda")
        d_q = torch.zeros(batch * n // 2, dtype=torch.uint8, device="cuda")
        d_s = torch.zeros(batch * n // 16, dtype=torch.uint8, device="cuda")
        pack.call(name, d_x, dev_f32(proj), dev_f32(w), d_out, d_q, d_s, n, eps, batch)
        torch.cuda.synchronize()
        res.append([t.cpu().numpy() for t in (d_x, d_out, d_q, d_s)])
    for a, b in zip(*res):
        assert np.array_equal(a, b)
    d = torch.zeros(64, dtype=torch.float32, device="cuda")
    assert pack.status("add_rmsnorm_nvf4_batch", d, None, d, d, d, d, 32, eps, 1) == 1
