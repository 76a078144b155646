"""FP8 E4M3 row-scaled path: quantizers bit-exact against the oracle, tcgen05
GEMM within 1e-2 (in practice ~1e-6) of an f64 matmul of the dequantized
operands (the FP8 prefill benchmark: 4096 tokens, K=5120)."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, cond_err, dev, dev_f32, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,k", [(1, 16), (3, 100), (64, 5120)])
def test_quantize_e4m3_row_bit_exact(pack, rows, k):
    x = oracle.fill_normal(rows * k, 400 + k, 1.0)
    x[0] *= 448.0
    q_ref, s_ref = oracle.quantize_e4m3_row_pow2(x, rows, k)
    d_q = torch.zeros(rows * k, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    pack.call("quantize_e4m3_row", dev_f32(x), d_q, d_s, k, rows)
    torch.cuda.synchronize()
    assert np.array_equal(d_s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(d_q.cpu().numpy().reshape(rows, k), q_ref)


def test_bf16_to_f8row_bit_exact(pack):
    rows, k = 37, 640
    w = oracle.bf16_round(oracle.fill_normal(rows * k, 410, 0.02))
    w[k:2 * k] = 0.0                     # an all-zero row keeps scale 1 and codes 0
    q_ref, s_ref = oracle.quantize_e4m3_row_pow2(w, rows, k)
    d_w = torch.from_numpy(w).cuda().to(torch.bfloat16)
    d_q = torch.zeros(rows * k, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    pack.call("bf16_to_f8row", d_w, d_q, d_s, k, rows)
    torch.cuda.synchronize()
    assert np.array_equal(d_s.cpu().numpy(), s_ref)
    assert np.array_equal(d_q.cpu().numpy().reshape(rows, k), q_ref)


def codes_agree(got, want, budget=2e-3):
    """e4m3 codes equal, or one step apart where the input sat within an ulp of a rounding tie."""
    got, want = np.asarray(got, np.int16), np.asarray(want, np.int16)
    off = got != want
    assert np.mean(off) < budget
    assert (np.abs(got[off] - want[off]) <= 1).all()


@pytest.mark.parametrize("rows,n", [(1, 64), (3, 5120), (70, 17408), (2, 40000)])
def test_quantize_e4m3_row_single_pass_route(pack, rows, n):
    """Rows of whole, aligned float4 take the register-resident kernel: same bytes as the oracle."""
    x = oracle.fill_normal(rows * n, 430 + n, 3.0)
    x[:n] *= 1e-3
    q_ref, s_ref = oracle.quantize_e4m3_row_pow2(x, rows, n)
    d_q = torch.zeros(rows * n, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    pack.call("quantize_e4m3_row", dev_f32(x), d_q, d_s, n, rows)
    torch.cuda.synchronize()
    assert np.array_equal(d_s.cpu().numpy(), s_ref)
    assert np.array_equal(d_q.cpu().numpy().reshape(rows, n), q_ref)


@pytest.mark.parametrize("rows,n", [(1, 64), (5, 5120), (80, 17408)])
def test_swiglu_quant_e4m3_row(pack, rows, n):
    """Slot 511: silu(gate) * up, then the row quantizer."""
    g = oracle.fill_normal(rows * n, 440 + n, 2.0).reshape(rows, n)
    u = oracle.fill_normal(rows * n, 441 + n, 1.0).reshape(rows, n)
    g[0, :32] = 0.0
    h = oracle.swiglu_silu(g, u)
    q_ref, s_ref = oracle.quantize_e4m3_row_pow2(h.reshape(-1), rows, n)
    d_q = torch.zeros(rows * n, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    pack.call("swiglu_quant_e4m3_row", dev_f32(g.reshape(-1)), dev_f32(u.reshape(-1)), d_q, d_s, n, rows)
    torch.cuda.synchronize()
    assert np.array_equal(d_s.cpu().numpy(), s_ref)
    codes_agree(d_q.cpu().numpy().reshape(rows, n), q_ref)


@pytest.mark.parametrize("rows,n,residual", [(1, 64, False), (4, 5120, True), (70, 5120, True), (3, 17408, False), (2, 32768, True)])
def test_rmsnorm_quant_e4m3_row(pack, rows, n, residual):
    """Slots 512 / 513: the summed row is written back bit-exactly, the normed row agrees with the
    oracle to an ulp of the norm scale, and the codes are exactly the row quantizer's on the normed
    row the kernel wrote."""
    x = oracle.fill_normal(rows * n, 450 + n, 1.5).reshape(rows, n)
    proj = oracle.fill_normal(rows * n, 451 + n, 0.5).reshape(rows, n) if residual else None
    w = (1.0 + 0.1 * oracle.fill_normal(n, 452, 1.0)).astype(np.float32)
    eps, pscale = 1e-6, 0.75
    v_ref, xn_ref = oracle.rmsnorm_scaled_add(x, proj, w, eps, pscale)
    d_x = dev_f32(x.reshape(-1))
    d_xn = torch.zeros(rows * n, dtype=torch.float32, device="cuda")
    d_q = torch.zeros(rows * n, dtype=torch.uint8, device="cuda")
    d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    if residual:
        pack.call("add_rmsnorm_scaled_quant_e4m3_row", d_x, dev_f32(proj.reshape(-1)), dev_f32(w), d_xn, d_q, d_s, n, eps,
                  pscale, rows)
    else:
        pack.call("rmsnorm_quant_e4m3_row", d_x, dev_f32(w), d_xn, d_q, d_s, n, eps, rows)
    torch.cuda.synchronize()
    assert np.array_equal(d_x.cpu().numpy().reshape(rows, n).view(np.uint32), v_ref.view(np.uint32))
    xn = d_xn.cpu().numpy().reshape(rows, n)
    assert np.allclose(xn, xn_ref, rtol=4e-7, atol=0)
    q_own, s_own = oracle.quantize_e4m3_row_pow2(xn.reshape(-1), rows, n)
    assert np.array_equal(d_s.cpu().numpy(), s_own)
    assert np.array_equal(d_q.cpu().numpy().reshape(rows, n), q_own)


def test_e4m3_producers_refuse_bad_shapes(pack):
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert pack.status("swiglu_quant_e4m3_row", buf, buf, buf, buf, 100, 2) == 1                 # n % 32
    assert pack.status("rmsnorm_quant_e4m3_row", buf.data_ptr() + 4, buf, buf, buf, buf, 64, 1e-6, 1) == 1
    assert pack.status("add_rmsnorm_scaled_quant_e4m3_row", buf, None, buf, buf, buf, buf, 64, 1e-6, 1.0, 1) == 1
    assert pack.status("rmsnorm_quant_e4m3_row", buf, buf, buf, buf, buf, 64, 1e-6, 0) == 0


def fp8_case(m, n, k, seed):
    w = oracle.fill_normal(n * k, seed, 0.02)
    x = oracle.bf16_round(oracle.fill_normal(m * k, seed + 1, 1.0))
    wq, ws = oracle.quantize_fp8_absmax(w, n, k)      # the FP8 benchmark recipe: scale = absmax / 448
    xq, xs = oracle.quantize_fp8_absmax(x, m, k)
    wd = oracle.dequant_fp8_channel(wq, ws, k, n)
    xd = oracle.dequant_fp8_channel(xq, xs, k, m)
    ref, ab = oracle.matmul_f64(wd, xd, k, n, m, with_abs=True)
    return wq, ws, xq, xs, ref, ab


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (256, 512, 5120), (1, 8, 64), (300, 260, 1040),
                                   (129, 257 * 4, 2048), (1024, 2048, 5120),
                                   # enough 256 x 256 tiles for every pair of SMs: the cta_group::2 kernel,
                                   # whole tiles and ragged ones (tokens, channels and K)
                                   (1024, 4864, 256), (1000, 4900, 400), (257, 19000, 128)])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_f8row_gemm(pack, m, n, k, out):
    if out == "bf16" and (m, n, k) == (1024, 2048, 5120):
        pytest.skip("large case once")
    wq, ws, xq, xs, ref, ab = fp8_case(m, n, k, 500 + m + n)
    d_y = torch.full((m * n,), float("nan"), dtype=torch.float32 if out == "f32" else torch.bfloat16, device="cuda")
    name = "f8row_gemm" if out == "f32" else "pdk_f8row_gemm_bf16"
    pack.call(name, dev(wq), dev_f32(ws), dev(xq), dev_f32(xs), d_y, k, n, m)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    y = d_y.float().cpu().numpy().reshape(m, n)
    assert np.isfinite(y).all()
    if out == "f32":
        assert cond_err(y, ref, ab) < 1e-5 < TOL
        assert rel_l2(y, ref) < 1e-5
    else:
        assert rel_l2(y, ref) < 4e-3 < TOL      # bf16 rounding of the output


def test_f8row_gemm_tc5x_slot_matches(pack):
    m, n, k = 128, 512, 1024
    wq, ws, xq, xs, ref, ab = fp8_case(m, n, k, 77)
    d_y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    pack.call("f8row_gemm_tc5x", dev(wq), dev_f32(ws), dev(xq), dev_f32(xs), d_y, k, n, m)
    torch.cuda.synchronize()
    assert cond_err(d_y.cpu().numpy().reshape(m, n), ref, ab) < 1e-5


def test_f8row_gemm_refuses_bad_shapes(pack):
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    assert pack.status("f8row_gemm", buf, buf, buf, buf, buf, 100, 8, 8) == 1        # K % 16
    assert pack.status("f8row_gemm", buf.data_ptr() + 8, buf, buf, buf, buf, 128, 8, 8) == 1
    assert pack.status("f8row_gemm", buf, buf, buf, buf, buf, 128, 0, 8) == 0


def test_bounded_wait_gives_up_and_reports(pack):
    """The wait under every tcgen05 kernel: a barrier nothing arrives on must time out after the
    budget, leave its code in the error word and let the kernel return; the context stays usable."""
    import time
    scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert pack.device_error() == 0
    t0 = time.perf_counter()
    assert pack.status("pdk_selftest_bounded_wait", 2000, scratch) == 0      # 2 ms budget
    dt = time.perf_counter() - t0
    assert 0.001 < dt < 1.0
    assert pack.device_error() == (5 << 8 | 7)
    assert pack.device_error() == 0                                          # read clears
    assert pack.status("pdk_selftest_bounded_wait", 0, scratch) == 1
    y = torch.ones(8, device="cuda") * 2                                     # the context still works
    assert float(y.sum()) == 16.0
