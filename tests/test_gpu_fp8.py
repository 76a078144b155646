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
