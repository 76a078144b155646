"""The C++ operator layer (libpaddock_exec.so) on a GPU: weights go from a GGUF file or a
checkpoint view through the loaders of crates/paddock-engine/src/gpu (load_quantw, upload_raw,
repack_kquant_bands / _concat, bf16_to_f8row, nvf4_upload) into resident planes, and the launch
wrappers are checked against the oracle like the slots underneath them."""
import struct

import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, bf16_activations, cond_err, dev, dev_f32, rel_l2
from paddock_b200 import executor as X
from paddock_b200 import formats as F
from test_formats import build_gguf, gstr
from test_gpu_gemv import raw_kquant

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ex():
    e = X.GpuExecutor()
    yield e
    e.close()


def run(ex, fn, *args):
    """Launch on the executor's stream once torch's stream has produced the operands."""
    torch.cuda.synchronize()
    fn(*args)
    ex.synchronize()


K, N = 1024, 48


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    """One GGUF file holding a tensor of every type the loaders dispatch on."""
    w = oracle.fill_normal(N * K, 9100, 0.02)
    t = {
        "q8.weight": (8, oracle.quantize_q8_0(w).tobytes(), [K, N]),
        "q4k.weight": (12, oracle.quantize_q4_k(w).tobytes(), [K, N]),
        "q5k.weight": (13, raw_kquant("q5_k", N * K // 256, 9101).tobytes(), [K, N]),
        "q6k.weight": (14, raw_kquant("q6_k", N * K // 256, 9102).tobytes(), [K, N]),
        "q40.weight": (2, raw_kquant("q4_0", N * K // 256, 9103).tobytes(), [K, N]),
        "q40_odd.weight": (2, raw_kquant("q4_0", N * 3, 9104)[: N * 96 // 32 * 18].tobytes(), [96, N]),
        "q4k_b.weight": (12, oracle.quantize_q4_k(oracle.fill_normal(16 * K, 9105, 0.02)).tobytes(), [K, 16]),
        "f32.weight": (0, np.ones(64, np.float32).tobytes(), [64]),
    }
    path = tmp_path_factory.mktemp("exec") / "model.gguf"
    path.write_bytes(build_gguf([(n, dims, ty, raw) for n, (ty, raw, dims) in t.items()],
                                [("general.architecture", 8, gstr("llama"))]))
    return F.MappedGguf(str(path)), t


DEQ = {8: oracle.dequant_q8_0, 12: oracle.dequant_q4_k, 13: lambda b: oracle.dequant_kquant("q5_k", b),
       14: lambda b: oracle.dequant_kquant("q6_k", b), 2: lambda b: oracle.dequant_kquant("q4_0", b)}


@pytest.mark.parametrize("name,kind", [("q8.weight", "Q8"), ("q4k.weight", "Kq"), ("q5k.weight", "Kq"), ("q6k.weight", "Kq"),
                                       ("q40.weight", "Kq"), ("q40_odd.weight", "Q8")])
def test_load_quantw_dispatches_per_tensor_and_the_gemv_matches(ex, model, name, kind):
    mapped, tensors = model
    ty, raw, dims = tensors[name]
    w = ex.load_quantw(mapped, name)
    assert w.kind == kind and w.dims == (dims[0], dims[1])
    k, n = dims
    want = DEQ[ty](np.frombuffer(raw, np.uint8))
    # resident bytes: exact, per stream
    per = {"Q8": 34 / 32, "Kq": {12: 152, 13: 184, 14: 216, 2: 152}.get(ty, 0) / 256}[kind]
    assert w.bytes() == int(n * k * per)
    for batch in (1, 3):
        x = bf16_activations(batch * k, 9200 + batch)
        d_x, d_y = dev_f32(x), torch.zeros(batch * n, dtype=torch.float32, device="cuda")
        if batch == 1:
            run(ex, ex.quantw_gemv, w, None, d_x, d_y)
        else:
            run(ex, ex.quantw_gemm, w, None, d_x, d_y, batch)
        ref, ab = oracle.matmul_f64(want, x, k, n, batch, with_abs=True)
        assert cond_err(d_y.cpu().numpy().reshape(batch, n), ref, ab) < 1e-5 < TOL


def test_load_quantw_refuses_a_type_without_a_kernel_class(ex, model):
    with pytest.raises(X.GpuError) as e:
        ex.load_quantw(model[0], "f32.weight")
    assert e.value.kind == "NoKernel"
    with pytest.raises(X.GpuError) as e:
        ex.load_quantw(model[0], "absent.weight")
    assert e.value.kind == "Format"


@pytest.mark.parametrize("name", ["q8.weight", "q4k.weight", "q6k.weight", "q40.weight"])
def test_upload_raw_keeps_the_bytes_and_dequantizes_row_slices(ex, model, name):
    mapped, tensors = model
    ty, raw, dims = tensors[name]
    k, n = dims
    t = ex.upload_raw(mapped, name)
    i = t.info()
    assert t.kind == "Raw" and i.ggml_type == (8 if ty == 2 else ty)      # Q4_0 lands as its Q8_0 transcode
    want = DEQ[ty](np.frombuffer(raw, np.uint8)).reshape(n, k)
    d_out = torch.zeros(5 * k, dtype=torch.float32, device="cuda")
    run(ex, ex.dequant_rows, t, 7, 5, d_out)
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32).reshape(5, k), want[7:12].view(np.uint32))
    with pytest.raises(X.GpuError):
        ex.dequant_rows(t, n - 2, 5, d_out)


def test_bands_and_concat_are_inverse_views_of_one_weight(ex, model):
    mapped, tensors = model
    want = oracle.dequant_q4_k(np.frombuffer(tensors["q4k.weight"][1], np.uint8)).reshape(N, K)
    x = bf16_activations(K, 9300)
    bands = ex.repack_kquant_bands(mapped, "q4k.weight", 2)
    assert [b.dims for b in bands] == [(K // 2, N)] * 2
    for b, plane in enumerate(bands):
        d_y = torch.zeros(N, dtype=torch.float32, device="cuda")
        run(ex, ex.quantw_gemv, plane, None, dev_f32(x[b * K // 2:(b + 1) * K // 2]), d_y)
        strip = np.ascontiguousarray(want[:, b * K // 2:(b + 1) * K // 2]).reshape(-1)
        ref, ab = oracle.matmul_f64(strip, x[b * K // 2:(b + 1) * K // 2], K // 2, N, 1, with_abs=True)
        assert cond_err(d_y.cpu().numpy().reshape(1, N), ref, ab) < 1e-5
    with pytest.raises(X.GpuError):
        ex.repack_kquant_bands(mapped, "q4k.weight", 3)          # 1024 / 3 is not whole super-blocks
    cat = ex.repack_kquant_concat(mapped, ["q4k.weight", "q4k_b.weight"])
    assert cat.dims == (K, N + 16)
    want_b = oracle.dequant_q4_k(np.frombuffer(tensors["q4k_b.weight"][1], np.uint8))
    d_y = torch.zeros(N + 16, dtype=torch.float32, device="cuda")
    run(ex, ex.quantw_gemv, cat, None, dev_f32(x), d_y)
    ref, ab = oracle.matmul_f64(np.concatenate([want.reshape(-1), want_b]), x, K, N + 16, 1, with_abs=True)
    assert cond_err(d_y.cpu().numpy().reshape(1, N + 16), ref, ab) < 1e-5
    with pytest.raises(X.GpuError):
        ex.repack_kquant_concat(mapped, ["q4k.weight", "q6k.weight"])


def test_staging_buffer_grows_to_the_largest_tensor_under_the_cap(ex, model):
    ex.release_staging()
    assert ex.staging_bytes() == 0
    ex.load_quantw(model[0], "q4k_b.weight")
    small = ex.staging_bytes()
    assert small == 16 * K // 256 * 144
    ex.load_quantw(model[0], "q6k.weight")
    assert ex.staging_bytes() == N * K // 256 * 210 > small
    ex.load_quantw(model[0], "q4k_b.weight")
    assert ex.staging_bytes() == N * K // 256 * 210            # reused, not shrunk


def test_f8row_plane_from_bf16_and_from_a_checkpoint_view(ex):
    m, n, k = 40, 192, 512
    w = oracle.bf16_round(oracle.fill_normal(n * k, 9400, 0.02))
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)
    plane = ex.bf16_to_f8row(bits, k, n)
    assert plane.kind == "F8Row" and plane.bytes() == n * k + 4 * n
    q_ref, s_ref = oracle.quantize_e4m3_row_pow2(w, n, k)
    x = oracle.bf16_round(oracle.fill_normal(m * k, 9401, 1.0))
    d_xq = torch.zeros(m * k, dtype=torch.uint8, device="cuda")
    d_xs = torch.zeros(m, dtype=torch.float32, device="cuda")
    d_y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    d_x = dev_f32(x)
    run(ex, ex.quantize_e4m3_row, d_x, d_xq, d_xs, k, m)
    run(ex, ex.f8row_gemm, plane, d_xq, d_xs, d_y, m)
    xq, xs = oracle.quantize_e4m3_row_pow2(x, m, k)
    assert np.array_equal(d_xq.cpu().numpy().reshape(m, k), xq)
    wd = oracle.dequant_fp8_channel(q_ref, s_ref, k, n)
    xd = oracle.dequant_fp8_channel(xq, xs, k, m)
    ref, ab = oracle.matmul_f64(wd, xd, k, n, m, with_abs=True)
    assert cond_err(d_y.cpu().numpy().reshape(m, n), ref, ab) < 1e-5 < TOL
    # the same weight as a per-channel FP8 checkpoint hands it over: codes + f32 row scales, no device pass
    plane2 = ex.f8row_upload(q_ref, s_ref, k, n)
    d_y2 = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    run(ex, ex.f8row_gemm, plane2, d_xq, d_xs, d_y2, m)
    assert torch.equal(d_y, d_y2)


def test_fused_e4m3_producers_feed_the_gemm(ex):
    """rmsnorm + quantize in one launch, then the FP8 GEMM on what it wrote: the chain the engine
    runs in front of every FP8 linear layer (gpu/fp8.rs:504-659)."""
    m, n, k, eps = 12, 128, 512, 1e-6
    x = oracle.fill_normal(m * k, 9600, 1.5).reshape(m, k)
    g = (1.0 + 0.1 * oracle.fill_normal(k, 9601, 1.0)).astype(np.float32)
    w = oracle.bf16_round(oracle.fill_normal(n * k, 9602, 0.02))
    plane = ex.bf16_to_f8row((w.view(np.uint32) >> 16).astype(np.uint16), k, n)
    d_x, d_xn = dev_f32(x.reshape(-1)), torch.zeros(m * k, dtype=torch.float32, device="cuda")
    d_q, d_s = torch.zeros(m * k, dtype=torch.uint8, device="cuda"), torch.zeros(m, dtype=torch.float32, device="cuda")
    d_y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert ex.rmsnorm_quant_e4m3_row(d_x, dev_f32(g), d_xn, d_q, d_s, k, eps, m) is True
    ex.f8row_gemm(plane, d_q, d_s, d_y, m)
    ex.synchronize()
    _, xn = oracle.rmsnorm_scaled_add(x, None, g, eps)
    assert np.allclose(d_xn.cpu().numpy().reshape(m, k), xn, rtol=4e-7, atol=0)
    wq, wsc = oracle.quantize_e4m3_row_pow2(w, n, k)
    xq, xsc = oracle.quantize_e4m3_row_pow2(d_xn.cpu().numpy(), m, k)
    ref, ab = oracle.matmul_f64(oracle.dequant_fp8_channel(wq, wsc, k, n), oracle.dequant_fp8_channel(xq, xsc, k, m), k, n, m,
                                with_abs=True)
    assert cond_err(d_y.cpu().numpy().reshape(m, n), ref, ab) < 1e-5 < TOL


def test_nvf4_upload_checks_geometry_tiles_scales_and_runs_both_lanes(ex):
    m, n, k = 24, 200, 768
    w = oracle.fill_normal(n * k, 9500, 0.02)
    scale2 = float(np.abs(w).max() / (6.0 * 448.0))
    q, s = oracle.quantize_nvf4(w, scale2)
    with pytest.raises(X.GpuError) as e:
        ex.nvf4_upload(q[:-1], s, scale2, n, k)
    assert e.value.kind == "Unsupported"
    plane = ex.nvf4_upload(q, s, scale2, n, k)
    i = plane.info()
    assert plane.kind == "Nvf4" and X.NVF4_LAYOUTS[i.layout] == "Row" and i.scale_tc5
    assert plane.bytes() == n * k // 2 + n * k // 16 + ((n + 127) // 128) * (k // 256) * 2048
    wd = oracle.dequant_nvfp4(q.reshape(n, k // 2), s.reshape(n, k // 16), scale2, k, n)
    x = oracle.bf16_round(oracle.fill_normal(m * k, 9501, 1.0))
    d_x = dev_f32(x)
    d_xq = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
    d_xs = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    d_y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    run(ex, ex.quantize_nvf4, d_x, d_xq, d_xs, m * k)
    run(ex, ex.nvf4_gemm_f4, plane, d_xq, d_xs, d_y, None, m)
    xq, xs = oracle.quantize_nvf4(x)
    xd = oracle.dequant_nvfp4(xq.reshape(m, k // 2), xs.reshape(m, k // 16), 1.0, k, m)
    ref, ab = oracle.matmul_f64(wd, xd, k, n, m, with_abs=True)
    assert cond_err(d_y.cpu().numpy().reshape(m, n), ref, ab) < 1e-5 < TOL
    # W4A16 decode lane on the same plane
    d_y1 = torch.zeros(n, dtype=torch.float32, device="cuda")
    run(ex, ex.nvf4_gemv, plane, None, dev_f32(x[:k]), d_y1)
    ref, ab = oracle.matmul_f64(wd, x[:k], k, n, 1, with_abs=True)
    assert cond_err(d_y1.cpu().numpy().reshape(1, n), ref, ab) < 1e-5
    # a row length that is not whole 256-element slabs: the plane loads, the tensor-core lane is refused
    q2, s2 = oracle.quantize_nvf4(w[: n * 96], scale2)
    odd = ex.nvf4_upload(q2, s2, scale2, n, 96)
    assert not odd.info().scale_tc5
    with pytest.raises(X.GpuError) as e:
        ex.nvf4_gemm_f4(odd, d_xq, d_xs, d_y, None, 1)
    assert e.value.kind == "MissingOp"


def test_has_probes_follow_the_table(ex):
    assert ex.has("kquant_gemv") and ex.has("nvf4_gemm_tc5w") and ex.has("pdk_kquant_gemm_f32")
    assert not ex.has("no_such_member")
