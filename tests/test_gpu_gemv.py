"""Decode GEMV / small-batch GEMM parity against the CPU oracle: outputs within
1e-2 (the stated tolerance) of an f64 matmul of the dequantized weights, both
as max |err| / sum|w x| and as rel-L2.  The kernels are held much tighter than
that: the weights' integer dot products are exact and the activations are
carried as 15-bit block floating point (error below 2^-15 of each 32-element
block's largest value), so rel-L2 stays under 1e-4 and the condition-aware
error under 1e-5."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import TOL, bf16_activations, cond_err, dev, dev_f32, rel_l2, seed_for

pytestmark = pytest.mark.gpu


def q8_planes(pack, w, n, k):
    raw = oracle.quantize_q8_0(w)
    nb = n * k // 32
    d_data = torch.zeros(nb * 32, dtype=torch.int8, device="cuda")
    d_scale = torch.zeros(nb, dtype=torch.float16, device="cuda")
    pack.call("q8_0_repack", dev(raw), d_data, d_scale, nb)
    return raw, d_data, d_scale


@pytest.mark.parametrize("k,n", [(32, 1), (512, 37), (2880, 100), (5120, 1024), (8192, 64)])
def test_q8_0_gemv_shapes(pack, k, n):
    w = oracle.fill_normal(n * k, seed_for(0, k + n), 0.02)
    x = bf16_activations(k, seed_for(0, 1))
    raw, d_data, d_scale = q8_planes(pack, w, n, k)
    bias = oracle.fill_normal(n, 9, 0.1)
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("q8_0_gemv_repacked", d_data, d_scale, dev_f32(bias), dev_f32(x), d_y, k, n)
    torch.cuda.synchronize()
    wd = oracle.dequant_q8_0(raw)
    ref, ab = oracle.matmul_f64(wd, x, k, n, 1, with_abs=True)
    y = d_y.cpu().numpy() - bias
    assert cond_err(y, ref[0], ab[0]) < 1e-5
    assert rel_l2(y, ref[0]) < 1e-4 < TOL
    # the reference CPU path (scalar f32, ascending k) agrees to the same bound
    y_cpu = oracle.matvec_f32(wd, x, k, n)
    assert rel_l2(y, y_cpu.astype(np.float64)) < 1e-4


def test_q8_0_gemv_k5120_rows(pack):
    """Q8_0 at the benchmark K=5120 with a 2048-row band of the 17408 rows."""
    k, n = 5120, 2048
    w = oracle.fill_normal(n * k, seed_for(1, 0), 0.02)
    x = bf16_activations(k, seed_for(1, 1))
    raw, d_data, d_scale = q8_planes(pack, w, n, k)
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("q8_0_gemv_repacked", d_data, d_scale, None, dev_f32(x), d_y, k, n)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_q8_0(raw), x, k, n, 1, with_abs=True)
    assert cond_err(d_y.cpu().numpy(), ref[0], ab[0]) < 1e-5


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7, 16])
def test_q8_0_gemm_small_batch(pack, batch):
    k, n = 1024, 96
    w = oracle.fill_normal(n * k, 31, 0.02)
    x = bf16_activations(batch * k, 32)
    raw, d_data, d_scale = q8_planes(pack, w, n, k)
    d_y = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    pack.call("q8_0_gemm_repacked", d_data, d_scale, None, dev_f32(x), d_y, k, n, batch)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_q8_0(raw), x, k, n, batch, with_abs=True)
    assert cond_err(d_y.cpu().numpy().reshape(batch, n), ref, ab) < 1e-5


@pytest.mark.parametrize("k,n", [(5120, 1000), (2048, 33), (6144, 160)])
@pytest.mark.parametrize("batch", [2, 4, 8, 9, 16])
def test_q8_0_gemm_tokens_as_columns(pack, k, n, batch):
    """K / 512 between 4 and 12: the ring kernel with the tokens as the mma's columns, one weight
    pass per eight tokens; rows that do not fill the last 16-row tile, a bias, tokens that do not
    fill the last group of eight."""
    w = oracle.fill_normal(n * k, 35 + k, 0.02)
    x = bf16_activations(batch * k, 36 + batch)
    x[:64] = 0.0                                   # all-zero activation blocks: step 1, limbs 0
    x[k + 32:k + 64] *= 1e-20
    bias = oracle.fill_normal(n, 37, 0.5)
    raw, d_data, d_scale = q8_planes(pack, w, n, k)
    d_y = torch.full((batch * n,), float("nan"), dtype=torch.float32, device="cuda")
    pack.call("q8_0_gemm_repacked", d_data, d_scale, dev_f32(bias), dev_f32(x), d_y, k, n, batch)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(oracle.dequant_q8_0(raw), x, k, n, batch, with_abs=True)
    y = d_y.cpu().numpy().reshape(batch, n) - bias[None, :]
    assert np.isfinite(y).all()
    assert cond_err(y, ref, ab) < 1e-5 < TOL
    # bit-identical from call to call (fixed fold order)
    d_y2 = torch.zeros_like(d_y)
    pack.call("q8_0_gemm_repacked", d_data, d_scale, dev_f32(bias), dev_f32(x), d_y2, k, n, batch)
    torch.cuda.synchronize()
    assert torch.equal(d_y, d_y2)


def test_q8_0_gemv_refuses_bad_shapes(pack):
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert pack.status("q8_0_gemv_repacked", buf, buf, None, buf, buf, 48, 4) == 1
    assert pack.status("q8_0_gemv_repacked", buf, buf, None, buf.data_ptr() + 4, buf, 64, 4) == 1
    assert pack.status("q8_0_gemv_repacked", buf, buf, None, buf, buf, 64, 0) == 0


def q4k_planes(pack, w, n, k):
    raw = oracle.quantize_q4_k(w)
    ns = n * k // 256
    d_data = torch.zeros(ns * 128, dtype=torch.uint8, device="cuda")
    d_sc = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
    pack.call("kquant_repack", dev(raw), d_data, d_sc, ns, 12)
    return raw, d_data, d_sc


@pytest.mark.parametrize("k,n", [(256, 1), (512, 33), (2560, 100), (5120, 1000), (14336, 16)])
def test_q4_k_gemv_shapes(pack, k, n):
    w = oracle.fill_normal(n * k, seed_for(2, k + n), 0.02)
    x = bf16_activations(k, seed_for(2, 1))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("kquant_gemv", d_data, d_sc, dev_f32(x), d_y, k, n, 12)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, 1, with_abs=True)
    y = d_y.cpu().numpy()
    assert cond_err(y, ref[0], ab[0]) < 1e-5
    assert rel_l2(y, ref[0]) < 1e-4 < TOL


# Shapes chosen for the ring-staged decode GEMV's plans: 8 units per row (the smallest it takes),
# stages that do not divide the row (18, 22, 68, 108 units), an odd unit count (43: the ring
# kernel declines Q4_K's 24-byte records there and the register-staged kernel runs), fewer than 16
# rows, a last tile of one row, and more tiles than SMs so that the ring wraps many times.
RING_SHAPES = [(2048, 7), (2048, 4099), (4608, 33), (5632, 100), (11008, 49), (17408, 161), (27648, 40), (4096, 16 * 148 * 3 + 1)]


@pytest.mark.parametrize("k,n", RING_SHAPES)
def test_q4_k_gemv_ring_plans(pack, k, n):
    w = oracle.fill_normal(n * k, seed_for(2, 7 * k + n), 0.02)
    x = bf16_activations(k, seed_for(2, 3))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_y = torch.full((n + 8,), 7.0, dtype=torch.float32, device="cuda")
    pack.call("kquant_gemv", d_data, d_sc, dev_f32(x), d_y, k, n, 12)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, 1, with_abs=True)
    y = d_y.cpu().numpy()
    assert (y[n:] == 7.0).all()          # nothing written past the last row
    assert cond_err(y[:n], ref[0], ab[0]) < 1e-5
    assert rel_l2(y[:n], ref[0]) < 1e-4 < TOL


@pytest.mark.parametrize("k,n", RING_SHAPES)
def test_q8_0_gemv_ring_plans(pack, k, n):
    w = oracle.fill_normal(n * k, seed_for(0, 7 * k + n), 0.02)
    x = bf16_activations(k, seed_for(0, 3))
    raw, d_data, d_scale = q8_planes(pack, w, n, k)
    bias = oracle.fill_normal(n, 9, 0.1)
    d_y = torch.full((n + 8,), 7.0, dtype=torch.float32, device="cuda")
    pack.call("q8_0_gemv_repacked", d_data, d_scale, dev_f32(bias), dev_f32(x), d_y, k, n)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(oracle.dequant_q8_0(raw), x, k, n, 1, with_abs=True)
    y = d_y.cpu().numpy()
    assert (y[n:] == 7.0).all()
    assert cond_err(y[:n] - bias, ref[0], ab[0]) < 1e-5
    assert rel_l2(y[:n] - bias, ref[0]) < 1e-4 < TOL


def test_gemv_ring_back_to_back_is_deterministic(pack):
    """Twenty dependent launches in a row (each starts its ring fill while its predecessor drains)
    leave bit-identical results."""
    k, n = 5120, 4000
    w = oracle.fill_normal(n * k, seed_for(2, 77), 0.02)
    x = dev_f32(bf16_activations(k, seed_for(2, 78)))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    ys = [torch.zeros(n, dtype=torch.float32, device="cuda") for _ in range(20)]
    for y in ys:
        pack.call("kquant_gemv", d_data, d_sc, x, y, k, n, 12)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    for y in ys[1:]:
        assert torch.equal(y, ys[0])


@pytest.mark.parametrize("batch", [1, 4, 16])
def test_q4_k_small_batch_k5120_band(pack, batch):
    """Q4_K K=5120 at 1 / 4 / 16 tokens on a 1536-row band of N=25600."""
    k, n = 5120, 1536
    w = oracle.fill_normal(n * k, seed_for(2, 0), 0.02)
    x = bf16_activations(batch * k, seed_for(2, 100 + batch))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_y = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    pack.call("pdk_kquant_gemm_f32", d_data, d_sc, dev_f32(x), d_y, k, n, batch, 12)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, batch, with_abs=True)
    y = d_y.cpu().numpy().reshape(batch, n)
    # up to 8 tokens: integer tensor path (15-bit activations); from 9 on the f16-weight tcgen05 path
    assert cond_err(y, ref, ab) < (1e-5 if batch <= 8 else 1e-4)
    assert rel_l2(y, ref) < (1e-4 if batch <= 8 else 1e-3) < TOL


@pytest.mark.parametrize("k,n,batch", [(5120, 1000, 2), (2048, 130, 8), (1024, 48, 5),      # int8 path, ragged rows
                                       (5120, 1000, 9), (2048, 300, 17), (4096, 257, 32),   # tcgen05, K halves
                                       (1536, 200, 16), (5120, 640, 40),                    # one K part; two launches
                                       (1280, 64, 16)])                                     # odd super-block count: int8 path
def test_q4_k_batch_shapes(pack, k, n, batch):
    """Every small-batch route of pdk_kquant_gemm_f32 on f32 activations that are not bf16 values."""
    w = oracle.fill_normal(n * k, seed_for(2, 900 + k + n), 0.02)
    x = oracle.fill_normal(batch * k, seed_for(2, 901 + batch), 1.0)
    x[:k] *= 1.0e4                       # one token far outside the f16 range, one tiny, one zero
    if batch > 2:
        x[k:2 * k] *= 1.0e-6
        x[2 * k:3 * k] = 0.0
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_y = torch.full((batch * n,), 3.0, dtype=torch.float32, device="cuda")
    pack.call("pdk_kquant_gemm_f32", d_data, d_sc, dev_f32(x), d_y, k, n, batch, 12)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, batch, with_abs=True)
    y = d_y.cpu().numpy().reshape(batch, n)
    for t in range(batch):               # per token: the tokens differ by ten orders of magnitude
        assert cond_err(y[t:t + 1], ref[t:t + 1], np.maximum(ab[t:t + 1], 1e-30)) < 1e-4, t
    if batch > 2:
        assert not y[2].any()


@pytest.mark.parametrize("k,n", [(5120, 1000), (6144, 72), (2048, 33)])
@pytest.mark.parametrize("batch", [2, 3, 8])
def test_q4_k_two_to_eight_tokens(pack, k, n, batch):
    """2 .. 8 tokens on the integer batch kernel: ragged rows, an all-zero token, a token of tiny
    values; bit-identical from call to call."""
    w = oracle.fill_normal(n * k, seed_for(2, 970 + k), 0.02)
    x = oracle.fill_normal(batch * k, seed_for(2, 971 + batch), 1.0)
    x[:k] = 0.0
    x[k:2 * k] *= 1.0e-12
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    outs = []
    for _ in range(2):
        d_y = torch.full((batch * n,), float("nan"), dtype=torch.float32, device="cuda")
        pack.call("pdk_kquant_gemm_f32", d_data, d_sc, dev_f32(x), d_y, k, n, batch, 12)
        torch.cuda.synchronize()
        outs.append(d_y.cpu().numpy())
    assert pack.device_error() == 0
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, batch, with_abs=True)
    y = outs[0].reshape(batch, n)
    assert np.isfinite(y).all() and not y[0].any()
    for t in range(1, batch):
        assert cond_err(y[t:t + 1], ref[t:t + 1], np.maximum(ab[t:t + 1], 1e-30)) < 2e-5 < TOL, t


def test_q4_k_batch_is_deterministic(pack):
    """The two K halves of a tile add into y in either order: the result must not depend on it."""
    k, n, batch = 5120, 2048, 16
    raw, d_data, d_sc = q4k_planes(pack, oracle.fill_normal(n * k, 77, 0.02), n, k)
    x = dev_f32(oracle.fill_normal(batch * k, 78, 1.0))
    outs = []
    for _ in range(3):
        d_y = torch.full((batch * n,), float(len(outs)), dtype=torch.float32, device="cuda")
        pack.call("pdk_kquant_gemm_f32", d_data, d_sc, x, d_y, k, n, batch, 12)
        torch.cuda.synchronize()
        outs.append(d_y.cpu().numpy().view(np.uint32).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_q4_k_gemv_general_f32_activations(pack):
    """Activations that are not bf16-representable keep f32 precision."""
    k, n = 2048, 64
    w = oracle.fill_normal(n * k, 55, 0.02)
    x = oracle.fill_normal(k, 56, 1.0)
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("kquant_gemv", d_data, d_sc, dev_f32(x), d_y, k, n, 12)
    torch.cuda.synchronize()
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, 1, with_abs=True)
    assert cond_err(d_y.cpu().numpy(), ref[0], ab[0]) < 1e-5


def test_q4_k_gemv_refuses_bad_shapes(pack):
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    assert pack.status("kquant_gemv", buf, buf, buf, buf, 128, 4, 12) == 1     # K not a multiple of 256
    assert pack.status("kquant_gemv", buf, buf, buf, buf, 256, 4, 99) == 1     # unknown dtype
    assert pack.status("kquant_gemv", buf, buf, buf, buf, 256, 4, 16) == 1     # IQ2_XXS: no kernel class in this pack
    assert pack.status("pdk_kquant_gemm_f32", buf, buf, buf, buf, 256, 4, 65, 12) == 1


# ---- int8 activation operands: slots 18 / 218 (quantizers) and 217 / 212 / 837 (W4A8 GEMV / GEMM)

@pytest.mark.parametrize("n", [32, 5120, 16 * 5120])
def test_quantize_q8_bit_exact(pack, n):
    x = oracle.fill_normal(n, 700 + n, 1.0)
    x[:32] = 0.0
    q_ref, s_ref, sums_ref = oracle.quantize_q8_act(x)
    d_q = torch.zeros(n, dtype=torch.int8, device="cuda")
    d_s = torch.zeros(n // 32, dtype=torch.float32, device="cuda")
    d_sum = torch.zeros(n // 16, dtype=torch.float32, device="cuda")
    pack.call("quantize_q8_sums", dev_f32(x), d_q, d_s, d_sum, n)
    torch.cuda.synchronize()
    assert np.array_equal(d_q.cpu().numpy(), q_ref)
    assert np.array_equal(d_s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(d_sum.cpu().numpy(), sums_ref)
    d_q2 = torch.zeros_like(d_q)
    d_s2 = torch.zeros_like(d_s)
    pack.call("quantize_q8", dev_f32(x), d_q2, d_s2, n)
    torch.cuda.synchronize()
    assert torch.equal(d_q, d_q2) and torch.equal(d_s, d_s2)


@pytest.mark.parametrize("k,n,batch", [(5120, 512, 1), (1024, 96, 1), (5120, 768, 4), (2048, 1000, 16)])
def test_q4k_w4a8_slots(pack, k, n, batch):
    """Slots 217 / 212 / 837 against an f64 matmul of the dequantized weights and q * scale."""
    raw, d_data, d_sc = q4k_planes(pack, oracle.fill_normal(n * k, 710 + n, 0.02), n, k)
    x = oracle.fill_normal(batch * k, 711, 1.0)
    q, s, sums = oracle.quantize_q8_act(x)
    xhat = (q.astype(np.float32).reshape(-1, 32) * s.reshape(-1, 1)).reshape(-1)
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), xhat, k, n, batch, with_abs=True)
    d_y = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    d_part = torch.zeros(8 * n * batch, dtype=torch.float32, device="cuda")
    names = ["kquant_gemm_mma_ks", "kquant_gemm_w4a8_sb"] + (["kquant_gemv_w4a8"] if batch == 1 else [])
    for name in names:
        d_y.zero_()
        if name == "kquant_gemv_w4a8":
            rc = pack.status(name, d_data, d_sc, dev(q), dev_f32(s), dev_f32(sums), d_y, k, n, 12)
            if rc == 801:
                continue                      # K outside the GEMV kernel's plan
            assert rc == 0
        else:
            pack.call(name, d_data, d_sc, dev(q), dev_f32(s), dev_f32(sums), d_part, d_y, k, n, batch, 12)
        torch.cuda.synchronize()
        y = d_y.cpu().numpy().reshape(batch, n)
        # up to 8 tokens run the integer path, more the f16-weight tcgen05 path
        assert cond_err(y, ref, ab) < 1e-4 < TOL, name


# ---- Q5_K, Q6_K, Q4_0 through the same slots

def raw_kquant(name, n_super, seed):
    """Random blocks of the raw ggml layout with finite f16 scales."""
    nbytes, elems = oracle.KQUANT_LAYOUT[name]
    n_blocks = n_super * 256 // elems
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, (n_blocks, nbytes), dtype=np.uint8)
    d = (rng.random(n_blocks) * 0.01 + 1e-4).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    if name == "iq4_xs":
        raw[:, 0:2] = (rng.random(n_blocks) * 0.001 + 1e-5).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    elif name == "q6_k":
        raw[:, 208:210] = d
    else:
        raw[:, 0:2] = d
        if name == "q5_k":
            raw[:, 2:4] = (rng.random(n_blocks) * 0.01).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    return raw.reshape(-1)


KQ = {"q5_k": (13, 160), "q6_k": (14, 192), "q4_0": (2, 128), "iq4_xs": (23, 128)}


@pytest.mark.parametrize("k,n", [(1024, 70), (5120, 333), (512, 40)])
@pytest.mark.parametrize("name", sorted(KQ))
def test_more_kquants_dequant_repack_gemv(pack, name, k, n):
    """(512, 40) is below the tensor-core GEMV's four super-blocks per row: the plain kernel's route."""
    dtype, datab = KQ[name]
    ns = n * k // 256
    raw = raw_kquant(name, ns, 720 + dtype)
    want = oracle.dequant_kquant(name, raw)
    d_y = torch.zeros(ns * 256, dtype=torch.float32, device="cuda")
    pack.call("kquant_dequant", dev(raw), d_y, ns, dtype)
    torch.cuda.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    d_data = torch.zeros(ns * datab, dtype=torch.uint8, device="cuda")
    d_sc = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
    pack.call("kquant_repack", dev(raw), d_data, d_sc, ns, dtype)
    for batch in (1, 5, 20):
        x = bf16_activations(batch * k, seed_for(2, 7 + batch))
        d_out = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
        if batch == 1:
            pack.call("kquant_gemv", d_data, d_sc, dev_f32(x), d_out, k, n, dtype)
        else:
            pack.call("pdk_kquant_gemm_f32", d_data, d_sc, dev_f32(x), d_out, k, n, batch, dtype)
        torch.cuda.synchronize()
        ref, ab = oracle.matmul_f64(want, x, k, n, batch, with_abs=True)
        # Q4_0 from four tokens on (and K a multiple of 512) runs the f16-weight tcgen05 kernel
        tol = 1e-4 if (name == "q4_0" and batch >= 4 and k % 512 == 0) else 1e-5
        assert cond_err(d_out.cpu().numpy().reshape(batch, n), ref, ab) < tol < TOL


@pytest.mark.parametrize("name", ["q5_k", "q6_k"])
@pytest.mark.parametrize("batch", [2, 8, 9, 16, 33])
def test_q5_k_q6_k_tokens_as_columns(pack, name, batch):
    """The integer batch kernels of Q5_K and Q6_K (eight or sixteen token columns per weight pass),
    whole and ragged passes, rows that are not a multiple of the 16-row tile."""
    dtype, datab = KQ[name]
    k, n = 2048, 203
    ns = n * k // 256
    raw = raw_kquant(name, ns, 760 + dtype + batch)
    want = oracle.dequant_kquant(name, raw)
    d_data = torch.zeros(ns * datab, dtype=torch.uint8, device="cuda")
    d_sc = torch.zeros(ns * 24, dtype=torch.uint8, device="cuda")
    pack.call("kquant_repack", dev(raw), d_data, d_sc, ns, dtype)
    x = oracle.fill_normal(batch * k, 761 + batch, 1.0)       # f32 activations that are not bf16 values
    d_out = torch.full((batch * n,), float("nan"), dtype=torch.float32, device="cuda")
    pack.call("pdk_kquant_gemm_f32", d_data, d_sc, dev_f32(x), d_out, k, n, batch, dtype)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(want, x, k, n, batch, with_abs=True)
    # f32 activations: the batch kernels' 15-bit block floating point per 256 elements (the Q4_K batch tests' bound)
    err = cond_err(d_out.cpu().numpy().reshape(batch, n), ref, ab)
    assert err < 1e-4 < TOL, ("batch kernel", err)
    # each token alone through the decode GEMV: the same value up to the activations' block-floating step
    d_one = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("kquant_gemv", d_data, d_sc, dev_f32(x[:k]), d_one, k, n, dtype)
    torch.cuda.synchronize()
    one = cond_err(d_one.cpu().numpy().reshape(1, n), ref[:1], ab[:1])
    assert one < 1e-4, ("decode GEMV", one)


def test_q4k_gemv_shard_stores_band_into_every_output(pack):
    """pdk_q4k_gemv_shard with two destination vectors on one GPU (the multi-GPU case points the
    second at a peer's buffer): both receive the band at row0, bit-identical to kquant_gemv."""
    import ctypes
    k, n, full, row0 = 5120, 512, 2048, 1024
    w = oracle.fill_normal(n * k, 730, 0.02)
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    x = dev_f32(bf16_activations(k, seed_for(2, 9)))
    d_ref = torch.zeros(n, dtype=torch.float32, device="cuda")
    pack.call("kquant_gemv", d_data, d_sc, x, d_ref, k, n, 12)
    outs = [torch.full((full,), -1.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(*[o.data_ptr() for o in outs])
    pack.call("pdk_q4k_gemv_shard", d_data, d_sc, x, ctypes.addressof(ptrs), 2, row0, k, n)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[row0:row0 + n], d_ref)
        assert bool((o[:row0] == -1.0).all()) and bool((o[row0 + n:] == -1.0).all())
    assert pack.status("pdk_q4k_gemv_shard", d_data, d_sc, x, ctypes.addressof(ptrs), 9, row0, k, n) == 1


def test_small_batch_scratch_is_per_stream(pack):
    """The small-batch Q4_K GEMM keeps its activation image in library scratch, one slice per
    (device, stream), two streams per device.  Three streams: the first two get slices, the third
    takes the scratch-free route (same results within its own precision class); releasing a
    stream hands its slice to the next newcomer."""
    k, n, batch = 2048, 300, 4
    w = oracle.fill_normal(n * k, seed_for(2, 900), 0.02)
    x = bf16_activations(batch * k, seed_for(2, 901))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, batch, with_abs=True)
    d_x = dev_f32(x)
    import ctypes
    rel = pack._lib.pdk_stream_release
    rel.argtypes, rel.restype = [ctypes.c_void_p], None
    streams = [torch.cuda.Stream() for _ in range(3)]
    outs = []
    torch.cuda.synchronize()
    rel(torch.cuda.current_stream().cuda_stream)    # earlier tests ran this route on the default stream
    for st in streams:
        y = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
        pack.call("pdk_kquant_gemm_f32", d_data, d_sc, d_x, y, k, n, batch, 12, stream=st.cuda_stream)
        outs.append(y)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    for y in outs:
        got = y.cpu().numpy().reshape(batch, n)
        assert cond_err(got, ref, ab) < 1e-4 and rel_l2(got, ref) < 1e-3 < TOL
    assert torch.equal(outs[0], outs[1])            # both on the integer tensor path
    rel(streams[0].cuda_stream)
    y3 = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    pack.call("pdk_kquant_gemm_f32", d_data, d_sc, d_x, y3, k, n, batch, 12, stream=streams[2].cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(y3, outs[0])                 # the third stream now runs the scratch route too
    for st in streams[1:]:
        rel(st.cuda_stream)


def test_q4k_gemv_shard_sync_raises_flags_and_wait_is_bounded(pack):
    """The sharded GEMV with its completion signal, two "ranks" played on one GPU (both y vectors and
    both flag arrays are local): the band lands in both outputs, word `rank` of both flag arrays
    reads the step, the CTA counter is back at zero, a wait for that step returns at once, and a
    wait for a step nobody signals gives up after its budget with its code in the error word.
    Explicit step numbers first, then the self-counting form a captured launch replays."""
    import ctypes
    k, n, row0 = 5120, 1030, 64
    w = oracle.fill_normal(n * k, seed_for(2, 950), 0.02)
    x = bf16_activations(k, seed_for(2, 951))
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    ys = [torch.full((row0 + n + 8,), 3.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    ctr = torch.zeros(2, dtype=torch.int32, device="cuda")
    yp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in ys])
    fp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
    d_x = dev_f32(x)
    for step in (1, 2, 7):
        pack.call("pdk_q4k_gemv_shard_sync", d_data, d_sc, d_x, ctypes.addressof(yp), ctypes.addressof(fp), ctr, 2, 1,
                  row0, step, k, n)
        torch.cuda.synchronize()
        assert [int(f[1]) for f in flags] == [step, step] and [int(f[0]) for f in flags] == [0, 0]
        assert ctr.tolist() == [0, 0]
    assert pack.device_error() == 0
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, 1, with_abs=True)
    for y in ys:
        got = y.cpu().numpy()
        assert (got[:row0] == 3.0).all() and (got[row0 + n:] == 3.0).all()
        assert cond_err(got[row0:row0 + n], ref[0], ab[0]) < 1e-5
    # a wait on word 1 for the step that was signalled passes; for the next step it runs out of budget
    only1 = flags[0][1:]
    pack.call("pdk_peer_flags_wait", only1, 1, 7, 1000)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    pack.call("pdk_peer_flags_wait", only1, 1, 8, 2000)                    # 2 ms budget, nobody signals step 8
    torch.cuda.synchronize()
    assert pack.device_error() == (0x16 << 8 | 0)
    assert pack.status("pdk_peer_flags_wait", only1, 9, 1, 1000) == 1       # more than 8 ranks
    # self-counting steps: rank 0 of one, three launches and three waits, arguments unchanged
    flags1 = torch.zeros(16, dtype=torch.int32, device="cuda")
    ctr1 = torch.zeros(2, dtype=torch.int32, device="cuda")
    fp1 = (ctypes.c_void_p * 1)(flags1.data_ptr())
    for i in range(3):
        pack.call("pdk_q4k_gemv_shard_sync", d_data, d_sc, d_x, ctypes.addressof(yp), ctypes.addressof(fp1), ctr1, 1, 0,
                  row0, 0, k, n)
        pack.call("pdk_peer_flags_wait", flags1, 1, 0, 100000)
    torch.cuda.synchronize()
    assert pack.device_error() == 0
    assert int(flags1[0]) == 3 and int(flags1[8]) == 3 and ctr1.tolist() == [0, 3]


def test_q4k_gemv_shard_lagged_checks_the_previous_step_on_the_device(pack):
    """The form for loops that rotate y buffers: a launch signals the PREVIOUS launch of its stream (when
    it starts) and checks that every rank's previous step has arrived (before it ends); the last launch
    is signalled by pdk_peer_flags_post.  One rank alone: every check passes, and a closing wait on "my
    own latest step" returns at once.  Two ranks of which the second never runs: the second launch gives
    up on rank 1 after its bounded wait and says so."""
    import ctypes
    import time
    k, n = 5120, 160
    w = oracle.fill_normal(n * k, seed_for(2, 960), 0.02)
    raw, d_data, d_sc = q4k_planes(pack, w, n, k)
    d_x = dev_f32(bf16_activations(k, seed_for(2, 961)))
    ys = [torch.zeros(n, dtype=torch.float32, device="cuda") for _ in range(2)]
    yp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in ys])
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    ctr = torch.zeros(2, dtype=torch.int32, device="cuda")
    fp = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    assert pack.device_error() == 0
    for i in range(4):
        pack.call("pdk_q4k_gemv_shard_lagged", d_data, d_sc, d_x, ctypes.addressof(yp), ctypes.addressof(fp), ctr, 1, 0,
                  0, 0, k, n)
    torch.cuda.synchronize()
    assert pack.device_error() == 0 and int(flags[0]) == 3 and ctr.tolist() == [0, 4]   # launch 4 signalled step 3
    pack.call("pdk_peer_flags_post", ctypes.addressof(fp), ctr, 1, 0)
    pack.call("pdk_peer_flags_wait", flags, 1, 0x80000000 | 0, 100000)
    torch.cuda.synchronize()
    assert pack.device_error() == 0 and int(flags[0]) == 4 and ctr.tolist() == [0, 4]
    ref, ab = oracle.matmul_f64(oracle.dequant_q4_k(raw), bf16_activations(k, seed_for(2, 961)), k, n, 1, with_abs=True)
    assert cond_err(ys[0].cpu().numpy(), ref[0], ab[0]) < 1e-5
    assert pack.status("pdk_peer_flags_post", ctypes.addressof(fp), ctr, 9, 0) == 1      # more than 8 ranks
    assert pack.status("pdk_peer_flags_post", ctypes.addressof(fp), ctr, 2, 2) == 1      # rank outside the group
    # rank 0 of two; nobody plays rank 1, so word 1 stays 0
    flags.zero_()
    ctr.zero_()
    pack.call("pdk_q4k_gemv_shard_lagged", d_data, d_sc, d_x, ctypes.addressof(yp), ctypes.addressof(fp), ctr, 2, 0, 0, 0, k, n)
    torch.cuda.synchronize()
    assert pack.device_error() == 0 and int(flags[0]) == 0                  # step 1 has no previous step
    t0 = time.perf_counter()
    pack.call("pdk_q4k_gemv_shard_lagged", d_data, d_sc, d_x, ctypes.addressof(yp), ctypes.addressof(fp), ctr, 2, 0, 0, 0, k, n)
    torch.cuda.synchronize()
    assert 0.5 < time.perf_counter() - t0 < 5.0                             # the one-second budget ran out
    assert pack.device_error() == (0x1c << 8 | 1)
    assert int(flags[0]) == 1                                               # step 1 was still signalled
    y = torch.ones(8, device="cuda") * 2                                    # the context still works
    assert float(y.sum()) == 16.0
