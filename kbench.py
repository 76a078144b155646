"""Per-kernel micro-benchmarks for the pack's launchers (the counterpart of the
reference's examples/*_kbench.rs): CUDA-event timing after warm-up, cold L2 for
the memory-bound operators (operand clones rotated so consecutive launches
never touch the same bytes), one JSON line per case.

    python kbench.py --op f8row_gemm --m 4096 --n 17408 --k 5120
    python kbench.py --op q4k_gemv --m 1
    python kbench.py --op q8_gemv
    python kbench.py --op f8row_gemm --out f32 --pack /path/to/another-pack.so

--pack times any library that exports the kernel-pack ABI (table slots only, so
--out f32 for the GEMMs); the default is this package's own library.
"""
import argparse
import json
import os

import torch

from paddock_b200 import synth
from paddock_b200.planes import GpuExecutor

L2_BYTES = 126 << 20


def peaks():
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


GRAPH_REPLAY = False  # --graph: the timed launches are captured once into a CUDA graph and replayed


def time_launches(fn, iters, warmup=5):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if GRAPH_REPLAY:
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn(0)                       # one launch on the capturing stream before capture (per-stream scratch)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for i in range(iters):
                    fn(i)
            g.replay()
            side.synchronize()
            e0.record()
            g.replay()
            e1.record()
            side.synchronize()
        return e0.elapsed_time(e1) / iters * 1e-3
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def rel_err(got, ref):
    """rel-L2 of a device result against a device reference (one host read)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = ref.float()
    return float((got.float() - ref).norm() / ref.norm().clamp_min(1e-30))


def clones_for(nbytes):
    return max(2, -(-2 * L2_BYTES // max(nbytes, 1)) + 1)


KQ_MORE = {"q5_k": (13, 176, 256), "q6_k": (14, 210, 256), "q4_0": (2, 18, 32), "iq4_xs": (23, 136, 256)}  # ggml id, block bytes, elements


def raw_kquant_blocks(name, n_elems):
    """Random raw ggml blocks with small finite f16 scales (there is no quantizer for these formats)."""
    _, nbytes, elems = KQ_MORE[name]
    n_blocks = n_elems // elems
    g = torch.Generator(device="cuda").manual_seed(7)
    raw = torch.randint(0, 256, (n_blocks, nbytes), dtype=torch.uint8, device="cuda", generator=g)
    d = (torch.rand(n_blocks, device="cuda", generator=g) * 0.01 + 1e-4).to(torch.float16).view(torch.uint8).view(n_blocks, 2)
    if name == "q6_k":
        raw[:, 208:210] = d
    else:
        raw[:, 0:2] = d
        if name == "q5_k":
            raw[:, 2:4] = d.flip(0)
    return raw.reshape(-1)


def bench_q4k(ex, a):
    k, n, m = a.k, a.n, a.m
    if a.dtype != "q4_k":
        ty, nbytes, elems = KQ_MORE[a.dtype]
        raw = raw_kquant_blocks(a.dtype, n * k)
        data_b = {"q5_k": 160, "q6_k": 192, "q4_0": 128, "iq4_xs": 128}[a.dtype]
        from paddock_b200.planes import RepackedKQ
        planes = []
        for _ in range(clones_for(n * k // 256 * (data_b + 24))):
            data = torch.empty(n * k // 256 * data_b, dtype=torch.uint8, device="cuda")
            scales = torch.empty(n * k // 256 * 24, dtype=torch.uint8, device="cuda")
            ex.pack.call("kquant_repack", raw, data, scales, n * k // 256, ty, stream=torch.cuda.current_stream().cuda_stream)
            planes.append(RepackedKQ(data, scales, (k, n), ty))
        x = synth.bf16_round(synth.normal(m * k, 2, 1.0, "cuda"))
        y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
        if m == 1:
            sec = time_launches(lambda i: ex.kquant_gemv(planes[i % len(planes)], x, y), a.iters)
        else:
            sec = time_launches(lambda i: ex.kquant_gemm_f32(planes[i % len(planes)], x, y, m), a.iters)
        return sec, {"bound": "hbm", "bytes": n * k // elems * nbytes + m * k * 2 + m * n * 4, "dtype": a.dtype}
    raw = synth.quantize_q4_k(synth.normal(n * k, 1, 0.02, "cuda"))
    planes = [ex.repack_kquant_raw(raw, k, n) for _ in range(clones_for(n * k // 256 * 152))]
    x = synth.bf16_round(synth.normal(m * k, 2, 1.0, "cuda"))
    y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    if m == 1:
        sec = time_launches(lambda i: ex.kquant_gemv(planes[i % len(planes)], x, y), a.iters)
    else:
        sec = time_launches(lambda i: ex.kquant_gemm_f32(planes[i % len(planes)], x, y, m), a.iters)
    nbytes = n * k // 256 * 144 + m * k * 2 + m * n * 4
    # spot check: the last call's first rows against an f32 product of the dequantized plane
    rows = min(n, 512)
    wd = torch.empty(rows * k, dtype=torch.float32, device="cuda")
    ex.pack.call("kquant_dequant", raw, wd, rows * k // 256, 12, stream=torch.cuda.current_stream().cuda_stream)
    err = rel_err(y.view(m, n)[:, :rows], x.view(m, k) @ wd.view(rows, k).t())
    return sec, {"bound": "hbm", "bytes": nbytes, "parity_rel_l2": err, "parity_ok": err < 1e-3}


def bench_q4k_w4a8(ex, a):
    """The reference's small-batch chain for a Q4_K plane (crates/paddock-engine/src/gpu/kquant.rs:1020-1038):
    quantize_q8_sums per token, then kquant_gemm_w4a8_sb (kquant_gemv_w4a8 at one token).  Table slots
    only, so --pack times another library on the same operands.  `us` is the GEMM alone; `us_chain`
    includes the per-token activation quantizers."""
    k, n, m = a.k, a.n, a.m
    st = torch.cuda.current_stream().cuda_stream
    raw = synth.quantize_q4_k(synth.normal(n * k, 1, 0.02, "cuda"))
    ours = GpuExecutor()
    planes = [ours.repack_kquant_raw(raw, k, n) for _ in range(clones_for(n * k // 256 * 152))]
    x = synth.bf16_round(synth.normal(m * k, 2, 1.0, "cuda"))
    xq = torch.zeros(m * k, dtype=torch.int8, device="cuda")
    xs = torch.zeros(m * k // 32, dtype=torch.float32, device="cuda")
    xsum = torch.zeros(m * k // 16, dtype=torch.float32, device="cuda")
    part = torch.zeros(8 * n * m, dtype=torch.float32, device="cuda")
    y = torch.zeros(m * n, dtype=torch.float32, device="cuda")

    def quant():
        for t in range(m):
            ex.pack.call("quantize_q8_sums", x[t * k:], xq[t * k:], xs[t * k // 32:], xsum[t * k // 16:], k, stream=st)

    def gemm(i):
        w = planes[i % len(planes)]
        if m == 1:
            ex.pack.call("kquant_gemv_w4a8", w.data, w.scales, xq, xs, xsum, y, k, n, 12, stream=st)
        else:
            ex.pack.call("kquant_gemm_w4a8_sb", w.data, w.scales, xq, xs, xsum, part, y, k, n, m, 12, stream=st)

    quant()
    sec = time_launches(gemm, a.iters)

    def chain(i):
        quant()
        gemm(i)
    sec_chain = time_launches(chain, a.iters)
    nbytes = n * k // 256 * 144 + m * k * 2 + m * n * 4
    return sec, {"bound": "hbm", "bytes": nbytes, "us_chain": sec_chain * 1e6}


def bench_tc5_probe(ex, a):
    """Issue rate of tcgen05.mma per operand kind with operands resident in shared memory
    (pdk_tc5_issue_probe): the measured tensor-core ceiling the FP8 / NVFP4 GEMM fractions
    can be read against.  --iters = MMAs per SM per launch."""
    n_mma = max(8, min(a.iters * 256, 1 << 20))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cyc = torch.zeros(sms, dtype=torch.int64, device="cuda")
    kinds = [("bf16_m128n256k16", 256, 16), ("e4m3_m128n256k32", 256, 32), ("nvf4_m128n128k64", 128, 64),
             ("nvf4_m128n128k64_with_scale_copies", 128, 64), ("e4m3_pair_m256n256k32", 256, 32),
             ("nvf4_pair_m256n128k64_with_scale_copies", 128, 64)]
    out = {}
    st = torch.cuda.current_stream().cuda_stream
    for kind, (name, n, k) in enumerate(kinds):
        for _ in range(3):
            ex.pack.call("pdk_tc5_issue_probe", kind, n_mma, cyc, stream=st)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ex.pack.call("pdk_tc5_issue_probe", kind, n_mma, cyc, stream=st)
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) * 1e-3
        flops = sms * n_mma * 2 * 128 * n * k          # a pair's MMA is M256 on two SMs: the same flops per SM
        per = cyc.float().median().item() / n_mma
        out[name] = {"tflops": flops / sec / 1e12, "ms": sec * 1e3, "sm_cycles_per_mma": per,
                     "tflops_at_cycle_rate_1965mhz": sms * 2 * 128 * n * k / per * 1.965e9 / 1e12}
    return sec, {"bound": "none", "mma_per_sm": n_mma, **out}


def bench_norm_nvf4(ex, a):
    """Slot 436, the fused residual-add + RMSNorm + NVFP4 quantizer in front of an NVFP4 GEMM:
    --m rows of --k elements.  Table slot only, so --pack times another library."""
    n, batch = a.k, a.m
    x = synth.normal(batch * n, 11, 1.0, "cuda")
    proj = synth.normal(batch * n, 12, 0.01, "cuda")
    w = torch.ones(n, dtype=torch.float32, device="cuda")
    out = torch.zeros(batch * n, dtype=torch.float32, device="cuda")
    q = torch.zeros(batch * n // 2, dtype=torch.uint8, device="cuda")
    s = torch.zeros(batch * n // 16, dtype=torch.uint8, device="cuda")
    sec = time_launches(lambda i: ex.pack.call("add_rmsnorm_quant_nvf4_batch", x, proj, w, out, q, s, n, 1e-6, batch,
                                               stream=torch.cuda.current_stream().cuda_stream), a.iters)
    return sec, {"bound": "hbm", "bytes": batch * n * (4 + 4 + 4 + 4) + batch * n * 9 // 16 + n * 4}


def bench_q8(ex, a):
    k, n = a.k, a.n
    raw = synth.quantize_q8_0(synth.normal(n * k, 3, 0.02, "cuda"))
    planes = [ex.repack_q8_blocks(raw, k, n) for _ in range(clones_for(n * k // 32 * 34))]
    m = a.m
    x = synth.bf16_round(synth.normal(m * k, 4, 1.0, "cuda"))
    y = torch.zeros(m * n, dtype=torch.float32, device="cuda")
    if m == 1:
        sec = time_launches(lambda i: ex.q8_0_gemv_repacked(planes[i % len(planes)], None, x, y), a.iters)
    else:
        sec = time_launches(lambda i: ex.q8_0_gemm_repacked(planes[i % len(planes)], None, x, y, m), a.iters)
    rows = min(n, 512)
    p = planes[(a.iters - 1) % len(planes)] if not GRAPH_REPLAY else planes[(a.iters - 1) % len(planes)]
    wd = p.data.view(n, k // 32, 32)[:rows].float() * p.scale.view(n, k // 32, 1)[:rows].float()
    err = rel_err(y.view(m, n)[:, :rows], x.view(m, k) @ wd.reshape(rows, k).t())
    return sec, {"bound": "hbm", "bytes": n * k // 32 * 34 + m * k * 2 + m * n * 4, "parity_rel_l2": err,
                 "parity_ok": err < 1e-3}


def bench_f8(ex, a):
    m, n, k = a.m, a.n, a.k
    w = torch.randint(0, 0x7E, (n * k,), dtype=torch.uint8, device="cuda")
    xq = torch.randint(0, 0x7E, (m * k,), dtype=torch.uint8, device="cuda")
    ws = torch.rand(n, device="cuda") + 0.5
    xs = torch.rand(m, device="cuda") + 0.5
    y = torch.zeros(m * n, dtype=torch.bfloat16 if a.out == "bf16" else torch.float32, device="cuda")
    name = "pdk_f8row_gemm_bf16" if a.out == "bf16" else "f8row_gemm"
    st = torch.cuda.current_stream().cuda_stream
    sec = time_launches(lambda i: ex.pack.call(name, w, ws, xq, xs, y, k, n, m, stream=st), a.iters)
    # spot check: a corner of y against an f32 product of the decoded operands
    rows, toks = min(n, 384), min(m, 96)
    wd = w.view(n, k)[:rows].view(torch.float8_e4m3fn).float() * ws[:rows, None]
    xd = xq.view(m, k)[:toks].view(torch.float8_e4m3fn).float() * xs[:toks, None]
    err = rel_err(y.view(m, n)[:toks, :rows], xd @ wd.t())
    return sec, {"bound": "tensor", "flops": 2.0 * m * n * k, "parity_rel_l2": err,
                 "parity_ok": err < (5e-3 if a.out == "bf16" else 1e-4)}


def bench_nvf4(ex, a):
    m, n, k = a.m, a.n, a.k
    st = torch.cuda.current_stream().cuda_stream
    nbytes_w = n * k // 2 + n * k // 16
    nc = clones_for(nbytes_w) if m <= 512 else 1
    ws = [(torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device="cuda"),
           torch.randint(0x20, 0x48, (((n + 127) // 128) * (k // 256) * 2048,), dtype=torch.uint8, device="cuda"))
          for _ in range(nc)]
    x = synth.bf16_round(synth.normal(m * k, 5, 1.0, "cuda"))
    xq = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    ex.pack.call("quantize_nvf4", x, xq, xs, m * k, stream=st)
    # the scale planes are tiled from a row-major plane, as the engine does at load time
    rowmajor = torch.randint(0x20, 0x48, (n * k // 16,), dtype=torch.uint8, device="cuda")
    for w in ws:
        ex.pack.call("nvf4_tc5_tile_scales", rowmajor, w[1], k, n, stream=st)
    if a.out == "bf16":
        y = torch.zeros(m * n, dtype=torch.bfloat16, device="cuda")
        call = lambda i: ex.pack.call("pdk_nvf4_gemm_bf16", ws[i % nc][0], ws[i % nc][1], None, xq, xs, y, 1.0, k, n, m,
                                      stream=torch.cuda.current_stream().cuda_stream)
    else:
        y = torch.zeros(m * n, dtype=torch.float32, device="cuda")   # the table slot writes f32
        call = lambda i: ex.pack.call("nvf4_gemm_tc5w", ws[i % nc][0], ws[i % nc][1], None, xq, xs, y, 1.0, k, n, m, None,
                                      0, stream=torch.cuda.current_stream().cuda_stream)
    sec = time_launches(call, a.iters)
    # spot check: clone 0's first rows against an f32 product of the dequantized operands
    call(0)
    rows, toks = min(n, 256), min(m, 64)
    wd = torch.empty(rows * k, dtype=torch.float32, device="cuda")
    xd = torch.empty(toks * k, dtype=torch.float32, device="cuda")
    ex.pack.call("nvf4_dequant", ws[0][0], rowmajor, 1.0, wd, k, rows, stream=st)
    ex.pack.call("nvf4_dequant", xq, xs, 1.0, xd, k, toks, stream=st)
    err = rel_err(y.view(m, n)[:toks, :rows], xd.view(toks, k) @ wd.view(rows, k).t())
    return sec, {"bound": "both", "flops": 2.0 * m * n * k, "bytes": nbytes_w + 4 + m * (k // 2 + k // 16) + m * n * 2,
                 "parity_rel_l2": err, "parity_ok": err < (5e-3 if a.out == "bf16" else 1e-4)}


def bench_moe_other_pack(ex, a):
    """The MXFP4 MoE block (128 experts, top-4) through another pack's int8-activation chain, the way the reference engine drives it
    (crates/paddock-engine/src/gpu_model/gpt_oss.rs:715-735, 2393-2440): gate|up interleaved once
    (slot 155), then per call top-k, align (32-row blocks), quantize_q8 (18), gate_up_mmq (88),
    down_mmq (89), slot_combine."""
    import ctypes as C
    from paddock_b200 import planes as P
    pk = ex.pack
    n_expert, k, embd, ff, T = 128, 4, a.k, a.n, a.m
    st = torch.cuda.current_stream().cuda_stream
    interleave = pk.fn_at(155, "pppuU")
    gate_up = pk.fn_at(88, "pppppppppppp" + "uuu" + "fff")
    down = pk.fn_at(89, "pppppppppp" + "uuuu")
    nblk = embd // 32
    blocks = n_expert * ff * nblk

    def rnd(n, lo, hi, seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        return torch.randint(lo, hi, (n,), dtype=torch.uint8, device="cuda", generator=g)

    g_data, u_data, d_data = rnd(blocks * 16, 0, 256, 1), rnd(blocks * 16, 0, 256, 2), rnd(blocks * 16, 0, 256, 3)
    g_scale, u_scale, d_scale = rnd(blocks, 118, 124, 4), rnd(blocks, 118, 124, 5), rnd(blocks, 118, 124, 6)
    gu = torch.zeros(n_expert * ff * ((nblk + 3) // 4) * 128, dtype=torch.uint8, device="cuda")
    rc = interleave(g_data.data_ptr(), u_data.data_ptr(), gu.data_ptr(), nblk, n_expert * ff, st)
    assert rc == 0, rc
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    zb_ff = torch.zeros(n_expert * ff, device="cuda")
    zb_embd = torch.zeros(n_expert * embd, device="cuda")
    pairs, bm = T * k, 32
    max_blocks = min(pairs, pairs // bm + n_expert)
    nb = max_blocks * bm
    idx = torch.zeros(pairs, dtype=torch.int32, device="cuda")
    w = torch.zeros(pairs, device="cuda")
    s_row = torch.zeros(nb, dtype=torch.int32, device="cuda")
    s_slot = torch.zeros(nb, dtype=torch.int32, device="cuda")
    b_exp = torch.zeros(max_blocks, dtype=torch.int32, device="cuda")
    x = synth.bf16_round(synth.normal(T * embd, 7, 1.0, "cuda"))
    xq = torch.zeros(T * embd, dtype=torch.int8, device="cuda")
    xs = torch.zeros(T * embd // 32, device="cuda")
    fq = torch.zeros(nb * ff, dtype=torch.int8, device="cuda")
    fs = torch.zeros(nb * ff // 32, device="cuda")
    part = torch.zeros(pairs * max(ff, embd), device="cuda")
    out = torch.zeros(T * embd, device="cuda")
    n_sets = 6 if T <= 64 else 1
    logits = [synth.normal(T * n_expert, 100 + i, 1.0, "cuda") for i in range(n_sets)]

    def step(i):
        pk.call("moe_topk_batch", logits[i % n_sets], None, n_expert, k, idx, w, T, stream=st)
        pk.call("moe_align", idx, s_row, s_slot, b_exp, T, k, n_expert, max_blocks, stream=st)
        pk.call("quantize_q8", x, xq, xs, T * embd, stream=st)
        rc = gate_up(gu.data_ptr(), g_scale.data_ptr(), zb_ff.data_ptr(), dummy.data_ptr(), u_scale.data_ptr(),
                     zb_ff.data_ptr(), s_row.data_ptr(), b_exp.data_ptr(), xq.data_ptr(), xs.data_ptr(), fq.data_ptr(),
                     fs.data_ptr(), embd, ff, max_blocks, 1.702, 7.0, 1.0, st)
        assert rc == 0, rc
        rc = down(d_data.data_ptr(), d_scale.data_ptr(), zb_embd.data_ptr(), s_row.data_ptr(), s_slot.data_ptr(),
                  b_exp.data_ptr(), w.data_ptr(), fq.data_ptr(), fs.data_ptr(), part.data_ptr(), ff, embd, k, max_blocks,
                  st)
        assert rc == 0, rc
        pk.call("moe_slot_combine", part, out, embd, k, T, stream=st)

    sec = time_launches(step, a.iters)
    distinct = 0
    for lg in logits:
        distinct += torch.unique(torch.topk(lg.view(T, n_expert), k, dim=1).indices).numel()
    distinct /= n_sets
    per_expert = 3 * embd * ff // 32 * 17
    return sec, {"bound": "hbm", "bytes": int(distinct * per_expert + T * embd * 2 * 2), "distinct_experts": distinct}


def bench_moe(ex, a):
    """MXFP4 MoE block: 128 experts, top-4, hidden = ff = 2880 by default, T = --m tokens."""
    from paddock_b200 import planes as P
    if a.pack:
        return bench_moe_other_pack(ex, a)
    n_expert, k, embd, ff, T = 128, 4, a.k, a.n, a.m
    bm = 8 if T * k <= 1024 else 32
    blocks_per_plane = n_expert * embd * ff // 32

    def plane(seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        data = torch.randint(0, 256, (blocks_per_plane * 16,), dtype=torch.uint8, device="cuda", generator=g)
        scale = torch.randint(118, 124, (blocks_per_plane,), dtype=torch.uint8, device="cuda", generator=g)
        return P.RepackedMxfp4(data, scale)

    planes = P.MoeMxfp4Planes(plane(1), plane(2), plane(3), n_expert, embd, ff)
    if a.moe_path == "tc5":
        P.prepare_tc5(ex, planes)
    x = synth.bf16_round(synth.normal(T * embd, 7, 1.0, "cuda"))
    ws = P.MoeWorkspace(ex, planes, T, k, bm)
    out = torch.zeros(T * embd, dtype=torch.float32, device="cuda")
    n_sets = 6 if T <= 64 else 1          # different routings so consecutive steps touch different experts
    logits = [synth.normal(T * n_expert, 100 + i, 1.0, "cuda") for i in range(n_sets)]
    if a.graph:
        # the block's launches replayed from CUDA graphs, one per routing set (what a serving
        # loop that captures its decode step does)
        graphs = []
        for lg in logits:
            P.moe_mxfp4_forward(ex, planes, ws, x, lg, out)     # first call outside capture
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                P.moe_mxfp4_forward(ex, planes, ws, x, lg, out)
            graphs.append(g)
        sec = time_launches(lambda i: graphs[i % n_sets].replay(), a.iters)
    else:
        sec = time_launches(lambda i: P.moe_mxfp4_forward(ex, planes, ws, x, logits[i % n_sets], out), a.iters)
    distinct = 0
    for lg in logits:
        distinct += torch.unique(torch.topk(lg.view(T, n_expert), k, dim=1).indices).numel()
    distinct /= n_sets
    per_expert = 3 * embd * ff // 32 * 17
    info = {"bound": "hbm", "bytes": int(distinct * per_expert + T * embd * 2 * 2), "distinct_experts": distinct}
    if a.moe_path == "tc5":
        # spot check: the same call through the other expert path (independent kernels: mma.sync on
        # weights decoded in registers), both starting from a zeroed output
        out.zero_()
        P.moe_mxfp4_forward(ex, planes, ws, x, logits[0], out)
        got = out.clone()
        saved, planes.tc5 = planes.tc5, None
        out.zero_()
        P.moe_mxfp4_forward(ex, planes, ws, x, logits[0], out)
        planes.tc5 = saved
        err = rel_err(got, out)
        info.update(parity_rel_l2=err, parity_ok=err < 5e-3)
    return sec, info


def bench_moe_ep(ex, a):
    """The MXFP4 MoE block, expert-parallel: run under torchrun, one rank per GPU; experts and tokens split over the ranks."""
    import torch.distributed as dist
    from paddock_b200 import moe_ep, planes as P
    world, rank = dist.get_world_size(), dist.get_rank()
    n_expert, k, embd, ff, T = 128, 4, a.k, a.n, a.m
    epr = n_expert // world
    bm = 8 if T * k <= 1024 else 32
    blocks = epr * embd * ff // 32

    def plane(seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed * 64 + rank)
        return P.RepackedMxfp4(torch.randint(0, 256, (blocks * 16,), dtype=torch.uint8, device="cuda", generator=g),
                               torch.randint(118, 124, (blocks,), dtype=torch.uint8, device="cuda", generator=g))

    local = P.MoeMxfp4Planes(plane(1), plane(2), plane(3), epr, embd, ff)
    if a.moe_path == "tc5":
        P.prepare_tc5(ex, local)
    cap = -(-T // world) * k                     # slots every rank sends every peer
    shard = moe_ep.GpuExpertShard(ex, local, max(T * k, world * cap), bm)
    lo, hi = (T * rank) // world, (T * (rank + 1)) // world
    x = synth.bf16_round(synth.normal(T * embd, 7, 1.0, "cuda")).view(T, embd)[lo:hi].contiguous()
    n_sets = 6 if T <= 64 else 1
    logits = [synth.normal(T * n_expert, 100 + i, 1.0, "cuda").view(T, n_expert)[lo:hi].contiguous()
              for i in range(n_sets)]
    out = torch.zeros(hi - lo, embd, device="cuda")

    def step(i):
        moe_ep.gpu_ep_forward(ex, shard, x, logits[i % n_sets], out, n_expert, k, capacity=cap)

    for i in range(5):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    if a.graph:
        # the fixed-capacity exchange never synchronizes the host, so a whole block call - routing,
        # both all-to-alls, the expert kernels - replays from one CUDA graph per routing set
        side = torch.cuda.Stream()
        graphs = []
        with torch.cuda.stream(side):
            for i in range(n_sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step(i)
                graphs.append(g)
        torch.cuda.synchronize()
        dist.barrier()
        run = lambda i: graphs[i % n_sets].replay()
    else:
        run = step
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.iters * 1e-3], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    per_expert = 3 * embd * ff // 32 * 17
    distinct = 0
    for i in range(n_sets):
        full = synth.normal(T * n_expert, 100 + i, 1.0, "cuda").view(T, n_expert)
        distinct += torch.unique(torch.topk(full, k, dim=1).indices).numel()
    distinct /= n_sets
    return float(t.item()), {"bound": "hbm", "bytes": int(distinct * per_expert + T * embd * 2 * 2),
                             "distinct_experts": distinct, "n_gpus": world}


def bench_f8_shard(ex, a):
    """FP8 row-scaled GEMM with the output channels sharded over the ranks (run under torchrun): each rank holds
    N / G weight rows and computes its band y[:, band] (bf16).  Three timings, max over ranks: the GEMM alone;
    GEMM + NCCL all-gather of the bands ([G][M][N/G], the baseline exchange); GEMM + peer stores, where the band
    is cut into M-chunks and every chunk is copied into its place in every rank's full [M][N] y (symmetric memory,
    plain stores over NVLink on side streams) while the next chunk's GEMM runs."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    world, rank = dist.get_world_size(), dist.get_rank()
    m, n, k = a.m, a.n, a.k
    nb = n // world
    g = torch.Generator(device="cuda")
    g.manual_seed(17 + rank)
    w = torch.randint(0, 0x7E, (nb * k,), dtype=torch.uint8, device="cuda", generator=g)
    g.manual_seed(5)
    xq = torch.randint(0, 0x7E, (m * k,), dtype=torch.uint8, device="cuda", generator=g)
    ws = torch.rand(nb, device="cuda") + 0.5
    xs = torch.rand(m, device="cuda") + 0.5
    y_band = torch.zeros(m, nb, dtype=torch.bfloat16, device="cuda")
    gathered = torch.zeros(world, m, nb, dtype=torch.bfloat16, device="cuda")
    y_full = symm_mem.empty(m * n, dtype=torch.bfloat16, device="cuda")
    hdl = symm_mem.rendezvous(y_full, dist.group.WORLD.group_name)
    peers = [hdl.get_buffer(p, (m, n), torch.bfloat16) for p in range(world)]
    st = torch.cuda.current_stream()
    chunks = 4 if m % 512 == 0 else 1
    mc = m // chunks
    evs = [torch.cuda.Event() for _ in range(chunks)]

    def gemm(rows0, rows):
        ex.pack.call("pdk_f8row_gemm_bf16", w, ws, xq[rows0 * k:], xs[rows0:], y_band[rows0:], k, nb, rows,
                     stream=st.cuda_stream)

    def step_gemm(i):
        gemm(0, m)

    def step_nccl(i):
        gemm(0, m)
        dist.all_gather_into_tensor(gathered.view(-1), y_band.view(-1))

    # 2-D copies through the CUDA runtime: the copy engines move the chunks over NVLink while the
    # SMs run the next chunk's GEMM (a strided torch copy kernel measured slower and takes SMs)
    import ctypes as C
    rt = None
    for nm in ("libcudart.so.12", "libcudart.so"):
        try:
            rt = C.CDLL(nm)
            break
        except OSError:
            continue
    rt.cudaMemcpy2DAsync.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]
    side = [torch.cuda.Stream() for _ in range(max(1, min(world, 4)))]
    dst_base = [peers[p].data_ptr() + rank * nb * 2 for p in range(world)]
    src_base = y_band.data_ptr()

    def step_peer(i):
        for c in range(chunks):
            gemm(c * mc, mc)
            evs[c].record(st)
            for d in range(world):
                p = (rank + d) % world            # start with the own copy, then walk the ring
                s2 = side[d % len(side)]
                s2.wait_event(evs[c])
                rc = rt.cudaMemcpy2DAsync(dst_base[p] + c * mc * n * 2, n * 2, src_base + c * mc * nb * 2, nb * 2, nb * 2, mc,
                                          4, s2.cuda_stream)       # 4 = cudaMemcpyDefault
                if rc != 0:
                    raise RuntimeError(f"cudaMemcpy2DAsync: {rc}")
        for s2 in side:
            st.wait_stream(s2)

    def timed(fn):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters * 1e-3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_gemm, t_nccl, t_peer = timed(step_gemm), timed(step_nccl), timed(step_peer)
    # the peer exchange must leave the same y everywhere as the all-gather does
    torch.cuda.synchronize()
    dist.barrier()
    want = gathered.permute(1, 0, 2).reshape(m, n)
    same = bool(torch.equal(want, y_full.view(m, n)))
    flag = torch.tensor([1 if same else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    # the record's time is the faster exchange's (the copy engines win at 2 ranks, NCCL from 4 on)
    return min(t_peer, t_nccl), {"bound": "tensor", "flops": 2.0 * m * n * k, "n_gpus": world, "us_gemm_only": t_gemm * 1e6,
                    "us_gemm_nccl_allgather": t_nccl * 1e6, "us_gemm_peer_stores": t_peer * 1e6, "m_chunks": chunks,
                    "exchange": "copy-engine peer stores" if t_peer <= t_nccl else "NCCL all-gather",
                    "exchange_bytes_per_rank": m * nb * 2 * (world - 1), "parity_ok": bool(flag.item())}


def bench_nvf4_gemv(ex, a):
    """Slot 394: W4A16 decode GEMV over an NVFP4 plane (f32 activations), K=5120 N=17408 by default."""
    n, k = a.n, a.k
    st = torch.cuda.current_stream().cuda_stream
    nbytes = n * k // 2 + n * k // 16
    nc = clones_for(nbytes)
    ws = [(torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device="cuda"),
           torch.randint(0x20, 0x48, (n * k // 16,), dtype=torch.uint8, device="cuda")) for _ in range(nc)]
    x = synth.bf16_round(synth.normal(k, 5, 1.0, "cuda"))
    y = torch.zeros(n, dtype=torch.float32, device="cuda")
    call = lambda i: ex.pack.call("nvf4_gemv", ws[i % nc][0], ws[i % nc][1], None, x, y, 1.0, k, n,
                                  stream=torch.cuda.current_stream().cuda_stream)
    sec = time_launches(call, a.iters)
    # spot check: clone 0's first rows against an f32 product of the dequantized weights
    call(0)
    rows = min(n, 256)
    wd = torch.empty(rows * k, dtype=torch.float32, device="cuda")
    ex.pack.call("nvf4_dequant", ws[0][0], ws[0][1], 1.0, wd, k, rows, stream=st)
    err = rel_err(y[:rows], wd.view(rows, k) @ x)
    return sec, {"bound": "hbm", "bytes": nbytes + 4 + k * 4 + n * 4, "parity_rel_l2": err, "parity_ok": err < 1e-3}


def bench_moe_nvf4(ex, a):
    """The MoE benchmark geometry (128 experts, top-4, 2880 / 2880) with NVFP4 expert planes (per-16 UE4M3 scales, scale2 per expert), plain SwiGLU."""
    from paddock_b200 import planes as P
    n_expert, k, embd, ff, T = 128, 4, a.k, a.n, a.m
    bm = 8 if T * k <= 1024 else 32

    def plane(rows, cols, seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        p = P.Nvf4MoePlane(
            torch.randint(0, 256, (n_expert * rows * cols // 2,), dtype=torch.uint8, device="cuda", generator=g),
            torch.randint(0x28, 0x40, (n_expert * rows * cols // 16,), dtype=torch.uint8, device="cuda", generator=g),
            torch.full((n_expert,), 1e-3, device="cuda"), n_expert, rows, cols)
        return P.nvf4_moe_prepare(ex, p)

    gate, up, down = plane(ff, embd, 1), plane(ff, embd, 2), plane(embd, ff, 3)

    class Shape:
        pass
    shape = Shape()
    shape.n_expert, shape.embd, shape.ff = n_expert, embd, ff
    ws = P.MoeWorkspace(ex, shape, T, k, bm)
    x = synth.bf16_round(synth.normal(T * embd, 7, 1.0, "cuda"))
    out = torch.zeros(T * embd, dtype=torch.float32, device="cuda")
    n_sets = 6 if T <= 64 else 1
    logits = [synth.normal(T * n_expert, 100 + i, 1.0, "cuda") for i in range(n_sets)]
    sec = time_launches(lambda i: P.moe_nvf4_forward(ex, gate, up, down, ws, x, logits[i % n_sets], out), a.iters)
    distinct = 0
    for lg in logits:
        distinct += torch.unique(torch.topk(lg.view(T, n_expert), k, dim=1).indices).numel()
    distinct /= n_sets
    per_expert = 3 * embd * ff // 16 * 9          # 4 bits + one scale byte per 16
    return sec, {"bound": "hbm", "bytes": int(distinct * per_expert + T * embd * 2 * 2), "distinct_experts": distinct}


OPS = {"tc5_probe": bench_tc5_probe, "f8_shard": bench_f8_shard, "norm_nvf4": bench_norm_nvf4, "q4k_w4a8": bench_q4k_w4a8, "nvf4_gemv": bench_nvf4_gemv, "moe_nvf4": bench_moe_nvf4, "moe_ep": bench_moe_ep, "moe_mxfp4": bench_moe, "nvf4_gemm": bench_nvf4, "q4k_gemv": bench_q4k, "q8_gemv": bench_q8, "f8row_gemm": bench_f8}
DEFAULTS = {"tc5_probe": (0, 0, 0), "f8_shard": (4096, 27648, 5120), "norm_nvf4": (64, 0, 5120), "q4k_w4a8": (4, 25600, 5120), "nvf4_gemv": (1, 17408, 5120), "moe_nvf4": (64, 2880, 2880), "moe_ep": (64, 2880, 2880), "moe_mxfp4": (64, 2880, 2880), "nvf4_gemm": (8192, 17408, 5120), "q4k_gemv": (1, 25600, 5120), "q8_gemv": (1, 17408, 5120), "f8row_gemm": (4096, 17408, 5120)}


class Case:
    """Arguments of one timed case (the command line's, or bench.py's)."""

    def __init__(self, op, m=None, n=None, k=None, iters=50, out="bf16", moe_path="tc5", graph=False, dtype="q4_k",
                 pack=None):
        dm, dn, dk = DEFAULTS[op]
        self.op, self.m, self.n, self.k = op, m or dm, n or dn, k or dk
        self.iters, self.out, self.moe_path, self.graph, self.dtype, self.pack = iters, out, moe_path, graph, dtype, pack


def run_case(ex, a):
    """Time one case; returns the JSON-able record the command line prints."""
    global GRAPH_REPLAY
    GRAPH_REPLAY = a.graph and a.op in ("q4k_gemv", "q8_gemv", "nvf4_gemv", "norm_nvf4", "nvf4_gemm")
    sec, info = OPS[a.op](ex, a)
    err = ex.pack.device_error() if not a.pack else 0
    hbm, bf16, kind = peaks()
    extra = {k: v for k, v in info.items() if k not in ("bound", "bytes", "flops")}
    line = {**extra, "op": a.op, "m": a.m, "n": a.n, "k": a.k, "us": sec * 1e6, "device_error": err, "peak_kind": kind,
            "pack": a.pack or "paddock_b200"}
    if info["bound"] in ("hbm", "both"):
        line.update(gbs=info["bytes"] / sec / 1e9, frac_of_hbm=info["bytes"] / sec / 1e9 / hbm)
    if info["bound"] in ("tensor", "both"):
        tf = info["flops"] / sec / 1e12
        line.update(tflops=tf, frac_of_2x_bf16=tf / (2 * bf16), frac_of_4x_bf16=tf / (4 * bf16))
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=sorted(OPS))
    ap.add_argument("--m", "--batch", dest="m", type=int, help="tokens (use --batch under torchrun, whose parser claims --m)")
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--moe-path", default="tc5", choices=["tc5", "mma"],
                    help="expert GEMMs: block-scaled tcgen05 (default) or the mma.sync kernels")
    ap.add_argument("--graph", action="store_true", help="replay the timed launches from a CUDA graph (moe_mxfp4, moe_ep, q4k_gemv, q8_gemv, nvf4_gemv, nvf4_gemm)")
    ap.add_argument("--dtype", default="q4_k", choices=["q4_k", "q5_k", "q6_k", "q4_0", "iq4_xs"], help="q4k_gemv: the plane's format")
    ap.add_argument("--pack", default=None, help="path of a kernel-pack library to time instead of this package's")
    args = ap.parse_args()
    a = Case(args.op, args.m, args.n, args.k, args.iters, args.out, args.moe_path, args.graph, args.dtype, args.pack)
    ep = a.op in ("moe_ep", "f8_shard")
    if ep:
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    if a.pack:
        from paddock_b200.pack import KernelPack
        ex = GpuExecutor(KernelPack.load(a.pack))
    else:
        ex = GpuExecutor()
    line = run_case(ex, a)
    if not ep or dist.get_rank() == 0:
        print(json.dumps(line), flush=True)
    if ep:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
