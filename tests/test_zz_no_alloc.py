"""The allocation-free MoE down + combine entry point (its partial buffer is a
static device array inside the library, for callers that cannot call
cudaMalloc) must give the same result as the ordinary pair of calls whose
partial buffer the caller allocates - on two calls in a row, since the second
call finds the first call's data in the shared buffer.

Collected last on purpose: with `-x` every other test has run before this one.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from gpu_util import dev, dev_f32
from paddock_b200 import planes as P

pytestmark = pytest.mark.gpu


def setup_case(pack, tokens, n_expert, k, embd, ff, bm, seed):
    ex = P.GpuExecutor(pack)
    raw = {n: oracle.quantize_mxfp4(oracle.fill_normal(n_expert * embd * ff, seed + i, 0.02))
           for i, n in enumerate(("gate", "up", "down"))}
    planes = P.MoeMxfp4Planes(*(P.repack_mxfp4(ex, dev(raw[n])) for n in ("gate", "up", "down")), n_expert, embd, ff)
    planes.down_bias = dev_f32(oracle.fill_normal(n_expert * embd, seed + 7, 0.02))
    x = oracle.bf16_round(oracle.fill_normal(tokens * embd, seed + 8, 1.0))
    logits = oracle.fill_normal(tokens * n_expert, seed + 9, 1.0)
    ws = P.MoeWorkspace(ex, planes, tokens, k, bm)
    out = torch.zeros(tokens * embd, dtype=torch.float32, device="cuda")
    P.moe_mxfp4_forward(ex, planes, ws, dev_f32(x), dev_f32(logits), out)   # fills ws (routing, hq, hscale)
    torch.cuda.synchronize()
    return planes, ws, out


def static_call(pack, planes, ws, residual, tokens, k, bm):
    pack.call("pdk_mxfp4_moe_down_combine_static", planes.down.data, planes.down.scale, planes.down_bias,
              ws.sorted_row, ws.sorted_slot, ws.block_expert, ws.w, ws.hq, ws.hscale, residual, planes.ff,
              planes.embd, k, tokens, bm, ws.max_blocks)


def test_static_scratch_matches_caller_allocated_path(pack):
    tokens, n_expert, k, embd, ff, bm = 6, 8, 4, 256, 320, 8
    planes, ws, want = setup_case(pack, tokens, n_expert, k, embd, ff, bm, 900)
    # a differently routed, larger problem first, so the shared buffer holds foreign data
    planes2, ws2, want2 = setup_case(pack, 13, n_expert, k, embd, ff, bm, 950)
    got2 = torch.zeros_like(want2)
    static_call(pack, planes2, ws2, got2, 13, k, bm)
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    for _ in range(2):                      # two calls in a row on the same buffer
        got = torch.zeros_like(want)
        static_call(pack, planes, ws, got, tokens, k, bm)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert np.isfinite(want.cpu().numpy()).all() and float(want.abs().max()) > 0


def test_static_scratch_refuses_oversize(pack):
    lib = C.CDLL(pack.origin)
    lib.pdk_static_part_capacity.restype = C.c_uint64
    lib.pdk_static_last_refusal.restype = C.c_char_p
    cap = lib.pdk_static_part_capacity()
    assert cap == 64 * 4096
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    rows = cap // (4 * 4096) + 1            # one token too many at top-4, embd 4096
    st = pack.status("pdk_mxfp4_moe_down_combine_static", buf, buf, None, buf, buf, buf, buf, buf, buf, buf,
                     2880, 4096, 4, rows, 8, 4)
    assert st == 1                          # cudaErrorInvalidValue, nothing launched
    assert b"exceeds the static partial buffer" in lib.pdk_static_last_refusal()
    # three factors whose product wraps past 2^64 (to 2^32 - 1 ... and below the capacity for some
    # triples) must be refused like any other oversize request
    for rows, k, embd in ((0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF), (0x80000000, 0x80000000, 4), (1 << 16, 1 << 16, 1 << 16)):
        st = pack.status("pdk_mxfp4_moe_down_combine_static", buf, buf, None, buf, buf, buf, buf, buf, buf, buf,
                         2880, embd, k, rows, 8, 4)
        assert st == 1
    torch.cuda.synchronize()
