"""Seeded synthetic weights in the on-disk (GGUF / safetensors) byte formats.

There are no checkpoints on the benchmark machine, so the benchmark and the
smoke run build their planes from a seeded normal draw quantized here with
torch ops (on whatever device the input lives on).  The recipes are the ones
the CPU oracle restates; tests/test_synth.py holds the two to byte equality.
"""
import torch


def normal(n, seed, sigma, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(n, generator=g, device=device, dtype=torch.float32) * sigma


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


def quantize_q8_0(w):
    """f32 [n] -> raw Q8_0 blocks, uint8 [n/32 * 34] = {f16 d, int8 q[32]}.
    d = amax/127 (f32), id = 1/d, q = round-half-away(w*id), d stored as f16
    (crates/paddock-engine/src/gpu_model/laguna/dflash.rs:233-253)."""
    b = w.reshape(-1, 32)
    amax = b.abs().amax(dim=1, keepdim=True)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    v = b * inv
    q = (torch.sign(v) * torch.floor(v.abs() + 0.5)).to(torch.int8)
    out = torch.empty(b.shape[0], 34, dtype=torch.uint8, device=w.device)
    out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(-1)


def quantize_q4_k(w):
    """f32 [n] -> raw Q4_K super-blocks, uint8 [n/256 * 144] (ggml block_q4_K:
    f16 d, f16 dmin, 12 packed 6-bit scale/min bytes, 128 nibble bytes).
    Per sub-block of 32: scale = (max - min0)/15 with min0 = min(0, min);
    d = max scale / 63, dmin = max(-min0) / 63, both rounded to f16;
    nibble = clamp(rint((w + dmin*m) / (d*sc)), 0, 15)."""
    b = w.reshape(-1, 8, 32)
    lo = torch.clamp(b.amin(dim=2), max=0.0)
    hi = torch.maximum(b.amax(dim=2), lo)
    scale = (hi - lo) / 15.0
    mn = 0.0 - lo
    d16 = (scale.amax(dim=1) / 63.0).to(torch.float16)
    m16 = (mn.amax(dim=1) / 63.0).to(torch.float16)
    d = d16.to(torch.float32).unsqueeze(1)
    dmin = m16.to(torch.float32).unsqueeze(1)
    zero = torch.zeros_like(scale)
    sc = torch.where(d > 0, torch.round(scale / d), zero).clamp(0, 63)
    m = torch.where(dmin > 0, torch.round(mn / dmin), zero).clamp(0, 63)
    dj = (d * sc).unsqueeze(2)
    mj = (dmin * m).unsqueeze(2)
    q = torch.where(dj > 0, torch.round((b + mj) / dj), torch.zeros_like(b)).clamp(0, 15).to(torch.uint8)
    sc = sc.to(torch.uint8)
    m = m.to(torch.uint8)
    out = torch.empty(b.shape[0], 144, dtype=torch.uint8, device=w.device)
    out[:, 0:2] = d16.view(torch.uint8).reshape(-1, 2)
    out[:, 2:4] = m16.view(torch.uint8).reshape(-1, 2)
    out[:, 4:8] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (m[:, 0:4] & 63) | ((m[:, 4:8] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:8] & 0xF) | ((m[:, 4:8] & 0xF) << 4)
    qg = q.reshape(-1, 4, 2, 32)
    out[:, 16:] = (qg[:, :, 0, :] | (qg[:, :, 1, :] << 4)).reshape(-1, 128)
    return out.reshape(-1)
