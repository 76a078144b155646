"""Helpers shared by the -m gpu parity tests: seeded synthetic planes, device
buffers (torch is only the allocator here) and the two error metrics the
reference's own GPU tests use."""
import numpy as np
import torch

import oracle

TOL = 1e-2  # max relative error for GEMV/GEMM outputs stated by the north star


def dev(a):
    """numpy array -> device tensor with the same bytes."""
    a = np.ascontiguousarray(a)
    return torch.from_numpy(a.view(np.uint8).reshape(-1)).cuda()


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def host(t, dtype):
    return t.cpu().numpy().view(dtype)


def seed_for(config, tensor_id):
    return 0x5EED0000 + 256 * config + tensor_id


def bf16_activations(n, seed):
    """N(0,1) rounded to bf16 and widened back to f32 (exact)."""
    return oracle.bf16_round(oracle.fill_normal(n, seed, 1.0))


def cond_err(y, ref, abs_sum):
    """max_i |y - ref| / sum_k |w x|  (tests/gpu_nvfp4_oracle.rs:140-153)."""
    return float(np.max(np.abs(y.astype(np.float64) - ref) / np.maximum(abs_sum, 1e-30)))


def rel_l2(y, ref):
    """rel-L2 (tests/gpu_kquant_parity.rs:145-153)."""
    return float(np.linalg.norm(y.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-12))
