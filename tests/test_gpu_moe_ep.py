"""Expert-parallel MoE block on two GPUs (NCCL): the combined output must be
bit-identical to the single-GPU block on the same kernels.  Skipped on a box
with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

N_EXPERT, K, EMBD, FF, BM = 16, 4, 256, 192, 8


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def build_planes(P, ex, dev, lo, hi, tc5):
    def plane(rows, cols, seed):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        nb = N_EXPERT * rows * cols // 32
        data = torch.randint(0, 256, (N_EXPERT, nb // N_EXPERT * 16), dtype=torch.uint8, generator=g)
        scale = torch.randint(118, 124, (N_EXPERT, nb // N_EXPERT), dtype=torch.uint8, generator=g)
        return P.RepackedMxfp4(data[lo:hi].reshape(-1).to(dev), scale[lo:hi].reshape(-1).to(dev))
    planes = P.MoeMxfp4Planes(plane(FF, EMBD, 1), plane(FF, EMBD, 2), plane(EMBD, FF, 3), hi - lo, EMBD, FF)
    return P.prepare_tc5(ex, planes) if tc5 else planes


def worker(rank, world, port, tokens, tc5, fixed, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from paddock_b200 import moe_ep, planes as P, synth
    ex = P.GpuExecutor()
    dev = ex.device
    x = synth.bf16_round(synth.normal(tokens * EMBD, 7, 1.0, dev)).view(tokens, EMBD)
    logits = synth.normal(tokens * N_EXPERT, 8, 1.0, dev).view(tokens, N_EXPERT)
    epr = N_EXPERT // world
    lo, hi = (tokens * rank) // world, (tokens * (rank + 1)) // world
    cap = -(-tokens // world) * K
    shard = moe_ep.GpuExpertShard(ex, build_planes(P, ex, dev, rank * epr, (rank + 1) * epr, tc5), max(tokens * K, world * cap), BM)
    out = torch.zeros(hi - lo, EMBD, device=dev)
    moe_ep.gpu_ep_forward(ex, shard, x[lo:hi].contiguous(), logits[lo:hi].contiguous(), out, N_EXPERT, K, capacity=cap,
                          fixed=fixed)
    torch.cuda.synchronize()
    parts = [torch.zeros(tokens, EMBD, device=dev) for _ in range(world)]
    padded = torch.zeros(tokens, EMBD, device=dev)
    padded[lo:hi] = out
    dist.all_gather(parts, padded)
    if rank == 0:
        y = sum(parts)
        full = build_planes(P, ex, dev, 0, N_EXPERT, tc5)
        ws = P.MoeWorkspace(ex, full, tokens, K, BM)
        ref = torch.zeros(tokens * EMBD, device=dev)
        P.moe_mxfp4_forward(ex, full, ws, x.reshape(-1), logits.reshape(-1), ref)
        torch.cuda.synchronize()
        np.save(out_path, np.stack([y.cpu().numpy().reshape(-1), ref.cpu().numpy()]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fixed", [False, True], ids=["counted", "fixed-capacity"])
@pytest.mark.parametrize("tc5", [False, True], ids=["mma", "tensor-core"])
@pytest.mark.parametrize("tokens", [1, 37])
def test_two_gpu_block_is_bit_identical(tmp_path, tokens, tc5, fixed):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "y.npy")
    mp.spawn(worker, args=(2, free_port(), tokens, tc5, fixed, out), nprocs=2, join=True)
    y, ref = np.load(out)
    assert np.isfinite(ref).all() and np.abs(ref).max() > 0
    assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))
