"""The row-sharded Q4_K decode GEMV on two GPUs (peer stores over NVLink, no collective in the
data path): a loop of launches with the deferred completion signal over three y buffers used in turn, a
different activation vector every step and a consumer right behind every launch, must see exactly what
GEMV + all-gather gives for every step, with no wait running out.  Skipped on a box with
fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

K_DIM, N_DIM, STEPS = 2048, 1056, 7      # bands of 33 row tiles: the last CTA of each rank has a short share


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from paddock_b200 import shard, synth
    from paddock_b200.planes import GpuExecutor
    ex = GpuExecutor()
    first_row, rows = shard.row_band(N_DIM, world, rank, align=16)
    raw = synth.quantize_q4_k(synth.normal(rows * K_DIM, 0x51 + rank, 0.02, dev))
    plane = ex.repack_kquant_raw(raw, K_DIM, rows)
    xs = [synth.bf16_round(synth.normal(K_DIM, 0x77 + s, 1.0, "cpu")).to(dev) for s in range(STEPS)]
    # shard.LaggedLoop owns three y buffers (a peer one launch ahead stores step s + 1 while this rank still
    # reads step s - 1) and the flag array / counters they share
    loop = shard.LaggedLoop(ex, N_DIM, first_row)
    chan = loop.chan
    seen = []
    for s in range(STEPS):
        y_prev = loop.launch(plane, xs[s])
        if y_prev is not None:                   # what follows launch s may read step s - 1 of every rank
            seen.append(y_prev.clone())
    seen.append(loop.close().clone())
    torch.cuda.synchronize()
    err = ex.pack.device_error()
    flags = chan.flags[:world].tolist()
    # reference: the local GEMV of every step, the bands put together by a sum of disjoint vectors
    ok = err == 0 and flags == [STEPS] * world
    y = torch.zeros(rows, dtype=torch.float32, device=dev)
    for s in range(STEPS):
        ex.pack.call("kquant_gemv", plane.data, plane.scales, xs[s], y, K_DIM, rows, 12)
        full = torch.zeros(N_DIM, dtype=torch.float32, device=dev)
        full[first_row:first_row + rows] = y
        dist.all_reduce(full)                    # disjoint bands: the sum is the concatenation, bit for bit
        ok = ok and torch.equal(full, seen[s])
    res = torch.tensor([1 if ok else 0, err], dtype=torch.int64, device=dev)
    dist.all_reduce(res)
    if rank == 0:
        np.save(out_path, res.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_lagged_loop_equals_gemv_plus_all_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "res.npy")
    mp.spawn(worker, args=(2, free_port(), out), nprocs=2, join=True)
    ok_count, err_sum = np.load(out).tolist()
    assert err_sum == 0
    assert ok_count == 2                         # both ranks saw every step of both ranks, bit for bit
