"""World-size-2 check (gloo, CPU) of the expert-parallel MoE block's host logic:
routing counts, dispatch / combine all-to-alls and the permutations around
them.  Each rank owns half of the experts and half of the tokens; the per-rank
expert computation is the CPU oracle (on GPUs it is the kernel pack), and the
combined result must equal the oracle's unsharded layer."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from paddock_b200 import moe_ep

N_EXPERT, K, EMBD, FF = 8, 2, 64, 96


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def layer():
    def plane(rows, cols, seed):
        return oracle.quantize_mxfp4(oracle.fill_normal(N_EXPERT * rows * cols, seed, 0.02)).reshape(N_EXPERT, -1)
    return plane(FF, EMBD, 1), plane(FF, EMBD, 2), plane(EMBD, FF, 3)


def worker(rank, world, port, tokens, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gate, up, down = layer()
    x = oracle.bf16_round(oracle.fill_normal(tokens * EMBD, 4, 1.0)).reshape(tokens, EMBD)
    logits = oracle.fill_normal(tokens * N_EXPERT, 5, 1.0)
    idx, w = oracle.moe_topk(logits, N_EXPERT, K)
    idx, w = idx.reshape(tokens, K), w.reshape(tokens, K)
    epr = N_EXPERT // world
    lo, hi = (tokens * rank) // world, (tokens * (rank + 1)) // world     # this rank's tokens (rank 1 may get none)
    mine = slice(rank * epr, (rank + 1) * epr)

    def expert_fn(rows, local_expert, weight):
        r = rows.shape[0]
        y = oracle.moe_mxfp4_layer(gate[mine], up[mine], down[mine], rows.numpy(), local_expert.numpy().reshape(r, 1),
                                   weight.numpy().reshape(r, 1), r, 1, EMBD, FF)
        return torch.from_numpy(y)

    slots, d = moe_ep.ep_moe_block(torch.from_numpy(x[lo:hi]), torch.from_numpy(idx[lo:hi].astype(np.int64)),
                                   torch.from_numpy(w[lo:hi]), N_EXPERT, expert_fn)
    out = moe_ep.combine_slots(slots, torch.zeros(hi - lo, EMBD))
    assert sum(d.send_counts) == (hi - lo) * K

    # the fixed-capacity exchange (no counts, unused slots marked) must give the same sums
    def expert_fn_padded(rows, local_expert, weight):
        live = local_expert >= 0
        y = torch.zeros(rows.shape[0], EMBD)
        if live.any():
            y[live] = expert_fn(rows[live], local_expert[live], weight[live])
        return y
    cap = ((tokens + world - 1) // world) * K              # the same on every rank
    slots_fixed = moe_ep.ep_moe_block_fixed(torch.from_numpy(x[lo:hi]), torch.from_numpy(idx[lo:hi].astype(np.int64)),
                                            torch.from_numpy(w[lo:hi]), N_EXPERT, expert_fn_padded, cap)
    assert torch.equal(slots_fixed, slots)
    gathered = [None] * world
    dist.all_gather_object(gathered, (lo, hi, out.numpy(), d.n_recv))
    if rank == 0:
        y = np.zeros((tokens, EMBD), np.float32)
        for a, b, part, _ in gathered:
            y[a:b] = part
        assert sum(g[3] for g in gathered) == tokens * K          # every routed pair arrived somewhere
        full = oracle.moe_mxfp4_layer(gate, up, down, x, idx, w, tokens, K, EMBD, FF)
        np.save(out_path, np.stack([y, full]))
    dist.destroy_process_group()


def run(tokens, tmp_path):
    out = str(tmp_path / f"y{tokens}.npy")
    mp.spawn(worker, args=(2, free_port(), tokens, out), nprocs=2, join=True)
    return np.load(out)


def test_expert_parallel_block_matches_unsharded(tmp_path):
    y, full = run(11, tmp_path)
    assert np.allclose(y, full, rtol=1e-5, atol=1e-6)


def test_single_token_lives_on_rank_0(tmp_path):
    y, full = run(1, tmp_path)
    assert np.allclose(y, full, rtol=1e-5, atol=1e-6)


def test_expert_owner():
    idx = torch.tensor([0, 15, 16, 127])
    assert moe_ep.expert_owner(idx, 16).tolist() == [0, 0, 1, 7]


def skew_worker(rank, world, port, out_path):
    """Every token routes both of its choices to rank 1's experts, and the capacity is smaller
    than what one rank sends there: the pairs beyond it must be dropped (zero contribution,
    counted), the others must come back exact, and nothing may spill into another rank's slots."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tokens, cap = 6, 5                                    # 12 pairs per rank, all bound for rank 1; 5 slots
    epr = N_EXPERT // world
    x = torch.from_numpy(oracle.bf16_round(oracle.fill_normal(tokens * EMBD, 40 + rank, 1.0)).reshape(tokens, EMBD))
    idx = torch.tensor([[epr + (t % epr), epr + ((t + 1) % epr)] for t in range(tokens)], dtype=torch.int64)
    w = torch.full((tokens, K), 0.5)

    def expert_fn(rows, local_expert, weight):            # "expert e" scales its rows by (e + 2) * weight
        live = local_expert >= 0
        assert not live.any() or rank == 1                # rank 0 owns none of the chosen experts
        y = torch.zeros(rows.shape[0], EMBD)
        y[live] = rows[live] * ((local_expert[live] + 2).float() * weight[live]).unsqueeze(1)
        return y
    dropped = torch.zeros(1, dtype=torch.int64)
    slots = moe_ep.ep_moe_block_fixed(x, idx, w, N_EXPERT, expert_fn, cap, dropped=dropped)
    want = torch.zeros(tokens, K, EMBD)
    for p in range(cap):                                  # the first `cap` pairs in token order survive
        t, s = divmod(p, K)
        want[t, s] = x[t] * ((idx[t, s] - epr + 2).float() * 0.5)
    ok = torch.equal(slots, want) and int(dropped) == tokens * K - cap
    gathered = [None] * world
    dist.all_gather_object(gathered, ok)
    if rank == 0:
        np.save(out_path, np.array(gathered))
    dist.destroy_process_group()


def test_fixed_capacity_overflow_is_dropped_and_counted(tmp_path):
    out = str(tmp_path / "skew.npy")
    mp.spawn(skew_worker, args=(2, free_port(), out), nprocs=2, join=True)
    assert np.load(out).all()


def test_fixed_capacity_rejects_negative():
    import pytest
    with pytest.raises(ValueError):
        # world size is read first: a single-process group is enough to reach the check
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
        dist.init_process_group("gloo", rank=0, world_size=1)
        try:
            moe_ep.ep_moe_block_fixed(torch.zeros(1, EMBD), torch.zeros(1, K, dtype=torch.int64), torch.zeros(1, K),
                                      N_EXPERT, lambda r, e, w: r, capacity=-1)
        finally:
            dist.destroy_process_group()
