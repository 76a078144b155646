"""Expert-parallel MXFP4 MoE block: experts split over the ranks of a process
group, routed tokens exchanged with two all-to-alls.

Each rank owns `n_expert / world` consecutive experts (weights resident on its
GPU only) and a shard of the tokens.  One block call:

  1. route the local tokens (top-k over all experts);
  2. count the (token, slot) pairs per destination rank, exchange the counts;
  3. dispatch: all-to-all of the token rows (bf16 - the activations are bf16
     values, so this is exact) with their local expert index and routing weight;
  4. run the grouped expert GEMMs on what arrived (one "slot" per row);
  5. combine: all-to-all of the weighted f32 outputs back to the token's owner,
     which sums a token's slots in slot order.

Step 5 keeps the single-GPU block's summation order, and a row's expert output
does not depend on which other rows share its block, so the result is
bit-identical to the single-GPU block on the same kernels.

The exchange goes through torch.distributed (NCCL over NVLink on GPUs, gloo on
CPU for the host-logic tests); the permutations around it are index_select
calls.  Received rows land in this rank's own memory before any kernel reads
them.  The expert computation is a callable, so the routing / exchange logic
runs without a GPU against any implementation of that step.
"""
import torch
import torch.distributed as dist


def expert_owner(idx, experts_per_rank):
    """Rank that owns each global expert index."""
    return torch.div(idx, experts_per_rank, rounding_mode="floor")


class Dispatch:
    """The permutation and split sizes of one block call (what step 5 needs to undo step 3)."""

    def __init__(self, order, send_counts, recv_counts, pairs):
        self.order, self.send_counts, self.recv_counts, self.pairs = order, send_counts, recv_counts, pairs

    @property
    def n_recv(self):
        return int(sum(self.recv_counts))


def plan_dispatch(idx, experts_per_rank, world, group=None):
    """idx int64[tokens][k] global expert choices -> Dispatch.  Pairs are ordered by destination rank,
    ties in (token, slot) order, so every rank's receive buffer is grouped by source rank."""
    dest = expert_owner(idx.reshape(-1), experts_per_rank)
    order = torch.argsort(dest, stable=True)
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return Dispatch(order, send.tolist(), recv.tolist(), idx.numel())


def exchange(rows, send_counts, recv_counts, group=None):
    """all-to-all of row blocks: rows [sum(send_counts)][...] -> [sum(recv_counts)][...]."""
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), list(recv_counts), list(send_counts), group=group)
    return out


def ep_moe_block(x, idx, w, n_expert, expert_fn, group=None):
    """One expert-parallel block call on this rank.

    x f32[tokens][embd] (bf16 values), idx int64[tokens][k] global expert choices, w f32[tokens][k]
    routing weights, expert_fn(rows f32[R][embd], local_expert int64[R], weight f32[R]) -> f32[R][embd]
    (the weighted expert outputs of this rank's experts).  Returns (sum over slots f32[tokens][embd],
    Dispatch)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if n_expert % world:
        raise ValueError(f"{n_expert} experts do not split over {world} ranks")
    epr = n_expert // world
    tokens, k = idx.shape
    d = plan_dispatch(idx, epr, world, group)
    token_of_pair = torch.div(d.order, k, rounding_mode="floor")
    flat_idx, flat_w = idx.reshape(-1), w.reshape(-1)
    send_x = x.index_select(0, token_of_pair).to(torch.bfloat16)
    send_e = (flat_idx.index_select(0, d.order) - expert_owner(flat_idx.index_select(0, d.order), epr) * epr)
    send_w = flat_w.index_select(0, d.order)
    recv_x = exchange(send_x, d.send_counts, d.recv_counts, group).to(torch.float32)
    recv_e = exchange(send_e, d.send_counts, d.recv_counts, group)
    recv_w = exchange(send_w, d.send_counts, d.recv_counts, group)
    part = expert_fn(recv_x, recv_e, recv_w) if d.n_recv else recv_x.new_zeros((0, x.shape[1]))
    back = exchange(part, d.recv_counts, d.send_counts, group)        # in `order` order
    slots = torch.empty((tokens * k, x.shape[1]), dtype=torch.float32, device=x.device)
    slots.index_copy_(0, d.order, back)
    return slots.view(tokens, k, x.shape[1]), d


PAD_EXPERT = -1  # local expert index of an unused slot of the fixed-capacity exchange


def ep_moe_block_fixed(x, idx, w, n_expert, expert_fn, capacity=None, group=None, dropped=None):
    """ep_moe_block without the host round trip: every rank sends every peer `capacity` row slots
    (default: all of its tokens*k pairs, which can never overflow), unused slots marked with
    PAD_EXPERT, so the split sizes are known without exchanging counts and nothing synchronizes
    the host.  One all-to-all each way: a slot is the token row as bf16 followed by 8 bytes
    (local expert i32, routing weight f32).  expert_fn must ignore rows whose expert is
    PAD_EXPERT (the kernels' alignment step drops indices outside [0, n_expert)); what it
    returns for them is never read.

    A capacity below tokens*k can overflow when routing is skewed: pairs beyond a destination's
    `capacity` slots (in token order) are dropped - they are not sent, contribute zero to their
    token, and are counted into `dropped` (a one-element int64 device tensor the caller reads
    whenever it likes; nothing here waits for it).  Every rank must pass the same capacity."""
    world = dist.get_world_size(group)
    if n_expert % world:
        raise ValueError(f"{n_expert} experts do not split over {world} ranks")
    epr = n_expert // world
    tokens, k = idx.shape
    embd = x.shape[1]
    pairs = tokens * k
    cap = pairs if capacity is None else int(capacity)
    if cap < 0:
        raise ValueError("capacity must not be negative")
    dev = x.device
    row_bytes = embd * 2 + 8
    n_slots = world * cap
    # one more row than is sent: the dump slot overflowing pairs are parked in
    send = torch.zeros((n_slots + 1, row_bytes), dtype=torch.uint8, device=dev)
    send[:, embd * 2:embd * 2 + 4] = 0xFF                      # expert = -1 everywhere
    if pairs:
        flat_idx, flat_w = idx.reshape(-1), w.reshape(-1)
        dest = expert_owner(flat_idx, epr)
        order = torch.argsort(dest, stable=True)
        # per-destination counts without bincount (which synchronizes the host to size its output)
        counts = (dest.unsqueeze(1) == torch.arange(world, device=dev).unsqueeze(0)).sum(0)
        starts = torch.cumsum(counts, 0) - counts
        dest_sorted = dest.index_select(0, order)
        rank_in_dest = torch.arange(pairs, device=dev) - starts.index_select(0, dest_sorted)
        overflow = rank_in_dest >= cap
        slot = torch.where(overflow, torch.full_like(rank_in_dest, n_slots), dest_sorted * cap + rank_in_dest)
        if dropped is not None:
            dropped += overflow.sum()
        token_of_pair = torch.div(order, k, rounding_mode="floor")
        rows = torch.empty((pairs, row_bytes), dtype=torch.uint8, device=dev)
        rows[:, :embd * 2] = x.index_select(0, token_of_pair).to(torch.bfloat16).view(torch.uint8).view(pairs, embd * 2)
        local_e = (flat_idx.index_select(0, order) - dest_sorted * epr).to(torch.int32)
        rows[:, embd * 2:embd * 2 + 4] = local_e.view(torch.uint8).view(pairs, 4)
        rows[:, embd * 2 + 4:] = flat_w.index_select(0, order).contiguous().view(torch.uint8).view(pairs, 4)
        send.index_copy_(0, slot, rows)                         # several dropped pairs may land on the dump row
    send = send[:n_slots]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    rx = recv[:, :embd * 2].contiguous().view(torch.bfloat16).view(n_slots, embd).to(torch.float32)
    re = recv[:, embd * 2:embd * 2 + 4].contiguous().view(torch.int32).view(-1).to(torch.int64)
    rw = recv[:, embd * 2 + 4:].contiguous().view(torch.float32).view(-1)
    part = expert_fn(rx, re, rw)
    back = torch.zeros((n_slots + 1, embd), dtype=torch.float32, device=dev)   # row n_slots stays zero: dropped pairs
    dist.all_to_all_single(back[:n_slots], part.contiguous(), group=group)
    slots = torch.zeros((pairs, embd), dtype=torch.float32, device=dev)
    if pairs:
        slots.index_copy_(0, order, back.index_select(0, slot))
    return slots.view(tokens, k, embd)


def combine_slots(slots, out):
    """out[t] += slots[t][0] + slots[t][1] + ... in slot order (the order of pd_moe_slot_combine)."""
    acc = slots[:, 0].clone()
    for s in range(1, slots.shape[1]):
        acc += slots[:, s]
    out += acc
    return out


class GpuExpertShard:
    """This rank's experts on its GPU: expert_fn for ep_moe_block built on the pack's kernels."""

    def __init__(self, ex, planes_local, max_rows, bm):
        from .planes import MoeWorkspace
        self.ex, self.planes, self.bm = ex, planes_local, bm
        self.ws = MoeWorkspace(ex, planes_local, max_rows, 1, bm)
        self.max_rows = max_rows
        self.launches = 0

    def __call__(self, rows, local_expert, weight):
        from .planes import moe_mxfp4_experts, moe_mxfp4_experts_tc5
        r = rows.shape[0]
        if r > self.max_rows:
            raise ValueError(f"{r} routed rows exceed the shard's workspace ({self.max_rows})")
        self.ws.idx[:r].copy_(local_expert.to(torch.int32))     # -1 (unused slot) is outside [0, n_expert): dropped
        self.ws.w[:r].copy_(weight)
        run = moe_mxfp4_experts_tc5 if self.planes.tc5 is not None else moe_mxfp4_experts
        self.launches += run(self.ex, self.planes, self.ws, rows.contiguous(), r)
        return self.ws.part[: r * self.planes.embd].view(r, self.planes.embd)


def gpu_ep_forward(ex, shard, x, router_logits, out, n_expert, k, group=None, router_bias=None, capacity=None,
                   fixed=True):
    """Route on this rank, exchange, compute, exchange back, combine into `out` (f32[tokens][embd]).
    fixed=True uses the fixed-capacity exchange (no host synchronization; every rank must pass the
    same `capacity`, by default the largest per-rank tokens*k, and the shard's workspace must hold
    world*capacity rows); fixed=False exchanges exact counts first."""
    tokens = x.shape[0]
    idx = torch.empty(tokens * k, dtype=torch.int32, device=x.device)
    w = torch.empty(tokens * k, dtype=torch.float32, device=x.device)
    st = torch.cuda.current_stream().cuda_stream
    ex.pack.call("moe_topk_batch", router_logits, router_bias, n_expert, k, idx, w, tokens, stream=st)
    d = None
    if fixed:
        slots = ep_moe_block_fixed(x, idx.view(tokens, k).to(torch.int64), w.view(tokens, k), n_expert, shard,
                                   capacity, group)
    else:
        slots, d = ep_moe_block(x, idx.view(tokens, k).to(torch.int64), w.view(tokens, k), n_expert, shard, group)
    ex.pack.call("moe_slot_combine", slots.contiguous(), out, x.shape[1], k, tokens, stream=st)
    return d
