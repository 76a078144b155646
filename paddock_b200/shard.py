"""Output-row sharding of a dense quantized layer across ranks (one process per GPU).

Rows (output channels) are independent units: rank r owns the contiguous band
[r*N/G, (r+1)*N/G) of W, repacks it locally and computes y_r = W_r x.  The one
exchange step is an all-gather of the y bands; because the bands are contiguous
and equal, the gathered [G][M][N/G] buffer is y for M = 1 and a strided view for
M > 1.  The reference has no multi-GPU path; this layer is new.
"""


def row_band(n_rows, world, rank, align=1):
    """(first_row, rows) of `rank`; bands are equal and `align`-row aligned."""
    if n_rows % (world * align) != 0:
        raise ValueError(f"{n_rows} rows do not split into {world} bands of a multiple of {align}")
    per = n_rows // world
    return rank * per, per


def raw_band_bytes(n_rows, in_dim, world, rank, block_elems, block_bytes):
    """Byte range of a rank's band inside a row-major block-quantized tensor."""
    first, rows = row_band(n_rows, world, rank)
    row_bytes = in_dim // block_elems * block_bytes
    return first * row_bytes, rows * row_bytes


def gathered_to_token_major(gathered, world, batch, rows_per_rank):
    """[G][M][N/G] all-gather result -> [M][N] view (no copy for M = 1)."""
    return gathered.view(world, batch, rows_per_rank).permute(1, 0, 2).reshape(batch, world * rows_per_rank)


class PeerOutput:
    """A full-length f32 output vector allocated symmetrically on every rank of `group`, with every
    rank's copy mapped into this process over NVLink, followed by the step flags of the exchange
    (one u32 per rank) and this rank's CTA counter.  `ptrs` / `flag_ptrs` are the host arrays of
    device pointers the sharded GEMV entry points take; `local` is this rank's copy of y as a
    tensor.  Multicast binding is switched off (only plain peer stores are used)."""

    def __init__(self, n, group=None):
        import ctypes
        import os
        import torch
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        pad = (-n) % 64
        self.n = n
        self.buf = symm_mem.empty(n + pad + 64, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        self.buf.zero_()
        self.local = self.buf[:n]
        self.flags = self.buf[n + pad:n + pad + 16].view(torch.int32)       # word p: the last step rank p completed; word 8: waits
        self.ctr = self.buf[n + pad + 32:n + pad + 34].view(torch.int32)      # CTA counter, this rank's signalled steps
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self.ptrs = (ctypes.c_void_p * self.world)(*bases)
        self.flag_ptrs = (ctypes.c_void_p * self.world)(*[b + (n + pad) * 4 for b in bases])
        torch.cuda.synchronize()
        dist.barrier(group)           # every rank's zeros are in place before anybody stores

    def ptrs_address(self):
        import ctypes
        return ctypes.addressof(self.ptrs)

    def flag_ptrs_address(self):
        import ctypes
        return ctypes.addressof(self.flag_ptrs)


def gemv_into_peers(ex, w, x, out, row0, signal=False, stream=None):
    """This rank's Q4_K row band times x, stored at rows row0.. of every rank's `out` (PeerOutput).
    signal: the kernel also raises this rank's flag on every rank when the band is there (the step
    numbers count up by themselves)."""
    import torch
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    if signal:
        ex.pack.call("pdk_q4k_gemv_shard_sync", w.data, w.scales, x, out.ptrs_address(), out.flag_ptrs_address(),
                     out.ctr, out.world, out.rank, row0, 0, w.dims[0], w.dims[1], stream=st)
    else:
        ex.pack.call("pdk_q4k_gemv_shard", w.data, w.scales, x, out.ptrs_address(), out.world, row0, w.dims[0], w.dims[1],
                     stream=st)


def wait_for_peers(ex, out, budget_us=200000, stream=None):
    """Device-side wait (in the stream) until every rank's band of the next step has landed in this rank's y."""
    import torch
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    ex.pack.call("pdk_peer_flags_wait", out.flags, out.world, 0, budget_us, stream=st)
