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


class LaggedLoop:
    """A decode loop over the row-sharded Q4_K GEMV with the deferred completion signal
    (pdk_q4k_gemv_shard_lagged): one launch per step and no fence inside it.  The loop owns its y buffers -
    three or more, used in turn, because a peer may be one launch ahead and already store step s + 1 while
    this rank reads step s - 1 - and the one flag array / counter pair they share.

        loop = LaggedLoop(ex, n_rows, first_row)
        for x in activations:
            y_prev = loop.launch(w, x)     # step s goes out; y_prev = the whole y of step s - 1 (None at first),
            ...                            # valid for work queued on the stream before the next launch
        y_last = loop.close()              # signals and awaits the last step

    `buffers` may be given (objects with ptrs_address(), flag_ptrs_address(), ctr, flags, local, world, rank:
    PeerOutput, or stand-ins in tests)."""

    def __init__(self, ex, n_rows, first_row, n_buffers=3, buffers=None):
        if buffers is None:
            if n_buffers < 3:
                raise ValueError("the deferred signal needs three or more y buffers")
            buffers = [PeerOutput(n_rows) for _ in range(n_buffers)]
        if len(buffers) < 3:
            raise ValueError("the deferred signal needs three or more y buffers")
        self.ex, self.bufs, self.first_row = ex, list(buffers), first_row
        self.chan = self.bufs[0]
        self.world, self.rank = self.chan.world, self.chan.rank
        self.steps = 0

    def _stream(self, stream):
        if stream is not None:
            return stream
        import torch
        return torch.cuda.current_stream().cuda_stream

    def launch(self, w, x, stream=None):
        b = self.bufs[self.steps % len(self.bufs)]
        self.ex.pack.call("pdk_q4k_gemv_shard_lagged", w.data, w.scales, x, b.ptrs_address(), self.chan.flag_ptrs_address(),
                          self.chan.ctr, self.world, self.rank, self.first_row, 0, w.dims[0], w.dims[1],
                          stream=self._stream(stream))
        self.steps += 1
        return self.bufs[(self.steps - 2) % len(self.bufs)].local if self.steps >= 2 else None

    def close(self, budget_us=2000000, stream=None):
        """Signals this rank's last step and waits (on the device, bounded) until every rank has caught up
        with it; returns the last step's y, or None if nothing was launched."""
        if self.steps == 0:
            return None
        st = self._stream(stream)
        self.ex.pack.call("pdk_peer_flags_post", self.chan.flag_ptrs_address(), self.chan.ctr, self.world, self.rank, stream=st)
        self.ex.pack.call("pdk_peer_flags_wait", self.chan.flags, self.world, 0x80000000 | self.rank, budget_us, stream=st)
        return self.bufs[(self.steps - 1) % len(self.bufs)].local
