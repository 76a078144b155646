"""World-size-2 check (gloo, CPU) of the output-row sharding convention the
multi-GPU benchmark uses: each rank computes its band of y from its band of
the raw quantized tensor, the bands are all-gathered, and the result must equal
the unsharded product.  The per-rank compute here is the CPU oracle; on GPUs it
is the kernel pack."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from paddock_b200 import shard


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, n, k, batch, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = oracle.fill_normal(n * k, 5, 0.02)
    raw = oracle.quantize_q4_k(w)                      # every rank derives the same full tensor
    x = oracle.bf16_round(oracle.fill_normal(batch * k, 6, 1.0))
    off, nbytes = shard.raw_band_bytes(n, k, world, rank, 256, 144)
    first, rows = shard.row_band(n, world, rank)
    band = oracle.dequant_q4_k(raw[off:off + nbytes])
    y_band = oracle.matmul_f64(band, x, k, rows, batch)          # [batch][rows]
    gathered = torch.empty(world * batch * rows, dtype=torch.float32)
    dist.all_gather_into_tensor(gathered, torch.from_numpy(np.ascontiguousarray(y_band)).reshape(-1))
    y = shard.gathered_to_token_major(gathered, world, batch, rows)
    if rank == 0:
        full = oracle.matmul_f64(oracle.dequant_q4_k(raw), x, k, n, batch)
        np.save(out_path, np.stack([y.numpy(), full]))
    dist.destroy_process_group()


def test_row_sharded_gemm_matches_unsharded(tmp_path):
    n, k, batch, world = 64, 512, 3, 2
    out = str(tmp_path / "y.npy")
    mp.spawn(worker, args=(world, free_port(), n, k, batch, out), nprocs=world, join=True)
    y, full = np.load(out)
    assert np.array_equal(y, full)


def test_band_helpers():
    assert shard.row_band(25600, 8, 3) == (9600, 3200)
    assert shard.raw_band_bytes(25600, 5120, 8, 1, 256, 144) == (3200 * 20 * 144, 3200 * 20 * 144)
    import pytest
    with pytest.raises(ValueError):
        shard.row_band(100, 8, 0)


class _FakeBuffer:
    def __init__(self, tag, world=2, rank=1):
        self.tag, self.world, self.rank = tag, world, rank
        self.ctr, self.flags, self.local = f"ctr{tag}", f"flags{tag}", f"y{tag}"

    def ptrs_address(self):
        return f"ptrs{self.tag}"

    def flag_ptrs_address(self):
        return f"flagptrs{self.tag}"


class _FakeExecutor:
    class _Pack:
        def __init__(self):
            self.calls = []

        def call(self, name, *args, stream=None):
            self.calls.append((name, args, stream))

    def __init__(self):
        self.pack = self._Pack()


class _FakePlane:
    data, scales, dims = "data", "scales", (512, 64)


def test_lagged_loop_rotates_three_buffers_over_one_flag_channel():
    """Host side of the deferred-signal loop: y buffers in turn, every launch on the first buffer's flag array and
    counters, the previous step's y handed back, post + wait at the end; fewer than three buffers refused."""
    import pytest
    ex = _FakeExecutor()
    bufs = [_FakeBuffer(i) for i in range(3)]
    loop = shard.LaggedLoop(ex, 128, 64, buffers=bufs)
    seen = [loop.launch(_FakePlane, f"x{s}", stream=7) for s in range(5)]
    assert seen == [None, "y0", "y1", "y2", "y0"]
    names = [c[0] for c in ex.pack.calls]
    assert names == ["pdk_q4k_gemv_shard_lagged"] * 5
    for s, (_, args, stream) in enumerate(ex.pack.calls):
        data, scales, x, yptrs, flagptrs, ctr, world, rank, row0, step, in_dim, out_dim = args
        assert (x, yptrs, flagptrs, ctr) == (f"x{s}", f"ptrs{s % 3}", "flagptrs0", "ctr0")
        assert (world, rank, row0, step, in_dim, out_dim, stream) == (2, 1, 64, 0, 512, 64, 7)
    assert loop.close(stream=7) == "y1"                      # step 5 went into buffer 4 % 3
    assert [c[0] for c in ex.pack.calls[5:]] == ["pdk_peer_flags_post", "pdk_peer_flags_wait"]
    assert ex.pack.calls[5][1] == ("flagptrs0", "ctr0", 2, 1)
    assert ex.pack.calls[6][1] == ("flags0", 2, 0x80000000 | 1, 2000000)
    with pytest.raises(ValueError):
        shard.LaggedLoop(ex, 128, 64, buffers=bufs[:2])
    assert shard.LaggedLoop(ex, 128, 64, buffers=bufs).close() is None
