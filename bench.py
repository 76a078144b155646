#!/usr/bin/env python
"""Benchmark of the quantized linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one Q4_K decode GEMV (M=1, K=5120, N=25600) through the
kernel-pack C ABI.  Prints ONE JSON line:

  value     weight GB/s = algorithmic bytes per step / device time per step,
            planes resident in HBM, cold L2 (the plane is cloned so that
            consecutive steps never touch the same bytes);
  e2e       the same metric with the step's activations coming from pinned
            host memory and its outputs read back, copies inside the timed
            region;
  roofline  achieved GB/s of the GEMV kernel (per-launch CUDA events) against
            the measured HBM copy bandwidth;
  cpu_baseline  the reference's CPU path (dequant + scalar f32 matvec), ported
            in oracle/, timed on this host's cores;
  configs   at N = 1, after the headline region: one record per further
            benchmark shape (Q8_0 GEMV, Q4_K at 4 / 16 tokens, FP8 and NVFP4
            GEMMs, the MXFP4 MoE block), each with its time, achieved GB/s or
            TFLOP/s, the fraction of the named denominator and a spot check of
            the result against an f32 product of the decoded operands.

With --gpus N > 1 (launched under torchrun) the N rows are sharded across the
ranks and the outputs are all-gathered with NCCL (strong scaling).
`--impl reference` times only the CPU path and prints the same line shape.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM = 5120
N_DIM = 25600
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch of the GEMV kernel from an
# ncu capture (scaled by rows when sharded): the planes as laid out in HBM (152 bytes per 256
# weights, of which 144 are the format's) plus y
NCU_TRAFFIC_BYTES = 79_990_000


def algorithmic_bytes(m, n=N_DIM, k=K_DIM):
    """Q4_K GEMV bytes per step: raw weights 144 B per 256 + bf16 x + f32 y."""
    return n * k // 256 * 144 + m * k * 2 + m * n * 4


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = get_reasons(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nv:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples), "reasons": sorted(self.reasons)}


class Cudart:
    """The handful of CUDA runtime calls the end-to-end loop makes per step, bound with ctypes."""

    def __init__(self):
        import ctypes as C
        self.C = C
        lib = None
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                lib = C.CDLL(name)
                break
            except OSError:
                continue
        if lib is None:
            raise RuntimeError("libcudart not found")
        self.lib = lib
        lib.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        lib.cudaEventCreateWithFlags.argtypes = [C.POINTER(C.c_void_p), C.c_uint]
        lib.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
        lib.cudaStreamWaitEvent.argtypes = [C.c_void_p, C.c_void_p, C.c_uint]
        lib.cudaEventSynchronize.argtypes = [C.c_void_p]

    def _ok(self, rc):
        if rc != 0:
            raise RuntimeError(f"CUDA runtime error {rc}")

    def event(self):
        e = self.C.c_void_p()
        self._ok(self.lib.cudaEventCreateWithFlags(self.C.byref(e), 2))      # cudaEventDisableTiming
        return e

    def copy(self, dst, src, n, kind, stream):                               # kind 1 = H2D, 2 = D2H
        self._ok(self.lib.cudaMemcpyAsync(dst, src, n, kind, stream))

    def record(self, ev, stream):
        self._ok(self.lib.cudaEventRecord(ev, stream))

    def wait(self, stream, ev):
        self._ok(self.lib.cudaStreamWaitEvent(stream, ev, 0))

    def sync_event(self, ev):
        self._ok(self.lib.cudaEventSynchronize(ev))


def cpu_baseline(steps, warmup, rows=N_DIM // 4):
    """Reference CPU path for one step: dequant_q4_k of the plane + scalar f32
    ascending-k matvec, on all host threads.  Returns (GB/s, cores, sample, ms)."""
    import numpy as np
    import oracle
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm uses every host core
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    w = oracle.fill_normal(rows * K_DIM, 0x5EED0200, 0.02)
    raw = oracle.quantize_q4_k(w)
    del w
    x = oracle.bf16_round(oracle.fill_normal(K_DIM, 0x5EED0201, 1.0))
    out = np.empty(rows * K_DIM, np.float32)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.dequant_q4_k(raw, out)
        oracle.matvec_f32(out, x, K_DIM, rows)
        t1 = time.perf_counter()
        if i >= warmup:
            times.append(t1 - t0)
    sec = sum(times) / len(times)
    gbs = algorithmic_bytes(1, rows) / sec / 1e9
    sample = f"{rows} of {N_DIM} rows x K={K_DIM}, dequant_q4_k + scalar f32 matvec, {len(times)} passes"
    return gbs, oracle.num_threads(), sample, sec * 1e3


def run_reference(args, rank):
    if rank != 0:
        return
    steps = min(args.steps, 20)
    warm = max(args.warmup, 3)
    rows = N_DIM // 4
    gbs, cores, sample, ms = cpu_baseline(steps, warm, rows)
    line = {
        "impl": "reference", "metric": "q4k_gemv_weight_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms * (N_DIM / rows),
        "ms_per_sample_pass": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.gpus, args.exchange),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, exchange="peer"):
    how = {"peer": "each rank's GEMV stores its band into every rank's y over NVLink (peer memory); y in three buffers used in turn; "
                   "every launch first raises the PREVIOUS step's flag on every rank (stream order puts that step's "
                   "stores before it, no fence inside the kernel) and checks on the device, bounded, that every rank's "
                   "previous step has arrived; the last step is signalled and awaited by two small kernels inside the "
                   "timed region",
           "peer-serial": "each rank's GEMV stores its band into every rank's y over NVLink (peer memory) and raises its flag "
                          "at the kernel's end, then a wait kernel for every rank's flag, then the next step (two y buffers "
                          "in turn)",
           "nccl": "NCCL all-gather of y"}[exchange]
    return {"workload": "Q4_K decode GEMV M=1 K=5120 N=25600, f32 activations holding bf16 values",
            "sharding": "none" if n_gpus == 1 else f"N rows / {n_gpus} ranks, {how}",
            "l2": "cold: steps rotate over weight-plane clones totalling > 2x the 126 MB L2"}


def other_configs(ex, quick):
    """One record per further benchmark shape, timed after the headline region (N = 1 only).
    Each is kbench's case for the shape: CUDA-event time, cold L2 for the memory-bound ones, and a
    spot check of the result against an f32 product of the decoded operands."""
    import gc
    import torch
    import kbench
    it = 10 if quick else 30
    # the tensor core's own issue rate per operand kind (operands resident in shared memory): the
    # measured denominator beside the 2x / 4x bf16 proxies of the FP8 and NVFP4 records
    probe = {}
    try:
        pr = kbench.run_case(ex, kbench.Case("tc5_probe", iters=128))
        probe = {k: round(v["tflops"], 1) for k, v in pr.items() if isinstance(v, dict)}
    except Exception as err:
        probe = {"error": str(err)[:200]}
    cases = [("q8_0_gemv_n17408", kbench.Case("q8_gemv", graph=True, iters=it)),
             ("q8_0_m4_n17408", kbench.Case("q8_gemv", m=4, graph=True, iters=it)),
             ("q8_0_m16_n17408", kbench.Case("q8_gemv", m=16, graph=True, iters=it)),
             ("q4k_m4_n25600", kbench.Case("q4k_gemv", m=4, graph=True, iters=it)),
             ("q4k_m16_n25600", kbench.Case("q4k_gemv", m=16, graph=True, iters=it))]
    cases += [(f"fp8_m4096_n{n}", kbench.Case("f8row_gemm", m=4096, n=n, iters=max(5, it // 3))) for n in (5120, 17408, 27648)]
    cases += [(f"nvf4_m{m}_n17408", kbench.Case("nvf4_gemm", m=m, graph=(m <= 64), iters=it if m <= 512 else max(5, it // 3)))
              for m in (1, 8, 64, 512, 8192)]
    cases += [("nvf4_w4a16_gemv_n17408", kbench.Case("nvf4_gemv", graph=True, iters=it))]
    cases += [(f"moe_mxfp4_t{t}", kbench.Case("moe_mxfp4", m=t, graph=(t == 1), iters=it if t <= 64 else max(5, it // 3)))
              for t in (1, 64, 1024)]
    out = {}
    for name, case in cases:
        try:
            r = kbench.run_case(ex, case)
            rec = {"us": r["us"], "parity_ok": r.get("parity_ok"), "parity_rel_l2": r.get("parity_rel_l2"),
                   "device_error": r["device_error"]}
            if case.op == "f8row_gemm":
                rec.update(achieved=r["tflops"], unit="TFLOP/s", frac=r["frac_of_2x_bf16"], denominator="2 x measured bf16 burst")
                if probe.get("e4m3_m128n256k32"):
                    rec.update(frac_of_probe=r["tflops"] / probe["e4m3_m128n256k32"], probe_denominator="tcgen05.mma e4m3 issue rate")
                    # shared-memory port (128 B per cycle and SM): per 128-byte K stage of the 256 x 256 pair tile
                    # 32 KB written by TMA + 4 MMAs x (4 + 4 + 4) KB read = 625 cycles for 512 tensor cycles
                    rec.update(frac_of_port_bound=r["tflops"] / (probe["e4m3_m128n256k32"] * 512.0 / 625.0),
                               port_bound="issue rate x 512 / 625: shared-memory bytes per K stage of the 256 x 256 pair tile")
            elif case.op == "nvf4_gemm" and case.m >= 512:
                rec.update(achieved=r["tflops"], unit="TFLOP/s", frac=r["frac_of_4x_bf16"], denominator="4 x measured bf16 burst",
                           gbs=r["gbs"], frac_of_hbm=r["frac_of_hbm"])
                # prefill widths run on pairs of SMs: the pair's rate is the denominator (the one-SM rate
                # with the same copies is a third lower)
                key = "nvf4_pair_m256n128k64_with_scale_copies"
                if probe.get(key):
                    # shared-memory port: per 256-element slab of the 256 x 256 pair tile 38 KB written + 4 MMAs x
                    # (4 + 4 + 4) KB + 6 KB of scale cells read = 720 cycles for 512 tensor cycles
                    rec.update(frac_of_port_bound=r["tflops"] / (probe[key] * 512.0 / 720.0),
                               port_bound="pair issue rate x 512 / 720: shared-memory bytes per K slab of the 256 x 256 pair tile")
                    rec.update(frac_of_probe=r["tflops"] / probe[key],
                               probe_denominator="tcgen05.mma NVFP4 issue rate on pairs of SMs with its scale-cell copies",
                               frac_of_one_sm_probe=r["tflops"] / probe.get("nvf4_m128n128k64_with_scale_copies", float("nan")))
            else:
                rec.update(achieved=r["gbs"], unit="GB/s", frac=r["frac_of_hbm"], denominator="measured HBM copy")
            if "distinct_experts" in r:
                rec["distinct_experts"] = r["distinct_experts"]
            out[name] = rec
        except Exception as err:                 # a failing case must not lose the headline line
            out[name] = {"error": str(err)[:200]}
        gc.collect()
        torch.cuda.empty_cache()
    out["tensor_core_probe_tflops"] = probe
    return out


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from paddock_b200 import synth
    from paddock_b200.planes import GpuExecutor

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from paddock_b200 import shard
    ex = GpuExecutor()
    _, rows = shard.row_band(N_DIM, world, rank, align=16)

    # ---- synthetic plane: this rank's row band, quantized to raw Q4_K, repacked
    w = synth.normal(rows * K_DIM, 0x5EED0200 + rank, 0.02, dev)
    raw = synth.quantize_q4_k(w)
    del w
    plane_bytes = rows * K_DIM // 256 * 152
    n_clones = max(2, -(-2 * L2_BYTES // plane_bytes) + 1)
    planes = [ex.repack_kquant_raw(raw, K_DIM, rows) for _ in range(n_clones)]
    del raw
    x_host = synth.bf16_round(synth.normal(K_DIM, 0x5EED0201, 1.0, "cpu")).pin_memory()
    x = x_host.to(dev)
    y = torch.zeros(rows, dtype=torch.float32, device=dev)
    y_all = torch.zeros(N_DIM, dtype=torch.float32, device=dev) if world > 1 else y
    y_host = torch.zeros(N_DIM, dtype=torch.float32).pin_memory()
    torch.cuda.synchronize()

    # N > 1: the row bands are exchanged by the GEMV kernel's own stores into every rank's y over
    # NVLink (peer memory); --exchange nccl keeps the kernel local and all-gathers y with NCCL.
    peer_out = peer_b = peer_c = None
    first_row, _ = shard.row_band(N_DIM, world, rank, align=16)
    if world > 1 and args.exchange in ("peer", "peer-serial"):
        peer_out = shard.PeerOutput(N_DIM)
        if args.exchange == "peer":
            # y in three buffers, used in turn: while this rank reads step s - 1 (after its launch s has observed
            # its arrival), a peer that is one launch ahead already stores step s + 1, and only its step s + 2,
            # which it cannot start before this rank's launch s + 1 has begun, returns to the buffer of s - 1
            peer_b, peer_c = shard.PeerOutput(N_DIM), shard.PeerOutput(N_DIM)
        else:
            # peer-serial: two buffers in turn, so that a peer that has passed its wait for step s and started
            # step s + 1 does not store into the y this rank is still reading
            peer_b = shard.PeerOutput(N_DIM)
        y_all = peer_out.local
        # the two exchanges must agree bit for bit
        ex.kquant_gemv(planes[0], x, y)
        check = torch.zeros(N_DIM, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(check, y)
        shard.gemv_into_peers(ex, planes[0], x, peer_out, first_row)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        if not torch.equal(check, y_all):
            raise RuntimeError("peer-store exchange differs from the all-gather")

    # One pre-bound launcher per plane clone (arguments converted once; the call is the C ABI entry).
    # N > 1, peer exchange (default): a step is ONE launch, the sharded GEMV.  y lives in three buffers
    # used in turn; all buffers share one flag array.  A launch signals nothing when it ends (the
    # system-scope fence for that costs an NVLink round trip behind which the next launch would wait);
    # instead every launch first stores - once the previous launch and its peer stores are complete -
    # the previous step's number into every rank's flags, and before it ends checks, on the device and
    # with a bounded wait, that every rank's previous step has arrived here.  Consecutive steps overlap
    # the way single-GPU launches do while every step's arrival is still observed on the device; the
    # last step is signalled by a post kernel and observed by a wait kernel at the end of the timed
    # region.  No step relies on a host barrier, and the calls count their steps on the device, so their
    # arguments never change and a captured sequence replays.
    # --exchange peer-serial is the single-buffered loop: GEMV that signals at its end, then a wait
    # kernel for every rank's flag, then the next GEMV (a consumer that must read y before the next step).
    st = torch.cuda.current_stream().cuda_stream
    bufs = [b for b in (peer_out, peer_b, peer_c) if b is not None]

    def bind_all(stream, xin, yout):
        """-> (launch(i) for step i, tail() that observes the arrival of the last steps)."""
        if peer_out is not None:
            serial = args.exchange == "peer-serial"
            name = "pdk_q4k_gemv_shard_sync" if serial else "pdk_q4k_gemv_shard_lagged"
            # one flag array and one counter pair (the first buffer's) for every buffer of the loop
            gem = [[ex.pack.bind(name, p.data, p.scales, xin, b.ptrs_address(), peer_out.flag_ptrs_address(), peer_out.ctr,
                                 world, rank, first_row, 0, p.dims[0], p.dims[1], stream=stream) for b in bufs] for p in planes]
            if serial:
                wait = ex.pack.bind("pdk_peer_flags_wait", peer_out.flags, world, 0, 2000000, stream=stream)
                return (lambda i: (gem[i % n_clones][i % len(bufs)](), wait())), (lambda: None)
            # closing: signal this rank's last step, then wait until every rank has caught up with it
            post = ex.pack.bind("pdk_peer_flags_post", peer_out.flag_ptrs_address(), peer_out.ctr, world, rank, stream=stream)
            wait = ex.pack.bind("pdk_peer_flags_wait", peer_out.flags, world, 0x80000000 | rank, 2000000, stream=stream)
            return (lambda i: gem[i % n_clones][i % len(bufs)]()), (lambda: (post(), wait()))
        ls = [ex.pack.bind("kquant_gemv", p.data, p.scales, xin, yout, p.dims[0], p.dims[1], p.ty, stream=stream)
              for p in planes]
        return (lambda i: ls[i % n_clones]()), (lambda: None)

    bound, bound_tail = bind_all(st, x, y)

    def step(i):
        bound(i)
        if world > 1 and peer_out is None:
            dist.all_gather_into_tensor(y_all, y)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()

    # ---- timed region: exactly K steps, device time, max over ranks
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The K steps are K launches through the C ABI either way; with --graph (default, and only
    # where no NCCL call sits inside a step) they are captured once into a CUDA graph and the
    # timed region replays it, the way a serving loop replays its captured decode step, so the
    # host's per-call cost (8 us from Python) does not pace a kernel that takes less.
    graph = None
    if args.graph and (world == 1 or peer_out is not None):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g_st = side.cuda_stream
            g_bound, g_tail = bind_all(g_st, x, y)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    g_bound(i)
                g_tail()
            torch.cuda.synchronize()
            graph.replay()                      # one untimed replay
            torch.cuda.synchronize()
        except Exception as err:                # capture not possible here: time the direct launches
            print(f"bench: graph capture failed ({err}); timing direct launches", file=sys.stderr)
            graph = None
    barrier()
    e0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(args.steps):
            step(i)
        bound_tail()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    # keep the same load running until the clock sampler has a few dozen samples (about 0.4 s).
    # The step count must be the same on every rank - a step holds a collective - so it is
    # derived from the slowest rank's timed region, not from each rank's own clock.
    agreed = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
    n_extra = int(min(50000, max(64, 400.0 / max(agreed.item() / args.steps, 1e-3))))
    for i in range(n_extra):
        step(i)
        if i % 64 == 63:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    sampler.stop()

    # ---- per-launch duration of the GEMV kernel alone (roofline)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i, (a, b) in enumerate(evs):
        a.record()
        ex.kquant_gemv(planes[i % n_clones], x, y)
        b.record()
    torch.cuda.synchronize()
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)

    # ---- end to end: pinned host activations in, outputs back, every step.
    # N = 1: the way a decode loop runs it - three steps in flight on three streams (copy in, kernel,
    # copy out), each step's input copied from pinned memory into its own device buffer and its
    # result read back and waited for by the host two steps later.  N > 1 keeps one step in flight.
    if world == 1:
        e2e_mode = "3 steps in flight: H2D / kernel / D2H on three streams, host waits for step i-2's result"
        s_in, s_k, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        D = 3  # buffers = steps in flight
        xb = [torch.empty_like(x) for _ in range(D)]
        yb = [torch.empty_like(y) for _ in range(D)]
        yh = [torch.zeros(N_DIM, dtype=torch.float32).pin_memory() for _ in range(D)]
        launch = [[ex.pack.bind("kquant_gemv", p.data, p.scales, xb[b], yb[b], p.dims[0], p.dims[1], p.ty,
                                stream=s_k.cuda_stream) for b in range(D)] for p in planes]
        # copies, events and waits go straight to the CUDA runtime (a torch call costs the host
        # several microseconds each, more than this step's kernel leaves room for)
        rt = Cudart()
        ev_in, ev_k, ev_out = ([rt.event() for _ in range(D)] for _ in range(3))
        q_in, q_k, q_out = s_in.cuda_stream, s_k.cuda_stream, s_out.cuda_stream
        x_src, x_bytes = x_host.data_ptr(), x_host.numel() * 4
        xd, yd, yhp = [t.data_ptr() for t in xb], [t.data_ptr() for t in yb], [t.data_ptr() for t in yh]
        y_bytes = y.numel() * 4

        def e2e_step(i):
            b = i % D
            rt.wait(q_in, ev_k[b])               # the kernel of step i-D has consumed this buffer
            rt.copy(xd[b], x_src, x_bytes, 1, q_in)
            rt.record(ev_in[b], q_in)
            rt.wait(q_k, ev_in[b])
            rt.wait(q_k, ev_out[b])              # step i-D's result has left this buffer
            launch[i % n_clones][b]()
            rt.record(ev_k[b], q_k)
            rt.wait(q_out, ev_k[b])
            rt.copy(yhp[b], yd[b], y_bytes, 2, q_out)
            rt.record(ev_out[b], q_out)
            if i >= D - 1:
                rt.sync_event(ev_out[(i + 1) % D])   # the host has step i-(D-1)'s result

        torch.cuda.synchronize()
        for i in range(2 * D):
            e2e_step(i)
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        for j in range(D):
            rt.sync_event(ev_out[j])
        e2e_ms = (time.perf_counter() - w0) * 1e3   # three streams: host clock around the fully drained loop
        torch.cuda.synchronize()
        host_paced_ms = e2e_ms
        # The same pipeline captured once and replayed, the way a serving loop replays its captured
        # step: per step an H2D copy node (pinned host activations), the kernel node and a D2H copy node
        # (the result into pinned host memory) on three captured streams with the same buffer
        # dependencies; the host launches the graph and waits for the last result.  Every step still
        # moves its input and its output over PCIe; what is gone is the host's per-call cost (12 runtime
        # calls a step from Python, about 30 us, more than the kernel takes).
        try:
            cap = torch.cuda.CUDAGraph()
            evi, evk, evo = ([rt.event() for _ in range(D)] for _ in range(3))
            fork, j_in, j_out = rt.event(), rt.event(), rt.event()
            with torch.cuda.graph(cap, stream=s_k):
                rt.record(fork, q_k)
                rt.wait(q_in, fork)
                rt.wait(q_out, fork)
                for i in range(args.steps):
                    b = i % D
                    if i >= D:
                        rt.wait(q_in, evk[b])        # the kernel of step i-D has consumed this input buffer
                    rt.copy(xd[b], x_src, x_bytes, 1, q_in)
                    rt.record(evi[b], q_in)
                    rt.wait(q_k, evi[b])
                    if i >= D:
                        rt.wait(q_k, evo[b])         # step i-D's result has left this output buffer
                    launch[i % n_clones][b]()
                    rt.record(evk[b], q_k)
                    rt.wait(q_out, evk[b])
                    rt.copy(yhp[b], yd[b], y_bytes, 2, q_out)
                    rt.record(evo[b], q_out)
                rt.record(j_in, q_in)
                rt.record(j_out, q_out)
                rt.wait(q_k, j_in)
                rt.wait(q_k, j_out)
            for t in yh:
                t.zero_()
            cap.replay()
            torch.cuda.synchronize()
            w0 = time.perf_counter()
            cap.replay()
            torch.cuda.synchronize()                 # the graph runs on the current stream: wait for the device
            graph_ms = (time.perf_counter() - w0) * 1e3
            if graph_ms < e2e_ms:
                e2e_ms = graph_ms
                e2e_mode = ("the K steps captured into one CUDA graph and replayed: per step an H2D copy node, the kernel "
                            "node and a D2H copy node on three captured streams, 3 steps in flight; the host launches "
                            "the graph and waits for the last result")
            # The same steps captured in groups of G: a group's H2D copies first (each into its own buffer), then
            # its kernels back to back - no cross-stream wait between two kernels of a group, so the dependent
            # launch that overlaps one kernel's start with the previous one's tail survives the capture - each
            # kernel followed by its D2H copy on the third stream.  Every step still copies its input in and
            # its result out; G results are in flight.
            G = 16
            xg = [torch.empty_like(x) for _ in range(G)]
            yg = [torch.empty_like(y) for _ in range(G)]
            yhg = [torch.zeros(N_DIM, dtype=torch.float32).pin_memory() for _ in range(G)]
            launch_g = [[ex.pack.bind("kquant_gemv", p.data, p.scales, xg[b], yg[b], p.dims[0], p.dims[1], p.ty,
                                      stream=s_k.cuda_stream) for b in range(G)] for p in planes]
            xgp, ygp, yhgp = [t.data_ptr() for t in xg], [t.data_ptr() for t in yg], [t.data_ptr() for t in yhg]
            cap2 = torch.cuda.CUDAGraph()
            gi, gk, go = ([rt.event() for _ in range(G)] for _ in range(3))
            fork2, j2_in, j2_out = rt.event(), rt.event(), rt.event()
            with torch.cuda.graph(cap2, stream=s_k):
                rt.record(fork2, q_k)
                rt.wait(q_in, fork2)
                rt.wait(q_out, fork2)
                for g0 in range(0, args.steps, G):
                    n = min(G, args.steps - g0)
                    for b in range(n):
                        if g0 > 0:
                            rt.wait(q_in, gk[b])     # the kernel of the previous group has consumed this input buffer
                        rt.copy(xgp[b], x_src, x_bytes, 1, q_in)
                        rt.record(gi[b], q_in)
                    for b in range(n):
                        rt.wait(q_k, gi[b])
                        if g0 > 0:
                            rt.wait(q_k, go[b])      # the previous group's result has left this output buffer
                    for b in range(n):
                        launch_g[(g0 + b) % n_clones][b]()
                        rt.record(gk[b], q_k)
                        rt.wait(q_out, gk[b])
                        rt.copy(yhgp[b], ygp[b], y_bytes, 2, q_out)
                        rt.record(go[b], q_out)
                rt.record(j2_in, q_in)
                rt.record(j2_out, q_out)
                rt.wait(q_k, j2_in)
                rt.wait(q_k, j2_out)
            cap2.replay()
            torch.cuda.synchronize()
            w0 = time.perf_counter()
            cap2.replay()
            torch.cuda.synchronize()
            grouped_ms = (time.perf_counter() - w0) * 1e3
            last = args.steps - 1
            ex.kquant_gemv(planes[last % n_clones], x, y)
            torch.cuda.synchronize()
            if not torch.equal(yhg[last % G][:y.numel()], y.cpu()):
                raise RuntimeError("grouped end-to-end graph returned a different y")
            if grouped_ms < e2e_ms:
                e2e_ms = grouped_ms
                e2e_mode = (f"the K steps captured into one CUDA graph in groups of {G}: a group's H2D copy nodes (pinned "
                            "host activations, one device buffer per step), then its kernel nodes back to back, each followed "
                            "by its D2H copy node into pinned host memory, on three captured streams; the host launches the "
                            "graph and waits for the last result")
        except Exception as err:
            print(f"bench: end-to-end graph capture failed ({err}); keeping the host-paced loop", file=sys.stderr)
        # the pipelined loop must produce the same y as a plain call
        ex.kquant_gemv(planes[(args.steps - 1) % n_clones], x, y)
        torch.cuda.synchronize()
        if not torch.equal(yh[(args.steps - 1) % D][:y.numel()], y.cpu()):
            raise RuntimeError("pipelined end-to-end loop returned a different y")
    else:
        # N > 1: one step in flight - the host reads every step's whole y before it launches the next one; the y
        # buffers are used in turn as in the timed loop, so a peer that is already a step ahead stores elsewhere;
        # copies and waits through the CUDA runtime directly, as at N = 1.
        e2e_mode = "1 step in flight: H2D, sharded GEMV + flag wait (or NCCL all-gather), D2H of the full y, host wait"
        rt = Cudart()
        ev = rt.event()
        x_src, x_bytes = x_host.data_ptr(), x_host.numel() * 4
        y_dst, y_bytes = y_host.data_ptr(), y_all.numel() * 4
        y_srcs = [b.local.data_ptr() for b in bufs] or [y_all.data_ptr()]
        e2e_tail = bound_tail if (peer_out is not None and args.exchange == "peer") else None

        def e2e_step(i):
            rt.copy(x.data_ptr(), x_src, x_bytes, 1, st)
            step(i)
            if e2e_tail is not None:
                e2e_tail()                       # the host reads this step's y: signal it, every band must be here
            rt.copy(y_dst, y_srcs[i % len(y_srcs)], y_bytes, 2, st)
            rt.record(ev, st)
            rt.sync_event(ev)

        for i in range(3):
            e2e_step(i)
        barrier()
        w0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        e2e_ms = (time.perf_counter() - w0) * 1e3
        barrier()

        # The pipelined form of the same loop for the peer exchange, captured into one CUDA graph in groups of
        # G steps: a group's H2D copies (one x buffer per step), then its sharded GEMVs back to back with the
        # deferred signal, each followed - one launch later, when its arrival from every rank has been observed
        # on the device - by the D2H copy of the whole y into pinned host memory.  y rotates over G + 2
        # buffers: step u stores into a buffer whose previous tenant, step u - G - 2, was copied out in an earlier
        # group, and a group's first kernel waits for the previous group's copies - so by the time ANY rank can
        # store step u (its launch u - 1 has ended, hence every rank's launch u - 1 has started), every rank has
        # its copy of that buffer out.  No cross-stream wait sits between two kernels of a group.
        if peer_out is not None and args.exchange == "peer":
            try:
                G = 8
                R = G + 2
                ybufs = [shard.PeerOutput(N_DIM) for _ in range(R)]
                s_in, s_k2, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
                q_in, q_k, q_out = s_in.cuda_stream, s_k2.cuda_stream, s_out.cuda_stream
                xg = [torch.empty_like(x) for _ in range(G)]
                yhg = [torch.zeros(N_DIM, dtype=torch.float32).pin_memory() for _ in range(G)]
                gi, gk, go = ([rt.event() for _ in range(G)] for _ in range(3))
                fork, j_in, j_out, tail_ev = rt.event(), rt.event(), rt.event(), rt.event()
                chan = peer_out
                cap3 = torch.cuda.CUDAGraph()
                s_k2.wait_stream(torch.cuda.current_stream())
                with torch.cuda.graph(cap3, stream=s_k2):
                    rt.record(fork, q_k)
                    rt.wait(q_in, fork)
                    rt.wait(q_out, fork)
                    prev_last_out = None
                    for g0 in range(0, args.steps, G):
                        n = min(G, args.steps - g0)
                        for b in range(n):
                            if g0 > 0:
                                rt.wait(q_in, gk[b])      # the kernel of the previous group has consumed this x buffer
                            rt.copy(xg[b].data_ptr(), x_src, x_bytes, 1, q_in)
                            rt.record(gi[b], q_in)
                        for b in range(n):
                            rt.wait(q_k, gi[b])
                        if prev_last_out is not None:
                            rt.wait(q_k, prev_last_out)   # the previous group's copies out (the stream is in order)
                        for b in range(n):
                            u = g0 + b
                            p = planes[u % n_clones]
                            ex.pack.call("pdk_q4k_gemv_shard_lagged", p.data, p.scales, xg[b], ybufs[u % R].ptrs_address(),
                                         chan.flag_ptrs_address(), chan.ctr, world, rank, first_row, 0, p.dims[0], p.dims[1],
                                         stream=q_k)
                            rt.record(gk[b], q_k)
                            if u >= 1:                    # launch u has observed every rank's step u - 1
                                rt.wait(q_out, gk[b])
                                rt.copy(yhg[(u - 1) % G].data_ptr(), ybufs[(u - 1) % R].local.data_ptr(), y_bytes, 2, q_out)
                                rt.record(go[b], q_out)
                                prev_last_out = go[b]
                    last = args.steps - 1
                    ex.pack.call("pdk_peer_flags_post", chan.flag_ptrs_address(), chan.ctr, world, rank, stream=q_k)
                    ex.pack.call("pdk_peer_flags_wait", chan.flags, world, 0x80000000 | rank, 2000000, stream=q_k)
                    rt.record(tail_ev, q_k)
                    rt.wait(q_out, tail_ev)
                    rt.copy(yhg[last % G].data_ptr(), ybufs[last % R].local.data_ptr(), y_bytes, 2, q_out)
                    rt.record(j_in, q_in)
                    rt.record(j_out, q_out)
                    rt.wait(q_k, j_in)
                    rt.wait(q_k, j_out)
                barrier()
                cap3.replay()
                barrier()
                w0 = time.perf_counter()
                cap3.replay()
                torch.cuda.synchronize()
                graph_ms = (time.perf_counter() - w0) * 1e3
                barrier()
                if not torch.equal(yhg[last % G], check.cpu()):
                    raise RuntimeError("pipelined sharded end-to-end graph returned a different y")
                if ex.pack.device_error() != 0:
                    raise RuntimeError(f"device error {ex.pack.device_error():#x} in the pipelined sharded loop")
                if graph_ms < e2e_ms:
                    e2e_ms = graph_ms
                    e2e_mode = (f"the K steps captured into one CUDA graph in groups of {G}: a group's H2D copy nodes, then its "
                                "sharded GEMVs back to back (deferred signal), each followed one launch later - its arrival "
                                f"from every rank observed on the device - by the D2H copy of the whole y; y rotates over {R} "
                                "buffers; the host launches the graph and waits for the last result")
            except Exception as err:
                print(f"bench: pipelined sharded end-to-end capture failed ({err}); keeping the one-step loop", file=sys.stderr)
            barrier()

    times = torch.tensor([total_ms, e2e_ms, kern_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kern_ms = times.tolist()

    if rank == 0:
        ms_step = total_ms / args.steps
        bytes_step = algorithmic_bytes(1)
        peak, peak_kind = measured_peak()
        kern_bytes = algorithmic_bytes(1, rows)
        # one step is one GEMV launch at N=1, so the timed region's average is the
        # kernel's back-to-back launch duration; with a collective in the step the
        # separately event-bracketed launches are used instead
        event_us = kern_ms * 1e3
        if graph is not None:
            kern_ms = ms_step       # the step is this rank's kernel (N > 1: plus the flag wait that follows it)
        achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": "q4k_gemv_weight_gbs", "value": bytes_step / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world, args.exchange),
            "e2e": {"value": bytes_step / (e2e_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": K_DIM * 4, "d2h_bytes_per_step": N_DIM * 4,
                    "ms_per_step": e2e_ms / args.steps, "mode": e2e_mode,
                    **({"host_paced_ms_per_step": host_paced_ms / args.steps} if world == 1 else {})},
            "gpu_launches": args.steps,
            "launch": "one replay of a CUDA graph holding the K launches" if graph is not None else "K direct launches",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES * rows // N_DIM, "peak_kind": peak_kind,
                         "kernel": "gemv_ring_kernel<RQ4K>", "us_per_launch": kern_ms * 1e3,
                         "us_per_launch_event_bracketed": event_us,
                         "algorithmic_bytes_per_launch": kern_bytes},
            "clocks": sampler.summary(),
        }
        if world == 1:
            gbs, cores, sample, _ = cpu_baseline(3, 1)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
            if args.configs:
                del planes, bound, bound_tail
                torch.cuda.empty_cache()
                line["configs"] = other_configs(ex, quick=args.steps < 50)
    if world > 1 and args.configs:
        # the other sharded shapes (every rank runs them; rank 0 reports): FP8 prefill GEMM with its
        # output channels sharded, and the expert-parallel MXFP4 MoE block
        import kbench
        del planes, bound, bound_tail
        torch.cuda.empty_cache()
        sharded = {}
        quick = args.steps < 50
        for name, case in (("fp8_m4096_n27648_nshard", kbench.Case("f8_shard", iters=5 if quick else 10)),
                           ("moe_mxfp4_t64_expert_parallel", kbench.Case("moe_ep", m=64, graph=True, iters=10 if quick else 30)),
                           ("moe_mxfp4_t1024_expert_parallel", kbench.Case("moe_ep", m=1024, graph=True, iters=5 if quick else 10))):
            try:
                r = kbench.run_case(ex, case)
                keep = ("us", "n_gpus", "us_gemm_only", "us_gemm_nccl_allgather", "us_gemm_peer_stores", "exchange", "m_chunks",
                        "exchange_bytes_per_rank", "parity_ok", "tflops", "gbs", "frac_of_hbm", "frac_of_2x_bf16",
                        "distinct_experts", "device_error")
                sharded[name] = {k: r[k] for k in keep if k in r}
            except Exception as err:
                sharded[name] = {"error": str(err)[:200]}
            torch.cuda.empty_cache()
        if rank == 0:
            line["configs"] = sharded
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="time K direct launches instead of one replay of a CUDA graph holding them")
    ap.add_argument("--no-configs", dest="configs", action="store_false",
                    help="N = 1: skip the records of the other benchmark shapes")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer-serial", "nccl"],
                    help="N > 1: how the row bands of y reach every rank")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with WORLD_SIZE={args.gpus} (got {world})")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
