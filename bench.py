"""Benchmark of the quantised GEMV hot path on B200: Q4_K decode sweep, Llama-7B layer shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass over the sweep: y = x W^T for the four Q4_K weight shapes 4096x4096, 11008x4096,
4096x11008 and 32000x4096 at batch M = 1 and M = 8 (eight launches). Weights are seeded N(0, 0.02)
values quantised to Q4_K, activations N(0, 1). Each launch reads a different copy of its weight from
a rotating pool several times the size of L2, so every weight byte comes from HBM.

The line printed (rank 0) carries:
  value      algorithmic GB/s of the whole job with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the C ABI with host buffers: pinned-host x copied in and y copied
             out inside every timed call
  roofline   achieved GB/s of the GEMV kernel against the measured HBM copy peak
  cpu_baseline  the CPU port of the reference's host arithmetic (oracle/), one thread, one step
With --gpus N > 1 every weight is split by output rows over the ranks and each launch is followed by
an NCCL all-gather of the output slices (strong scaling: the job is the same at every N).
With --impl reference the CPU port runs the sweep on all host threads instead (the reference's own
backend for these operators is its scalar host loop; it has no JVM here to run in).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]  # [N out, K in]
BATCHES = [1, 8]
TYPE = "Q4_K"
BYTES_PER_WEIGHT = 144.0 / 256.0
POOL_COPIES = 4  # distinct copies of every weight; 4 x 134 MB = 537 MB, about 4x the 126 MB L2
METRIC = "q4k_gemv_sweep_GBps"
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one step of this sweep, per linear: not measured by the run
# itself but taken from an ncu capture of the same command line (`--steps 20 --warmup 3 --no-cpu --no-decode --eager`, one pass,
# --clock-control none); the line names the source beside the figure.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 269226240 // 8
NCU_TRAFFIC_SOURCE = "ncu capture of the sweep (the 12 launches of one eager step), not measured by this run"
WORKLOAD = "Q4_K GEMV sweep: [N,K] in 4096x4096, 11008x4096, 4096x11008, 32000x4096, M in {1,8}; 8 launches per step"


def algorithmic_bytes(n, k, m):
    """Quantised weights once + FP32 x + FP32 y."""
    return n * k * BYTES_PER_WEIGHT + 4.0 * m * k + 4.0 * m * n


def step_bytes():
    return sum(algorithmic_bytes(n, k, m) for n, k in SHAPES for m in BATCHES)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms from its creation until stop()."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append((time.time(), parts))

    def stop(self, t0, t1):
        """Summary over the samples taken in [t0, t1] (the timed region); if the region was too short to
        catch one, over the samples of the whole run under load, and `window` says so."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for ts, r in self.rows if t0 <= ts <= t1 + 0.05]
        window = "timed region"
        if not inside:
            inside = [r for ts, r in self.rows]
            window = "whole run (timed region shorter than the sampling period)"
        sm, mx, power, reasons = [], [], [], set()
        for r in inside:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm), "window": window}


def make_weights(torch, device, rank, world):
    """Seeded N(0, 0.02) weights quantised to Q4_K on the GPU; each rank uploads its row shard."""
    from jitnn_b200 import Tensor, synth
    pools, samples = [], []
    for si, (n, k) in enumerate(SHAPES):
        copies = []
        for c in range(POOL_COPIES):
            g = torch.Generator(device=device).manual_seed(1234 + 17 * si + c)
            wf = torch.randn(n, k, generator=g, device=device) * 0.02
            raw = synth.quantize_q4_k(wf).cpu().numpy()
            del wf
            lo, hi = rank * n // world, (rank + 1) * n // world
            copies.append(Tensor.quantized(TYPE, raw, n, k, device=device.index, rows=(lo, hi)) if world > 1
                          else Tensor.quantized(TYPE, raw, n, k, device=device.index))
            if c == 0:
                rows = guard_rows(n, world)
                samples.append((rows, raw[rows].copy()))
        pools.append(copies)
    return pools, samples


def guard_rows(n, world):
    """Rows the parity guard compares with the oracle: the first and last rows of the weight and the rows on both sides of every
    shard border (at 8 ranks, whatever the run's world size: the same rows at every N)."""
    rows = set(range(16)) | set(range(n - 16, n))
    for g in range(1, 8):
        b = g * n // 8
        rows |= {b - 2, b - 1, b, b + 1}
    return sorted(rows)


def launches_per_step(L, step, side, torch, device):
    """Kernels one eager step launches (the graph replays exactly these)."""
    with torch.cuda.stream(side):
        before = L.jq_launch_count()
        step(0)
        torch.cuda.synchronize(device)
        return L.jq_launch_count() - before


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import jitnn_b200
    from jitnn_b200 import _lib, sharded

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run for N > 1" % (args.gpus, world))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback for the product path"
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    L = jitnn_b200.load()

    if args.leg in ("prefill", "decode", "formats", "decode70b"):
        # one leg alone, for profiler captures: no sweep, a short line of its own
        out = (prefill_leg(torch, device, L, _lib) if args.leg == "prefill" else
               formats_leg(torch, device, L, _lib, reps=max(1, min(25, args.steps))) if args.leg == "formats" else  # --steps 1: a short run for profiler captures
               decode_70b_leg(torch, device, rank, world, args.decode_shape) if args.leg == "decode70b" else
               decode_leg(torch, device, args.decode_shape))
        if rank == 0:
            print(json.dumps({"leg": args.leg, "result": out}), flush=True)
        if world > 1:
            torch.cuda.synchronize(device)
            dist.barrier()
            sys.stdout.flush()
            os._exit(0)
        return

    pools, samples = make_weights(torch, device, rank, world)
    g = torch.Generator(device=device).manual_seed(99)
    xs = {(k, m): torch.randn(m, k, generator=g, device=device) for _, k in SHAPES for m in BATCHES}
    ys = {}
    for n, k in SHAPES:
        for m in BATCHES:
            ys[(n, k, m)] = torch.empty(m, n // world, device=device)

    # With several ranks y [m, n] is completed on every rank after each linear: by the library's peer-store exchange
    # (every rank writes its slice into every rank's y over NVLink, then a bounded wait for the others' flags) or, with
    # --gather nccl, by an NCCL all-gather.
    peers, gather_kind = {}, "none"
    if world > 1:
        gather_kind = args.gather
        if gather_kind == "peer":
            try:
                for n, k in SHAPES:
                    for m in BATCHES:
                        peers[(n, k, m)] = sharded.PeerGather(n, m, device=device.index)
            except Exception as exc:  # no CUDA IPC between these processes: every rank fails alike
                sys.stderr.write("peer gather unavailable (%s): using the NCCL all-gather\n" % exc)
                peers, gather_kind = {}, "nccl"

    def step(i):
        sp = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        for si, (n, k) in enumerate(SHAPES):
            for mi, m in enumerate(BATCHES):
                w = pools[si][(i * len(BATCHES) + mi) % POOL_COPIES]
                y = ys[(n, k, m)]
                if gather_kind == "peer":
                    peers[(n, k, m)].linear(w, xs[(k, m)])  # y [m, n] complete on every rank
                    continue
                _lib.check(L.jq_linear_f32(w._handle(), xs[(k, m)].data_ptr(), m, None, y.data_ptr(), _lib.JQ_MEM_DEVICE, sp))
                if gather_kind == "nccl":
                    sharded.gather_rows(y, n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # Parity guard, at every N and on every rank (not timed): one pass over the sweep on copy 0 of every weight, through the same
    # calls the timed steps make; sampled rows of the complete y (first, last, both sides of every shard border) against the
    # CPU oracle. The weights are the same at every N (seeded by shape and copy; a rank uploads its rows of them).
    from oracle import oracle
    worst = 0.0
    for si, (n, k) in enumerate(SHAPES):
        rows, raw_rows = samples[si]
        for m in BATCHES:
            w = pools[si][0]
            x0 = xs[(k, m)]
            if gather_kind == "peer":
                full = peers[(n, k, m)].linear(w, x0)
            else:
                y = ys[(n, k, m)]
                sp0 = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
                _lib.check(L.jq_linear_f32(w._handle(), x0.data_ptr(), m, None, y.data_ptr(), _lib.JQ_MEM_DEVICE, sp0))
                full = sharded.gather_rows(y, n) if gather_kind == "nccl" else y
            torch.cuda.synchronize(device)
            got = full.cpu().numpy()
            if gather_kind == "none" and world > 1:  # diagnosis mode: every rank only has its own rows
                lo = rank * n // world
                keep = [i for i, r in enumerate(rows) if lo <= r < (rank + 1) * n // world]
                ref = oracle.linear(TYPE, raw_rows[keep], x0.cpu().numpy(), None, threads=4)
                got = got[:, [rows[i] - lo for i in keep]]
            else:
                ref = oracle.linear(TYPE, raw_rows, x0.cpu().numpy(), None, threads=4)
                got = got[:, rows]
            worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    if world > 1:
        t = torch.tensor([worst], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = float(t.item())
    assert worst <= 1e-3, "GEMV differs from the oracle: max relative error %g" % worst
    parity_check = {"against": "CPU oracle (ops/Gguf.java:187-205 semantics)", "max_rel_err": worst, "tolerance": 1e-3, "ranks_checked": world,
                    "rows_per_shape": len(samples[0][0]), "shapes": len(SHAPES) * len(BATCHES), "ok": True}

    # The weight rotation repeats every `period` steps. That many steps are captured into a CUDA graph (the launches of
    # a step are a few microseconds each, less than the host needs to issue them) and the graph is replayed; with
    # several ranks the NCCL all-gathers are part of each rank's graph.
    period = POOL_COPIES // len(BATCHES) if POOL_COPIES % len(BATCHES) == 0 else POOL_COPIES
    use_graph = not args.eager
    side = torch.cuda.Stream(device)
    graph = None
    with torch.cuda.stream(side):
        for i in range(args.warmup):
            step(i)
        torch.cuda.synchronize(device)
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(period):
                    step(i)
            for _ in range(3):
                graph.replay()
    timed_steps = args.steps if not use_graph else max(period, args.steps // period * period)
    # The region of `timed_steps` steps is timed `regions` times back to back, each with its own pair of events; the line
    # reports the median region (and the spread), so that a region of a few milliseconds still sits inside a window long
    # enough for the clock sampler.
    regions = max(1, min(200, -(-2000 // timed_steps)))
    sampler = ClockSampler(local) if rank == 0 else None
    time.sleep(0.2)  # lets the sampler take its first readings; every rank waits, then all start together
    barrier()
    t_start = time.time()
    launches0 = L.jq_launch_count()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(regions)]
    with torch.cuda.stream(side):
        for e0, e1 in events:
            e0.record(side)
            if use_graph:
                for _ in range(timed_steps // period):
                    graph.replay()
            else:
                for i in range(timed_steps):
                    step(args.warmup + i)
            e1.record(side)
    barrier()
    t_end = time.time()
    region_ms = [e0.elapsed_time(e1) for e0, e1 in events]
    # kernels of this library that ran in the timed regions: counted at launch, or launches per captured step x replays
    launches = (L.jq_launch_count() - launches0) if not use_graph else regions * timed_steps * launches_per_step(L, step, side, torch, device)
    if world > 1:
        t = torch.tensor(region_ms, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every region: the slowest rank
        region_ms = [float(v) for v in t.tolist()]
    ms = statistics.median(region_ms)
    clocks = sampler.stop(t_start, t_end) if sampler else None
    ms_per_step = ms / timed_steps
    spread = {"regions": regions, "steps_per_region": timed_steps, "ms_per_step_min": round(min(region_ms) / timed_steps, 5),
              "ms_per_step_median": round(ms_per_step, 5), "ms_per_step_max": round(max(region_ms) / timed_steps, 5)}
    args.steps = timed_steps
    value = step_bytes() / (ms_per_step * 1e-3) / 1e9
    stream = torch.cuda.current_stream(device)
    sp = ctypes.c_void_p(stream.cuda_stream)

    # With several ranks: the same sweep without the exchange (every rank computes its rows into a private y), so that the
    # line names what the exchange costs per linear at this N.
    exchange = None
    if world > 1 and gather_kind == "peer":
        def shard_step(i):
            sps = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            for si, (n, k) in enumerate(SHAPES):
                for mi, m in enumerate(BATCHES):
                    w = pools[si][(i * len(BATCHES) + mi) % POOL_COPIES]
                    _lib.check(L.jq_linear_f32(w._handle(), xs[(k, m)].data_ptr(), m, None, ys[(n, k, m)].data_ptr(), _lib.JQ_MEM_DEVICE, sps))
        with torch.cuda.stream(side):
            for i in range(period):
                shard_step(i)
            torch.cuda.synchronize(device)
            runner = None
            if use_graph:
                runner = torch.cuda.CUDAGraph()
                with torch.cuda.graph(runner, stream=side):
                    for i in range(period):
                        shard_step(i)
                runner.replay()
            barrier()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(20)]
            for e0, e1 in ev:
                e0.record(side)
                for rep in range(timed_steps // period):
                    if use_graph:
                        runner.replay()
                    else:
                        for i in range(period):
                            shard_step(i)
                e1.record(side)
            barrier()
        tt = torch.tensor([e0.elapsed_time(e1) for e0, e1 in ev], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        alone = statistics.median(float(v) for v in tt.tolist()) / (timed_steps // period * period)
        n_lin = len(SHAPES) * len(BATCHES)
        exchange = {"ms_per_step_rows_only": round(alone, 5), "ms_per_step_with_exchange": round(ms_per_step, 5),
                    "exchange_us_per_linear": round((ms_per_step - alone) * 1e3 / n_lin, 3),
                    "note": "rows only = every rank multiplies its rows and keeps them (jq_linear_f32 on the shard); with exchange = jq_linear_f32_peer, "
                            "whose kernel stores into every rank's y, announces its part and ends when all ranks' parts have arrived"}

    # per-shape kernel times (device-resident, same rotation, graph replay), for the roofline breakdown
    per_shape = {}
    if world == 1:
        with torch.cuda.stream(side):
            sps = ctypes.c_void_p(side.cuda_stream)
            for si, (n, k) in enumerate(SHAPES):
                for m in BATCHES:
                    def rot():
                        for r in range(POOL_COPIES):
                            _lib.check(L.jq_linear_f32(pools[si][r]._handle(), xs[(k, m)].data_ptr(), m, None, ys[(n, k, m)].data_ptr(), 1, sps))
                    rot()
                    torch.cuda.synchronize(device)
                    reps = 10
                    if use_graph:
                        gs = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(gs, stream=side):
                            rot()
                        gs.replay()
                    a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize(device)
                    a.record(side)
                    for r in range(reps):
                        if use_graph:
                            gs.replay()
                        else:
                            rot()
                    b2.record(side)
                    torch.cuda.synchronize(device)
                    us = a.elapsed_time(b2) * 1e3 / (reps * POOL_COPIES)
                    per_shape["%dx%d_m%d" % (n, k, m)] = {"us": round(us, 3), "GBps": round(algorithmic_bytes(n, k, m) / us / 1e3, 1)}

    # end to end through the C ABI with host buffers (pinned), copies inside the timed region
    e2e = None
    e2e_steps = min(args.steps, 200)
    if world == 1:
        hx = {key: torch.randn(key[1], key[0], generator=torch.Generator().manual_seed(5)).pin_memory() for key in xs}
        hy = {key: torch.empty(key[2], key[0]).pin_memory() for key in ys}

        # the arguments of every call, looked up once (a caller holds its handles and buffers): per step phase, the eight linears
        linear_f32, mem_host = L.jq_linear_f32, _lib.JQ_MEM_HOST
        phases = [[(pools[si][(ph * len(BATCHES) + mi) % POOL_COPIES]._handle(), hx[(k, m)].data_ptr(), m, hy[(n, k, m)].data_ptr())
                   for si, (n, k) in enumerate(SHAPES) for mi, m in enumerate(BATCHES)] for ph in range(POOL_COPIES)]

        def host_step(i):
            for handle, xp, m, yp in phases[i % POOL_COPIES]:
                rc = linear_f32(handle, xp, m, None, yp, mem_host, None)
                if rc != 0:
                    _lib.check(rc)

        for i in range(args.warmup):
            host_step(i)
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            host_step(args.warmup + i)
        torch.cuda.synchronize(device)
        dt = (time.perf_counter() - t0) / e2e_steps
        e2e = {"value": round(step_bytes() / dt / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": int(sum(4 * m * k for _, k in SHAPES for m in BATCHES)),
               "d2h_bytes_per_step": int(sum(4 * m * n for n, _ in SHAPES for m in BATCHES)),
               "ms_per_step": round(dt * 1e3, 4), "steps": e2e_steps,
               "path": "jq_linear_f32 with page-locked host x and y, one blocking call per linear: x (up to 1 MB) is read by the kernels "
                       "across PCIe in place, y up to 256 KB is written in place, larger y through a device-to-host copy"}
    elif gather_kind == "peer":
        # N > 1: every rank's process holds x in its own page-locked host memory and copies it in; the row-sharded linear with
        # the peer exchange completes y on every rank; rank 0 reads the whole y back to its host memory. One call per linear,
        # the stream synchronised after each (the result is needed on the host), max over ranks of the wall clock.
        hx = {key: torch.randn(key[1], key[0], generator=torch.Generator().manual_seed(5)).pin_memory() for key in xs}
        hy = {key: torch.empty(key[2], key[0]).pin_memory() for key in ys} if rank == 0 else {}
        dx = {key: torch.empty_like(xs[key]) for key in xs}

        def host_step(i):
            for si, (n, k) in enumerate(SHAPES):
                for mi, m in enumerate(BATCHES):
                    w = pools[si][(i * len(BATCHES) + mi) % POOL_COPIES]
                    dx[(k, m)].copy_(hx[(k, m)], non_blocking=True)
                    full = peers[(n, k, m)].linear(w, dx[(k, m)])
                    if rank == 0:
                        hy[(n, k, m)].copy_(full, non_blocking=True)
                    torch.cuda.current_stream(device).synchronize()

        for i in range(args.warmup):
            host_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            host_step(args.warmup + i)
        barrier()
        t = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        e2e = {"value": round(step_bytes() / dt / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": int(world * sum(4 * m * k for _, k in SHAPES for m in BATCHES)),
               "d2h_bytes_per_step": int(sum(4 * m * n for n, _ in SHAPES for m in BATCHES)),
               "ms_per_step": round(dt * 1e3, 4), "steps": e2e_steps,
               "path": "every rank copies x from its page-locked host memory, jq_linear_f32_peer (row shard + peer-store exchange), rank 0 copies "
                       "the whole y to its host memory; one call and one stream synchronisation per linear, max over ranks"}

    prefill = prefill_leg(torch, device, L, _lib) if (rank == 0 and world == 1 and not args.only) else None
    formats = formats_leg(torch, device, L, _lib) if (rank == 0 and world == 1 and not args.only) else None
    sharded_layer = sharded_layer_leg(torch, device, rank, world, L, _lib) if (not args.only and gather_kind != "nccl") else None
    decode = None
    if rank == 0 and world == 1 and not args.only and not args.no_decode:
        for copies in pools:
            for w in copies:
                w.release()  # make room: the decoder holds 5 GB of weights and 1 GB of cache
        decode = decode_leg(torch, device)
    decode_70b = None
    if not args.only and not args.no_decode and gather_kind != "nccl":
        # every rank takes part (the decoder is split by rows over the ranks); a failure is reported, not fatal to the line
        for copies in pools:
            for w in copies:
                w.release()
        for p in peers.values():
            p.close()
        peers = {}
        try:
            decode_70b = decode_70b_leg(torch, device, rank, world)
        except Exception as exc:  # noqa: BLE001 - whatever it is, the sweep's numbers above are still valid
            decode_70b = {"error": "%s: %s" % (type(exc).__name__, exc)}
    cpu = None
    if rank == 0 and not args.no_cpu:
        # the reference's CPU backend runs these operators on one thread (engine/CpuExecutor.java:233-239): that is the baseline;
        # the same loops over all host cores are printed beside it as a courtesy figure. Thread counts are explicit: the
        # environment (OMP_NUM_THREADS, which the multi-rank launcher sets to 1) does not change them.
        cpu = cpu_baseline_leg(threads=1, fraction=8, steps=1)
        cores = host_cores()
        allc = cpu_baseline_leg(threads=cores, fraction=1 if cores >= 8 else 4, steps=1)
        cpu["all_cores"] = {"value": allc["value"], "unit": "GB/s", "cores": cores, "sample": allc["sample"],
                            "note": "the same loops split by output rows over every host core: something the reference does not do"}

    if rank == 0:
        peak, which = measured_peaks()
        n_launch = len(SHAPES) * len(BATCHES)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "weights": "seeded N(0,0.02) quantised to Q4_K, x ~ N(0,1) fp32",
                       "l2": "every launch reads a different copy from a pool of %d copies per shape (%.0f MB > 126 MB L2)"
                             % (POOL_COPIES, POOL_COPIES * sum(n * k for n, k in SHAPES) * BYTES_PER_WEIGHT / 1e6),
                       "launch": ("CUDA graph of %d steps, replayed" % period) if use_graph else "eager launches through the C ABI",
                       "parallelism": "single GPU" if world == 1 else "output rows split over %d GPUs + %s per launch" % (
                           world, "peer-store all-gather in the GEMV epilogue (jq_linear_f32_peer)" if gather_kind == "peer" else "NCCL all-gather")},
            "roofline": {"bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s", "frac": round(value / world / peak, 4),
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (world == 1 and not args.only) else None,
                         "traffic_source": NCU_TRAFFIC_SOURCE if (world == 1 and not args.only) else None, "peak_source": "of " + which, "frac_of_nominal_8TBps": round(value / world / 8000.0, 4),
                         "bytes_per_launch": round(step_bytes() / n_launch / world), "us_per_launch": round(ms_per_step * 1e3 / n_launch, 3),
                         "per_shape": per_shape},
            "formats": formats, "sharded_70b_layer": sharded_layer, "prefill": prefill, "decode": decode, "decode_70b": decode_70b, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "parity_check": parity_check, "timing": spread,
            "exchange": exchange,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing NCCL down under captured graphs: everything measured is printed, all ranks are in step
        graph = None
        torch.cuda.synchronize(device)
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


PREFILL_SHAPES = [("Q4_K", 4096, 4096), ("Q4_K", 11008, 4096), ("Q6_K", 4096, 11008), ("Q6_K", 32000, 4096)]  # BASELINE.json configs[2]
PREFILL_M = 512


def prefill_leg(torch, device, L, _lib):
    """Mixed-format prefill GEMM (M = 512 bf16 activations) through jq_linear_bf16: TFLOP/s per shape."""
    from jitnn_b200 import Tensor, synth
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        which = "measured sustained"
    except Exception:
        peak, which = 1400.0, "fallback"
    out = {"m": PREFILL_M, "peak_tflops": peak, "peak_source": "of " + which, "shapes": {}}
    stream = torch.cuda.current_stream(device)
    sp = ctypes.c_void_p(stream.cuda_stream)
    for t, n, k in PREFILL_SHAPES:
        g = torch.Generator(device=device).manual_seed(n + k)
        wf = torch.randn(n, k, generator=g, device=device) * 0.02
        raw = synth.QUANTIZERS[t](wf).cpu().numpy()
        del wf
        w = Tensor.quantized(t, raw, n, k, device=device.index)
        x = torch.randn(PREFILL_M, k, generator=g, device=device).to(torch.bfloat16)
        y = torch.empty(PREFILL_M, n, device=device)
        for _ in range(3):
            _lib.check(L.jq_linear_bf16(w._handle(), x.data_ptr(), PREFILL_M, None, y.data_ptr(), 1, sp))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        reps = 20
        a.record(stream)
        for _ in range(reps):
            _lib.check(L.jq_linear_bf16(w._handle(), x.data_ptr(), PREFILL_M, None, y.data_ptr(), 1, sp))
        b.record(stream)
        torch.cuda.synchronize(device)
        us = a.elapsed_time(b) * 1e3 / reps
        tf = 2.0 * PREFILL_M * n * k / us / 1e6
        out["shapes"]["%s_%dx%d" % (t, n, k)] = {"us": round(us, 2), "TFLOPs": round(tf, 1), "frac": round(tf / peak, 4)}
        w.release()
    return out


FORMAT_CASES = [("Q8_0", 4096, 4096), ("Q8_0", 32000, 4096), ("Q4_0", 32000, 4096), ("Q4_1", 32000, 4096), ("Q5_K", 32000, 4096),
                ("Q6_K", 4096, 11008), ("Q6_K", 32000, 4096)]
FORMAT_BPW = {"Q8_0": 34 / 32, "Q4_0": 18 / 32, "Q4_1": 20 / 32, "Q4_K": 144 / 256, "Q5_K": 176 / 256, "Q6_K": 210 / 256}


def formats_leg(torch, device, L, _lib, reps=25):
    """The decode GEMV of the other formats of the path at M = 1, 8 and 16: BASELINE.json configs[0] (Q8_0, 4096x4096, weights
    from the reference's host quantiser as restated in jq_quantize_q8_0) and one large layer per format. Four copies of every
    weight in rotation (so that no launch finds its weight in L2), replayed from a CUDA graph; GB/s over the algorithmic
    bytes N K bytes-per-weight + 4 M K + 4 M N against the measured HBM copy peak. The top-level figures of a case are those
    of M = 1; `m8` and `m16` sit beside them (a format whose kernel takes fewer rows per pass reads its weights several times)."""
    import jitnn_b200
    from jitnn_b200 import Tensor, synth
    peak, which = measured_peaks()
    out = {"m": [1, 8, 16], "peak_GBps": peak, "peak_source": "of " + which, "cases": {}}
    side = torch.cuda.Stream(device)
    for t, n, k in FORMAT_CASES:
        g = torch.Generator(device=device).manual_seed(n + 3 * k + len(t))
        ws = []
        for c in range(POOL_COPIES):
            wf = torch.randn(n, k, generator=g, device=device) * 0.02
            raw = (jitnn_b200.Quant.quantizeQ8Blocks(wf, device.index) if t == "Q8_0" else synth.QUANTIZERS[t](wf)).cpu().numpy()
            del wf
            ws.append(Tensor.quantized(t, raw, n, k, device=device.index))
        case = {}
        for m in (1, 8, 16):
            x = torch.randn(m, k, generator=g, device=device)
            y = torch.empty(m, n, device=device)
            with torch.cuda.stream(side):
                sp = ctypes.c_void_p(side.cuda_stream)

                def rot():
                    for w in ws:
                        _lib.check(L.jq_linear_f32(w._handle(), x.data_ptr(), m, None, y.data_ptr(), _lib.JQ_MEM_DEVICE, sp))
                rot()
                torch.cuda.synchronize(device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    rot()
                graph.replay()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize(device)
                a.record(side)
                for _ in range(reps):
                    graph.replay()
                b.record(side)
                torch.cuda.synchronize(device)
            us = a.elapsed_time(b) * 1e3 / (reps * POOL_COPIES)
            nbytes = n * k * FORMAT_BPW[t] + 4 * m * k + 4 * m * n
            gbps = nbytes / us / 1e3
            res = {"us": round(us, 2), "GBps": round(gbps, 1), "frac": round(gbps / peak, 4)}
            if m == 1:
                case.update(res)
            else:
                case["m%d" % m] = res
            del graph
        out["cases"]["%s_%dx%d" % (t, n, k)] = case
        for w in ws:
            w.release()
    return out


LAYER_70B = [("wq", 8192, 8192), ("wk", 1024, 8192), ("wv", 1024, 8192), ("wo", 8192, 8192), ("w1", 28672, 8192), ("w3", 28672, 8192),
             ("w2", 8192, 28672)]


def sharded_layer_leg(torch, device, rank, world, L, _lib):
    """The seven linears of one 70B-shape decoder layer (BASELINE.json configs[4]: d 8192, 64 / 8 heads, FFN 28672, all
    Q4_K), each split by output rows over the ranks and completed on every rank by the peer-store exchange, at batch 1
    and 16. Every rank quantises only its own rows of weights that are the same at every N (seeded by shape); two copies per weight in rotation; one
    CUDA graph per batch size holds two passes over the layer and is replayed. Reports microseconds per linear and per
    layer (max over ranks) and the layer's aggregate GB/s over the whole weights' bytes."""
    import torch.distributed as dist
    from jitnn_b200 import Tensor, sharded, synth
    out = {"world": world, "exchange": "peer stores in the GEMV epilogue (batch 1), scatter kernel (batch 16)" if world > 1 else "none", "batches": {}}
    weights, peers = {}, {}
    for name, n, k in LAYER_70B:
        lo, hi = sharded.row_range(n, rank, world)
        copies = []
        for c in range(2):
            g = torch.Generator(device=device).manual_seed(7000 + n + 3 * k + c)  # the same weight at every N: a rank takes its rows of it
            wf = torch.randn(n, k, generator=g, device=device) * 0.02
            raw = synth.quantize_q4_k(wf[lo:hi]).cpu().numpy()
            del wf
            copies.append(Tensor.quantized("Q4_K", raw, hi - lo, k, device=device.index))
        weights[name] = copies
    side = torch.cuda.Stream(device)
    for m in (1, 16):
        g = torch.Generator(device=device).manual_seed(70 + m)
        xs = {k: torch.randn(m, k, generator=g, device=device) for k in (8192, 28672)}
        ys = {name: torch.empty(m, weights[name][0].shape()[0], device=device) for name, _, _ in LAYER_70B}
        if world > 1:
            peers = {name: sharded.PeerGather(n, m, device=device.index) for name, n, _ in LAYER_70B}

        def one(name, k, c, sp):
            w = weights[name][c]
            if world > 1:
                peers[name].linear(w, xs[k])
            else:
                _lib.check(L.jq_linear_f32(w._handle(), xs[k].data_ptr(), m, None, ys[name].data_ptr(), _lib.JQ_MEM_DEVICE, sp))

        per = {}
        with torch.cuda.stream(side):
            sp = ctypes.c_void_p(side.cuda_stream)
            for c in range(2):  # warm-up: scratch buffers, peer tables
                for name, n, k in LAYER_70B:
                    one(name, k, c, sp)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for c in range(2):
                    for name, n, k in LAYER_70B:
                        one(name, k, c, sp)
            graph.replay()
            torch.cuda.synchronize(device)
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 50
            a.record(side)
            for _ in range(reps):
                graph.replay()
            b.record(side)
            torch.cuda.synchronize(device)
            t = torch.tensor([a.elapsed_time(b) * 1e3 / (2 * reps)], device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            layer_us = float(t.item())
        layer_bytes = sum(n * k * BYTES_PER_WEIGHT + 4 * m * k + 4 * m * n for _, n, k in LAYER_70B)
        out["batches"]["m%d" % m] = {"layer_us": round(layer_us, 2), "GBps": round(layer_bytes / layer_us / 1e3, 1),
                                      "us_per_linear": round(layer_us / len(LAYER_70B), 2)}
        del graph
        for p in peers.values():
            p.close()
        peers = {}
    for copies in weights.values():
        for w in copies:
            w.release()
    return out


def decode_70b_leg(torch, device, rank, world, shape=None):
    """BASELINE.json configs[4]: Llama-style decoder, 70B shape (80 layers, d 8192, 64 query / 8 key-value heads, FFN
    28672, vocab 32000, all linears Q4_K), split by output rows over the ranks (jitnn_b200.LlamaDecoder sharded: local
    heads, peer-store exchanges), a 256-token uniform-random prompt per sequence, then greedy decode at batch 16 (16
    sequences in lockstep) and at batch 1. Every rank quantises only its own rows; the 80 layers cycle through 4
    distinct seeded weight sets, each layer with a device copy of its own (the bytes streamed per token are those of 80
    distinct layers). Wall-clock per step around the call that returns the next tokens, max over ranks."""
    import numpy as np
    import torch.distributed as dist
    from jitnn_b200 import LlamaDecoder, synth
    layers, dim, heads, kv_heads, hidden, vocab, prompt_len, gen, seqs = 80, 8192, 64, 8, 28672, 32000, 256, 34, 16
    if shape:  # "layers,prompt,gen": a cut-down run for trials, not a bench number
        layers, prompt_len, gen = (int(v) for v in shape.split(","))
    kv_dim = kv_heads * (dim // heads)
    dec = LlamaDecoder(layers, dim, heads, kv_heads, hidden, vocab, max_seq=prompt_len + 2 * gen + 8, device=device.index, sharded=world > 1)
    dec.set_sequences(seqs)
    names = [("wq", dim, dim), ("wk", kv_dim, dim), ("wv", kv_dim, dim), ("wo", dim, dim), ("w1", hidden, dim), ("w3", hidden, dim), ("w2", dim, hidden)]

    def rows(n, k, seed):
        # the model is the same at every N (seeded by weight, not by rank): a rank quantises its rows of it
        g = torch.Generator(device=device).manual_seed(seed)
        wf = torch.randn(n, k, generator=g, device=device) * 0.02
        per = n // world
        return ("Q4_K", synth.quantize_q4_k(wf[rank * per:(rank + 1) * per]).cpu().numpy().reshape(-1), per, k)

    parity = sharded_decoder_check(torch, device, rank, world) if world > 1 else None
    sets = [{name: rows(n, k, 9000 + 100 * c + 10 * i) for i, (name, n, k) in enumerate(names)} for c in range(min(4, layers))]
    ones = np.ones(dim, np.float32)
    for l in range(layers):
        w = {"layers.%d.%s" % (l, name): sets[l % len(sets)][name] for name, _, _ in names}
        dec.load(w, local=True)
        dec.load({"layers.%d.attention_norm" % l: ones, "layers.%d.ffn_norm" % l: ones})
    dec.load({"output": rows(vocab, dim, 9900)}, local=True)
    g = torch.Generator(device=device).manual_seed(2025)  # the same table on every rank
    dec.load({"norm": ones, "tok_embeddings": (torch.randn(vocab, dim, generator=g, device=device) * 0.02).cpu().numpy()})
    del sets
    weight_bytes = (layers * sum(n * k for _, n, k in names) + vocab * dim) * BYTES_PER_WEIGHT
    prompts = np.random.default_rng(13).integers(0, vocab, (seqs, prompt_len)).astype(np.int32)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    first = np.zeros(seqs, np.int32)
    for b in range(seqs):
        for i in range(0, prompt_len - 16, 16):
            dec.enqueue(prompts[b, i:i + 16], i, seq=b)
        _, nxt = dec.forward(prompts[b, prompt_len - 16:], prompt_len - 16, want_logits=False, seq=b)
        first[b] = nxt[-1]
    t_prompt = time.perf_counter() - t0

    def timed(step_fn, toks, pos):
        out = []
        for _ in range(2):  # untimed: the first runs eagerly, the second captures the step into a CUDA graph
            toks = step_fn(toks, pos)
            pos += 1
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(gen - 2):
            toks = step_fn(toks, pos)
            out.append(int(toks[0]))
            pos += 1
        dt = torch.tensor([(time.perf_counter() - t0) / (gen - 2)], device=device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return float(dt.item()), toks, pos, out

    dt16, toks, pos, out16 = timed(lambda t, p: dec.forward_batch(t, p, want_logits=False)[1], first, prompt_len)
    dt1, _, _, out1 = timed(lambda t, p: dec.forward([int(t[0])], p, want_logits=False)[1], toks[:1], pos)
    dec.close()
    peak, which = measured_peaks()
    kv1 = 2 * layers * (prompt_len + gen + gen // 2) * kv_dim * 4
    kv16 = 16 * 2 * layers * (prompt_len + gen // 2) * kv_dim * 4
    return {"world": world,
            "batch1": {"tokens_per_s": round(1.0 / dt1, 1), "ms_per_token": round(dt1 * 1e3, 4),
                       "hbm_roofline_tokens_per_s": round(world * peak * 1e9 / (weight_bytes + kv1), 1),
                       "frac": round((weight_bytes + kv1) / world / dt1 / 1e9 / peak, 4)},
            "batch16": {"tokens_per_s": round(16.0 / dt16, 1), "ms_per_step": round(dt16 * 1e3, 4),
                        "hbm_roofline_tokens_per_s": round(16 * world * peak * 1e9 / (weight_bytes + kv16), 1),
                        "frac": round((weight_bytes + kv16) / world / dt16 / 1e9 / peak, 4)},
            "prompt_tokens_per_s": round(seqs * prompt_len / t_prompt, 1), "weight_bytes_per_token": int(weight_bytes), "peak_source": "of " + which,
            "config": "70B shape, %d layers, all Q4_K, rows split over %d GPU(s), 16 prompts of %d tokens in groups of 16, %d timed greedy steps "
                      "per batch size, fp32 KV cache; batch 1: the fused single-token step (8 launches per layer; with several GPUs the attention and "
                      "SwiGLU kernels store the next linear's activation image into every rank, wo / w2 store their rows into every rank's "
                      "vector, the consumers wait for the flags themselves); batch 16: general kernels, the linears of enough weight rows on the tcgen05 "
                      "GEMV (16 rows of x in one pass), the others in two passes of 8; both replayed as CUDA graphs" % (layers, world, prompt_len, gen - 2),
            "first_tokens": {"batch16_seq0": out16[:6], "batch1": out1[:6]}, "parity_check": parity}


def sharded_decoder_check(torch, device, rank, world):
    """Before the timed run at N > 1: a two-layer decoder of the 70B layer shape (d 8192, 64 / 8 heads, FFN 28672, vocab 32000,
    all Q4_K, seeded) split over the ranks against the same decoder on this rank's GPU alone, on the general kernels
    (option decoder_fused = 0), where both do the same arithmetic per output row: logits and greedy tokens of a prompt of 12
    tokens must agree within 2e-5, those of the same tokens in calls of at most eight and of 3 single-token steps bitwise, on every rank."""
    import numpy as np
    import torch.distributed as dist
    import jitnn_b200
    from jitnn_b200 import LlamaDecoder, synth
    layers, dim, heads, kv_heads, hidden, vocab = 2, 8192, 64, 8, 28672, 32000
    kv_dim = kv_heads * (dim // heads)
    L = jitnn_b200.load()
    L.jq_set_option(b"decoder_fused", 0)
    whole = LlamaDecoder(layers, dim, heads, kv_heads, hidden, vocab, max_seq=32, device=device.index)
    split = LlamaDecoder(layers, dim, heads, kv_heads, hidden, vocab, max_seq=32, device=device.index, sharded=True)
    g = torch.Generator(device=device).manual_seed(4242)
    ones = np.ones(dim, np.float32)
    for l in range(layers):
        for name, n, k in [("wq", dim, dim), ("wk", kv_dim, dim), ("wv", kv_dim, dim), ("wo", dim, dim), ("w1", hidden, dim), ("w3", hidden, dim), ("w2", dim, hidden)]:
            raw = synth.quantize_q4_k(torch.randn(n, k, generator=g, device=device) * 0.02).cpu().numpy().reshape(-1)
            for d in (whole, split):
                d.load({"layers.%d.%s" % (l, name): ("Q4_K", raw, n, k)})
        for d in (whole, split):
            d.load({"layers.%d.attention_norm" % l: ones, "layers.%d.ffn_norm" % l: ones})
    raw = synth.quantize_q4_k(torch.randn(vocab, dim, generator=g, device=device) * 0.02).cpu().numpy().reshape(-1)
    table = (torch.randn(vocab, dim, generator=g, device=device) * 0.02).cpu().numpy()
    for d in (whole, split):
        d.load({"output": ("Q4_K", raw, vocab, dim), "norm": ones, "tok_embeddings": table})
    prompt = np.random.default_rng(3).integers(0, vocab, 12).astype(np.int32)
    # twelve tokens in one call: from eleven rows on the kernel of a linear is chosen by its number of weight rows (the tcgen05
    # GEMV where they are many), so a shard may sum in another order than the whole weight: equal within 2e-5 of the largest logit
    a, na = whole.forward(prompt, 0)
    b, nb = split.forward(prompt, 0)
    ok = bool(np.abs(a - b).max() <= 2e-5 * np.abs(a).max())
    # the same tokens in calls of at most eight (one kernel whatever the rows): bitwise
    for lo, hi in ((0, 8), (8, 12)):
        a, na = whole.forward(prompt[lo:hi], lo)
        b, nb = split.forward(prompt[lo:hi], lo)
        ok = ok and bool(np.array_equal(a, b) and np.array_equal(na, nb))
    tok, pos = int(na[-1]), 12
    for _ in range(3):
        a, na = whole.forward([tok], pos)
        b, nb = split.forward([tok], pos)
        ok = ok and bool(np.array_equal(a, b)) and int(na[0]) == int(nb[0])
        tok, pos = int(na[0]), pos + 1
    whole.close()
    split.close()
    L.jq_set_option(b"decoder_fused", 1)
    t = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    all_ok = bool(int(t.item()))
    assert all_ok, "the row-sharded decoder differs from the single-GPU decoder"
    return {"against": "the same 2-layer 70B-shape decoder on one GPU, general kernels", "bitwise_equal": all_ok, "ranks_checked": world,
            "tokens": 12 + 3, "note": "bitwise: the 12 tokens in calls of 8 and 4, and 3 single-token steps; the 12 tokens in one call within 2e-5"}


def decode_leg(torch, device, shape=None):
    """BASELINE.json configs[3]: Llama-style decoder, 7B shape (32 layers, d 4096, 32 heads, FFN 11008, vocab 32000),
    seeded N(0, 0.02) weights quantised Q4_K_M-style (Q6_K for wv, w2 and the output projection, Q4_K elsewhere),
    512 uniform-random prompt tokens, then 128 greedy tokens at batch 1. Reports decode tokens/s."""
    import numpy as np
    from jitnn_b200 import LlamaDecoder, synth
    layers, dim, heads, hidden, vocab, prompt_len, gen = 32, 4096, 32, 11008, 32000, 512, 128
    if shape:  # "layers,prompt,gen": a cut-down run for profiler captures, not a bench number
        layers, prompt_len, gen = (int(v) for v in shape.split(","))
    dec = LlamaDecoder(layers, dim, heads, heads, hidden, vocab, max_seq=prompt_len + gen + 8, device=device.index)
    g = torch.Generator(device=device).manual_seed(2024)

    def lin(n, k, t):
        wf = torch.randn(n, k, generator=g, device=device) * 0.02
        return (t, synth.QUANTIZERS[t](wf).cpu().numpy().reshape(-1), n, k)

    weight_bytes = 0
    bpw = {"Q4_K": 144 / 256, "Q6_K": 210 / 256}
    for l in range(layers):
        w = {}
        p = "layers.%d." % l
        for name, n, k, t in [("wq", dim, dim, "Q4_K"), ("wk", dim, dim, "Q4_K"), ("wv", dim, dim, "Q6_K"), ("wo", dim, dim, "Q4_K"),
                              ("w1", hidden, dim, "Q4_K"), ("w3", hidden, dim, "Q4_K"), ("w2", dim, hidden, "Q6_K")]:
            w[p + name] = lin(n, k, t)
            weight_bytes += n * k * bpw[t]
        w[p + "attention_norm"] = np.ones(dim, np.float32)
        w[p + "ffn_norm"] = np.ones(dim, np.float32)
        dec.load(w)
    dec.load({"output": lin(vocab, dim, "Q6_K"), "norm": np.ones(dim, np.float32),
              "tok_embeddings": (torch.randn(vocab, dim, generator=g, device=device) * 0.02).cpu().numpy()})
    weight_bytes += vocab * dim * bpw["Q6_K"]
    prompt = np.random.default_rng(11).integers(0, vocab, prompt_len).astype(np.int32)
    torch.cuda.synchronize(device)
    # the prompt twice: in one pass over the weights on the tensor-core path (bfloat16 operands; the first call also allocates
    # its workspace, so it is run once untimed), then in groups of 8 on the FP32 path, whose cache the greedy steps go on from
    dec.prompt(prompt, 0, want_logits=False)
    t0 = time.perf_counter()
    _, nxt_bf16 = dec.prompt(prompt, 0, want_logits=False)
    t_prompt_bf16 = time.perf_counter() - t0
    t0 = time.perf_counter()
    for i in range(0, prompt_len - 8, 8):
        dec.enqueue(prompt[i:i + 8], i)
    _, nxt = dec.forward(prompt[prompt_len - 8:], prompt_len - 8, want_logits=False)
    t_prompt = time.perf_counter() - t0
    tok = int(nxt[-1])
    out = []
    # two untimed steps: the first runs eagerly, the second captures the decode step into a CUDA graph
    pos = prompt_len
    for _ in range(2):
        _, nxt = dec.forward([tok], pos, want_logits=False)
        tok = int(nxt[0])
        out.append(tok)
        pos += 1
    t0 = time.perf_counter()
    for _ in range(gen - 2):
        _, nxt = dec.forward([tok], pos, want_logits=False)
        tok = int(nxt[0])
        out.append(tok)
        pos += 1
    dt = (time.perf_counter() - t0) / (gen - 2)
    dec.close()
    peak, which = measured_peaks()
    kv_bytes = 2 * layers * (prompt_len + gen // 2) * dim * 4
    return {"tokens_per_s": round(1.0 / dt, 1), "ms_per_token": round(dt * 1e3, 4), "prompt_tokens_per_s": round(prompt_len / t_prompt, 1),
            "prompt_tokens_per_s_tensor_core": round(prompt_len / t_prompt_bf16, 1),
            "prompt_note": "prompt_tokens_per_s: FP32 operands, groups of 8 tokens through the decode kernels; ..._tensor_core: jq_decoder_prompt, the whole "
                           "prompt in one pass, linears on the tcgen05 prefill kernel with bfloat16 operands (next token %s the FP32 path's)"
                           % ("equals" if int(nxt_bf16) == int(nxt[-1]) else "differs from"),
            "weight_bytes_per_token": int(weight_bytes), "kv_cache_bytes_per_token": int(kv_bytes),
            "hbm_roofline_tokens_per_s": round(peak * 1e9 / (weight_bytes + kv_bytes), 1),
            "frac": round((weight_bytes + kv_bytes) / dt / 1e9 / peak, 4), "peak_source": "of " + which,
            "config": "7B shape, 32 layers, Q4_K + Q6_K (wv, w2, output), prompt 512 in groups of 8, 128 greedy tokens, fp32 KV cache",
            "first_tokens": out[:8]}


def host_cores():
    """Cores this process may run on, whatever OMP_NUM_THREADS says."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline_leg(threads, fraction, steps=1, warmup=0):
    """Times the CPU port of the reference's host loops on the sweep (rows [0, N/fraction) of every shape)."""
    import numpy as np
    import torch
    from jitnn_b200 import synth
    from oracle import oracle
    work = []
    total_bytes = 0.0
    for si, (n, k) in enumerate(SHAPES):
        rows = max(1, n // fraction)
        g = torch.Generator().manual_seed(1234 + 17 * si)
        raw = synth.quantize_q4_k(torch.randn(rows, k, generator=g) * 0.02).numpy()
        for m in BATCHES:
            x = torch.randn(m, k, generator=g).numpy()
            work.append((raw, x, rows))
            total_bytes += algorithmic_bytes(rows, k, m)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for raw, x, rows in work:
            oracle.linear(TYPE, raw, x, None, n=rows, threads=threads)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    return {"value": round(total_bytes / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "%d step(s) of the sweep on rows [0, N/%d) of every shape, %.2f s per step" % (steps, fraction, dt),
            "seconds_per_step": round(dt, 3)}


def run_reference(args):
    """The reference's CPU implementation of the path: its scalar host loops (ops/Gguf.java:187-205),
    restated in C (oracle/) because no JVM exists here, on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_cores()  # explicit: the launcher's OMP_NUM_THREADS does not decide this
    # size the per-step sample so that the whole run stays within about two minutes: time rows [0, N/64) once,
    # then take the largest power-of-two share of the rows that fits
    probe = cpu_baseline_leg(threads=threads, fraction=64, steps=1, warmup=0)
    total_steps = args.steps + min(args.warmup, 1)
    fraction = 1
    while fraction < 64 and probe["seconds_per_step"] * 64 / fraction * total_steps > 100.0:
        fraction *= 2
    cpu = cpu_baseline_leg(threads=threads, fraction=fraction, steps=args.steps, warmup=min(args.warmup, 1))
    one = cpu_baseline_leg(threads=1, fraction=64, steps=1, warmup=0)
    cpu["one_thread"] = {"value": one["value"], "unit": "GB/s", "cores": 1, "sample": one["sample"],
                         "note": "the reference's CPU backend as shipped runs these operators on one thread (engine/CpuExecutor.java:233-239)"}
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(cpu["seconds_per_step"] * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "weights": "seeded N(0,0.02) quantised to Q4_K, x ~ N(0,1) fp32",
                   "sample": "rows [0, N/%d) of every shape per step, %d host threads" % (fraction, threads)},
        "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the one-thread CPU baseline leg")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl", "none"],
                    help="N > 1: how every rank gets the whole y after each sharded linear (the library's peer-store exchange, or NCCL; none = no exchange, for diagnosis only)")
    ap.add_argument("--leg", default="all", choices=["all", "prefill", "decode", "formats", "decode70b"],
                    help="run only the prefill GEMM leg, the format table, the 7B-shape decode leg (one GPU; for profiler captures) or the sharded 70B-shape decoder leg (any N)")
    ap.add_argument("--no-decode", action="store_true", help="skip the decoder tokens/s legs (7B shape on one GPU, 70B shape row-sharded at any N)")
    ap.add_argument("--decode-shape", default=None, metavar="LAYERS,PROMPT,GEN",
                    help="with --leg decode: fewer layers / a shorter prompt and run, for profiler captures")
    ap.add_argument("--eager", action="store_true", help="issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--only", default=None, metavar="NxKxM",
                    help="restrict the sweep to one shape and batch, e.g. 32000x4096x1 (a small case for profiler captures)")
    args = ap.parse_args()
    if args.only:
        n, k, m = (int(v) for v in args.only.lower().split("x"))
        SHAPES[:] = [(n, k)]
        BATCHES[:] = [m]
        args.no_cpu = True
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
