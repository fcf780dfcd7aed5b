#!/usr/bin/env python
"""Benchmark of the NVFP4 decode GEMV path: achieved HBM GB/s of the batch-1 weight-only linear.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (the decode GEMV shape sweep at M=1): the four shapes
(K,N) in {(4096,6144),(4096,4096),(4096,28672),(14336,4096)}, x bf16 ~ N(0,1), weights bf16 ~ N(0,0.02)
quantized to NVFP4 (global 448*6/amax).  One graph replay = one pass over `copies` distinct weight sets
of all four shapes (~3.9 GB of weights, far larger than the 126 MB L2: every launch reads cold
weights).  One STEP = `replays_per_step` replays, chosen once so that a step lasts ~0.1 s and the timed
region of K steps is long enough for the clock sampler to see it.  value = algorithmic bytes of the
step / device time, where bytes(M,N,K) = N*K/2 + N*K/16 + 2*M*K + 2*M*N + 4.

At N > 1 the same matrices are sharded tensor-parallel over the ranks (strong scaling): the QKV and
gate+up shapes column-parallel (rows split, output left sharded for the consumer), the o_proj and
down shapes row-parallel (K split, all-reduce of the partial y with NCCL, or over peer memory with
--collective peer), one process per GPU.

`--impl reference` times the reference's CPU path for the same linears (weights dequantized to
bf16 once, then bf16 x bf16 -> f32 -> bf16, all host cores) through the CPU oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

SHAPES_KN = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)]  # (K, N)
ROW_PARALLEL = {(4096, 4096), (14336, 4096)}  # o_proj / down: split along K at N > 1, all-reduce of y;
# the other two (QKV, gate+up) split along N and their outputs stay sharded into the consumer
COPIES = 32            # distinct weight sets per shape in one graph replay
STEP_TARGET_S = 0.1    # a step is as many replays as make it last about this long
METRIC = "nvfp4_decode_gemv_hbm_gbs"
# sizes of the two layer-stack legs (hidden, q width, kv width, FFN, vocabulary; experts, expert FFN, top-k)
STACK_DIMS = {"H": 5120, "QO": 8192, "KV": 1024, "F": 25600, "V": 151936, "layers": 64}
MOE_DIMS = {"E": 128, "H": 2048, "F": 768, "TOPK": 8, "layers": 48}


def algo_bytes(m: int, n: int, k: int) -> int:
    return n * k // 2 + n * k // 16 + 2 * m * k + 2 * m * n + 4


def step_bytes(copies: int) -> int:
    return copies * sum(algo_bytes(1, n, k) for k, n in SHAPES_KN)


# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs.  Every sample carries
    nvidia-smi's own timestamp; `stop(t0, t1)` keeps the samples taken between the two host times."""

    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int, period_ms: int = 100):
        self.idx, self.period_ms = gpu_index, period_ms
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    @classmethod
    def parse(cls, text: str, t0=None, t1=None) -> dict:
        """Summary of nvidia-smi's CSV lines; with t0/t1 (datetime) only the samples between them count."""
        import datetime
        sm, mx, power, reasons, total = [], [], [], set(), 0
        for line in text.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 10:
                continue
            try:
                when = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                clk, cmax = float(f[2]), float(f[3])
            except ValueError:
                continue
            total += 1
            if t0 is not None and not (t0 <= when <= t1):
                continue
            sm.append(clk)
            mx.append(cmax)
            try:
                power.append(float(f[4]))
            except ValueError:
                pass
            for name, v in zip(cls.NAMES, f[6:10]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples_in_region": len(sm), "samples_total": total,
                "reasons": sorted(reasons)}

    def stop(self, t0=None, t1=None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples_in_region": 0, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        return self.parse(out, t0, t1)


# ------------------------------------------------------------------------------------------------
def run_b200(args) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    import speaches_plus_b200 as sp
    from speaches_plus_b200 import tp as tpmod

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    def mark(msg):
        if os.environ.get("NVK_BENCH_VERBOSE"):
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    if world > 1:
        tpmod.init_process_group_for_node(dev)  # NVLS off, see tp.init_process_group_for_node
    sp.ffi.lib()
    mark("process group up")

    peer_ar = None
    if world > 1 and args.collective == "peer":
        try:
            peer_ar = tpmod.PeerAllReduce(None, 64 * 5120, dev)
            mark("peer all-reduce ready")
        except RuntimeError as e:  # raised on every rank together; the sums then go through NCCL
            args.collective = f"nccl ({e})"
            mark(str(e))

    peer_fused = None
    if world > 1 and args.collective == "fused":
        try:
            peer_fused = tpmod.PeerFusedLinear(None, dev)
            mark("fused linear + all-reduce ready")
        except RuntimeError as e:
            args.collective = f"nccl ({e})"
            mark(str(e))

    # ---- synthetic weights: seeded, identical on every rank, then sharded ----
    copies = COPIES
    layers = []  # (K, N, [TpLinear per copy])
    for si, (k, n) in enumerate(SHAPES_KN):
        mode = "row" if (k, n) in ROW_PARALLEL else "column"
        per_copy = []
        for c in range(copies):
            gen = torch.Generator(device=dev).manual_seed(1000 * si + c)
            w = (torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            lin = tpmod.TpNvfp4Linear.from_bf16(w, mode, rank, world)
            lin.peer_ar = peer_ar
            lin.peer_fused = peer_fused
            per_copy.append(lin)
            del w
        layers.append((k, n, per_copy))
    gen = torch.Generator(device=dev).manual_seed(7)
    xs = {k: torch.randn((1, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
          for k in {k for k, _ in SHAPES_KN}}
    torch.cuda.synchronize()

    def one_step():
        for k, n, per_copy in layers:
            x = xs[k]
            for lin in per_copy:
                lin.forward(x, gather=False)

    launches_per_replay = copies * len(SHAPES_KN)
    n_row_parallel = sum(1 for k, n in SHAPES_KN if (k, n) in ROW_PARALLEL)
    mark("weights ready")

    # ---- device-resident timing: one pass captured as a CUDA graph, a step = `rps` replays ----
    import datetime
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):
            one_step()
        stream.synchronize()
        mark("eager warm-up done")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_step()
        mark("graph captured")
        # how many replays make a step of about STEP_TARGET_S (decided on rank 0, the same on every rank)
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(5):
            graph.replay()
        b.record(stream)
        stream.synchronize()
        rps_t = torch.tensor([max(1, min(400, int(round(STEP_TARGET_S / max(a.elapsed_time(b) / 5 * 1e-3, 1e-6)))))],
                             dtype=torch.int32, device=dev)
        if world > 1:
            dist.broadcast(rps_t, 0)
        rps = int(rps_t.item())
        warm = max(args.warmup, 3)
        for _ in range(warm):           # warm-up steps (>= 10 warm replays of every launch)
            for _ in range(rps):
                graph.replay()
        stream.synchronize()
        mark(f"graph warm-up done, {rps} replays per step")
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
            time.sleep(0.25)            # let the sampler produce its first line before the region opens
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        t_open = datetime.datetime.now()
        ev[0].record(stream)
        for i in range(args.steps):
            for _ in range(rps):
                graph.replay()
            ev[i + 1].record(stream)
        stream.synchronize()
        t_close = datetime.datetime.now()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop(t_open, t_close) if rank == 0 else None
        ms = ev[0].elapsed_time(ev[-1])
        step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
        mark("timed region done")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    total_bytes = step_bytes(copies) * rps
    launches_per_step = launches_per_replay * rps
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- time of each GEMV inside a graph replay, from GPU timestamps between the launches ----
    stamped = stamped_graph_leg(dev, stream, layers, xs) if world == 1 else None
    # ... and the same with every launch kept at one CTA per 128-row tile (no dealing of 16-row units over a
    # full-GPU grid): the pair shows what the dealt launch is worth on the shapes where it is chosen
    stamped_per_tile = None
    if world == 1:
        sp.ffi.check("nvk_b200_set_row_balance", 2)
        try:
            stamped_per_tile = stamped_graph_leg(dev, stream, layers, xs)
        finally:
            sp.ffi.check("nvk_b200_set_row_balance", 0)

    # ---- per-shape breakdown (each shape's copies timed as their own region) ----
    per_shape = {}
    with torch.cuda.stream(stream):
        for k, n, per_copy in layers:
            reps = 20
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # interleave with the other shapes' weights between repetitions to keep L2 cold
            times = []
            for _ in range(reps):
                for kk, nn, pc in layers:
                    if (kk, nn) != (k, n):
                        pc[0].forward(xs[kk])
                a.record(stream)
                for lin in per_copy:
                    lin.forward(xs[k])
                b.record(stream)
                stream.synchronize()
                times.append(a.elapsed_time(b) / len(per_copy))
            us = statistics.median(times) * 1e3
            per_shape[f"K{k}_N{n}"] = {"us_per_launch_eager": round(us, 3),
                                        "gbs": round(algo_bytes(1, n, k) / (us * 1e-6) / 1e9, 1)}

    mark("per-shape done")
    if peer_ar is not None:
        peer_ar.check()
    if peer_fused is not None:
        peer_fused.check()
    # ---- end to end through the public API with host buffers ----
    pin_x = {k: torch.randn((1, k), dtype=torch.float32).to(torch.bfloat16).pin_memory() for k in xs}
    pin_y = {(k, n): torch.empty((1, n), dtype=torch.bfloat16).pin_memory() for k, n in SHAPES_KN}
    dx = {k: torch.empty((1, k), dtype=torch.bfloat16, device=dev) for k in xs}
    h2d = sum(2 * k for k, n in SHAPES_KN) * copies     # per pass over the weight sets
    d2h = sum(2 * n for k, n in SHAPES_KN) * copies

    def e2e_step():
        for k, n, per_copy in layers:
            for lin in per_copy:
                dx[k].copy_(pin_x[k], non_blocking=True)
                y = lin.forward(dx[k])
                pin_y[(k, n)].copy_(y, non_blocking=True)

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_steps = max(3, min(args.steps, 20))
        a.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        b.record(stream)
        stream.synchronize()
        e2e_ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = step_bytes(copies) / (e2e_ms / e2e_steps * 1e-3) / 1e9   # an e2e step is ONE pass

    out = None
    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        peak, peak_src = 6650.0, "fallback"
        if pk.exists():
            peaks = json.loads(pk.read_text())
            peak, peak_src = float(peaks["hbm_gbs"]), "measured"
        per_gpu_gbs = value / world
        step_ms_sorted = sorted(step_ms)
        # kernels of this library inside the timed region: the GEMVs, plus one all-reduce kernel per
        # row-parallel GEMV when the sums go over peer memory
        own_collectives = copies * n_row_parallel * rps if (world > 1 and peer_ar is not None) else 0
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "e2m1*ue4m3 x bf16 -> f32",
            "data": "synthetic",
            "config": bench_config(world, args.collective if world > 1 else None),
            "step": {"passes_per_step": rps, "step_bytes": total_bytes, "launches_per_step": launches_per_step,
                     "timing": "CUDA events around every step; a step = passes_per_step replays of a CUDA graph of "
                               "one pass"},
            "step_ms": {"median": round(statistics.median(step_ms), 4), "best": round(step_ms_sorted[0], 4),
                        "worst": round(step_ms_sorted[-1], 4),
                        "gbs_median": round(total_bytes / (statistics.median(step_ms) * 1e-3) / 1e9 / 1, 1),
                        "gbs_best": round(total_bytes / (step_ms_sorted[0] * 1e-3) / 1e9, 1),
                        "timed_replays_of_every_launch": rps * args.steps, "note": "rank 0's own steps"},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "path": "Nvfp4Linear.forward per GEMV: pinned x -> device, launch, y -> pinned host; an e2e "
                            "step is one pass over the weight sets"},
            "e2e_check": {"copies_declared": True, "h2d_copies_per_step": launches_per_replay,
                          "d2h_copies_per_step": launches_per_replay},
            "gpu_launches": (launches_per_step + own_collectives) * args.steps,
            "roofline": {"bound": "hbm", "achieved": round(per_gpu_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu_gbs / peak, 4), "peak_source": peak_src,
                         "frac_of_nominal_8TBs": round(per_gpu_gbs / 8000.0, 4),
                         # DRAM read+write bytes per launch: the ncu capture of the K=4096, N=28672 case
                         # (profiles/) measured 1.012 x the algorithmic bytes; scaled to the average launch.
                         # Per GPU: each rank's launch streams 1/world of the matrix.
                         "traffic": int(1.012 * (total_bytes // launches_per_step // world)),
                         "traffic_source": "ncu dram__bytes_read+write on K4096_N28672_M1, scaled by bytes",
                         "kernel": "w4a16_mma_kernel",
                         "bytes_per_launch_avg": total_bytes // launches_per_step // world,
                         "us_per_launch_avg": round(ms_per_step * 1e3 / launches_per_step, 3)},
            "per_shape": per_shape,
            "per_shape_in_graph": stamped,
            "per_shape_in_graph_one_cta_per_tile": stamped_per_tile,
            "clocks": clocks,
        }
        if args.cpu_baseline:
            out["cpu_baseline"] = cpu_reference_leg(passes=15, warm=2)
    if args.persistent and world == 1 and out is not None:
        out["persistent_step"] = persistent_step_leg(dev, layers, xs, max(args.steps, 5))
    if args.extras:
        # free the sweep's weights before the larger workloads
        del graph
        layers.clear()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        stack = [decode_stack_leg(dev, rank, world, b, peer_ar=peer_ar, peer_fused=peer_fused) for b in (1, 16)]
        peer_combine = None
        if world > 1 and args.collective == "fused":
            try:
                peer_combine = tpmod.PeerMoeCombine(None, dev)
            except RuntimeError as e:
                mark(str(e))
        moe = [moe_decode_leg(dev, b, rank=rank, world=world, peer_combine=peer_combine) for b in (1, 16, 64)]
        if peer_combine is not None:
            peer_combine.check()
            peer_combine.close()
        pre = None
        if world == 1:
            pre = (prefill_leg(dev) if sp.ffi.prefill_available()
                   else "unavailable: libnvk_b200_prefill.so is not part of this run")
        if out is not None:
            out["decode_stack"] = stack
            if moe is not None:
                out["moe_decode"] = moe
            if pre is not None:
                out["prefill_gemm"] = pre
        graph = None
    mark("results ready")
    if out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        # Tear down in dependency order: captured graphs (they hold collective work) first, then the
        # peer mappings, then the process group.
        graph = None
        if peer_ar is not None:
            peer_ar.close()
        if peer_fused is not None:
            peer_fused.close()
        clean = tpmod.shutdown_process_group()
        mark(f"process group destroyed: {clean}")
        sys.stdout.flush()
        sys.stderr.flush()
        if not clean:
            os._exit(0)  # every rank is past the final barrier; nothing of ours is mapped any more
    return None


# ------------------------------------------------------------------------------------------------
def bench_config(world: int, collective) -> dict:
    """The workload both arms are run on (the reference arm samples it; see its `cpu_baseline.sample`).
    The two arms print the same dict."""
    return {"workload": "NVFP4 decode GEMV shape sweep, M=1 (x bf16 [1,K], W [N,K] NVFP4, y bf16, fp32 accumulate)",
            "shapes_KN": SHAPES_KN, "weight_copies_per_shape": COPIES,
            "launches_per_pass": COPIES * len(SHAPES_KN), "pass_bytes": step_bytes(COPIES),
            "parallelism": f"tp{world}" if world > 1 else "single", "collective": collective,
            "l2": f"inputs larger than L2: {step_bytes(COPIES) / 1e6:.0f} MB of cold weights per pass",
            "step": "as many passes as last about 0.1 s on the device that runs them (see `step`)"}


def stamped_graph_leg(dev, stream, layers, xs, copies_used: int = 8, reps: int = 9) -> dict:
    """Per-GEMV time INSIDE a graph replay: a second graph of the same launches with a GPU timestamp
    (nv_kernels_prof_timestamp, %globaltimer) before each one and after the last.  A stamp is a kernel
    of its own without programmatic dependent launch, so consecutive GEMVs do not overlap here as they
    do in the timed graph: these are serialised per-kernel times (their SHARES are what carries over)."""
    import torch

    import speaches_plus_b200 as sp
    seq = [(k, n, lin) for k, n, per_copy in layers for lin in per_copy[:copies_used]]
    stamps = torch.zeros(len(seq) + 1, dtype=torch.int64, device=dev)

    def body():
        s = torch.cuda.current_stream().cuda_stream
        for i, (k, n, lin) in enumerate(seq):
            sp.ffi.check("nv_kernels_prof_timestamp", s, stamps.data_ptr() + 8 * i)
            lin.forward(xs[k], gather=False)
        sp.ffi.check("nv_kernels_prof_timestamp", s, stamps.data_ptr() + 8 * len(seq))

    per = {}
    with torch.cuda.stream(stream):
        body()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            body()
        samples = {}
        for _ in range(reps):
            g.replay()
            stream.synchronize()
            t = stamps.cpu().numpy()
            for i, (k, n, _) in enumerate(seq):
                samples.setdefault((k, n), []).append(float(t[i + 1] - t[i]) * 1e-3)   # ns -> us
        total = sum(statistics.median(v) for v in samples.values())
        for (k, n), v in samples.items():
            us = statistics.median(v)
            per[f"K{k}_N{n}"] = {"us_per_launch": round(us, 3), "gbs": round(algo_bytes(1, n, k) / (us * 1e-6) / 1e9, 1),
                                 "share": round(us / total, 4)}
        del g
    per["note"] = "serialised (a timestamp kernel sits between launches); cold weights: distinct copies in sequence"
    return per


# ------------------------------------------------------------------------------------------------
def persistent_step_leg(dev, layers, xs, replays: int) -> dict:
    """The M=1 shape sweep as one persistent launch: the same GEMVs, each made to wait for the one
    before it (as consecutive linears of a decode step do), timed over graph replays."""
    import torch

    import speaches_plus_b200 as sp
    step = sp.DecodeStep(1, dev)
    dep, outs = -1, []
    for k, n, per_copy in layers:
        for lin in per_copy:
            y = torch.empty((1, n), dtype=torch.bfloat16, device=dev)
            outs.append(y)
            dep = step.add(lin.local, xs[k], y, dep=dep)
    step.build()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step.run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step.run()
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1) / replays
    step.check()
    n_ops = sum(len(pc) for _, _, pc in layers)
    nbytes = sum(algo_bytes(1, n, k) * len(pc) for k, n, pc in layers)
    out = {"launches_per_step": 1, "operations": n_ops, "ms_per_step": round(ms, 4),
           "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1), "us_per_gemv": round(ms * 1e3 / n_ops, 3),
           "grid": step._launch[0], "smem_bytes": step._launch[1]}
    del graph
    return out


# ------------------------------------------------------------------------------------------------
def decode_stack_leg(dev, rank: int, world: int, batch: int, replays: int = 5, peer_ar=None, peer_fused=None) -> dict:
    """Dense 64-layer decoder linear stack (hidden 5120, 64 q / 8 kv heads of 128, SwiGLU
    25600, bf16 lm_head 151936), random-init NVFP4 weights, one decode step of `batch` tokens through
    every linear.  Attention itself is outside the path: o_proj is fed the q slice of the QKV output.
    Tensor parallel: QKV and gate/up column-parallel (outputs stay sharded into the row-parallel
    consumer), o_proj and down row-parallel followed by an all-reduce, lm_head column-parallel +
    all-gather.  Each rank holds random weights of its shard's shape."""
    import torch
    import torch.distributed as dist

    import speaches_plus_b200 as sp
    ffi = sp.ffi
    H, QO, KV, F, V, layers = (STACK_DIMS[k] for k in ("H", "QO", "KV", "F", "V", "layers"))
    q_l, kv_l, f_l = QO // world, KV // world, F // world
    v_l = (V // world + 127) // 128 * 128 if world > 1 else V

    def rand_lin(n, k, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        w = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        lin = sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w)
        del w
        return lin

    stack = []
    for li in range(layers):
        b = 10 * li + 1000 * rank
        stack.append((rand_lin(q_l + 2 * kv_l, H, b), rand_lin(H, q_l, b + 1), rand_lin(f_l, H, b + 2),
                      rand_lin(f_l, H, b + 3), rand_lin(H, f_l, b + 4)))
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    lm_head = sp.Bf16Linear((torch.randn((v_l, H), generator=g, device=dev, dtype=torch.float32) * 0.02)
                            .to(torch.bfloat16))
    x0 = torch.randn((batch, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    bf = dict(dtype=torch.bfloat16, device=dev)
    qkv = torch.empty((batch, q_l + 2 * kv_l), **bf)
    q_in = torch.empty((batch, q_l), **bf)
    o_out, d_out = torch.empty((batch, H), **bf), torch.empty((batch, H), **bf)
    gate, up = torch.empty((batch, f_l), **bf), torch.empty((batch, f_l), **bf)
    logits_l = torch.empty((batch, v_l), **bf)
    logits = torch.empty((world * batch, v_l), **bf) if world > 1 else logits_l

    from speaches_plus_b200 import linear as L

    def lin_call(lin, lin_b, x, x2, y, y_b):
        L.linear_w4a16(lin, lin_b, x, x2, y, y_b, batch)

    def reduce_(t):
        if peer_ar is not None:
            peer_ar.all_reduce_(t)
        else:
            dist.all_reduce(t)

    def step():
        for (w_qkv, w_o, w_g, w_u, w_d) in stack:
            lin_call(w_qkv, None, x0, None, qkv, None)
            if batch == 1:
                q_view = qkv[:, :q_l]
            else:
                q_in.copy_(qkv[:, :q_l])
                q_view = q_in
            # row-parallel linears: the partials meet inside the linear's launch when that fits (<= 8 rows)
            if not (peer_fused is not None and peer_fused.linear_(w_o, q_view, o_out)):
                lin_call(w_o, None, q_view, None, o_out, None)
                if world > 1:
                    reduce_(o_out)
            lin_call(w_g, w_u, o_out, None, gate, up)
            if not (peer_fused is not None and peer_fused.linear_(w_d, gate, d_out, up=up)):
                lin_call(w_d, None, gate, up, d_out, None)
                if world > 1:
                    reduce_(d_out)
        lm_head.forward_into(d_out, logits_l)   # M = 1: the GEMV; M > 1: one pass over the matrix for all rows
        if world > 1:
            dist.all_gather_into_tensor(logits, logits_l)

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(2):
            graph.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1) / replays
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    per_layer = (algo_bytes(batch, q_l + 2 * kv_l, H) + algo_bytes(batch, H, q_l) + 2 * algo_bytes(batch, f_l, H)
                 + algo_bytes(batch, H, f_l))
    bytes_rank = layers * per_layer + 2 * v_l * H + batch * 2 * (v_l + H)
    out = {"batch": batch, "layers": layers, "tp": world, "ms_per_step": round(ms, 4),
           "tok_s": round(batch / (ms * 1e-3), 1), "bytes_per_step_per_gpu": bytes_rank,
           "gbs_per_gpu": round(bytes_rank / (ms * 1e-3) / 1e9, 1),
           "launches_per_step": layers * 4 + 1, "collectives_per_step": (2 * layers + 1) if world > 1 else 0}
    if world > 1 and peer_fused is not None and batch <= peer_fused.MAX_ROWS:
        # the row-parallel sums happen inside the linears' own launches; only the lm_head's gather is left
        out["collectives_per_step"] = 1
        out["row_parallel_sum"] = "inside the linear's launch"

    if world == 1 and batch == 1:
        # The same stack with both RMSNorms and both residual adds of every layer inside its four launches:
        # normed QKV -> o_proj + residual (+ 1/rms for the next norm) -> normed gate/up -> SiLU*up + down +
        # residual (+ 1/rms).  Same weights, same launch count, a little more arithmetic per launch.
        s_ = lambda: torch.cuda.current_stream().cuda_stream
        hid = x0.clone()
        pack = torch.zeros(3, dtype=torch.float32, device=dev)
        nw = torch.ones((2 * layers, H), **bf)
        eps = 1e-6

        def normed(lin_a, lin_b, x, w_row, rstd, y_a, y_b):
            ffi.check("nvk_b200_linear_nvfp4_w4a16_normed", s_(), lin_a.weight_u8.data_ptr(),
                      lin_a.weight_scales.data_ptr(), lin_b.weight_u8.data_ptr() if lin_b else None,
                      lin_b.weight_scales.data_ptr() if lin_b else None, x.data_ptr(), w_row.data_ptr(),
                      rstd.data_ptr() if rstd is not None else None, eps, y_a.data_ptr(),
                      y_b.data_ptr() if y_b is not None else None, lin_a.alpha_w4a16,
                      lin_b.alpha_w4a16 if lin_b else 0.0, 1, lin_a.out_features, lin_a.in_features)

        def residual_emit(lin, x, x2):
            ffi.check("nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit", s_(), lin.weight_u8.data_ptr(),
                      lin.weight_scales.data_ptr(), x.data_ptr(), x2.data_ptr() if x2 is not None else None,
                      hid.data_ptr(), hid.data_ptr(), lin.alpha_w4a16, pack.data_ptr(), eps, lin.out_features,
                      lin.in_features)

        def fused_step():
            for li, (w_qkv, w_o, w_g, w_u, w_d) in enumerate(stack):
                normed(w_qkv, None, hid, nw[2 * li], pack if li > 0 else None, qkv, None)
                residual_emit(w_o, qkv[:, :q_l], None)
                normed(w_g, w_u, hid, nw[2 * li + 1], pack, gate, up)
                residual_emit(w_d, gate, up)
            lm_head.forward_into(hid, logits_l)

        with torch.cuda.stream(stream):
            fused_step()
            stream.synchronize()
            fgraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(fgraph, stream=stream):
                fused_step()
            for _ in range(2):
                fgraph.replay()
            stream.synchronize()
            e0.record(stream)
            for _ in range(replays):
                fgraph.replay()
            e1.record(stream)
            stream.synchronize()
            fms = e0.elapsed_time(e1) / replays
            del fgraph
        out["with_norms_and_residuals_fused"] = {"ms_per_step": round(fms, 4), "tok_s": round(1.0 / (fms * 1e-3), 1),
                                                 "launches_per_step": layers * 4 + 1}
    del graph, stack, lm_head
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return out


def moe_decode_leg(dev, batch: int, replays: int = 5, rank: int = 0, world: int = 1, peer_combine=None) -> dict:
    """MoE expert decode: 48 layers x 128 experts (hidden 2048, SwiGLU 768), top-8 with
    softmax over the winners, router logits ~ N(0,1); one decode step of `batch` tokens through
    route -> sort -> grouped gate+up -> grouped down (SiLU prologue) -> combine in every layer.
    Algorithmic bytes count each distinct routed expert once per layer (from the actual routing).
    With world > 1 the experts are dealt out in blocks (16 per GPU at 8): every rank routes all
    tokens, runs the slots of its own experts and the f32 partial outputs are summed with one
    all-reduce per layer."""
    import numpy as np
    import torch

    import torch.distributed as dist

    import speaches_plus_b200 as sp
    from speaches_plus_b200 import linear as L
    ffi = sp.ffi
    E, H, F, TOPK, layers = (MOE_DIMS[k] for k in ("E", "H", "F", "TOPK", "layers"))

    def bank(n, k, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        w = (torch.randn((E * n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        amax = w.view(E, -1).abs().amax(1).float()
        globals_ = (torch.full_like(amax, 448.0 * 6.0) / amax).contiguous()
        packed = torch.empty((E * n, k // 2), dtype=torch.uint8, device=dev)
        scales = torch.zeros(L.swizzled_scale_bytes(E * n, k), dtype=torch.uint8, device=dev)
        ffi.check("nv_kernels_quantize_nvfp4_bf16_per_expert", torch.cuda.current_stream().cuda_stream, w.data_ptr(),
                  packed.data_ptr(), scales.data_ptr(), globals_.data_ptr(), n, E * n, k)
        return packed.view(E, n, k // 2), scales.view(E, -1), (1.0 / globals_).contiguous()

    mods = []
    for li in range(layers):
        w = sp.MoeGroupedWeights(bank(F, H, 3 * li), bank(F, H, 3 * li + 1), bank(H, F, 3 * li + 2), H, F, E)
        if world > 1:  # keep this rank's block of experts only
            v = w.shard_experts(rank, world)
            w = sp.MoeGroupedWeights(*[tuple(t.clone() for t in b) for b in (v.gate, v.up, v.down)], H, F,
                                     v.num_experts, v.first_expert, E)
            del v
        g = torch.Generator(device=dev).manual_seed(7000 + li)
        logits = torch.randn((batch, E), generator=g, device=dev, dtype=torch.float32)
        mods.append((w, logits))
    ctx = sp.GroupedDecodeContext(mods[0][0], max(batch, 1), TOPK, dev)
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((batch, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    distinct = 0
    for w, logits in mods:
        distinct += int(torch.unique(torch.topk(logits, TOPK, dim=1).indices).numel())

    def step():
        for w, logits in mods:
            sp.forward_grouped_decode(w, ctx, x, logits, peer_combine=peer_combine)

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(2):
            graph.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1) / replays
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # the same step with every expert's K range kept in one CTA per row tile (no cluster split of K): the pair
    # shows, per batch size, what the split is worth -- its rule looks at one expert's tiles only, so that a
    # slot's bits never depend on the batch, and is therefore the same at every batch size
    ms_unsplit = None
    if world == 1:
        sp.ffi.check("nvk_b200_set_tuning", 1, 0)
        try:
            with torch.cuda.stream(stream):
                step()
                stream.synchronize()
                graph1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph1, stream=stream):
                    step()
                for _ in range(2):
                    graph1.replay()
                stream.synchronize()
                e0.record(stream)
                for _ in range(replays):
                    graph1.replay()
                e1.record(stream)
                stream.synchronize()
                ms_unsplit = e0.elapsed_time(e1) / replays
                del graph1
        finally:
            sp.ffi.check("nvk_b200_set_tuning", 0, 0)
    per_expert = mods[0][0].per_expert_bytes()
    nbytes = distinct * per_expert
    out = {"batch": batch, "layers": layers, "experts": E, "top_k": TOPK, "ep": world, "ms_per_step": round(ms, 4),
           "ms_per_step_no_k_split": round(ms_unsplit, 4) if ms_unsplit is not None else None,
           "tok_s": round(batch / (ms * 1e-3), 1), "distinct_experts_per_layer": round(distinct / layers, 2),
           "bytes_per_step": nbytes, "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
           "launches_per_step": layers * (4 if world == 1 else 5), "collectives_per_step": layers if world > 1 else 0}
    del graph, mods, ctx
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return out


def prefill_leg(dev, m: int = 2048, reps: int = 10) -> dict:
    """Prefill block-scaled GEMM: M=2048 tokens through FFN up (K=5120, N=25600) and down (K=25600, N=5120),
    activations quantized online to NVFP4 (global 1.0), FP4 x FP4 tensor-core GEMM, bf16 out -- for both
    tiles of the prefill library (this is a single-GPU process, so the 2-SM tile may be selected).
    The tensor peak these are set against is MEASURED here: the same kernel on a problem that stays in
    L2 (4096^3, 48 MB of operands and output), best of several runs; the nominal 9 PFLOP/s is quoted
    beside it."""
    import torch

    import speaches_plus_b200 as sp

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def make(n, k, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        w = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        lin = sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w)
        del w
        return lin, g

    out = {"tiles": {}}
    for cfg, name in ((1, "1sm_128x128x256"), (2, "2sm_256x128x256_cluster2")):
        sp.ffi.check("nvk_b200_set_prefill_config", cfg)
        # proxy peak: L2-resident problem, GEMM alone (activations quantized beforehand)
        lin, g = make(4096, 4096, 1)
        xq = torch.randn((4096, 4096), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        a_packed, a_scales = sp.linear.quantize_nvfp4_bf16(xq, 1.0, m_padded=4096)
        y = torch.empty((4096, 4096), dtype=torch.bfloat16, device=dev)
        peak_ms = min(timed(lambda: lin._fp4_gemm(a_packed, a_scales, y, 4096), 20) for _ in range(3))
        peak_tf = 2.0 * 4096 ** 3 / (peak_ms * 1e-3) / 1e12
        del lin, xq, a_packed, a_scales, y
        rows = []
        for k, n in ((5120, 25600), (25600, 5120)):
            lin, g = make(n, k, k)
            x = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            ms_all = timed(lambda: lin.forward_prefill_into(x, y), reps)
            a_packed, a_scales = sp.linear.quantize_nvfp4_bf16(x, lin.input_stored_global, m_padded=m)
            ms_gemm = timed(lambda: lin._fp4_gemm(a_packed, a_scales, y, m), reps)
            flop = 2.0 * m * n * k
            tf = flop / (ms_gemm * 1e-3) / 1e12
            rows.append({"M": m, "K": k, "N": n, "ms_gemm": round(ms_gemm, 4), "ms_quantize_plus_gemm": round(ms_all, 4),
                         "tflops_gemm": round(tf, 1), "frac_of_measured_proxy_peak": round(tf / peak_tf, 4),
                         "frac_of_nominal_fp4_dense_9000": round(tf / 9000.0, 4)})
            del lin, x, y, a_packed, a_scales
            torch.cuda.empty_cache()
        out["tiles"][name] = {"proxy_peak_tflops_L2_resident_4096cubed": round(peak_tf, 1), "shapes": rows}
    sp.ffi.check("nvk_b200_set_prefill_config", 1)
    return out


# ------------------------------------------------------------------------------------------------
_CPU_CACHE = {}


def _cpu_weights():
    """bf16 weights of the four shapes as the reference's Cpu backend holds them: quantized to NVFP4,
    then dequantized to bf16 (done once, not timed)."""
    import numpy as np

    from oracle import ref
    if "w" not in _CPU_CACHE:
        ws = []
        for si, (k, n) in enumerate(SHAPES_KN):
            rng = np.random.default_rng(1000 * si)
            w = ref.f32_to_bf16((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)))
            packed, sw, alpha = ref.quantize_weight_bf16(w)
            ws.append((k, n, ref.dequantize_to_bf16(packed, sw, n, k, alpha)))
        rng = np.random.default_rng(7)
        xs = {k: ref.f32_to_bf16(rng.standard_normal((1, k), dtype=np.float32)) for k, _ in SHAPES_KN}
        _CPU_CACHE["w"] = (ws, xs)
    return _CPU_CACHE["w"]


def cpu_pass(scalar_one_core: bool = False) -> float:
    """One pass over the four shapes on the host cores; returns seconds.  The timed linear keeps 16
    partial sums per output, the order a SIMD matmul such as the reference's adds in, on every host
    thread; `scalar_one_core` times the sequential scalar dot of the reference's hand-written CPU GEMV
    on one thread instead."""
    from oracle import ref
    ws, xs = _cpu_weights()
    t0 = time.perf_counter()
    for k, n, w in ws:
        if scalar_one_core:
            ref.linear_cpu_backend(w, xs[k], threads=1)
        else:
            ref.linear_cpu_backend_lanes16(w, xs[k], threads=0)
    return time.perf_counter() - t0


def cpu_reference_leg(passes: int, warm: int) -> dict:
    from oracle import ref
    for _ in range(warm):
        cpu_pass()
    ts = [cpu_pass() for _ in range(passes)]
    t = statistics.median(ts)
    t1 = cpu_pass(scalar_one_core=True)
    b = sum(algo_bytes(1, n, k) for k, n in SHAPES_KN)
    return {"value": round(b / t / 1e9, 3), "unit": "GB/s", "cores": ref.num_threads(), "kind": "port",
            "sample": f"one weight set of each of the 4 shapes (M=1), median of {passes} passes; weights "
                      "dequantized to bf16 beforehand (untimed), as the reference's Cpu backend holds them; "
                      "16 partial sums per output (SIMD order), all host threads",
            "ms_per_pass": round(t * 1e3, 2),
            "scalar_one_core": {"value": round(b / t1 / 1e9, 3), "unit": "GB/s", "cores": 1,
                                "sample": "the same pass with the sequential scalar dot on one thread"}}


def run_reference(args) -> dict | None:
    """The reference's own CPU implementation of the path (the oracle's port of its Cpu-backend linear),
    all host threads, on the B200 arm's workload and config.  A step is a bounded SAMPLE of that
    arm's step -- one weight set of each shape instead of replays_per_step x COPIES of them -- and the
    metric (GB/s of algorithmic bytes) does not depend on how many sets a step covers."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from oracle import ref
    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        cpu_pass()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_pass()
    dt = (time.perf_counter() - t0) / steps
    b = sum(algo_bytes(1, n, k) for k, n in SHAPES_KN)
    v = round(b / dt / 1e9, 3)
    sample = ("each step = one weight set of each of the 4 shapes at M=1 (1/%d of one pass of the B200 arm), CPU oracle "
              "port of the reference's Cpu-backend linear (16 partial sums per output), all host threads" % COPIES)
    return {"impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16 x bf16 -> f32",
            "data": "synthetic",
            "config": bench_config(args.gpus, (args.collective if args.gpus > 1 else None)),
            "step": {"passes_per_step": 1.0 / COPIES, "step_bytes": b, "launches_per_step": 0,
                     "timing": "host clock around the steps"},
            "cpu_baseline": {"value": v, "unit": "GB/s", "cores": ref.num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def profile_case(spec: str, copies: int) -> None:
    """A few eager launches of one (K,N,M) case on cold weights: the small, self-ending workload that
    profiler captures are taken on (see profiles/)."""
    import torch

    import speaches_plus_b200 as sp
    from speaches_plus_b200 import linear as L
    k, n, m = (int(v) for v in spec.split(","))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    lins = []
    for c in range(copies):
        g = torch.Generator(device=dev).manual_seed(c)
        w = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        lins.append(sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w))
        del w
    x = torch.randn((m, k), device=dev, dtype=torch.float32).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    for _ in range(2):
        for lin in lins:
            lin.forward_into(x, y)
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": {"K": k, "N": n, "M": m, "copies": copies, "launches": 2 * copies,
                                       "bytes_per_launch": algo_bytes(m, n, k)}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="skip the decode-stack, MoE and prefill legs")
    ap.add_argument("--collective", default="nccl", choices=["peer", "nccl", "fused"],
                    help="row-parallel sum at --gpus > 1: NCCL (default; in-switch multicast off), this library's "
                         "one-shot all-reduce over CUDA-IPC peer memory, or the exchange fused into the linear's "
                         "own launch (peer stores from the GEMV's epilogue)")
    ap.add_argument("--profile-case", default=None, metavar="K,N,M",
                    help="run a few eager launches of one case and exit (for profiler captures)")
    ap.add_argument("--copies", type=int, default=4)
    ap.add_argument("--persistent", action="store_true",
                    help="also time the sweep as ONE persistent launch (DecodeStep); reported as 'persistent_step'")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case, args.copies)
        return
    if args.impl == "reference":
        out = run_reference(args)
        if out is not None:
            print(json.dumps(out), flush=True)
    else:
        if args.gpus > 1:
            args.cpu_baseline = False
        run_b200(args)  # prints its own line (before the multi-GPU teardown)


if __name__ == "__main__":
    main()
