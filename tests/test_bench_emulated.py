"""bench.py's B200 arm, run end to end on the host emulation with toy sizes: the control flow (graph
capture, steps of several passes, per-step events, in-graph timestamps, the end-to-end leg, the
decode-stack and MoE legs) and the JSON contract are exercised where no GPU is present.  The numbers
it prints mean nothing; on a GPU the same code runs unmodified at the real sizes."""
import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]

_SCRIPT = r"""
import sys, argparse
sys.path.insert(0, {root!r})
from tests.emu import torch_shim
torch_shim.install()
import bench
bench.SHAPES_KN = [(256, 384), (256, 256), (512, 128)]
bench.ROW_PARALLEL = {{(256, 256), (512, 128)}}
bench.COPIES = 2
bench.STEP_TARGET_S = 1e-4
bench.STACK_DIMS = {{"H": 256, "QO": 256, "KV": 128, "F": 512, "V": 1000, "layers": 2}}
bench.MOE_DIMS = {{"E": 16, "H": 256, "F": 128, "TOPK": 4, "layers": 2}}
bench.cpu_reference_leg = lambda passes, warm: {{"value": 1.0, "unit": "GB/s", "cores": 1, "kind": "port", "sample": "stub"}}
args = argparse.Namespace(gpus=1, steps=3, warmup=3, impl="b200", cpu_baseline=True, extras=True, collective="peer",
                          profile_case=None, copies=2, persistent=True)
bench.run_b200(args)
"""


def test_b200_arm_runs_on_the_emulator_and_prints_the_contract():
    r = subprocess.run([sys.executable, "-c", _SCRIPT.format(root=str(ROOT))], capture_output=True, text=True,
                       timeout=1200, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    j = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "roofline", "cpu_baseline", "clocks",
                "step", "step_ms", "per_shape", "per_shape_in_graph", "per_shape_in_graph_one_cta_per_tile", "decode_stack", "moe_decode", "persistent_step"):
        assert key in j, key
    assert j["steps"] == 3 and j["warmup"] >= 3 and j["n_gpus"] == 1 and j["value"] > 0
    assert set(j["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac", "traffic"}
    assert set(j["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert j["e2e_check"]["copies_declared"] is True
    rps = j["step"]["passes_per_step"]
    assert j["gpu_launches"] == 3 * rps * 2 * 3        # steps x passes x copies x shapes
    assert "workload" in j["config"] and "model" not in j["config"]
    assert [d["batch"] for d in j["decode_stack"]] == [1, 16] and [d["batch"] for d in j["moe_decode"]] == [1, 16, 64]
    fused = j["decode_stack"][0]["with_norms_and_residuals_fused"]
    assert fused["launches_per_step"] == j["decode_stack"][0]["launches_per_step"] and fused["ms_per_step"] > 0


def test_both_arms_print_the_same_config_block():
    sys.path.insert(0, str(ROOT))
    import bench
    assert bench.bench_config(1, None) == bench.bench_config(1, None)
    assert "replays" not in json.dumps(bench.bench_config(1, None))


def test_clock_sampler_keeps_only_samples_inside_the_timed_region():
    sys.path.insert(0, str(ROOT))
    import datetime

    import bench
    rows = ["2026/01/02 10:00:00.100, 0, 1200, 1965, 400.1, 0x0, Not Active, Not Active, Not Active, Not Active",
            "2026/01/02 10:00:00.600, 0, 1900, 1965, 900.0, 0x4, Not Active, Not Active, Not Active, Active",
            "2026/01/02 10:00:01.100, 0, 1800, 1965, 950.5, 0x4, Not Active, Not Active, Not Active, Active",
            "2026/01/02 10:00:02.100, 0, 300, 1965, 100.0, 0x1, Not Active, Not Active, Not Active, Not Active",
            "garbage line"]
    t0 = datetime.datetime(2026, 1, 2, 10, 0, 0, 500000)
    t1 = datetime.datetime(2026, 1, 2, 10, 0, 1, 500000)
    got = bench.ClockSampler.parse("\n".join(rows), t0, t1)
    assert got["samples_in_region"] == 2 and got["samples_total"] == 4
    assert got["sm_mhz"] == 1850.0 and got["sm_max_mhz"] == 1965.0 and got["reasons"] == ["sw_power_cap"]
    assert got["power_w_max"] == 950.5


_SCRIPT_TWO_RANKS = r"""
import sys, argparse, datetime
sys.path.insert(0, {root!r})
from tests.emu import torch_shim
torch_shim.install()
import torch.distributed as dist
import bench
from speaches_plus_b200 import tp as tpmod
tpmod.init_process_group_for_node = lambda device, timeout_s=90: dist.init_process_group(
    "gloo", timeout=datetime.timedelta(seconds=timeout_s))
bench.SHAPES_KN = [(256, 512), (256, 256), (512, 256)]
bench.ROW_PARALLEL = {{(256, 256), (512, 256)}}
bench.COPIES = 2
bench.STEP_TARGET_S = 1e-4
bench.STACK_DIMS = {{"H": 256, "QO": 256, "KV": 128, "F": 512, "V": 1000, "layers": 2}}
bench.MOE_DIMS = {{"E": 16, "H": 256, "F": 128, "TOPK": 4, "layers": 2}}
args = argparse.Namespace(gpus=2, steps=3, warmup=3, impl="b200", cpu_baseline=False, extras=True, collective="nccl",
                          profile_case=None, copies=2, persistent=False)
bench.run_b200(args)
"""


def test_two_ranks_run_the_b200_arm_and_rank_0_prints_the_line():
    """The N > 1 control flow of the bench -- sharded weight sets, the all-reduce after row-parallel linears,
    max-over-ranks timing, the tensor-parallel decode stack and the expert-parallel MoE leg, the orderly
    shutdown -- with two emulated ranks over gloo."""
    import os
    import socket
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", _SCRIPT_TWO_RANKS.format(root=str(ROOT))], env=env, cwd=ROOT,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=900) for p in procs]
    for p, (so, se) in zip(procs, outs):
        assert p.returncode == 0, (so + se)[-4000:]
    lines0 = [ln for ln in outs[0][0].splitlines() if ln.startswith("{")]
    lines1 = [ln for ln in outs[1][0].splitlines() if ln.startswith("{")]
    assert len(lines0) == 1 and not lines1            # rank 0 alone prints
    j = json.loads(lines0[0])
    assert j["n_gpus"] == 2 and j["scaling"] == "strong" and j["config"]["parallelism"] == "tp2" and j["value"] > 0
    assert j["per_shape_in_graph"] is None            # the stamped legs are single-GPU
    assert [d["batch"] for d in j["decode_stack"]] == [1, 16] and [d["batch"] for d in j["moe_decode"]] == [1, 16, 64]
