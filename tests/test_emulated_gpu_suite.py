"""Runs the tests marked `gpu` on the host emulation of the CUDA library (tests/emu).

Where no GPU is present this is how the kernels' index arithmetic, barriers, cp.async ordering and
buffer bounds get executed at all: the product's own .cu sources, compiled for the host, called through
the same C ABI by the same parity tests, against the same CPU oracle.  It does not replace the GPU
run -- float rounding of device math functions, real asynchrony and the hardware's own checks are not
modelled -- and nothing in the product package can load the emulated library.  Full-size shapes and the
tests that need a real CUDA runtime (graph capture, the CUTLASS prefill library) are skipped.
"""
import pathlib
import re
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _run(extra_env=None):
    import os
    env = dict(os.environ)
    env.update(extra_env or {})
    r = subprocess.run([sys.executable, "-m", "pytest", "tests", "-m", "gpu", "--emu", "-x", "-q", "-p",
                        "no:cacheprovider"], cwd=ROOT, capture_output=True, text=True, timeout=1500, env=env)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    m = re.search(r"(\d+) passed", r.stdout)
    assert m and int(m.group(1)) >= 200, tail
    return int(m.group(1))


def test_gpu_suite_passes_on_the_emulator():
    # cp.async copies land at the matching wait_group: the latest moment the ISA allows
    _run()


def test_gpu_linear_tests_also_pass_with_copies_landing_at_once():
    # ... and the earliest: a slot overwritten while another thread still reads it would show here
    import os
    env = dict(os.environ, NVK_EMU_CP_ASYNC_EARLY="1")
    # (the bf16 linears copy nothing asynchronously, and the two largest GEMV shapes add only time)
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_linear.py", "-m", "gpu", "--emu", "-x", "-q",
                        "-p", "no:cacheprovider", "-k", "not bf16 and not 5376-5376 and not config0"], cwd=ROOT,
                       capture_output=True, text=True, timeout=1500, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
