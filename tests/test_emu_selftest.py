"""The host emulation must itself catch what it is used to catch: an access past the end of a buffer
ends the process with exit code 98 and a message, and results of an in-bounds call are unaffected by
where in its guard-paged mapping a buffer sits."""
import subprocess
import sys
import pathlib

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[1]

_OOB = r"""
import sys
sys.path.insert(0, {root!r})
import numpy as np
from tests.emu import harness as H
x = H.Buf(np.zeros((4, 256), np.uint16))
idx = H.Buf(np.array([0, 1, 2, 3, 0, 1], np.int32))
out = H.Buf(np.zeros((4, 256), np.uint16))          # room for 4 rows ...
rc = H.call("nv_kernels_gather_rows_bf16", None, x, idx, out, 6, 256, 4)   # ... asked to write 6
print("returned", rc)
"""


def test_a_write_past_the_end_of_a_buffer_is_caught():
    r = subprocess.run([sys.executable, "-c", _OOB.format(root=str(ROOT))], capture_output=True, text=True, timeout=300)
    assert r.returncode == 98, (r.returncode, r.stdout, r.stderr)
    assert "memory fault" in r.stderr and "out-of-bounds" in r.stderr


def test_front_and_back_guarded_buffers_give_the_same_result():
    from oracle import ref
    from tests.emu import harness as H
    rng = np.random.default_rng(5)
    m, k = 3, 128
    x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    outs = []
    for front in (False, True):
        bx = H.Buf(x, front=front)
        bp = H.Buf(np.zeros((m, k // 2), np.uint8), front=front)
        bs = H.Buf(np.zeros(ref.swizzled_len(m, k // 16), np.uint8), front=front)
        assert H.call("nv_kernels_quantize_nvfp4_bf16", None, bx, bp, bs, 2.0, m, m, k) == 0
        outs.append((bp.read(), bs.read()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    packed, lin = ref.quantize_rows_bf16(x, 2.0)
    assert np.array_equal(outs[0][0], packed) and np.array_equal(outs[0][1], ref.swizzle_scales(lin))


_RACE = r"""
import sys
sys.path.insert(0, {root!r})
import ctypes as C
import numpy as np
from tests.emu import harness as H
L = H.lib()
L.emu_selftest_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
a = H.Buf(np.arange(64, dtype=np.int32))
o = H.Buf(np.zeros(64, np.int32))
rc = L.emu_selftest_rotate(a.ptr, o.ptr, {synced})
print("returned", rc, int(np.array_equal(o.read(), (np.arange(64) + 33) % 64)))
"""


def _run_under_race_checker(synced: int):
    import os
    import shutil
    import pytest
    tsan_rt = subprocess.run(["gcc", "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
    if not shutil.which("gcc") or not os.path.isabs(tsan_rt):
        pytest.skip("no ThreadSanitizer runtime on this machine")
    from tests.emu import harness as H
    lib = H._build_module().build(tsan=True)
    env = dict(os.environ, LD_PRELOAD=tsan_rt, NVK_EMU_LIB=str(lib),
               TSAN_OPTIONS="halt_on_error=1 exitcode=66 report_signal_unsafe=0")
    return subprocess.run([sys.executable, "-c", _RACE.format(root=str(ROOT), synced=synced)], capture_output=True,
                          text=True, timeout=600, env=env)


def test_the_race_checker_passes_a_kernel_with_its_barrier():
    r = _run_under_race_checker(1)
    assert r.returncode == 0 and "returned 0 1" in r.stdout, (r.returncode, r.stdout, r.stderr[-2000:])


def test_the_race_checker_reports_a_missing_barrier():
    r = _run_under_race_checker(0)
    assert r.returncode == 66, (r.returncode, r.stdout, r.stderr[-2000:])
    assert "data race" in r.stderr and "rotate_kernel<false>" in r.stderr
