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
