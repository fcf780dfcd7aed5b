"""The peer all-reduce's protocol (push to every peer's inbox, per-CTA flags that carry the call number,
two inbox parities, sum in rank order) with every rank running AT THE SAME TIME -- on the host
emulation, where each rank's kernel is a group of host threads.  On GPUs the ranks are processes on
different devices; kernels that wait for each other must never share one GPU, so this concurrent form
exists only here (the single-device GPU tests cover the bounded wait and the data path one rank at a
time)."""
import ctypes as C
import threading

import numpy as np
import pytest

from oracle import ref
from tests.emu import harness as H


@pytest.mark.parametrize("world,n", [(2, 256), (4, 8192 + 64), (8, 5120)])
def test_all_ranks_get_the_fp32_sum_in_rank_order_over_several_calls(world, n):
    max_elems = (n + 7) // 8 * 8
    nbytes = H.lib().nvk_b200_tp_allreduce_buffer_bytes(world, max_elems)
    bufs = [H.Buf(np.zeros(nbytes, np.uint8)) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.ptr for b in bufs])
    epochs = [H.Buf(np.zeros(32, np.uint32)) for _ in range(world)]
    errs = [H.Buf(np.zeros(1, np.int32)) for _ in range(world)]
    rng = np.random.default_rng(world * 1000 + n)
    calls = 5   # odd and even call numbers: both inbox halves get used, flags are never reset
    for call in range(calls):
        xs = [ref.f32_to_bf16(rng.standard_normal(n).astype(np.float32)) for _ in range(world)]
        dx = [H.Buf(x) for x in xs]
        ys = [H.Buf(np.zeros(n, np.uint16)) for _ in range(world)]
        rcs = [None] * world

        def run(r):
            rcs[r] = H.call("nvk_b200_tp_allreduce_bf16", None, C.addressof(ptrs), r, world, dx[r], ys[r], n, max_elems,
                            epochs[r], errs[r])

        th = [threading.Thread(target=run, args=(r,)) for r in range(world)]
        for t in th:
            t.start()
        for t in th:
            t.join(timeout=300)
            assert not t.is_alive()
        assert rcs == [0] * world
        acc = np.zeros(n, np.float32)
        for x in xs:                       # rank order, fp32, one rounding at the end
            acc = acc + ref.bf16_to_f32(x)
        want = ref.f32_to_bf16(acc)
        for r in range(world):
            assert int(errs[r].read()[0]) == 0
            assert np.array_equal(ys[r].read(), want), (call, r)
        ctas = -(-n // 8192)
        assert all(np.all(e.read()[:ctas] == call + 1) for e in epochs)
