"""Emulation mode of the GPU test suite (`pytest -m gpu --emu`): the tests marked `gpu` run unchanged,
with "device" tensors that are host tensors and the C ABI calls of the package redirected -- by this
test harness, never by the package -- to the host emulation of the CUDA library (tests/emu).

What is patched, for the test process only:
  * torch factory functions and Tensor.cuda()/to(): device "cuda" means host memory taken from the
    emulation's guard-paged allocator, so a kernel that reads or writes past the end of a "device"
    tensor (at the 256-byte granularity of a device allocation) ends the run with a message;
  * torch.cuda.synchronize / current_stream / is_available: no-ops with the obvious answers;
  * Tensor.is_cuda: True (the package asserts it on its inputs);
  * speaches_plus_b200._ffi: its library handle is the emulated library.
Tests that need a real CUDA runtime (graph capture, the CUTLASS prefill library) are skipped in this
mode by tests/conftest.py."""
from __future__ import annotations

import types

import torch

_installed = False


def _is_cuda_dev(d) -> bool:
    if d is None:
        return False
    if isinstance(d, torch.device):
        return d.type == "cuda"
    return isinstance(d, str) and d.startswith("cuda")


def install() -> None:
    global _installed
    if _installed:
        return
    _installed = True
    import speaches_plus_b200 as sp

    from . import harness

    import ctypes as C

    orig_frombuffer = torch.frombuffer

    def to_device(t: torch.Tensor) -> torch.Tensor:
        """A copy of `t` in guard-paged memory (kept alive by the tensor's storage)."""
        t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        if nbytes == 0:
            return t
        buf = harness.Buf.__new__(harness.Buf)
        buf.ptr = harness.lib().emu_alloc(nbytes, 0)
        assert buf.ptr
        arr = (C.c_ubyte * nbytes).from_address(buf.ptr)
        arr._keep = buf   # freed when the storage lets go of the ctypes array
        g = orig_frombuffer(arr, dtype=torch.uint8).view(t.dtype).reshape(t.shape)
        g.copy_(t)
        return g

    def wrap_factory(fn):
        def inner(*a, **k):
            if _is_cuda_dev(k.get("device")):
                k["device"] = "cpu"
                return to_device(fn(*a, **k))
            return fn(*a, **k)
        inner.__name__ = getattr(fn, "__name__", "factory")
        return inner

    for name in ("full", "zeros", "empty", "ones", "tensor", "arange", "randn", "rand", "zeros_like", "empty_like",
                 "full_like", "ones_like", "as_tensor"):
        setattr(torch, name, wrap_factory(getattr(torch, name)))

    torch.Tensor.cuda = lambda self, *a, **k: to_device(self)
    orig_to = torch.Tensor.to

    def to(self, *a, **k):
        moved = any(_is_cuda_dev(x) for x in a) or _is_cuda_dev(k.get("device"))
        a = tuple("cpu" if _is_cuda_dev(x) else x for x in a)
        if _is_cuda_dev(k.get("device")):
            k["device"] = "cpu"
        out = orig_to(self, *a, **k)
        return to_device(out) if moved else out

    torch.Tensor.to = to
    torch.Tensor.is_cuda = property(lambda self: True)
    torch.cuda.is_available = lambda: True
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.set_device = lambda *a, **k: None
    torch.cuda.current_stream = lambda *a, **k: types.SimpleNamespace(cuda_stream=0)
    torch.cuda.empty_cache = lambda: None
    torch.Tensor.pin_memory = lambda self, *a, **k: self

    # Streams, events and graphs for code that times itself (bench.py): launches are synchronous here,
    # so a "captured" graph is simply its body run once and a replay does nothing; events read the
    # host clock.  Good for exercising the control flow and the output contract, not for numbers.
    import contextlib
    import time as _time

    class Stream:
        cuda_stream = 0

        def synchronize(self):
            pass

        def wait_stream(self, other):
            pass

    class Event:
        def __init__(self, enable_timing=False):
            self.t = None

        def record(self, stream=None):
            self.t = _time.perf_counter()

        def synchronize(self):
            pass

        def elapsed_time(self, other):
            return max(1e-3, (other.t - self.t) * 1e3)

    class CUDAGraph:
        def replay(self):
            pass

    torch.cuda.Stream = Stream
    torch.cuda.Event = Event
    torch.cuda.CUDAGraph = CUDAGraph
    torch.cuda.stream = lambda s: contextlib.nullcontext()
    torch.cuda.graph = lambda g, stream=None, **k: contextlib.nullcontext()
    orig_generator = torch.Generator
    torch.Generator = lambda device=None: orig_generator()

    # the package's binding now talks to the emulated library (same symbols, same argument types)
    sp.ffi._lib = harness.lib()
    sp.ffi.EMULATED = True
    sp.ffi.prefill_available = lambda: False   # the CUTLASS library needs a GPU
    import os
    if os.environ.get("NVK_EMU_CP_ASYNC_EARLY") == "1":
        harness.set_option("cp_async_early", 1)
