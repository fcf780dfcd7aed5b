"""Loads the host emulation of the CUDA library (tests/emu/build_emu.py) and gives the tests
guard-paged "device" buffers to call it with.  The emulated library exports the product's C ABI
unchanged, so the tests call the same symbols with the same arguments as on a GPU.  Test
infrastructure only: nothing in the product package imports this."""
from __future__ import annotations

import ctypes as C
import importlib.util
import pathlib

import numpy as np

import speaches_plus_b200 as sp

_HERE = pathlib.Path(__file__).resolve().parent
_lib = None


def _build_module():
    spec = importlib.util.spec_from_file_location("_nvk_emu_build", _HERE / "build_emu.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        import os
        # NVK_EMU_LIB: a prebuilt emulation library to use instead (e.g. one built with -fsanitize=...)
        path = os.environ.get("NVK_EMU_LIB") or _build_module().build()
        L = C.CDLL(str(path))
        for name, args in sp.ffi.SIGNATURES.items():
            fn = getattr(L, name)   # the emulated library must export every symbol of the product's
            fn.argtypes = args
            fn.restype = C.c_size_t if name.endswith("_bytes") else C.c_int
        L.emu_alloc.argtypes = [C.c_size_t, C.c_int]
        L.emu_alloc.restype = C.c_void_p
        L.emu_free.argtypes = [C.c_void_p]
        L.emu_free.restype = None
        L.emu_set_option.argtypes = [C.c_char_p, C.c_int]
        L.emu_install_fault_handler()
        _lib = L
    return _lib


def set_option(name: str, value: int) -> None:
    assert lib().emu_set_option(name.encode(), int(value)) == 0


def call(name: str, *args) -> int:
    conv = [a.ptr if isinstance(a, Buf) else a for a in args]
    return int(getattr(lib(), name)(*conv))


class Buf:
    """A buffer in guard-paged memory: an access one byte past its end (256-byte granularity, like a
    device allocation) or -- with front=True -- one byte before its start ends the process with a
    message.  Filled from `a`; `read()` copies it back out."""

    def __init__(self, a: np.ndarray, front: bool = False):
        a = np.ascontiguousarray(a)
        self.dtype, self.shape, self.nbytes = a.dtype, a.shape, a.nbytes
        self.ptr = lib().emu_alloc(max(self.nbytes, 1), 1 if front else 0)
        assert self.ptr
        if self.nbytes:
            C.memmove(self.ptr, a.ctypes.data, self.nbytes)

    def read(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        if self.nbytes:
            C.memmove(out.ctypes.data, self.ptr, self.nbytes)
        return out

    def write(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a, dtype=self.dtype)
        assert a.nbytes == self.nbytes
        C.memmove(self.ptr, a.ctypes.data, self.nbytes)

    def __del__(self):
        try:
            if self.ptr:
                lib().emu_free(self.ptr)
                self.ptr = None
        except Exception:
            pass


def full(shape, value, dtype) -> Buf:
    return Buf(np.full(shape, value, dtype))
