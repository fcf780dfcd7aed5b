"""A decode step's NVFP4 linears as one persistent launch (nvk_b200_stack_*; no counterpart in the
reference, which launches one kernel per linear).

    step = DecodeStep(m=1, device="cuda")
    gu = step.add(gate, x, y_gate, lin_b=up, y_b=y_up)              # gate + up share x
    dn = step.add(down, y_gate, y_down, x2=y_up, dep=gu)            # SiLU(gate) * up is the down input
    step.build()
    step.run(); step.check()

Each operation may depend on ONE earlier operation (the one that writes its activations); a buffer may
be overwritten only by an operation that (transitively) depends on every reader of the old contents.
`run` enqueues on the current stream and can be captured in a CUDA graph; `build` is a set-up call."""
from __future__ import annotations

import ctypes as C

import torch

from . import _ffi
from .linear import Nvfp4Linear


class DecodeStep:
    def __init__(self, m: int, device):
        if not 1 <= m <= 8:
            raise ValueError(f"DecodeStep: m={m} tokens; the persistent step takes 1..8")
        self.m, self.device = m, torch.device(device)
        self._ops: list[_ffi.NvkStackOp] = []
        self._keep = []          # tensors the operations point into
        self._plan = None
        self._launch = None
        self.err = None

    def add(self, lin_a: Nvfp4Linear, x: torch.Tensor, y_a: torch.Tensor, lin_b: Nvfp4Linear | None = None,
            y_b: torch.Tensor | None = None, x2: torch.Tensor | None = None, dep: int = -1,
            rows_per_item: int = 0) -> int:
        """Append y_a = lin_a(act), and y_b = lin_b(act) when given, with act = x or bf16(SiLU(x) * x2).
        Returns the operation's index (to be named as a later operation's `dep`)."""
        if self._plan is not None:
            raise RuntimeError("DecodeStep: already built")
        if (lin_b is None) != (y_b is None):
            raise ValueError("DecodeStep.add: lin_b and y_b come together")
        if lin_b is not None and (lin_b.in_features, lin_b.out_features) != (lin_a.in_features, lin_a.out_features):
            raise ValueError("DecodeStep.add: the two arms must have the same shape")
        if not -1 <= dep < len(self._ops):
            raise ValueError(f"DecodeStep.add: dep={dep} does not name an earlier operation")
        for t, cols in ((x, lin_a.in_features), (x2, lin_a.in_features), (y_a, lin_a.out_features),
                        (y_b, lin_a.out_features)):
            if t is None:
                continue
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != (self.m, cols):
                raise ValueError(f"DecodeStep.add: expected a contiguous bf16 [{self.m}, {cols}] tensor, "
                                 f"got {t.dtype} {tuple(t.shape)}")
        op = _ffi.NvkStackOp()
        op.wq_a, op.sc_a = lin_a.weight_u8.data_ptr(), lin_a.weight_scales.data_ptr()
        op.wq_b = lin_b.weight_u8.data_ptr() if lin_b is not None else None
        op.sc_b = lin_b.weight_scales.data_ptr() if lin_b is not None else None
        op.x, op.x2 = x.data_ptr(), (x2.data_ptr() if x2 is not None else None)
        op.y_a, op.y_b = y_a.data_ptr(), (y_b.data_ptr() if y_b is not None else None)
        op.alpha_a = lin_a.alpha_w4a16
        op.alpha_b = lin_b.alpha_w4a16 if lin_b is not None else 0.0
        op.N, op.K, op.dep, op.rows_per_item = lin_a.out_features, lin_a.in_features, dep, rows_per_item
        self._ops.append(op)
        self._keep.append((lin_a, lin_b, x, x2, y_a, y_b))
        return len(self._ops) - 1

    def build(self) -> None:
        n = len(self._ops)
        nbytes = int(_ffi.lib().nvk_b200_stack_plan_bytes(n))
        if nbytes == 0:
            raise ValueError(f"DecodeStep: {n} operations (1..1024 are accepted)")
        arr = (_ffi.NvkStackOp * n)(*self._ops)
        self._plan = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        launch = (C.c_int * 2)()
        _ffi.check("nvk_b200_stack_build", C.addressof(arr), n, self.m, self._plan.data_ptr(), nbytes,
                   C.addressof(launch))
        self._launch = (int(launch[0]), int(launch[1]))

    def run(self) -> None:
        """Enqueue one step on the current stream."""
        if self._plan is None:
            raise RuntimeError("DecodeStep: build() first")
        _ffi.check("nvk_b200_stack_run", torch.cuda.current_stream().cuda_stream, self._plan.data_ptr(), len(self._ops),
                   self.m, self._launch[0], self._launch[1], self.err.data_ptr())

    def check(self) -> None:
        """Raise if a wait inside a step gave up since the last check (reads one int back; synchronises)."""
        if int(self.err.item()):
            self.err.zero_()
            raise RuntimeError("DecodeStep: a dependency wait inside the kernel ran out")
