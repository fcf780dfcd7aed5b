"""Tensor-parallel sharding of NVFP4 linears across the GPUs of one node (one process per GPU,
torch.distributed / NCCL).  The reference has no multi-GPU code for this path; this is new design.

Column-parallel (QKV, gate/up, lm_head): output rows are split.  A shard is a whole number of
128-row scale tiles, so the packed rows and the swizzled scale tiles of a shard are both contiguous
slices.  y shards are all-gathered only where the full vector is needed.

Row-parallel (o_proj, down): K is split at multiples of 64 (one scale k-tile).  Each rank produces a
partial y over its K slice and the partials are summed with an all-reduce on the same stream.

The weight is quantized once with the global of the WHOLE matrix and then sliced, so a sharded
linear uses exactly the bytes the unsharded one does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import linear as L


def column_shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [r0, r1) of a column-parallel shard: 128-row tiles dealt out as evenly as possible."""
    tiles = -(-n // 128)
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * 128, n), min(t1 * 128, n)


def row_shard_cols(k: int, rank: int, world: int) -> tuple[int, int]:
    """K range [k0, k1) of a row-parallel shard: 64-element scale k-tiles dealt out evenly."""
    tiles = -(-k // 64)
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * 64, k), min(t1 * 64, k)


def shard_nvfp4(packed: torch.Tensor, scales_swz: torch.Tensor, n: int, k: int, mode: str, rank: int, world: int):
    """Slice (packed [n, k/2] u8, swizzled scales) for one rank.  Returns (packed, scales, n_local, k_local,
    offset) where offset is the first row (column mode) or first K index (row mode) of the shard."""
    k_tiles = -(-(k // 16) // 4)
    m_tiles = -(-n // 128)
    sc = scales_swz[: m_tiles * k_tiles * 512].reshape(m_tiles, k_tiles, 512)
    if mode == "column":
        r0, r1 = column_shard_rows(n, rank, world)
        return (packed[r0:r1].contiguous(), sc[r0 // 128: -(-r1 // 128)].reshape(-1).contiguous(), r1 - r0, k, r0)
    if mode == "row":
        k0, k1 = row_shard_cols(k, rank, world)
        return (packed[:, k0 // 2: k1 // 2].contiguous(), sc[:, k0 // 64: -(-k1 // 64)].reshape(-1).contiguous(), n,
                k1 - k0, k0)
    raise ValueError(f"unknown tensor-parallel mode {mode!r}")


def shard_nvfp4_fused(packed: torch.Tensor, scales_swz: torch.Tensor, parts: int, n_each: int, k: int, rank: int,
                      world: int):
    """Column shard of a matrix that is `parts` matrices of `n_each` rows stacked ([gate; up],
    [q; k; v] with equal parts): every rank takes its row range of EACH part, so outputs that are
    combined element by element (SiLU(gate) * up) stay on one rank.  `n_each` must be a multiple of
    128 so that each part is whole scale tiles.  Returns (packed, scales, rows per part on this rank,
    first row within a part)."""
    if n_each % 128 != 0:
        raise ValueError(f"fused column shard: each part needs a multiple of 128 rows, got {n_each}")
    k_tiles = -(-(k // 16) // 4)
    sc = scales_swz[: parts * (n_each // 128) * k_tiles * 512].reshape(parts, n_each // 128, k_tiles * 512)
    pk = packed.reshape(parts, n_each, k // 2)
    r0, r1 = column_shard_rows(n_each, rank, world)
    return (pk[:, r0:r1].reshape(parts * (r1 - r0), k // 2).contiguous(),
            sc[:, r0 // 128: r1 // 128].reshape(-1).contiguous(), r1 - r0, r0)


class PeerAllReduce:
    """One-shot all-reduce over peer memory (nvk_b200_tp_allreduce_bf16) for vectors of up to
    `max_elems` bf16 values.  Each rank's exchange buffer is plain device memory that the other ranks
    of the node map through CUDA IPC handles (exchanged over the process group's host side); no
    memory is bound to a multicast object.  Call `close()` on every rank before the process group is
    torn down."""

    def __init__(self, group, max_elems: int, device):
        import ctypes as C

        from . import _ffi
        self._C, self._ffi = C, _ffi
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.max_elems = (max_elems + 7) // 8 * 8
        nbytes = self._buffer_bytes()
        own = C.c_void_p(0)
        _ffi.check("nvk_b200_tp_buffer_alloc", nbytes, C.addressof(own))   # zero-filled
        self._own = own.value
        handle = (C.c_ubyte * 64)()
        _ffi.check("nvk_b200_tp_ipc_export", self._own, C.addressof(handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        self._opened = []
        ptrs = []
        failure = None
        for r in range(self.world):
            if r == self.rank:
                ptrs.append(self._own)
                continue
            raw = (C.c_ubyte * 64).from_buffer_copy(handles[r])
            peer = C.c_void_p(0)
            rc = _ffi.call("nvk_b200_tp_ipc_open", C.addressof(raw), C.addressof(peer))
            if rc != 0:
                failure = f"opening rank {r}'s buffer failed with CUDA error {rc}"
                break
            self._opened.append(peer.value)
            ptrs.append(peer.value)
        # Every rank learns whether every mapping succeeded, so that all of them either go on or
        # all of them give the buffers back and raise.
        ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self.close()
            raise RuntimeError("peer all-reduce unavailable: " + (failure or "a peer could not map the buffers"))
        self._ptr_array = (C.c_void_p * self.world)(*ptrs)
        self.epoch = torch.zeros(self._epoch_words(), dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every inbox exists and is zeroed before anyone pushes

    def _buffer_bytes(self) -> int:
        return int(self._ffi.lib().nvk_b200_tp_allreduce_buffer_bytes(self.world, self.max_elems))

    def _epoch_words(self) -> int:
        return 32

    def all_reduce_(self, y: torch.Tensor) -> torch.Tensor:
        """In-place sum of a contiguous bf16 tensor across the group."""
        n = y.numel()
        self._ffi.check("nvk_b200_tp_allreduce_bf16", torch.cuda.current_stream().cuda_stream,
                        self._C.addressof(self._ptr_array), self.rank, self.world, y.data_ptr(), y.data_ptr(), n,
                        self.max_elems, self.epoch.data_ptr(), self.err.data_ptr())
        return y

    def check(self) -> None:
        """Raise if any wait gave up since the last check (reads one int back; synchronises)."""
        e = int(self.err.item())
        if e:
            self.err.zero_()
            raise RuntimeError(f"peer all-reduce: rank {e - 1} never arrived within the wait limit")

    def close(self) -> None:
        """Unmap the peers' buffers and free ours.  Collective: every rank calls it, with no
        all-reduce in flight; peers unmap before anyone frees."""
        if self._own is None:
            return
        torch.cuda.synchronize()
        dist.barrier(self.group)
        for p in self._opened:
            self._ffi.call("nvk_b200_tp_ipc_close", p)
        self._opened = []
        dist.barrier(self.group)
        self._ffi.call("nvk_b200_tp_buffer_free", self._own)
        self._own = None


class PeerFusedLinear(PeerAllReduce):
    """Exchange buffers of the fused row-parallel linear + all-reduce
    (nvk_b200_tp_linear_nvfp4_w4a16_allreduce): the same plain-device-memory / CUDA IPC set-up as
    PeerAllReduce, sized for launches of up to `max_ctas` CTAs.  One object serves every row-parallel
    linear of a step (calls on one stream are ordered); every rank makes the same sequence of calls, with
    K slices of equal length (the launch geometry, and with it the pairing of CTAs across the ranks, follows
    from N and the slice's K)."""

    def __init__(self, group, device, max_ctas: int = 512, max_rows: int = 16):
        self.max_ctas, self.MAX_ROWS = int(max_ctas), int(max_rows)
        super().__init__(group, 8, device)

    def _buffer_bytes(self) -> int:
        return int(self._ffi.lib().nvk_b200_tp_fused_buffer_bytes(self.world, self.max_ctas, self.MAX_ROWS))

    def _epoch_words(self) -> int:
        return self.max_ctas

    def all_reduce_(self, y):
        raise TypeError("PeerFusedLinear exchanges inside the linear's launch: use linear_()")

    def linear_(self, lin: "L.Nvfp4Linear", xs: torch.Tensor, y: torch.Tensor, up: torch.Tensor | None = None,
                residual: torch.Tensor | None = None) -> bool:
        """y [m, N] = sum over ranks of this rank's partial (+ residual), m <= max_rows; `lin` holds this rank's K
        slice, xs [m, K_local] (row stride = its own).  False when the launch does not fit (more rows, or
        more CTAs than the buffers hold): the caller then runs the linear and the all-reduce separately."""
        m = xs.shape[0]
        if m > self.MAX_ROWS or lin.in_features % 32 != 0 or (m > 1 and not xs.is_contiguous()):
            return False
        rc = self._ffi.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", torch.cuda.current_stream().cuda_stream,
                            self._C.addressof(self._ptr_array), self.rank, self.world, lin.weight_u8.data_ptr(),
                            lin.weight_scales.data_ptr(), xs.data_ptr(), up.data_ptr() if up is not None else None,
                            residual.data_ptr() if residual is not None else None, y.data_ptr(), lin.alpha_w4a16, m,
                            lin.out_features, lin.in_features, self.max_ctas, self.MAX_ROWS, self.epoch.data_ptr(),
                            self.err.data_ptr())
        if rc == -3:
            return False      # more CTAs than the buffers hold
        if rc != 0:
            raise self._ffi.NvkError("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", rc)
        return True


class PeerMoeCombine(PeerAllReduce):
    """Exchange buffers of the expert-parallel combine that sums over the GPUs inside its own launch
    (nvk_b200_moe_combine_allreduce); set up like PeerAllReduce."""

    def __init__(self, group, device, max_ctas: int = 512):
        self.max_ctas = int(max_ctas)
        super().__init__(group, 8, device)

    def _buffer_bytes(self) -> int:
        return int(self._ffi.lib().nvk_b200_moe_combine_buffer_bytes(self.world, self.max_ctas))

    def _epoch_words(self) -> int:
        return self.max_ctas

    def all_reduce_(self, y):
        raise TypeError("PeerMoeCombine sums inside the combine's launch: use combine_()")

    def combine_(self, down_out: torch.Tensor, topk_weights: torch.Tensor, inv_perm: torch.Tensor, y_acc: torch.Tensor,
                 n: int, k: int, hidden: int, slots: int, status: torch.Tensor) -> bool:
        """False when the launch does not fit the buffers (the caller then combines and all-reduces)."""
        if hidden % 8 != 0:
            return False
        rc = self._ffi.call("nvk_b200_moe_combine_allreduce", torch.cuda.current_stream().cuda_stream,
                            self._C.addressof(self._ptr_array), self.rank, self.world, down_out.data_ptr(),
                            topk_weights.data_ptr(), inv_perm.data_ptr(), y_acc.data_ptr(), n, k, hidden, hidden, slots,
                            status.data_ptr(), self.max_ctas, self.epoch.data_ptr(), self.err.data_ptr())
        if rc == -3:
            return False
        if rc != 0:
            raise self._ffi.NvkError("nvk_b200_moe_combine_allreduce", rc)
        return True


def init_process_group_for_node(device, timeout_s: int = 90):
    """NCCL process group for the GPUs of one node with in-switch multicast (NVLS) turned off: on
    shared machines a rank that goes away while its memory is bound to an NVLink multicast object
    disturbs its peers' GPUs, and nothing on this path needs it."""
    import datetime
    import os
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=timeout_s))


def shutdown_process_group(join_s: float = 30.0) -> bool:
    """Orderly end of a multi-GPU run: the caller has deleted its CUDA graphs and closed its
    PeerAllReduce; this synchronises, meets the other ranks at a barrier and destroys the process
    group.  Returns False if the destroy call did not come back within `join_s` seconds (every rank
    is past the barrier by then, so the caller may simply exit)."""
    import threading
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dist.barrier()
    done = threading.Event()

    def _destroy():
        try:
            dist.destroy_process_group()
        finally:
            done.set()

    th = threading.Thread(target=_destroy, daemon=True)
    th.start()
    return done.wait(join_s)


class TpNvfp4Linear:
    """One rank's shard of an NVFP4 linear plus the collective that completes it."""

    def __init__(self, local: L.Nvfp4Linear | None, mode: str, rank: int, world: int, n: int, k: int, offset: int,
                 group=None, peer_ar: "PeerAllReduce | None" = None):
        self.local, self.mode, self.rank, self.world = local, mode, rank, world
        self.n, self.k, self.offset, self.group = n, k, offset, group
        self.peer_ar = peer_ar  # when set, row-parallel sums go over peer memory instead of NCCL
        self._bufs = {}

    @classmethod
    def from_bf16(cls, w: torch.Tensor, mode: str, rank: int, world: int, group=None):
        n, k = w.shape
        packed, scales, alpha, _ = L.quantize_weight_nvfp4(w)
        return cls.from_parts(packed, scales, alpha, n, k, mode, rank, world, group)

    @classmethod
    def from_parts(cls, packed, scales, alpha, n, k, mode, rank, world, group=None, input_stored_global=1.0,
                   device=None):
        """Shard (packed [n, k/2], swizzled scales) for this rank; with `device`, the shard is cut
        where the tensors are (e.g. on the host) and only the shard is moved there."""
        def place(t):
            return t if device is None else t.to(device)
        if world == 1:
            return cls(L.Nvfp4Linear(place(packed), place(scales), alpha, k, n, None, input_stored_global), mode, 0,
                       1, n, k, 0, group)
        if mode == "column" and n % (128 * world) != 0:
            raise ValueError(f"column-parallel needs N={n} to be a multiple of 128*{world}")
        if mode == "row" and k % (64 * world) != 0:
            raise ValueError(f"row-parallel needs K={k} to be a multiple of 64*{world}")
        p, s, nl, kl, off = shard_nvfp4(packed, scales, n, k, mode, rank, world)
        return cls(L.Nvfp4Linear(place(p), place(s), alpha, kl, nl, None, input_stored_global), mode, rank, world, n, k,
                   off, group)

    @classmethod
    def from_disk(cls, weights, module: str, n: int, k: int, mode: str, rank: int, world: int, device, sfx=None,
                  group=None):
        """One rank's shard of a checkpoint module: read and swizzle on the host, cut the shard there,
        upload only the shard."""
        import numpy as np

        from . import weights as W
        parts = W.read_nvfp4_module(weights, module, n, k, sfx or W.Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS)
        packed = torch.from_numpy(np.array(parts.packed, copy=True))
        scales = torch.from_numpy(np.array(parts.scales_swizzled, copy=True))
        return cls.from_parts(packed, scales, float(parts.weight_alpha), n, k, mode, rank, world, group,
                              float(parts.stored_input_global), device)

    def _buf(self, name, shape, device):
        key = (name, tuple(shape))
        if key not in self._bufs:
            self._bufs[key] = torch.empty(shape, dtype=torch.bfloat16, device=device)
        return self._bufs[key]

    def forward(self, x: torch.Tensor, gather: bool = True) -> torch.Tensor:
        """x [M, K] (full K on every rank) -> y.  Column mode returns the full [M, N] when `gather`
        (else this rank's [M, N/world] shard); row mode returns the all-reduced [M, N]."""
        m = x.shape[0]
        if self.world == 1:
            y = self._buf("y", (m, self.n), x.device)
            self.local.forward_into(x, y)
            return y
        # Sharded: the prefill library (cluster-multicast tile) is off limits, whatever M is.
        if self.mode == "column":
            yl = self._buf("yl", (m, self.local.out_features), x.device)
            self.local.forward_into(x, yl, allow_prefill=False)
            if not gather:
                return yl
            nl = self.local.out_features
            full = self._buf("yg", (self.world * m, nl), x.device)  # rank-major: [world, m, nl]
            dist.all_gather_into_tensor(full, yl, group=self.group)
            if m == 1:
                return full.reshape(1, self.n)
            return full.reshape(self.world, m, nl).permute(1, 0, 2).reshape(m, self.n)
        xs = x[:, self.offset: self.offset + self.local.in_features]
        if m > 1:
            xs = xs.contiguous()
        y = self._buf("yr", (m, self.n), x.device)
        fused = getattr(self, "peer_fused", None)
        # the fused form needs the same launch geometry on every rank: equal K slices
        if fused is not None and self.k % (64 * self.world) == 0 and fused.linear_(self.local, xs, y):
            return y          # the partials met inside the linear's own launch
        self.local.forward_into(xs, y, allow_prefill=False)
        if self.peer_ar is not None and y.numel() % 8 == 0 and y.numel() <= self.peer_ar.max_elems:
            self.peer_ar.all_reduce_(y)
        else:
            dist.all_reduce(y, group=self.group)
        return y
