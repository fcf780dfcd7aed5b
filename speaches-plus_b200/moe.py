"""Host-side mirror of the reference's grouped MoE decode path for NVFP4 experts
(rust/crates/nv-layers/src/moe_grouped.rs: `MoeGroupedWeights`, `GroupedDecodeContext`,
`forward_grouped_decode`), on the W4A16 route: activations stay bf16 and the tokens routed to one
expert share one pass over that expert's weights.

Step: route (top-k, softmax over the winners) -> sort the routed slots by expert -> gate+up grouped
linear (gathering each slot's token row) -> down grouped linear with SiLU(gate)*up as its prologue ->
weighted combine back to token order.  Every buffer is allocated once in the context, every launch
goes to the current stream, nothing synchronises: the step can be captured in a CUDA graph.
"""
from __future__ import annotations

import dataclasses

import torch

from . import _ffi
from . import linear as L


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def expert_shard_range(num_experts: int, rank: int, world: int) -> tuple[int, int]:
    """Experts [e0, e1) held by `rank` when a layer's experts are dealt out in contiguous blocks, as
    evenly as possible (128 experts over 8 GPUs: 16 each)."""
    base, extra = divmod(num_experts, world)
    e0 = rank * base + min(rank, extra)
    return e0, e0 + base + (1 if rank < extra else 0)


class MoeGroupedWeights:
    """Expert banks addressable by expert id: packed weights [E, N, K/2], swizzled scales
    [E, sc_bytes], alphas [E] for gate, up ([inter, hidden]) and down ([hidden, inter])."""

    def __init__(self, gate, up, down, hidden: int, inter: int, num_experts: int, first_expert: int = 0,
                 total_experts: int | None = None, input_globals_gate_up=None, input_globals_down=None):
        self.gate, self.up, self.down = gate, up, down  # each: (packed, scales, alphas)
        # stored activation globals per expert for the route that quantizes activations (f32 [E] on the
        # banks' device; ones when a checkpoint carries none) -- moe_grouped.rs `input_globals_*`
        dev = gate[0].device
        self.folded_shared = gate[0].shape[0] == num_experts + 1   # a shared expert stored as bank entry E
        ones = lambda: torch.ones(gate[0].shape[0], dtype=torch.float32, device=dev)   # noqa: E731
        self.input_globals_gate_up = ones() if input_globals_gate_up is None else input_globals_gate_up
        self.input_globals_down = ones() if input_globals_down is None else input_globals_down
        self.hidden, self.inter, self.num_experts = hidden, inter, num_experts
        # expert parallelism: this object holds experts [first_expert, first_expert + num_experts) of
        # a layer with total_experts routed experts
        self.first_expert = first_expert
        self.total_experts = num_experts if total_experts is None else total_experts
        if not (0 <= first_expert and first_expert + num_experts <= self.total_experts):
            raise ValueError("MoeGroupedWeights: local expert range outside the layer's experts")

    @property
    def sharded(self) -> bool:
        return self.num_experts != self.total_experts

    def shard_experts(self, rank: int, world: int) -> "MoeGroupedWeights":
        """This rank's contiguous block of experts (views of the banks, no copy)."""
        if self.sharded:
            raise ValueError("MoeGroupedWeights: already sharded")
        e0, e1 = expert_shard_range(self.num_experts, rank, world)

        def cut(bank):
            return tuple(t[e0:e1] for t in bank)

        return MoeGroupedWeights(cut(self.gate), cut(self.up), cut(self.down), self.hidden, self.inter, e1 - e0, e0,
                                 self.num_experts)

    @classmethod
    def build_from_experts(cls, experts, shared=None):
        """experts: list of (gate, up, down) Nvfp4Linear triples; `shared`: one more triple of the same
        shapes stored after them as bank entry E (the shared expert folded into the routed step,
        moe_grouped.rs `folded_shared`)."""
        n_routed = len(experts)
        if shared is not None:
            experts = list(experts) + [shared]
        e0 = experts[0]
        hidden, inter = e0[0].in_features, e0[0].out_features

        def bank(idx):
            lins = [e[idx] for e in experts]
            packed = torch.stack([l.weight_u8.reshape(l.out_features, l.in_features // 2) for l in lins]).contiguous()
            nbytes = L.swizzled_scale_bytes(lins[0].out_features, lins[0].in_features)
            scales = torch.stack([l.weight_scales[:nbytes] for l in lins]).contiguous()
            alphas = torch.tensor([l.alpha_w4a16 for l in lins], dtype=torch.float32, device=packed.device)
            return packed, scales, alphas

        return cls(bank(0), bank(1), bank(2), hidden, inter, n_routed)

    def per_expert_bytes(self) -> int:
        """Packed + scale bytes of one expert (rust/crates/nv-layers/src/moe_grouped.rs `per_expert_bytes`)."""
        return sum(t[0][0].numel() + t[1][0].numel() for t in (self.gate, self.up, self.down))


class GroupedDecodeContext:
    """Pre-allocated intermediates for up to `max_tokens` tokens with `top_k` routed experts each."""

    def __init__(self, w: MoeGroupedWeights, max_tokens: int, top_k: int, device):
        slots = max_tokens * top_k
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tokens, self.top_k = max_tokens, top_k
        self.topk_ids = torch.zeros((max_tokens, top_k), **i32)
        self.topk_weights = torch.zeros((max_tokens, top_k), dtype=torch.float32, device=device)
        self.perm_token = torch.zeros(slots, **i32)
        self.offsets = torch.zeros(w.total_experts + 1, **i32)
        self.inv_perm = torch.zeros(slots, **i32)
        self.counts = torch.zeros(w.total_experts, **i32)
        self.gate_out = torch.zeros((slots, w.inter), dtype=torch.bfloat16, device=device)
        self.up_out = torch.zeros((slots, w.inter), dtype=torch.bfloat16, device=device)
        self.down_out = torch.zeros((slots, w.hidden), dtype=torch.bfloat16, device=device)
        self.y_acc = torch.zeros((max_tokens, w.hidden), dtype=torch.float32, device=device)
        # experts that received slots (written by the fused router; lets the expert launches cover
        # only those) and the word in which the kernels report a routing table they refused to follow
        self.active = torch.zeros(max(1, min(w.total_experts, slots)), **i32)
        self.n_active = torch.zeros(1, **i32)
        self.status = torch.zeros(1, **i32)

    def check_status(self) -> None:
        """Raise if a kernel met an offset or row index outside its buffers since the last check
        (bit 0: expert offset, bit 1: gathered row, bit 2: combine row).  Reads one int back."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
            raise RuntimeError(f"MoE decode step: a routing table pointed outside its buffers (status {v:#x}); "
                               "the affected slots were skipped")


def forward_grouped_decode(w: MoeGroupedWeights, ctx: GroupedDecodeContext, x: torch.Tensor,
                           router_logits: torch.Tensor, bias=None, mode: int = 0, softcap: float = 0.0,
                           norm_topk: bool = True, routed_scaling: float = 1.0, group=None,
                           peer_combine=None) -> torch.Tensor:
    """x [n, hidden] bf16, router_logits [n, E] f32 -> y_acc [n, hidden] f32 (the view of ctx.y_acc).

    Expert parallelism: when `w` holds only a block of the layer's experts (`shard_experts`), every
    rank routes all tokens over all E experts (the router is replicated), runs the slots that landed
    on ITS experts, leaves zeros in the other slots' rows, combines, and the ranks' f32 partial
    outputs are summed with one all-reduce over `group` -- or, with a `tp.PeerMoeCombine`, inside the
    combine's own launch (peer stores from the combine kernel, no separate collective)."""
    n, k, E = x.shape[0], ctx.top_k, w.total_experts
    assert n <= ctx.max_tokens and x.dtype == torch.bfloat16 and x.is_contiguous()
    assert router_logits.dtype == torch.float32 and router_logits.is_contiguous()
    s = _stream()
    bias_p = bias.data_ptr() if bias is not None else None
    fused = E <= 256 and n * k <= 4096
    if fused:
        # decode-sized: router, slot sort and the list of active experts in one launch
        _ffi.check("nvk_b200_moe_route_permute", s, router_logits.data_ptr(), bias_p, ctx.topk_ids.data_ptr(),
                   ctx.topk_weights.data_ptr(), ctx.perm_token.data_ptr(), ctx.offsets.data_ptr(),
                   ctx.inv_perm.data_ptr(), ctx.active.data_ptr(), ctx.n_active.data_ptr(), n, E, k, mode,
                   float(softcap), int(norm_topk), float(routed_scaling))
    else:
        _ffi.check("nv_kernels_moe_route_topk", s, router_logits.data_ptr(), bias_p, ctx.topk_ids.data_ptr(),
                   ctx.topk_weights.data_ptr(), n, E, k, mode, float(softcap), int(norm_topk), float(routed_scaling))
        _ffi.check("nv_kernels_moe_permute", s, ctx.topk_ids.data_ptr(), ctx.perm_token.data_ptr(),
                   ctx.offsets.data_ptr(), ctx.inv_perm.data_ptr(), ctx.counts.data_ptr(), n, k, E)
    g, u, d = w.gate, w.up, w.down
    # Local expert i owns the sorted slots [offsets[first + i], offsets[first + i + 1]): the same offsets
    # array, entered at this rank's first expert.  Slot positions stay global.  The active-expert list
    # holds layer-wide ids, so it is used only when this object holds the whole layer.
    offsets = ctx.offsets.data_ptr() + 4 * w.first_expert
    use_active = fused and not w.sharded
    act = ctx.active.data_ptr() if use_active else None
    n_act = ctx.n_active.data_ptr() if use_active else None
    slots = n * k
    if w.sharded:
        ctx.down_out[:slots].zero_()   # rows of slots routed to other ranks' experts contribute nothing
    _ffi.check("nvk_b200_moe_grouped_w4a16", s, g[0].data_ptr(), g[1].data_ptr(), u[0].data_ptr(), u[1].data_ptr(),
               g[2].data_ptr(), u[2].data_ptr(), x.data_ptr(), None, ctx.perm_token.data_ptr(), offsets, act, n_act,
               ctx.gate_out.data_ptr(), ctx.up_out.data_ptr(), w.num_experts, w.inter, w.hidden, slots, n,
               ctx.status.data_ptr())
    _ffi.check("nvk_b200_moe_grouped_w4a16", s, d[0].data_ptr(), d[1].data_ptr(), None, None, d[2].data_ptr(), None,
               ctx.gate_out.data_ptr(), ctx.up_out.data_ptr(), None, offsets, act, n_act, ctx.down_out.data_ptr(),
               None, w.num_experts, w.hidden, w.inter, slots, slots, ctx.status.data_ptr())
    if w.sharded and peer_combine is not None and peer_combine.combine_(
            ctx.down_out, ctx.topk_weights, ctx.inv_perm, ctx.y_acc, n, k, w.hidden, slots, ctx.status):
        return ctx.y_acc[:n]      # combined and summed over the ranks in one launch
    _ffi.check("nvk_b200_moe_combine", s, ctx.down_out.data_ptr(), ctx.topk_weights.data_ptr(),
               ctx.inv_perm.data_ptr(), ctx.y_acc.data_ptr(), n, k, w.hidden, w.hidden, slots, ctx.status.data_ptr())
    if w.sharded:
        import torch.distributed as dist
        dist.all_reduce(ctx.y_acc[:n], group=group)
    return ctx.y_acc[:n]


# ------------------------------------------------------------------------------------------------
# decode on the route that quantizes activations (FP4 x FP4), every (token, winner) pair a tile
class TiledDecodeContext:
    """Buffers of `forward_grouped_decode_into` (rust/crates/nv-layers/src/moe_grouped.rs:575-782): every
    (token, winner) pair -- plus one pair per token for a shared expert folded in as expert id E --
    owns a 128-row tile of which row 0 is live.  Everything is allocated here, once; the step itself
    allocates nothing.  Inputs are written into `x_in` / `logits_f32`, the result is read from `y_acc`."""

    def __init__(self, w: MoeGroupedWeights, n_tokens: int, top_k: int, device, folded_shared: bool = False):
        if top_k <= 0 or n_tokens <= 0:
            raise ValueError("TiledDecodeContext: k and n_tokens must be > 0")
        self.k, self.n_tokens, self.folded_shared = top_k, n_tokens, folded_shared
        self.tiles_per_token = top_k + (1 if folded_shared else 0)
        tiles = n_tokens * self.tiles_per_token
        m_total = tiles * MIN_TILE
        self.hidden, self.inter, self.num_experts = w.hidden, w.inter, w.total_experts
        i32 = dict(dtype=torch.int32, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        u8 = dict(dtype=torch.uint8, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        src = torch.full((m_total,), -1, dtype=torch.int32)
        src[::MIN_TILE] = torch.arange(tiles, dtype=torch.int32) // self.tiles_per_token
        self.src_idx = src.to(device)                                       # tile row 0 <- its token
        self.inv_perm = (torch.arange(tiles, dtype=torch.int32) * MIN_TILE).to(device)
        self.topk_ids = torch.zeros(tiles, **i32)
        self.topk_weights = torch.zeros(tiles, **f32)
        self.input_gu_mini = torch.zeros(tiles, **f32)
        self.input_dn_mini = torch.zeros(tiles, **f32)
        self.x_sorted = torch.zeros((m_total, w.hidden), **bf)
        self.x_fp4 = torch.zeros((m_total, w.hidden // 2), **u8)
        self.x_sf = torch.zeros(L.swizzled_scale_bytes(m_total, w.hidden), **u8)
        self.y_gate = torch.zeros((m_total, w.inter), **bf)
        self.y_up = torch.zeros((m_total, w.inter), **bf)
        self.y_act_fp4 = torch.zeros((m_total, w.inter // 2), **u8)
        self.y_act_sf = torch.zeros(L.swizzled_scale_bytes(m_total, w.inter), **u8)
        self.y_down = torch.zeros((m_total, w.hidden), **bf)
        self.x_in = torch.zeros((n_tokens, w.hidden), **bf)
        self.logits_f32 = torch.zeros((n_tokens, w.total_experts), **f32)
        self.y_acc = torch.zeros((n_tokens, w.hidden), **f32)
        # FP4 x FP4 multipliers: the reciprocal of the weight global times the reciprocal of the
        # activation global the tile was quantized with
        self.alphas = tuple((bank[2] / g).contiguous() for bank, g in
                            ((w.gate, w.input_globals_gate_up), (w.up, w.input_globals_gate_up),
                             (w.down, w.input_globals_down)))


def forward_grouped_decode_into(w: MoeGroupedWeights, ctx: TiledDecodeContext, bias=None, mode: int = 0,
                                softcap: float = 0.0, norm_topk: bool = True, routed_scaling: float = 1.0,
                                run_scatter: bool = True, prof_base: int | None = None) -> None:
    """One decode step over the context's own buffers (moe_grouped.rs:1137-1495): route; each tile's
    activation globals; quantize the token's row per tile; gate and up as grouped M = 1 FP4 GEMVs;
    SiLU(gate) * up quantized per tile; down; f32 weighted combine into ctx.y_acc.  A single token with
    at most 256 experts routes, gathers and quantizes in one launch.  `prof_base`: device address of
    u64 slots that receive GPU timestamps after the route, the quantize, gate/up, activation, down."""
    if w.sharded:
        raise ValueError("forward_grouped_decode_into: expert-parallel shards use forward_grouped_decode")
    if (ctx.hidden, ctx.inter, ctx.num_experts) != (w.hidden, w.inter, w.num_experts):
        raise ValueError("TiledDecodeContext shape mismatch")
    if ctx.folded_shared and not w.folded_shared:
        raise ValueError("TiledDecodeContext folds the shared expert but the grouped weights were built without it")
    s = _stream()
    E, k, n, tpt = w.num_experts, ctx.k, ctx.n_tokens, ctx.tiles_per_token
    tiles = n * tpt
    m_total = tiles * MIN_TILE
    hidden, inter = w.hidden, w.inter
    tail = E if ctx.folded_shared else -1
    bias_p = bias.data_ptr() if bias is not None else None

    def mark(slot):
        if prof_base is not None:
            _ffi.check("nv_kernels_prof_timestamp", s, prof_base + 8 * slot)

    if n == 1 and E <= 256:
        _ffi.check("nv_kernels_moe_route_gather_quant_m1", s, ctx.logits_f32.data_ptr(), bias_p, ctx.x_in.data_ptr(),
                   w.input_globals_gate_up.data_ptr(), w.input_globals_down.data_ptr(), ctx.topk_ids.data_ptr(),
                   ctx.topk_weights.data_ptr(), ctx.input_gu_mini.data_ptr(), ctx.input_dn_mini.data_ptr(),
                   ctx.x_fp4.data_ptr(), ctx.x_sf.data_ptr(), E, k, mode, float(softcap), int(norm_topk),
                   float(routed_scaling), tail, hidden, MIN_TILE)
        mark(0)
        mark(1)
    else:
        if ctx.folded_shared:
            _ffi.check("nv_kernels_moe_route_topk_shared_tail", s, ctx.logits_f32.data_ptr(), bias_p,
                       ctx.topk_ids.data_ptr(), ctx.topk_weights.data_ptr(), n, E, k, mode, float(softcap),
                       int(norm_topk), float(routed_scaling), tail)
        else:
            _ffi.check("nv_kernels_moe_route_topk", s, ctx.logits_f32.data_ptr(), bias_p, ctx.topk_ids.data_ptr(),
                       ctx.topk_weights.data_ptr(), n, E, k, mode, float(softcap), int(norm_topk),
                       float(routed_scaling))
        mark(0)
        for src, dst in ((w.input_globals_gate_up, ctx.input_gu_mini), (w.input_globals_down, ctx.input_dn_mini)):
            _ffi.check("nv_kernels_gather_f32_by_ids", s, src.data_ptr(), ctx.topk_ids.data_ptr(), dst.data_ptr(), tiles)
        _ffi.check("nv_kernels_gather_rows_bf16_strided", s, ctx.x_in.data_ptr(), ctx.src_idx.data_ptr(),
                   ctx.x_sorted.data_ptr(), m_total, hidden, n, MIN_TILE)
        _ffi.check("nv_kernels_quantize_nvfp4_bf16_per_expert_strided", s, ctx.x_sorted.data_ptr(), ctx.x_fp4.data_ptr(),
                   ctx.x_sf.data_ptr(), ctx.input_gu_mini.data_ptr(), MIN_TILE, m_total, hidden)
        mark(1)
    n_ids = E + (1 if ctx.folded_shared else 0)   # a folded shared expert is bank entry E

    def gemv(a_fp4, a_sf, bank, alphas, out, n_out, k_in):
        _ffi.check("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", s, a_fp4.data_ptr(), a_sf.data_ptr(), bank[0].data_ptr(),
                   bank[1].data_ptr(), alphas.data_ptr(), out.data_ptr(), ctx.topk_ids.data_ptr(), tiles, n_ids, n_out,
                   k_in, MIN_TILE, MIN_TILE * n_out)

    gemv(ctx.x_fp4, ctx.x_sf, w.gate, ctx.alphas[0], ctx.y_gate, inter, hidden)
    gemv(ctx.x_fp4, ctx.x_sf, w.up, ctx.alphas[1], ctx.y_up, inter, hidden)
    mark(2)
    _ffi.check("nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert_strided", s, ctx.y_gate.data_ptr(),
               ctx.y_up.data_ptr(), ctx.y_act_fp4.data_ptr(), ctx.y_act_sf.data_ptr(), ctx.input_dn_mini.data_ptr(),
               MIN_TILE, m_total, inter)
    mark(3)
    gemv(ctx.y_act_fp4, ctx.y_act_sf, w.down, ctx.alphas[2], ctx.y_down, hidden, inter)
    mark(4)
    if run_scatter:
        _ffi.check("nv_kernels_moe_unpermute_scatter", s, ctx.y_down.data_ptr(), ctx.topk_weights.data_ptr(),
                   ctx.inv_perm.data_ptr(), ctx.y_acc.data_ptr(), n, tpt, hidden, hidden)


# ------------------------------------------------------------------------------------------------
# prefill-sized steps: block-scaled FP4 x FP4 grouped GEMM (activations quantized online)
MIN_TILE = 128               # rows of one expert tile (rust/crates/nv-quant/src/nvfp4.rs:2)
MAX_GROUPS_PER_CALL = 1024   # groups one grouped-GEMM call takes


def plan_routing(topk_ids, num_experts: int) -> dict:
    """Host-side plan of a prefill-sized routed step (rust/crates/nv-layers/src/moe_grouped.rs:310-350):
    every expert that received tokens gets one 128-row tile; `src_idx[row]` is the token a tile row
    reads (-1 for padding), `inv_perm[token, slot]` the tile row that holds that routed slot.  Rows of
    one expert keep (token, slot) order.  `overflow` is set when an expert received more than 128
    rows: the caller must split the token range."""
    import numpy as np
    ids = np.asarray(topk_ids).astype(np.int64)
    n, k = ids.shape
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")                 # by expert, (token, slot) order inside
    counts = np.bincount(flat, minlength=num_experts)
    active = np.nonzero(counts)[0]
    tile_of = np.full(num_experts, -1, np.int64)
    tile_of[active] = np.arange(active.size)
    first = np.concatenate([[0], np.cumsum(counts)[:-1]])   # first sorted position of each expert
    pos_in_expert = np.arange(flat.size) - first[flat[order]]
    rows = tile_of[flat[order]] * MIN_TILE + pos_in_expert
    ok = pos_in_expert < MIN_TILE
    src_idx = np.full(active.size * MIN_TILE, -1, np.int32)
    inv_perm = np.full(n * k, -1, np.int32)
    src_idx[rows[ok]] = (order[ok] // k).astype(np.int32)
    inv_perm[order[ok]] = rows[ok].astype(np.int32)
    return {"active_experts": active.astype(np.int32), "real_m_per_active": counts[active].astype(np.int32),
            "m_total_padded": int(active.size * MIN_TILE), "src_idx": src_idx, "inv_perm": inv_perm.reshape(n, k),
            "overflow": bool((~ok).any())}


def grouped_gemm_chunked(a_packed, a_scales, bank, alphas_w4a4, d, active_ids, n: int, k: int, meta_scratch,
                         gemm_ws) -> None:
    """One grouped-GEMM call per chunk of active experts, each expert a 128-row tile of the stacked
    activations (moe_grouped.rs:1656-1760)."""
    import ctypes as C
    import numpy as np
    dev = d.device
    total = int(active_ids.numel())
    kb_pad = -(-(k // 16) // 4) * 4
    s = _stream()
    for c0 in range(0, total, MAX_GROUPS_PER_CALL):
        g = min(MAX_GROUPS_PER_CALL, total - c0)
        rows0 = c0 * MIN_TILE
        offs = torch.arange(g, dtype=torch.int32, device=dev) * MIN_TILE
        sizes = torch.tensor(np.tile(np.array([MIN_TILE, n, k], np.int32), g), dtype=torch.int32, device=dev)
        need = C.c_size_t(0)
        _ffi.check("nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16", s,
                   a_packed.data_ptr() + rows0 * (k // 2), a_scales.data_ptr() + rows0 * kb_pad, bank[0].data_ptr(),
                   bank[1].data_ptr(), alphas_w4a4.data_ptr(), d.data_ptr() + rows0 * n * 2, offs.data_ptr(),
                   offs.data_ptr(), sizes.data_ptr(), active_ids[c0:].data_ptr(), n, k, g, k, k, n,
                   meta_scratch.data_ptr(), meta_scratch.numel(), gemm_ws.data_ptr(), gemm_ws.numel(),
                   C.addressof(need))


def forward_grouped(w: MoeGroupedWeights, x: torch.Tensor, topk_ids, topk_weights, input_globals_gate_up=None,
                    input_globals_down=None) -> torch.Tensor:
    """Prefill-shaped MoE step on the FP4 x FP4 route (moe_grouped.rs:352-573): gather the routed rows
    into one 128-row tile per active expert, quantize them with that expert's input global, gate and up
    as grouped block-scaled GEMMs, SiLU(gate)*up quantized in one pass, down as a grouped GEMM, f32
    weighted combine.  x [n, hidden] bf16; topk_ids [n, k] (host or device integers); topk_weights
    [n, k] f32.  Returns [n, hidden] f32.  `input_globals_*`: per-expert activation globals (host
    sequences of num_experts floats; 1.0 when omitted); `w`'s alphas are reciprocals of the weight
    globals alone, so the GEMM multiplier is alpha / input_global."""
    import numpy as np
    if w.sharded:
        raise ValueError("forward_grouped: expert-parallel shards run through forward_grouped_decode")
    dev = x.device
    n, hidden, inter, E = x.shape[0], w.hidden, w.inter, w.num_experts
    ids_host = topk_ids.cpu().numpy() if isinstance(topk_ids, torch.Tensor) else np.asarray(topk_ids)
    k = ids_host.shape[1]
    plan = plan_routing(ids_host, E)
    if plan["overflow"]:
        raise ValueError(f"forward_grouped: an expert received more than {MIN_TILE} rows -- split the token range")
    a = int(plan["active_experts"].size)
    if a == 0:
        return torch.zeros((n, hidden), dtype=torch.float32, device=dev)
    m_total = plan["m_total_padded"]
    gu = np.ones(E, np.float32) if input_globals_gate_up is None else np.asarray(input_globals_gate_up, np.float32)
    dn = np.ones(E, np.float32) if input_globals_down is None else np.asarray(input_globals_down, np.float32)
    act = plan["active_experts"]
    gu_dev = torch.from_numpy(gu[act].copy()).to(dev)
    dn_dev = torch.from_numpy(dn[act].copy()).to(dev)
    active_ids = torch.from_numpy(act.copy()).to(dev)
    src_idx = torch.from_numpy(plan["src_idx"]).to(dev)
    inv_perm = torch.from_numpy(np.ascontiguousarray(plan["inv_perm"])).to(dev)
    wts = topk_weights.to(device=dev, dtype=torch.float32).contiguous()
    s = _stream()
    b = _grouped_buffers(w, m_total, n, dev)
    x_sorted, x_fp4, x_sf, meta, ws = b["x_sorted"], b["x_fp4"], b["x_sf"], b["meta"], b["ws"]
    y_gate, y_up, act_fp4, act_sf, y_down = b["y_gate"], b["y_up"], b["act_fp4"], b["act_sf"], b["y_down"]
    _ffi.check("nv_kernels_gather_rows_bf16", s, x.data_ptr(), src_idx.data_ptr(), x_sorted.data_ptr(), m_total,
               hidden, n)
    _ffi.check("nv_kernels_quantize_nvfp4_bf16_per_expert", s, x_sorted.data_ptr(), x_fp4.data_ptr(), x_sf.data_ptr(),
               gu_dev.data_ptr(), MIN_TILE, m_total, hidden)
    gu_all, dn_all = torch.from_numpy(gu).to(dev), torch.from_numpy(dn).to(dev)
    grouped_gemm_chunked(x_fp4, x_sf, w.gate, (w.gate[2] / gu_all).contiguous(), y_gate, active_ids, inter, hidden,
                         meta, ws)
    grouped_gemm_chunked(x_fp4, x_sf, w.up, (w.up[2] / gu_all).contiguous(), y_up, active_ids, inter, hidden, meta, ws)
    _ffi.check("nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert", s, y_gate.data_ptr(), y_up.data_ptr(),
               act_fp4.data_ptr(), act_sf.data_ptr(), dn_dev.data_ptr(), MIN_TILE, m_total, inter)
    grouped_gemm_chunked(act_fp4, act_sf, w.down, (w.down[2] / dn_all).contiguous(), y_down, active_ids, hidden,
                         inter, meta, ws)
    y_acc = torch.empty((n, hidden), dtype=torch.float32, device=dev)
    _ffi.check("nv_kernels_moe_unpermute_scatter", s, y_down.data_ptr(), wts.data_ptr(), inv_perm.data_ptr(),
               y_acc.data_ptr(), n, k, hidden, hidden)
    return y_acc


def _grouped_buffers(w: MoeGroupedWeights, m_total: int, n: int, dev) -> dict:
    """The intermediates of a prefill-shaped step, kept on the weights object and grown on demand: a
    step of a size seen before allocates only its result (moe_grouped.rs keeps them in its context for
    the same reason)."""
    cache = w.__dict__.setdefault("_grouped_bufs", {})
    st = cache.get("b")
    if st is None or st["rows"] < m_total or st["x_sorted"].device != torch.device(dev):
        hidden, inter = w.hidden, w.inter
        u8 = dict(dtype=torch.uint8, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        st = {"rows": m_total,
              "x_sorted": torch.empty((m_total, hidden), **bf), "x_fp4": torch.empty((m_total, hidden // 2), **u8),
              "x_sf": torch.zeros(L.swizzled_scale_bytes(m_total, hidden), **u8),
              "y_gate": torch.empty((m_total, inter), **bf), "y_up": torch.empty((m_total, inter), **bf),
              "act_fp4": torch.empty((m_total, inter // 2), **u8),
              "act_sf": torch.zeros(L.swizzled_scale_bytes(m_total, inter), **u8),
              "y_down": torch.empty((m_total, hidden), **bf),
              "meta": torch.empty(512 * 1024, **u8), "ws": torch.empty(16 * 1024 * 1024, **u8)}
        cache["b"] = st
    # views of exactly this step's size (the scale buffers' size depends on the row count)
    hidden, inter = w.hidden, w.inter
    return {"x_sorted": st["x_sorted"][:m_total], "x_fp4": st["x_fp4"][:m_total],
            "x_sf": st["x_sf"][:L.swizzled_scale_bytes(m_total, hidden)],
            "y_gate": st["y_gate"][:m_total], "y_up": st["y_up"][:m_total], "act_fp4": st["act_fp4"][:m_total],
            "act_sf": st["act_sf"][:L.swizzled_scale_bytes(m_total, inter)], "y_down": st["y_down"][:m_total],
            "meta": st["meta"], "ws": st["ws"]}


# ------------------------------------------------------------------------------------------------
# the MoE block around the expert dispatch
@dataclasses.dataclass(frozen=True)
class MoeConfig:
    """rust/crates/nv-layers/src/moe.rs:12-19."""
    hidden_size: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int = 0


class MoeBlock:
    """Router + routed experts + gated shared expert (rust/crates/nv-layers/src/moe.rs:21-401):

        y = sum_j softmax(top-k logits)_j * expert_j(x)  +  sigmoid(x . w_shared_gate) * shared_expert(x)

    `gate` is the bf16 router linear [num_experts, hidden]; `experts` the routed experts' banks
    (`MoeGroupedWeights`); `shared_expert` an `Nvfp4Mlp` with its bf16 gate linear [1, hidden], or both
    None.  Up to `decode_tokens` tokens run the capture-safe decode path (tokens grouped per expert,
    activations kept in bf16); larger batches take the prefill route (`forward_grouped`)."""

    def __init__(self, cfg: MoeConfig, gate: L.Bf16Linear, experts: MoeGroupedWeights, shared_expert=None,
                 shared_expert_gate=None, decode_tokens: int = 64):
        if experts.total_experts != cfg.num_experts:
            raise ValueError(f"MoeBlock: experts={experts.total_experts} != cfg.num_experts={cfg.num_experts}")
        if cfg.num_experts_per_tok == 0 or cfg.num_experts_per_tok > cfg.num_experts:
            raise ValueError(f"MoeBlock: num_experts_per_tok={cfg.num_experts_per_tok} invalid for "
                             f"num_experts={cfg.num_experts}")
        if gate.in_features != cfg.hidden_size or gate.out_features != cfg.num_experts:
            raise ValueError(f"MoeBlock: gate shape mismatch -- expected [{cfg.num_experts}, {cfg.hidden_size}], "
                             f"got [{gate.out_features}, {gate.in_features}]")
        if (experts.hidden, experts.inter) != (cfg.hidden_size, cfg.moe_intermediate_size):
            raise ValueError("MoeBlock: expert banks do not have the configured sizes")
        if (shared_expert is None) != (shared_expert_gate is None):
            raise ValueError("MoeBlock: the shared expert and its gate come together")
        if shared_expert_gate is not None and (shared_expert_gate.out_features != 1 or
                                               shared_expert_gate.in_features != cfg.hidden_size):
            raise ValueError("MoeBlock: shared_expert_gate must be [1, hidden]")
        self.cfg, self.gate, self.experts = cfg, gate, experts
        self.shared_expert, self.shared_expert_gate = shared_expert, shared_expert_gate
        self.decode_tokens = decode_tokens
        self._ctx = None

    def shared_contribution(self, x_flat: torch.Tensor) -> torch.Tensor:
        """sigmoid(gate logit) * shared_expert(x), f32 [n, hidden] (moe.rs:386-398)."""
        out = self.shared_expert.forward(x_flat).float().contiguous()
        gate_logits = self.shared_expert_gate.forward(x_flat).float().contiguous()   # [n, 1]
        _ffi.check("nv_kernels_mul_sigmoid_rowgate_f32", _stream(), out.data_ptr(), gate_logits.data_ptr(),
                   out.data_ptr(), out.shape[0], out.shape[1])
        return out

    def forward(self, x: torch.Tensor, group=None) -> torch.Tensor:
        cfg = self.cfg
        if x.shape[-1] != cfg.hidden_size:
            raise ValueError(f"MoeBlock: last dim {x.shape[-1]} != hidden_size {cfg.hidden_size}")
        lead = x.shape[:-1]
        x_flat = x.reshape(-1, cfg.hidden_size).to(torch.bfloat16).contiguous()
        n = x_flat.shape[0]
        logits = self.gate.forward(x_flat).float().contiguous()     # the router's bf16 output, widened
        if n <= self.decode_tokens:
            if self._ctx is None or self._ctx.topk_ids.device != x.device:
                self._ctx = GroupedDecodeContext(self.experts, self.decode_tokens, cfg.num_experts_per_tok, x.device)
            y = forward_grouped_decode(self.experts, self._ctx, x_flat, logits, group=group).clone()
        else:
            ids = torch.zeros((n, cfg.num_experts_per_tok), dtype=torch.int32, device=x.device)
            wts = torch.zeros((n, cfg.num_experts_per_tok), dtype=torch.float32, device=x.device)
            _ffi.check("nv_kernels_moe_route_topk", _stream(), logits.data_ptr(), None, ids.data_ptr(),
                       wts.data_ptr(), n, cfg.num_experts, cfg.num_experts_per_tok, 0, 0.0, 1, 1.0)
            y = self._forward_prefill(x_flat, ids, wts)
        if self.shared_expert is not None:
            y = y + self.shared_contribution(x_flat)
        return y.reshape(*lead, cfg.hidden_size).to(x.dtype)

    __call__ = forward

    def _forward_prefill(self, x_flat, ids, wts):
        """Token ranges small enough that no expert receives more than one 128-row tile."""
        n = x_flat.shape[0]
        out = torch.empty((n, self.cfg.hidden_size), dtype=torch.float32, device=x_flat.device)
        ids_host = ids.cpu().numpy()
        r0 = 0
        while r0 < n:
            r1 = min(n, r0 + MIN_TILE)   # at most 128 tokens: no expert can receive more than 128 rows
            out[r0:r1] = forward_grouped(self.experts, x_flat[r0:r1].contiguous(), ids_host[r0:r1],
                                         wts[r0:r1].contiguous())
            r0 = r1
        return out

    @classmethod
    def from_loader(cls, cfg: MoeConfig, prefix: str, weights, qconfig, device, sfx=None, decode_tokens: int = 64):
        """`<prefix>.gate.weight`, `<prefix>.experts.<i>.{gate,up,down}_proj.*`,
        `<prefix>.shared_expert.{gate,up,down}_proj.*`, `<prefix>.shared_expert_gate.weight`
        (moe.rs:176-290)."""
        from . import weights as W
        sfx = sfx or W.Nvfp4Suffixes.QWEN_COMPRESSED_TENSORS
        gate = W.load_linear(weights, f"{prefix}.gate.weight", cfg.num_experts, cfg.hidden_size, device)
        banks = W.moe_grouped_weights_from_disk(weights, [f"{prefix}.experts.{i}" for i in range(cfg.num_experts)],
                                                cfg.hidden_size, cfg.moe_intermediate_size, device, sfx)
        shared = shared_gate = None
        if cfg.shared_expert_intermediate_size:
            f, h = cfg.shared_expert_intermediate_size, cfg.hidden_size
            mk = lambda name, n, k: W.nvfp4_linear_from_disk_with_suffixes(  # noqa: E731
                weights, f"{prefix}.shared_expert.{name}", n, k, device, sfx)
            shared = L.Nvfp4Mlp(mk("gate_proj", f, h), mk("up_proj", f, h), mk("down_proj", h, f))
            shared_gate = W.load_linear(weights, f"{prefix}.shared_expert_gate.weight", 1, h, device)
        return cls(cfg, gate, banks, shared, shared_gate, decode_tokens)
