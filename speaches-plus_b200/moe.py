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
                 total_experts: int | None = None):
        self.gate, self.up, self.down = gate, up, down  # each: (packed, scales, alphas)
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
    def build_from_experts(cls, experts):
        """experts: list of (gate, up, down) Nvfp4Linear triples."""
        e0 = experts[0]
        hidden, inter = e0[0].in_features, e0[0].out_features

        def bank(idx):
            lins = [e[idx] for e in experts]
            packed = torch.stack([l.weight_u8.reshape(l.out_features, l.in_features // 2) for l in lins]).contiguous()
            nbytes = L.swizzled_scale_bytes(lins[0].out_features, lins[0].in_features)
            scales = torch.stack([l.weight_scales[:nbytes] for l in lins]).contiguous()
            alphas = torch.tensor([l.alpha_w4a16 for l in lins], dtype=torch.float32, device=packed.device)
            return packed, scales, alphas

        return cls(bank(0), bank(1), bank(2), hidden, inter, len(experts))

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


def forward_grouped_decode(w: MoeGroupedWeights, ctx: GroupedDecodeContext, x: torch.Tensor,
                           router_logits: torch.Tensor, bias=None, mode: int = 0, softcap: float = 0.0,
                           norm_topk: bool = True, routed_scaling: float = 1.0, group=None) -> torch.Tensor:
    """x [n, hidden] bf16, router_logits [n, E] f32 -> y_acc [n, hidden] f32 (the view of ctx.y_acc).

    Expert parallelism: when `w` holds only a block of the layer's experts (`shard_experts`), every
    rank routes all tokens over all E experts (the router is replicated), runs the slots that landed
    on ITS experts, leaves zeros in the other slots' rows, combines, and the ranks' f32 partial
    outputs are summed with one all-reduce over `group`."""
    n, k, E = x.shape[0], ctx.top_k, w.total_experts
    assert n <= ctx.max_tokens and x.dtype == torch.bfloat16 and x.is_contiguous()
    assert router_logits.dtype == torch.float32 and router_logits.is_contiguous()
    s = _stream()
    bias_p = bias.data_ptr() if bias is not None else None
    if E <= 256 and n * k <= 4096:
        # decode-sized: router and permutation in one launch
        _ffi.check("nvk_b200_moe_route_permute", s, router_logits.data_ptr(), bias_p, ctx.topk_ids.data_ptr(),
                   ctx.topk_weights.data_ptr(), ctx.perm_token.data_ptr(), ctx.offsets.data_ptr(),
                   ctx.inv_perm.data_ptr(), n, E, k, mode, float(softcap), int(norm_topk), float(routed_scaling))
    else:
        _ffi.check("nv_kernels_moe_route_topk", s, router_logits.data_ptr(), bias_p, ctx.topk_ids.data_ptr(),
                   ctx.topk_weights.data_ptr(), n, E, k, mode, float(softcap), int(norm_topk), float(routed_scaling))
        _ffi.check("nv_kernels_moe_permute", s, ctx.topk_ids.data_ptr(), ctx.perm_token.data_ptr(),
                   ctx.offsets.data_ptr(), ctx.inv_perm.data_ptr(), ctx.counts.data_ptr(), n, k, E)
    g, u, d = w.gate, w.up, w.down
    # Local expert i owns the sorted slots [offsets[first + i], offsets[first + i + 1]): the same offsets
    # array, entered at this rank's first expert.  Slot positions stay global.
    offsets = ctx.offsets.data_ptr() + 4 * w.first_expert
    if w.sharded:
        ctx.down_out[: n * k].zero_()   # rows of slots routed to other ranks' experts contribute nothing
    _ffi.check("nvk_b200_moe_grouped_w4a16", s, g[0].data_ptr(), g[1].data_ptr(), u[0].data_ptr(), u[1].data_ptr(),
               g[2].data_ptr(), u[2].data_ptr(), x.data_ptr(), None, ctx.perm_token.data_ptr(), offsets,
               ctx.gate_out.data_ptr(), ctx.up_out.data_ptr(), w.num_experts, w.inter, w.hidden)
    _ffi.check("nvk_b200_moe_grouped_w4a16", s, d[0].data_ptr(), d[1].data_ptr(), None, None, d[2].data_ptr(), None,
               ctx.gate_out.data_ptr(), ctx.up_out.data_ptr(), None, offsets, ctx.down_out.data_ptr(),
               None, w.num_experts, w.hidden, w.inter)
    _ffi.check("nv_kernels_moe_unpermute_scatter", s, ctx.down_out.data_ptr(), ctx.topk_weights.data_ptr(),
               ctx.inv_perm.data_ptr(), ctx.y_acc.data_ptr(), n, k, w.hidden, w.hidden)
    if w.sharded:
        import torch.distributed as dist
        dist.all_reduce(ctx.y_acc[:n], group=group)
    return ctx.y_acc[:n]
