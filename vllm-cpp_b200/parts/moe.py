"""A feed-forward of routed experts.

    s = softmax(W_r h)  or  sigmoid(W_r h)  float32, over ``num_experts`` + ``num_identity`` router outputs (``score``)
    chosen = the ``top`` outputs with the largest s + correction (``correction`` False: no such tensor); with
             ``groups`` > ``keep_groups`` only outputs of the ``keep_groups`` best of ``groups`` equal groups of neighbours
             may be chosen, a group's score being the sum of its ``group_top`` largest
    weights = s[chosen]; with ``normalize`` divided by (their sum + ``sum_eps``); times ``route_scale``
    out = sum over chosen of weight * expert(h)

Outputs 0 .. num_experts - 1 are small gated feed-forwards with tensors ``e<i>.gate``, ``e<i>.up``, ``e<i>.down``.
``activation`` "clamped_swish": g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
W_down (g * sigmoid(alpha * g) * (u + 1)); "silu": W_down (silu(W_gate h) * W_up h).  The last ``num_identity`` outputs
are identity experts, expert(h) = h, without tensors.

``router_bias``: a tensor ``router.b`` joins the router's logits.  ``shared``: the PartSpec of a registered feed-forward
(tensors under ``shared.``) that every token takes beside its chosen experts; its result is added.  With softmax
scores and ``normalize``, the weights are the softmax over the chosen logits alone.

Everything runs on the device (csrc/moe.cu): the router (logits, then selection), a sort of the (token, choice) pairs by expert, one product
per tile of an expert's rows for gate-and-up (with the activation) and one for down, and the weighted sum.  The
grids are sized for the most tiles a step can have, so a step's launches do not depend on the routing and the host
never reads it.  The reference has no routed feed-forward (src/layers/mlp.cpp).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from . import mlp as _mlp  # noqa: F401  (registers the feed-forwards a shared expert may be)
from .base import FEED_FORWARDS, FeedForward, ParamSpec, build_part, register_feed_forward, workspace_piece


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    ACTIVATIONS = ("clamped_swish", "silu")

    def __init__(self, hidden_size: int, expert_size: int, num_experts: int, num_identity: int, top: int, limit: float,
                 dtype, device, alpha: float = 1.702, activation: str = "clamped_swish", score: str = "softmax",
                 correction: bool = True, groups: int = 1, keep_groups: int = 1, group_top: int = 1, normalize: bool = False,
                 sum_eps: float = 0.0, route_scale: float = 1.0, router_bias: bool = False, shared=None):
        if min(hidden_size, expert_size, num_experts, top) <= 0 or num_identity < 0:
            raise ValueError("routed_experts: sizes must be positive")
        if top > num_experts + num_identity:
            raise ValueError(f"routed_experts: {top} of {num_experts + num_identity} router outputs cannot be chosen")
        if not limit > 0:
            raise ValueError("routed_experts: limit must be positive")
        if activation not in self.ACTIVATIONS or score not in ops.ROUTER_SCORES:
            raise ValueError(f"routed_experts: activation one of {self.ACTIVATIONS}, score one of {sorted(ops.ROUTER_SCORES)}")
        outputs = num_experts + num_identity
        if groups < 1 or outputs % groups or not 1 <= keep_groups <= groups or not 1 <= group_top <= ops.ROUTER_GROUP_TOP_MAX:
            raise ValueError(f"routed_experts: {outputs} router outputs in {groups} equal groups of which {keep_groups} stay, "
                             f"a group's score from its {group_top} (at most {ops.ROUTER_GROUP_TOP_MAX}) best")
        if top > outputs // groups * keep_groups:
            raise ValueError(f"routed_experts: {top} choices do not fit the {keep_groups} groups that stay")
        self.hidden, self.ff, self.E, self.I, self.top = hidden_size, expert_size, num_experts, num_identity, top
        if activation == "silu":
            self.limit, self.alpha, self.up_shift = float("inf"), 1.0, 0.0
        else:
            self.limit, self.alpha, self.up_shift = float(limit), float(alpha), 1.0
        self.activation, self.score, self.has_correction = activation, score, bool(correction)
        self.rule = dict(score=score, groups=int(groups), keep_groups=int(keep_groups), group_top=int(group_top),
                         normalize=bool(normalize), sum_eps=float(sum_eps), scale=float(route_scale))
        self.dtype, self.device = dtype, device
        self.has_router_bias = bool(router_bias)
        self.shared = None if shared is None else build_part(FEED_FORWARDS, "feed-forward", shared, dtype=dtype, device=device)
        self.w_gate_up = self.w_down = self.w_router = self.correction = self.router_bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {}
        for e in range(self.E):
            specs[f"e{e}.gate"] = ParamSpec((self.ff, self.hidden))
            specs[f"e{e}.up"] = ParamSpec((self.ff, self.hidden))
            specs[f"e{e}.down"] = ParamSpec((self.hidden, self.ff))
        specs["router"] = ParamSpec((self.E + self.I, self.hidden), "bias")       # held in float32: the router is
        if self.has_router_bias:
            specs["router.b"] = ParamSpec((self.E + self.I,), "bias")
        if self.has_correction:
            specs["correction"] = ParamSpec((self.E + self.I,), "bias")
        if self.shared is not None:
            for name, ps in self.shared.param_specs().items():
                specs["shared." + name] = ps
        return specs

    def load_params(self, tensors):
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.E)]).contiguous()
        self.w_router = tensors["router"].contiguous()
        self.correction = tensors["correction"].contiguous() if self.has_correction else None
        self.router_bias = tensors["router.b"].contiguous() if self.has_router_bias else None
        if self.shared is not None:
            self.shared.load_params({name: tensors["shared." + name] for name in self.shared.param_specs()})

    def product_weights(self):
        # the experts' products are this part's own kernels; only a shared feed-forward has products to measure or tile
        return self.shared.product_weights() if self.shared is not None else []

    def step_arrays(self):
        return self.shared.step_arrays() if self.shared is not None else {}

    def reserve(self, n_tokens, n_reqs, device):
        if self.shared is not None:
            self.shared.reserve(n_tokens, n_reqs, device)

    def workspace_bytes(self, n_tokens, n_reqs):
        pairs = n_tokens * self.top
        tiles = max(ops.moe_max_tiles(n_tokens, self.top, self.E, tm) for tm in ops.MOE_TILE_ROWS)
        ints = 3 * workspace_piece((pairs,), torch.int32) + 3 * workspace_piece((tiles,), torch.int32) + workspace_piece((4,), torch.int32)
        also = 0 if self.shared is None else workspace_piece((n_tokens, self.hidden), self.dtype) + self.shared.workspace_bytes(n_tokens, n_reqs)
        return (ints + workspace_piece((pairs,), torch.float32) + workspace_piece((n_tokens, self.E + self.I), torch.float32)
                + workspace_piece((pairs, self.ff), self.dtype)
                + workspace_piece((pairs, self.hidden), torch.float32) + also)

    def forward(self, x, out, step, ws):
        n = x.shape[0]
        mark = ws.mark()
        pairs = n * self.top
        tm = ops.moe_tile_rows(n, self.top, self.E)
        tiles = ops.moe_max_tiles(n, self.top, self.E, tm)
        ids = ws.take((n, self.top), torch.int32)
        weights = ws.take((n, self.top), torch.float32)
        sorted_token = ws.take((pairs,), torch.int32)
        pos = ws.take((pairs,), torch.int32)
        tile_expert, tile_row0, tile_rows = (ws.take((tiles,), torch.int32) for _ in range(3))
        meta = ws.take((4,), torch.int32)
        logits = ws.take((n, self.E + self.I), torch.float32)
        ops.moe_router(x, self.w_router, self.correction, ids, weights, logits, logit_bias=self.router_bias, **self.rule)
        ops.moe_sort(ids, self.E, tm, sorted_token, pos, tile_expert, tile_row0, tile_rows, meta)
        act = ws.take((pairs, self.ff), self.dtype)
        lists = (sorted_token, tile_expert, tile_row0, tile_rows, meta, tiles, tm)
        ops.moe_expert_gemm(x, self.w_gate_up, act, *lists, gated=True, limit=self.limit, alpha=self.alpha, up_shift=self.up_shift)
        y = ws.take((pairs, self.hidden), torch.float32)
        ops.moe_expert_gemm(act, self.w_down, y, *lists, gated=False)
        also = None
        if self.shared is not None:
            also = ws.take((n, self.hidden), self.dtype)
            self.shared.forward(x, also, step, ws)
        ops.moe_combine(y, x, pos, weights, out, add=also)
        ws.release(mark)
