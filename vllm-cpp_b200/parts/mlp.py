"""Gated feed-forward: down( act(gate(x)) * up(x) ), no biases
(src/layers/mlp.cpp:49-64; silu of src/kernels/activation.cu:8-10).

gate and up are one product against the row-wise concatenation [W_gate; W_up],
made at load; the reference runs them as two.

``activation`` "clamped_swish" is another rule for the pair: g = min(gate, limit),
u = clamp(up, -limit, limit), act = g * sigmoid(alpha * g) * (u + 1); ``biases`` gives
all three projections a bias (tensors named as the matrices plus ``bias_suffix``),
added in float before the clamps and after the down product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec, register_feed_forward, workspace_piece


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: arrangements that allow it skip the sublayer."""

    def __init__(self, dtype=None, device=None):
        pass


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    ACTIVATIONS = ("silu", "clamped_swish")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, dtype, device,
                 tensor_names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), limit: float = 0.0,
                 alpha: float = 1.702, biases: bool = False, bias_suffix: str = ".b"):
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"gated_mlp: activation {activation!r} is not built (known: {self.ACTIVATIONS})")
        if activation == "clamped_swish" and not limit > 0:
            raise ValueError("gated_mlp: the clamped activation needs a positive limit")
        if biases and activation == "silu":
            raise ValueError("gated_mlp: biases are built for the clamped activation only")
        self.hidden, self.inter = hidden_size, intermediate_size
        self.names = tuple(tensor_names)          # local names of the gate, up and down matrices
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.biases, self.bias_suffix = bool(biases), bias_suffix
        self.dtype, self.device = dtype, device
        self.w_gate_up = None     # [2*inter, hidden]
        self.w_down = None        # [hidden, inter]
        self.b_gate_up = None     # float32 [2*inter]
        self.b_down = None        # float32 [hidden]

    def param_specs(self) -> Dict[str, ParamSpec]:
        gate, up, down = self.names
        specs = {gate: ParamSpec((self.inter, self.hidden)),
                 up: ParamSpec((self.inter, self.hidden)),
                 down: ParamSpec((self.hidden, self.inter))}
        if self.biases:
            specs.update({gate + self.bias_suffix: ParamSpec((self.inter,), "bias"), up + self.bias_suffix: ParamSpec((self.inter,), "bias"),
                          down + self.bias_suffix: ParamSpec((self.hidden,), "bias")})
        return specs

    def load_params(self, tensors):
        gate, up, down = self.names
        self.w_gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
        self.w_down = tensors[down].contiguous()
        if self.biases:
            sfx = self.bias_suffix
            self.b_gate_up = torch.cat([tensors[gate + sfx], tensors[up + sfx]]).contiguous()
            self.b_down = tensors[down + sfx].contiguous()

    def product_weights(self):
        return [(self.w_gate_up, self.inter if self.activation == "silu" else 0), (self.w_down, 0)]

    def fuses_norm(self, n_tokens):
        if self.activation != "silu":
            return False
        return ops.linear_fuses_norm(n_tokens, self.w_gate_up) and ops.linear_fuses_norm(n_tokens, self.w_down)

    def workspace_bytes(self, n_tokens, n_reqs):
        # the activations, and the gate-and-up product where the activation is a kernel of its own
        return workspace_piece((n_tokens, self.inter), self.dtype) + workspace_piece((n_tokens, 2 * self.inter), self.dtype)

    def forward(self, x, out, step, ws, x_scale=None, fuse=None):
        n = x.shape[0]
        mark = ws.mark()
        act = ws.take((n, self.inter), self.dtype)
        if self.activation == "clamped_swish":
            gate_up = ws.take((n, 2 * self.inter), self.dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.clamped_swish_mul(gate_up, self.b_gate_up, act, limit=self.limit, alpha=self.alpha)
            ops.linear(act, self.w_down, out)
            if self.b_down is not None:
                ops.add_bias(out, self.b_down)
            ws.release(mark)
            return
        if ops.linear_gated_fuses(n, self.w_gate_up):
            ops.linear_gated(x, self.w_gate_up, act, x_scale=x_scale)       # product and activation in one kernel
        else:
            gate_up = ws.take((n, 2 * self.inter), self.dtype)
            ops.linear(x, self.w_gate_up, gate_up, x_scale=x_scale)
            ops.silu_mul(gate_up, act)
        ops.linear(act, self.w_down, out, fuse=fuse)
        ws.release(mark)
