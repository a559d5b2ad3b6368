"""Recurrent mixers whose inputs pass a short causal convolution: a real-gated linear recurrent unit and the gated
delta rule.  Both keep, per request, the recurrence's state and the convolution's last inputs in slots of the cache
manager (StateSpec; zero at admission, which is also "zeros before the start" for the convolution), read them at the
start of a request's portion and leave them at its end, so a prompt may be cut anywhere.

"rglru": two branches of ``width`` channels,
    y = gelu_tanh(W_y h + b_y),   u = conv(W_x h + b_x) + b_conv            (per channel, ``taps`` long, causal)
    r = sigmoid(A_b u_b + a_b),   i = sigmoid(I_b u_b + i_b)                 per block b of width / blocks channels
    a = exp(-c r softplus(lam)),  S_t = a S_(t-1) + sqrt(1 - a^2) i u,       out = W_o (S_t * y)
with c = ``gate_constant``.  State: S [width] and the convolution's taps - 1 inputs, one StateSpec of taps rows.

"gated_delta": q = W_q h, k = W_k h (``num_qk_heads`` heads of ``head_dim``), v = W_v h (``num_heads`` x ``v_head_dim``),
each through its own causal convolution and silu; q and k made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q
times head_dim^(-1/2); beta = sigmoid(W_b h) per head; a decay per head and key channel
g = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias)); per head (head h reads qk head h // (heads / qk heads))
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
then o RMS-normed per head with one gain vector, times sigmoid(W_g2 (W_g1 h)), then W_o.  State: S [heads, dk, dv] and
the convolutions' inputs [taps - 1, channels of q, k and v].

Everything between the projections and the recurrence's result is float32 in both precisions (csrc/gated_recurrence.cu).
The reference has no recurrent mixer (src/layers/attention.cpp is its only one).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import CompositeSpec, Mixer, ParamSpec, StateSpec, register_mixer, workspace_piece

DEFAULT_LOW_RANK = 32        # inner width of the low-rank products where no checkpoint gives it (random weights)
UNIT_NORM_EPS = 1e-6


@register_mixer("rglru")
class RealGatedLinearRecurrence(Mixer):
    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, dtype, device, gate_constant: float = 8.0):
        if min(hidden_size, width, blocks) <= 0 or width % blocks:
            raise ValueError(f"rglru: width {width} is no multiple of its {blocks} blocks")
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"rglru: a convolution of 1 to {ops.CONV_MAX_TAPS} taps, got {taps}")
        self.hidden, self.width, self.blocks, self.taps, self.c = hidden_size, width, blocks, taps, float(gate_constant)
        self.dtype, self.device = dtype, device
        self.w_in = self.w_o = self.b_y = self.b_x = self.conv = self.conv_b = None
        self.w_ra = self.w_ri = self.b_ra = self.b_ri = self.lam = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        W, B, D = self.width, self.blocks, self.hidden
        bs = W // B
        return {"y": ParamSpec((W, D)), "y.b": ParamSpec((W,), "bias"), "x": ParamSpec((W, D)), "x.b": ParamSpec((W,), "bias"),
                "conv": ParamSpec((W, self.taps), "bias"), "conv.b": ParamSpec((W,), "bias"),
                "ra": ParamSpec((B, bs, bs)), "ra.b": ParamSpec((B, bs), "bias"),
                "ri": ParamSpec((B, bs, bs)), "ri.b": ParamSpec((B, bs), "bias"),
                "lam": ParamSpec((W,), "bias"), "o": ParamSpec((D, W))}

    def load_params(self, t):
        self.w_in = torch.cat([t["y"], t["x"]], dim=0).contiguous()
        self.b_y, self.b_x = t["y.b"].contiguous(), t["x.b"].contiguous()
        self.conv, self.conv_b = t["conv"].contiguous(), t["conv.b"].contiguous()
        self.w_ra, self.w_ri = t["ra"].contiguous(), t["ri"].contiguous()
        self.b_ra, self.b_ri = t["ra.b"].reshape(-1).contiguous(), t["ri.b"].reshape(-1).contiguous()
        self.lam = t["lam"].contiguous()
        self.w_o = t["o"].contiguous()

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    def cache_spec(self):
        # row 0: the recurrence's state; rows 1 .. taps - 1: the convolution's last inputs, oldest first
        return StateSpec((self.taps, self.width), torch.float32)

    def workspace_bytes(self, n_tokens, n_reqs):
        W = self.width
        return (workspace_piece((n_tokens, 2 * W), self.dtype) + 3 * workspace_piece((n_tokens, W), torch.float32)
                + workspace_piece((n_tokens, W), self.dtype))

    def forward(self, x, out, step, cache, writes_cache, ws):
        n, W = x.shape[0], self.width
        mark = ws.mark()
        proj = ws.take((n, 2 * W), self.dtype)
        ops.linear(x, self.w_in, proj)
        u = ws.take((n, W), torch.float32)
        slots = cache.slots                                   # [slots, taps, W]
        ops.causal_conv(proj[:, W:], self.conv, slots[:, 1:], u, step.q_start, step.state_slots, step.n_reqs, step.max_q_len,
                        pre_bias=self.b_x, bias=self.conv_b)
        decay = ws.take((n, W), torch.float32)
        drive = ws.take((n, W), torch.float32)
        ops.gate_blocks(u, self.w_ra, self.w_ri, self.b_ra, self.b_ri, self.lam, decay, drive, self.c)
        act = ws.take((n, W), self.dtype)
        ops.linear_recurrence(decay, drive, proj[:, :W], self.b_y, slots[:, 0], act, step.q_start, step.state_slots, step.n_reqs,
                              step.max_q_len)
        ops.linear(act, self.w_o, out)
        ws.release(mark)


@register_mixer("gated_delta")
class GatedDeltaRule(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int, taps: int, eps: float,
                 dtype, device):
        if min(hidden_size, num_heads, num_qk_heads, head_dim, v_head_dim) <= 0 or num_heads % num_qk_heads:
            raise ValueError(f"gated_delta: {num_heads} heads cannot share {num_qk_heads} query/key heads")
        if head_dim > 1024:
            raise ValueError("gated_delta: key heads of up to 1024 channels")
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"gated_delta: convolutions of 1 to {ops.CONV_MAX_TAPS} taps, got {taps}")
        if not eps > 0:
            raise ValueError("gated_delta: eps must be positive")
        self.hidden, self.H, self.G, self.dk, self.dv, self.taps, self.eps = (hidden_size, num_heads, num_qk_heads, head_dim,
                                                                              v_head_dim, taps, float(eps))
        self.dtype, self.device = dtype, device
        self.rank_a = self.rank_g = None      # inner widths of the low-rank products: the checkpoint's tensors give them
        self.w_in = self.w_a2 = self.w_g2 = self.w_o = self.conv = self.a_log = self.dt_bias = self.w_norm = None

    @property
    def conv_channels(self) -> int:
        return 2 * self.G * self.dk + self.H * self.dv

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, vv, D, r, J = self.G * self.dk, self.H * self.dv, self.hidden, DEFAULT_LOW_RANK, self.taps
        return {"q": ParamSpec((qk, D)), "q.conv": ParamSpec((qk, J), "bias"), "k": ParamSpec((qk, D)), "k.conv": ParamSpec((qk, J), "bias"),
                "v": ParamSpec((vv, D)), "v.conv": ParamSpec((vv, J), "bias"), "b": ParamSpec((self.H, D)),
                "A_log": ParamSpec((self.H,), "bias"), "norm": ParamSpec((self.dv,), "gain"),
                "a1": ParamSpec((-1, D), default_shape=(r, D)), "a2": ParamSpec((self.H * self.dk, -1), default_shape=(self.H * self.dk, r)),
                "dt_bias": ParamSpec((self.H * self.dk,), "bias"),
                "g1": ParamSpec((-1, D), default_shape=(r, D)), "g2": ParamSpec((vv, -1), default_shape=(vv, r)),
                "o": ParamSpec((D, vv))}

    def load_params(self, t):
        if t["a1"].shape[0] != t["a2"].shape[1] or t["g1"].shape[0] != t["g2"].shape[1]:
            raise ValueError(f"gated_delta: the low-rank products do not fit: a1 {tuple(t['a1'].shape)}, a2 {tuple(t['a2'].shape)}, "
                             f"g1 {tuple(t['g1'].shape)}, g2 {tuple(t['g2'].shape)}")
        self.rank_a, self.rank_g = int(t["a1"].shape[0]), int(t["g1"].shape[0])
        self.w_in = torch.cat([t[n] for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
        self.conv = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).contiguous()
        self.w_a2, self.w_g2 = t["a2"].contiguous(), t["g2"].contiguous()
        self.a_log, self.dt_bias = t["A_log"].contiguous(), t["dt_bias"].contiguous()
        self.w_norm = t["norm"].contiguous()
        self.w_o = t["o"].contiguous()

    def product_weights(self):
        return [(self.w_in, 0), (self.w_a2, 0), (self.w_g2, 0), (self.w_o, 0)]

    def cache_spec(self):
        return CompositeSpec((StateSpec((self.H, self.dk, self.dv), torch.float32),
                              StateSpec((max(1, self.taps - 1), self.conv_channels), torch.float32)))

    def in_width(self) -> int:
        ra = self.rank_a if self.rank_a is not None else DEFAULT_LOW_RANK
        rg = self.rank_g if self.rank_g is not None else DEFAULT_LOW_RANK
        return self.conv_channels + self.H + ra + rg

    def workspace_bytes(self, n_tokens, n_reqs):
        vv = self.H * self.dv
        return (workspace_piece((n_tokens, self.in_width()), self.dtype) + workspace_piece((n_tokens, self.conv_channels), torch.float32)
                + workspace_piece((n_tokens, self.H * self.dk), self.dtype) + 2 * workspace_piece((n_tokens, vv), self.dtype)
                + workspace_piece((n_tokens, vv), torch.float32)
                + workspace_piece((n_tokens, ops.gated_delta_work_row(self.H, self.G, self.dk)), torch.float32))

    def forward(self, x, out, step, cache, writes_cache, ws):
        n, H, G, dk, dv, C = x.shape[0], self.H, self.G, self.dk, self.dv, self.conv_channels
        matrix, window = cache.views
        mark = ws.mark()
        proj = ws.take((n, self.in_width()), self.dtype)
        ops.linear(x, self.w_in, proj)
        beta_pre = proj[:, C: C + H]
        low_a = proj[:, C + H: C + H + self.rank_a]
        low_g = proj[:, C + H + self.rank_a:]
        decay_pre = ws.take((n, H * dk), self.dtype)
        ops.linear(low_a, self.w_a2, decay_pre)
        gate_pre = ws.take((n, H * dv), self.dtype)
        ops.linear(low_g, self.w_g2, gate_pre)
        qkv = ws.take((n, C), torch.float32)
        ops.causal_conv(proj[:, :C], self.conv, window.slots, qkv, step.q_start, step.state_slots, step.n_reqs, step.max_q_len,
                        act="silu")
        o = ws.take((n, H * dv), torch.float32)
        work = ws.take((n, ops.gated_delta_work_row(H, G, dk)), torch.float32) if step.max_q_len >= ops.DELTA_PORTIONS_FROM else None
        ops.gated_delta_scan(qkv[:, : G * dk], qkv[:, G * dk: 2 * G * dk], qkv[:, 2 * G * dk:], beta_pre, decay_pre, self.a_log,
                             self.dt_bias, matrix.slots, o, step.q_start, step.state_slots, step.n_reqs, num_heads=H,
                             num_qk_heads=G, q_scale=float(dk) ** -0.5, unit_eps=UNIT_NORM_EPS, max_q_len=step.max_q_len, work=work)
        act = ws.take((n, H * dv), self.dtype)
        ops.gated_group_norm(o, gate_pre, self.w_norm, act, group=dv, eps=self.eps, gate_act="sigmoid")
        ops.linear(act, self.w_o, out)
        ws.release(mark)
