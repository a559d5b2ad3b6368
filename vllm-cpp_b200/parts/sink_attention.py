"""Grouped-query attention over the paged cache with a sink in its softmax and a gate per head:

    q = rms_head(W_q h) * w_q,  k = rms_head(W_k h) * w_k     RMS norm head by head over ``head_dim``, one gain vector for all heads
    q, k rotated by position (any registered rotary encoding with ``inv_freq``; "none": no rotation)
    v = W_v h                                                 heads of ``v_head_dim``, which may differ from ``head_dim``
    p(i, j) = exp(scale * q_i . k_j) / (sum_{j' <= i} exp(scale * q_i . k_j') + exp(sink_head))
    out = W_o concat_heads(sigmoid(W_g h)_head * sum_j p(i, j) v_j)

The sink is a learned logit per head that takes part in the denominator only: it has no key and no value, is not
scaled, and counts once.  ``window`` > 0 restricts the keys to the last ``window``.  q, k, v and the gate are one product;
norm, rotation and the cache write are one kernel (csrc/attention_biased.cu, qk_head_rope_cache_write_kernel); bfloat16
heads of 64 or 128 with keys as wide as values run the tensor-core kernels (csrc/attention_mma.cu: tcgen05 for portions,
split-KV for single tokens) with the sink and the gate in their epilogues and, with ``precise_weights``, the softmax
weights as two bfloat16 terms in the product with the values (the weights are float up to there; one term would round them
to 8 bits of mantissa); everything else runs the plain paged kernel of attention_biased.cu, whose weights stay float.  The cache holds rows of
max(head_dim, v_head_dim) elements.  The reference's attention (src/layers/attention.cpp) has rotation and none of the
rest.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.model_spec import PartSpec
from ..csrc import ops
from .attention import PagedAttentionKernels
from .base import POSITION_ENCODINGS, PagedKVSpec, ParamSpec, build_part, register_mixer, workspace_piece


@register_mixer("sink_attention")
class SinkAttention(PagedAttentionKernels):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 eps: float, position: PartSpec, dtype, device, window: int = 0, qk_norm: bool = True, sink: bool = True,
                 head_gate: bool = True, precise_weights: bool = True):
        if min(hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"sink_attention: {num_heads} heads cannot share {num_kv_heads} kv heads")
        if v_head_dim > 256 or head_dim > 1024:
            raise ValueError("sink_attention: head sizes up to 1024 (keys) and 256 (values)")
        if window < 0 or not eps > 0:
            raise ValueError("sink_attention: window must not be negative, eps positive")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim
        self.row = max(head_dim, v_head_dim)
        self.d = self.row
        self.scale, self.window, self.eps = float(scale), int(window), float(eps)
        self.qk_norm, self.has_sink, self.head_gate = bool(qk_norm), bool(sink), bool(head_gate)
        self.precise_weights = bool(precise_weights)
        self.dtype, self.device = dtype, device
        self.position = build_part(POSITION_ENCODINGS, "position encoding", position, dtype=dtype, device=device)
        fused = self.position.fused()
        if fused is None or (fused["rotary_dim"] and (fused["pairing"] != 0 or not hasattr(self.position, "inv_freq"))):
            raise ValueError("sink_attention: positions enter by a rotation of half-split pairs with given frequencies, or not at all")
        self.rot = int(fused["rotary_dim"])
        if self.rot > head_dim:
            raise ValueError(f"sink_attention: {self.rot} rotated coordinates in heads of {head_dim}")
        self.inv_freq = self.position.inv_freq if self.rot else None
        self.w_in = self.w_o = self.w_qn = self.w_kn = self.sink = None

    def _tensor_core_path(self) -> bool:
        # bfloat16 heads of 64 and 128 with keys as wide as values: the tensor-core kernels, sink and gate in their epilogues
        return self.dk == self.dv and super()._tensor_core_path()

    def score_shaping(self):
        # the design wants its attention weights in 32-bit: the tensor-core kernels take them as two bfloat16 terms
        return dict({"sink": self.sink} if self.has_sink else {}, precise_weights=self.precise_weights)

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q": ParamSpec((self.nh * self.dk, self.hidden)), "k": ParamSpec((self.nkv * self.dk, self.hidden)),
                 "v": ParamSpec((self.nkv * self.dv, self.hidden))}
        if self.qk_norm:
            specs["q.norm"] = ParamSpec((self.dk,), "gain")
            specs["k.norm"] = ParamSpec((self.dk,), "gain")
        if self.has_sink:
            specs["sink"] = ParamSpec((self.nh,), "bias")
        if self.head_gate:
            specs["g"] = ParamSpec((self.nh, self.hidden))
        specs["o"] = ParamSpec((self.hidden, self.nh * self.dv))
        return specs

    def load_params(self, tensors):
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.head_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        if self.qk_norm:
            self.w_qn, self.w_kn = tensors["q.norm"].contiguous(), tensors["k.norm"].contiguous()
        if self.has_sink:
            self.sink = tensors["sink"].contiguous()
        if self.dk == self.dv:
            self.warn_if_plain()

    def tensors(self):
        return super().tensors() + self.position.tensors()

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.row, self.window)

    def in_width(self) -> int:
        return self.nh * self.dk + self.nkv * (self.dk + self.dv) + (self.nh if self.head_gate else 0)

    def workspace_bytes(self, n_tokens, n_reqs):
        return (workspace_piece((n_tokens, self.in_width()), self.dtype) + workspace_piece((n_tokens, self.nh * self.dk), self.dtype)
                + workspace_piece((n_tokens, self.nh * self.dv), self.dtype))

    def forward(self, x, out, step, cache, writes_cache, ws):
        n = x.shape[0]
        mark = ws.mark()
        proj = ws.take((n, self.in_width()), self.dtype)
        ops.linear(x, self.w_in, proj)
        k_off = self.nh * self.dk
        v_off = k_off + self.nkv * self.dk
        g_off = v_off + self.nkv * self.dv
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        sizes = dict(num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.dk, v_head_dim=self.dv, row=self.row,
                     page_size=cache.page_size)
        q = ws.take((n, self.nh * self.dk), self.dtype)
        ops.qk_head_rope_cache_write(proj, 0, k_off, v_off, self.w_qn, self.w_kn, self.inv_freq, q, pages, step.positions,
                                     step.req_of_token, block_table, eps=self.eps, write_kv=writes_cache, **sizes)
        attn = ws.take((n, self.nh * self.dv), self.dtype)
        gate = proj[:, g_off:] if self.head_gate else None
        if self._tensor_core_path() and cache.page_size % 8 == 0:
            self.attend(q, attn, step, cache, block_table, head_gate=gate)
        else:
            ops.attention_biased(q, pages, attn, gate, step.positions, step.req_of_token, block_table, None, window=self.window,
                                 scale=self.scale, cap=0.0, sink=self.sink, gate_per_head=True, **sizes)
        ops.linear(attn, self.w_o, out)
        ws.release(mark)
