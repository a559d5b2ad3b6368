"""Latent attention: keys and values of every head are projections of one low-rank row per token, and
only that row (the latent) is cached.

    q_h = Wq_h s                                    per head, `head_dim` wide; no position enters
    c   = rms(Wdkv s) * w_c                         the latent, `kv_rank` wide, RMS-normed in float
    k_h = Wuk_h c,  v_h = Wuv_h c                   `head_dim` and `v_head_dim` wide
    p   = softmax_j((q_h . k_h[j]) * scale),  j in the window (the query's own position included)
    out = Wo (concat_h(sum_j p v_h[j]) * sigmoid(Wg s))

Since q_h . (Wuk_h c) = (Wuk_h^T q_h) . c and sum_j p (Wuv_h c_j) = Wuv_h (sum_j p c_j), the queries are
moved into the latent space, attention runs against the cached rows themselves (multi-query attention
with one row per token that is key and value at once, PagedKVSpec.planes = 1, on the engine's paged
attention kernels), and its result is moved out again; keys and values are never formed.

A layer may read another layer's cached latents (a run-order entry with ``writes_cache`` False): it then
has no down-projection of its own (``owns_latent`` False), but its own queries, window and up-projections.
``cache_window`` is the window the cache layer is kept for (the widest of its readers).  The reference
has no such mixer (its one mixer is src/layers/attention.cpp).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.model_spec import PartSpec
from ..csrc import ops
from . import position as _position  # noqa: F401  (registers the position encodings)
from .attention import PagedAttentionKernels
from .base import POSITION_ENCODINGS, PagedKVSpec, ParamSpec, build_part, register_mixer, workspace_piece


@register_mixer("latent_attention")
class LatentAttention(PagedAttentionKernels):
    planes = 1

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, kv_rank: int, scale: float,
                 window: int, cache_window: int, owns_latent: bool, eps: float, output_gate: bool, dtype, device):
        if min(hidden_size, num_heads, head_dim, v_head_dim, kv_rank) <= 0:
            raise ValueError("latent_attention: sizes must be positive")
        if kv_rank > ops.SIMT_MAX_HEAD_DIM:
            raise ValueError(f"latent_attention: kv_rank {kv_rank} exceeds {ops.SIMT_MAX_HEAD_DIM}, the widest row the attention kernels take")
        if window < 0 or cache_window < 0 or (cache_window and (window == 0 or window > cache_window)):
            raise ValueError("latent_attention: the cache must be kept for at least the mixer's window")
        if not eps > 0:
            raise ValueError("latent_attention: eps must be positive")
        self.hidden, self.heads, self.qk, self.vd, self.rank = hidden_size, num_heads, head_dim, v_head_dim, kv_rank
        # as the attention kernels see it: every head reads the one cached row of a token
        self.nh, self.nkv, self.d = num_heads, 1, kv_rank
        self.scale, self.window, self.cache_window = float(scale), int(window), int(cache_window)
        self.owns_latent, self.eps, self.output_gate = bool(owns_latent), float(eps), bool(output_gate)
        self.dtype, self.device = dtype, device
        self.w_in = None          # [q | dkv | g] rows: one product on the mixer's input
        self.w_c = None           # gain of the latent's norm
        self.w_uk_t = None        # [heads, kv_rank, head_dim]: Wuk_h^T
        self.w_uv = None          # [heads, v_head_dim, kv_rank]
        self.w_o = None

    # -- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        h = self.heads
        specs = {"q": ParamSpec((h * self.qk, self.hidden))}
        if self.owns_latent:
            specs["dkv"] = ParamSpec((self.rank, self.hidden))
            specs["dkv.norm"] = ParamSpec((self.rank,), "gain")
        specs["uk"] = ParamSpec((h * self.qk, self.rank))
        specs["uv"] = ParamSpec((h * self.vd, self.rank))
        if self.output_gate:
            specs["g"] = ParamSpec((h * self.vd, self.hidden))
        specs["o"] = ParamSpec((self.hidden, h * self.vd))
        return specs

    def load_params(self, tensors):
        rows = [tensors["q"]] + ([tensors["dkv"]] if self.owns_latent else []) + ([tensors["g"]] if self.output_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_c = tensors["dkv.norm"].contiguous() if self.owns_latent else None
        self.w_uk_t = tensors["uk"].unflatten(0, (self.heads, self.qk)).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].unflatten(0, (self.heads, self.vd)).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.warn_if_plain()

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    # -- cache
    def cache_spec(self):
        return PagedKVSpec(1, self.rank, self.cache_window, planes=1)

    def workspace_bytes(self, n_tokens, n_reqs):
        h = self.heads
        return (workspace_piece((n_tokens, self.w_rows()), self.dtype) + 2 * workspace_piece((n_tokens, h * self.rank), self.dtype)
                + workspace_piece((n_tokens, h * self.vd), self.dtype))

    def w_rows(self) -> int:
        return self.heads * self.qk + (self.rank if self.owns_latent else 0) + (self.heads * self.vd if self.output_gate else 0)

    # -- run
    def forward(self, x, out, step, cache, writes_cache, ws):
        if writes_cache != self.owns_latent:
            raise ValueError("latent_attention: a layer writes the cache layer it reads exactly when it has a down-projection")
        n, h = x.shape[0], self.heads
        mark = ws.mark()
        proj = ws.take((n, self.w_rows()), self.dtype)
        ops.linear(x, self.w_in, proj)
        q0 = h * self.qk
        g0 = q0 + (self.rank if self.owns_latent else 0)
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        if self.owns_latent:
            ops.latent_cache_write(proj[:, q0:g0], self.w_c, step.positions, step.req_of_token, block_table, pages,
                                   page_size=cache.page_size, eps=self.eps)
        q_lat = ws.take((n, h * self.rank), self.dtype)
        ops.headwise_linear(proj[:, :q0], self.w_uk_t, q_lat)
        o_lat = ws.take((n, h * self.rank), self.dtype)
        self.attend(q_lat, o_lat, step, cache, block_table)
        o = ws.take((n, h * self.vd), self.dtype)
        ops.headwise_linear(o_lat, self.w_uv, o, gate=proj[:, g0:] if self.output_gate else None)
        ops.linear(o, self.w_o, out)
        ws.release(mark)


@register_mixer("rotary_latent_attention")
class RotaryLatentAttention(PagedAttentionKernels):
    """Latent attention whose positions enter through one rotated key part that all heads share, with queries that may
    come through a normed low-rank row themselves:

        c_q = rms(Wdq s) * w_q,  q_h = Wuq_h c_q        (``q_rank`` 0: q_h = Wq_h s); a head's query is laid out
                                                          [head_dim plain | rot_dim rotated]
        [c_raw | kr] = Wdkv s;  c = rms(c_raw) * w_c      the latent, ``kv_rank`` wide; kr, ``rot_dim`` wide, is not normed
        score_h(i, j) = scale * (q_h,plain . (Wuk_h c_j) + rot(q_h,rot, i) . rot(kr_j, j))
        out = Wo concat_h(sigmoid(gate) * sum_j softmax_j(score_h) Wuv_h c_j)

    ``position`` is a rotation with given frequencies (parts/position.py "scaled_rope": its ``inv_freq`` and pairing) over
    ``rot_dim`` coordinates.  ``gate``: "head" (W_g has one row per head), "channel" (one per output channel) or "none".
    Only [c | rot(kr)] is cached, one row of kv_rank + rot_dim per token (PagedKVSpec.planes = 1): the plain query part is
    moved into the latent space and the rotated part rides along, both by one per-head product with the block matrix
    [[Wuk_h^T, 0], [0, I]], so that attention is multi-query attention over the cached rows; its result leaves the latent
    space by Wuv_h (zero columns where the rotated part sat), with the gate in that product's epilogue."""
    planes = 1
    GATES = ("head", "channel", "none")

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int, q_rank: int,
                 scale: float, eps: float, position: PartSpec, dtype, device, gate: str = "head", window: int = 0):
        if min(hidden_size, num_heads, head_dim, v_head_dim, kv_rank) <= 0 or q_rank < 0 or rot_dim < 0 or rot_dim % 2:
            raise ValueError("rotary_latent_attention: sizes must be positive, rot_dim even")
        if kv_rank + rot_dim > ops.SIMT_MAX_HEAD_DIM:
            raise ValueError(f"rotary_latent_attention: kv_rank + rot_dim exceeds {ops.SIMT_MAX_HEAD_DIM}, the widest row the attention kernels take")
        if gate not in self.GATES or window < 0 or not eps > 0:
            raise ValueError(f"rotary_latent_attention: gate one of {self.GATES}, window not negative, eps positive")
        self.hidden, self.heads, self.qk, self.rot, self.vd = hidden_size, num_heads, head_dim, rot_dim, v_head_dim
        self.rank, self.q_rank = kv_rank, q_rank
        self.nh, self.nkv, self.d = num_heads, 1, kv_rank + rot_dim        # as the attention kernels see it
        self.scale, self.window, self.eps, self.gate = float(scale), int(window), float(eps), gate
        self.dtype, self.device = dtype, device
        self.position = build_part(POSITION_ENCODINGS, "position encoding", position, dtype=dtype, device=device)
        self.pairing, self.inv_freq = 0, None
        if rot_dim:
            fused = self.position.fused()
            if fused is None or fused["rotary_dim"] != rot_dim or not hasattr(self.position, "inv_freq"):
                raise ValueError("rotary_latent_attention: the position encoding must rotate rot_dim coordinates with given frequencies")
            self.pairing, self.inv_freq = int(fused["pairing"]), self.position.inv_freq
        self.w_in = self.w_uq = self.w_qn = self.w_c = self.w_qk = self.w_uv = self.w_o = None

    # -- tensors
    def score_shaping(self):
        # attention weights are wanted in 32-bit: the tensor-core kernels take them as two bfloat16 terms
        return {"precise_weights": True}

    def gate_rows(self) -> int:
        return {"head": self.heads, "channel": self.heads * self.vd, "none": 0}[self.gate]

    def param_specs(self) -> Dict[str, ParamSpec]:
        h, qd = self.heads, self.qk + self.rot
        specs = {}
        if self.q_rank:
            specs.update({"dq": ParamSpec((self.q_rank, self.hidden)), "dq.norm": ParamSpec((self.q_rank,), "gain"),
                          "uq": ParamSpec((h * qd, self.q_rank))})
        else:
            specs["q"] = ParamSpec((h * qd, self.hidden))
        specs.update({"dkv": ParamSpec((self.rank + self.rot, self.hidden)), "dkv.norm": ParamSpec((self.rank,), "gain"),
                      "uk": ParamSpec((h * self.qk, self.rank)), "uv": ParamSpec((h * self.vd, self.rank))})
        if self.gate != "none":
            specs["g"] = ParamSpec((self.gate_rows(), self.hidden))
        specs["o"] = ParamSpec((self.hidden, h * self.vd))
        return specs

    def load_params(self, tensors):
        rows = [tensors["dq"] if self.q_rank else tensors["q"], tensors["dkv"]] + ([tensors["g"]] if self.gate != "none" else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        if self.q_rank:
            self.w_uq, self.w_qn = tensors["uq"].contiguous(), tensors["dq.norm"].contiguous()
        self.w_c = tensors["dkv.norm"].contiguous()
        h, qd = self.heads, self.qk + self.rot
        uk = tensors["uk"].unflatten(0, (h, self.qk))                     # [h, qk, rank]
        w_qk = torch.zeros((h, self.d, qd), dtype=uk.dtype, device=uk.device)
        w_qk[:, :self.rank, :self.qk] = uk.transpose(1, 2)
        if self.rot:
            w_qk[:, self.rank:, self.qk:] = torch.eye(self.rot, dtype=uk.dtype, device=uk.device)
        self.w_qk = w_qk.contiguous()                                      # per head [[Wuk^T, 0], [0, I]]
        w_uv = torch.zeros((h, self.vd, self.d), dtype=uk.dtype, device=uk.device)
        w_uv[:, :, :self.rank] = tensors["uv"].unflatten(0, (h, self.vd))
        self.w_uv = w_uv.contiguous()
        self.w_o = tensors["o"].contiguous()
        self._no_freq = torch.zeros(0, dtype=torch.float32, device=self.w_c.device)
        self.warn_if_plain()

    def tensors(self):
        return super().tensors() + self.position.tensors()

    def product_weights(self):
        return [(self.w_in, 0)] + ([(self.w_uq, 0)] if self.q_rank else []) + [(self.w_o, 0)]

    # -- cache
    def cache_spec(self):
        return PagedKVSpec(1, self.d, self.window, planes=1)

    def w_rows(self) -> int:
        return (self.q_rank or self.heads * (self.qk + self.rot)) + self.rank + self.rot + self.gate_rows()

    def workspace_bytes(self, n_tokens, n_reqs):
        h = self.heads
        return (workspace_piece((n_tokens, self.w_rows()), self.dtype) + workspace_piece((n_tokens, max(self.q_rank, 1)), self.dtype)
                + workspace_piece((n_tokens, h * (self.qk + self.rot)), self.dtype) + 2 * workspace_piece((n_tokens, h * self.d), self.dtype)
                + workspace_piece((n_tokens, h * self.vd), self.dtype))

    # -- run
    def forward(self, x, out, step, cache, writes_cache, ws):
        n, h, qd = x.shape[0], self.heads, self.qk + self.rot
        mark = ws.mark()
        proj = ws.take((n, self.w_rows()), self.dtype)
        ops.linear(x, self.w_in, proj)
        q0 = self.q_rank or h * qd
        g0 = q0 + self.rank + self.rot
        if self.q_rank:
            cq = ws.take((n, self.q_rank), self.dtype)
            ops.rows_rmsnorm(proj[:, :q0], self.w_qn, cq, self.eps)
            q = ws.take((n, h * qd), self.dtype)
            ops.linear(cq, self.w_uq, q)
        else:
            q = proj[:, :q0]
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        inv_freq = self.inv_freq if self.rot else self._no_freq
        ops.latent_rope_cache_write(proj[:, q0:g0], self.w_c, q if self.rot else None, inv_freq, step.positions, step.req_of_token,
                                    block_table, pages, rank=self.rank, num_heads=h, q_stride=qd, q_off=self.qk,
                                    pairing=self.pairing, page_size=cache.page_size, eps=self.eps, write_kv=writes_cache)
        q_lat = ws.take((n, h * self.d), self.dtype)
        ops.headwise_linear(q, self.w_qk, q_lat)
        o_lat = ws.take((n, h * self.d), self.dtype)
        self.attend(q_lat, o_lat, step, cache, block_table)
        o = ws.take((n, h * self.vd), self.dtype)
        gate = proj[:, g0:] if self.gate != "none" else None
        ops.headwise_linear(o_lat, self.w_uv, o, gate=gate, gate_per_head=self.gate == "head")
        ops.linear(o, self.w_o, out)
        ws.release(mark)
