"""Grouped-query attention over the paged cache whose heads talk to one another before the softmax, without
rotation and without a value projection:

    q = W_q h,  k = W_k h                            heads of ``head_dim``; query head g reads kv head g // (heads / kv_heads)
    v = k                                            the unnormed key projection doubles as the value
    qn, kn = q, k divided by their root mean square per head (eps inside the root; no gain)
    raw_g(i, j) = scale * (qn_i,g . kn_j) - slope_g * (i - j),   slope_g = 2^(-slope_span * (g + 1) / heads)
    s_h(i, j)   = sum_g talk[h, g] * raw_g(i, j)     the heads' scores mixed by a learned heads x heads matrix
    out = W_o (concat_h(softmax_j(s_h) v) * sigmoid(W_g h))

``slope_span`` 0 switches the distance bias off, ``talk`` False the mixing (the identity is used), ``qk_norm`` False
the division, ``output_gate`` False the gate; ``window`` > 0 restricts a query to the last ``window`` keys.  The cache
holds the normed keys in its key plane and the unnormed key projection in its value plane.  q, k and the gate are one product;
the norms and the cache write are the kernel that attention with head norms uses (csrc/attention_biased.cu,
qk_head_rope_cache_write_kernel with a gain of ones and no rotation); attention is csrc/attention_talking.cu: in
bfloat16 with up to 16 heads of 64 or 128 the tensor-core kernel over work items that the host lists per step (16 query
rows of a request each; in steps of single tokens a request's keys are cut into runs that fill the device, joined by a
second kernel), otherwise the plain kernel.  Scores, bias, mixing, softmax and the weighted sums are float in both
precisions; the tensor cores take the weights as two bfloat16 terms.  The reference's attention
(src/layers/attention.cpp) has independent heads, rotation and a value projection.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, ParamSpec, register_mixer, workspace_piece


def distance_slopes(heads: int, span: float) -> np.ndarray:
    """slope_g = 2^(-span * (g + 1) / heads) for g = 0 .. heads - 1, in double."""
    return np.power(2.0, -float(span) * (np.arange(heads, dtype=np.float64) + 1.0) / heads)


@register_mixer("talking_heads_attention")
class TalkingHeadsAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float, eps: float, dtype, device,
                 slope_span: float = 8.0, talk: bool = True, qk_norm: bool = True, output_gate: bool = True, window: int = 0):
        if min(hidden_size, num_heads, num_kv_heads, head_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"talking_heads_attention: {num_heads} heads cannot share {num_kv_heads} kv heads")
        if num_heads > ops.TALKING_MAX_HEADS or head_dim > 256:
            raise ValueError(f"talking_heads_attention: at most {ops.TALKING_MAX_HEADS} heads of at most 256")
        if window < 0 or slope_span < 0 or not eps > 0:
            raise ValueError("talking_heads_attention: window and slope_span must not be negative, eps positive")
        self.hidden, self.nh, self.nkv, self.d = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.eps, self.window, self.slope_span = float(scale), float(eps), int(window), float(slope_span)
        self.talk, self.qk_norm, self.output_gate = bool(talk), bool(qk_norm), bool(output_gate)
        self.dtype, self.device = dtype, device
        self.w_in = self.w_o = self.mix = self.slopes = self.ones = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q": ParamSpec((self.nh * self.d, self.hidden)), "k": ParamSpec((self.nkv * self.d, self.hidden))}
        if self.talk:
            specs["talk"] = ParamSpec((self.nh, self.nh), "identity")
        if self.output_gate:
            specs["g"] = ParamSpec((self.nh * self.d, self.hidden))
        specs["o"] = ParamSpec((self.hidden, self.nh * self.d))
        return specs

    def load_params(self, tensors):
        rows = [tensors["q"], tensors["k"]] + ([tensors["g"]] if self.output_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        dev = self.w_o.device
        self.mix = (tensors["talk"].to(torch.float32) if self.talk else torch.eye(self.nh, dtype=torch.float32, device=dev)).contiguous()
        self.slopes = (torch.from_numpy(distance_slopes(self.nh, self.slope_span).astype(np.float32)).to(dev)
                       if self.slope_span > 0 else None)
        self.ones = torch.ones(self.d, dtype=torch.float32, device=dev) if self.qk_norm else None

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    # -- the tensor-core kernel's work lists
    def _tensor_core_path(self) -> bool:
        return self.dtype == torch.bfloat16 and ops.talking_mma_fits(self.nh, self.nkv, self.d)

    def _items_key(self) -> str:
        return f"talk_items_w{self.window}"

    SPLIT_LADDER = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)

    def step_arrays(self):
        """Work items of the tensor-core kernel, [items, 6] int32 (ops.attention_talking_mma).  Portions: tiles of 16 rows;
        a tile that sees many more keys than a CTA's fair share of the step (causal work is triangular) is cut along its
        keys into items of equal runs, each with a slot for its partial sums, and listed in a second array
        [entries, 5] = (request, first row, rows, first slot, slots) for the kernel that joins them; the items that see the
        most keys go first.  A step of single tokens: every request's keys cut into as many runs (the same number for
        all, from a short ladder) as fill the device once with two CTAs an SM, a run being at least four key tiles.  The
        numbers of items, runs and entries are launch shapes of the step."""
        if not self._tensor_core_path():
            return {}
        key = self._items_key()

        def plan(host):
            if getattr(host, "_talk_plan", None) is not None and host._talk_plan[0] == key:
                return host._talk_plan[1:]
            rows, tile = ops.TALKING_ITEM_ROWS, ops.TALKING_KEY_TILE
            out, merges = [], []
            if all(q == 1 for q in host.q_lens):
                hi = [c + 1 for c in host.ctx_lens]
                lo = [max(0, h - self.window) if self.window > 0 else 0 for h in hi]
                longest = max(-(-(h - l) // tile) for h, l in zip(hi, lo))
                want = max(1, min(2 * ops.sm_count() // len(hi), longest // 4, ops.TALKING_MAX_SPLITS))
                nsplit = max(s for s in self.SPLIT_LADDER if s <= want)
                for r, (l, h) in enumerate(zip(lo, hi)):
                    per = -(-(-(-(h - l) // nsplit)) // tile) * tile           # keys of a run, whole tiles
                    for s in range(nsplit):
                        a, b = min(h, l + s * per), min(h, l + (s + 1) * per)
                        out.append((r, 0, 1, a, b, r * nsplit + s if nsplit > 1 else -1))
            else:
                nsplit = 1
                whole = []
                for r, (q, ctx) in enumerate(zip(host.q_lens, host.ctx_lens)):
                    for q0 in range(0, q, rows):
                        nq = min(rows, q - q0)
                        k_lo = max(0, ctx + q0 - self.window + 1) if self.window > 0 else 0
                        whole.append((r, q0, nq, k_lo, ctx + q0 + nq))
                tiles = [-(-(it[4] - it[3]) // tile) for it in whole]
                share = max(8, -(-sum(tiles) // ops.sm_count()))                # key tiles of a CTA if all had the same
                slots = 0
                for it, n in zip(whole, tiles):
                    parts = min(ops.TALKING_MAX_PARTS, -(-n // share)) if n > share + share // 4 else 1
                    if parts == 1 or slots + parts > self.max_wide_slots():
                        out.append(it + (-1,))
                        continue
                    per = -(-n // parts) * tile
                    for s in range(parts):
                        out.append((it[0], it[1], it[2], min(it[4], it[3] + s * per), min(it[4], it[3] + (s + 1) * per), slots + s))
                    merges.append((it[0], it[1], it[2], slots, parts))
                    slots += parts
                out.sort(key=lambda it: it[3] - it[4])                        # the longest first (a stable sort)
            host._talk_plan = (key, out, merges, nsplit)
            return out, merges, nsplit

        def items(host):
            out, merges, nsplit = plan(host)
            host.shapes[key] = len(out)
            host.shapes[key + "_runs"] = nsplit
            host.shapes[key + "_joins"] = len(merges)
            return np.asarray(out, dtype=np.int32).reshape(-1, ops.TALKING_ITEM_INTS)

        def joins(host):
            return np.asarray(plan(host)[1], dtype=np.int32).reshape(-1, 5)

        return {key: items, key + "_joins": joins}

    def max_wide_slots(self) -> int:
        """Most slots for partial sums of portions cut along their keys (each holds 16 rows of every head)."""
        return 2 * ops.sm_count()

    def reserve(self, n_tokens, n_reqs, device):
        if self._tensor_core_path():
            most = max(n_reqs * ops.TALKING_MAX_SPLITS, self.max_wide_slots() * ops.TALKING_ITEM_ROWS) * self.nh
            ops.scratch("talk_part_o", most * self.d, device)
            ops.scratch("talk_part_ml", most * 2, device)

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window)

    def in_width(self) -> int:
        return (self.nh + self.nkv) * self.d + (self.nh * self.d if self.output_gate else 0)

    def workspace_bytes(self, n_tokens, n_reqs):
        return workspace_piece((n_tokens, self.in_width()), self.dtype) + 2 * workspace_piece((n_tokens, self.nh * self.d), self.dtype)

    def forward(self, x, out, step, cache, writes_cache, ws):
        n = x.shape[0]
        mark = ws.mark()
        proj = ws.take((n, self.in_width()), self.dtype)
        ops.linear(x, self.w_in, proj)
        k_off = self.nh * self.d
        g_off = k_off + self.nkv * self.d
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        sizes = dict(num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.d, v_head_dim=self.d, row=self.d, page_size=cache.page_size)
        q = ws.take((n, self.nh * self.d), self.dtype)
        # keys normed per head into the key plane, the same keys, unnormed, into the value plane
        ops.qk_head_rope_cache_write(proj, 0, k_off, k_off, self.ones, self.ones, None, q, pages, step.positions, step.req_of_token,
                                     block_table, eps=self.eps, write_kv=writes_cache, **sizes)
        attn = ws.take((n, self.nh * self.d), self.dtype)
        gate = proj[:, g_off:] if self.output_gate else None
        key = self._items_key()
        if self._tensor_core_path() and key in step.extras and key in step.shapes:
            nsplit = step.shapes[key + "_runs"]
            n_joins = step.shapes.get(key + "_joins", 0)
            part_o = part_ml = None
            if nsplit > 1 or n_joins:
                need = max(step.n_reqs * nsplit, self.max_wide_slots() * ops.TALKING_ITEM_ROWS if n_joins else 0) * self.nh
                part_o = ops.scratch("talk_part_o", need * self.d, q.device)
                part_ml = ops.scratch("talk_part_ml", need * 2, q.device)
            ops.attention_talking_mma(q, pages, attn, gate, step.extras[key], step.shapes[key], step.q_start, step.ctx_lens, block_table,
                                      self.mix, self.slopes, nsplit=nsplit, n_reqs=step.n_reqs, num_heads=self.nh,
                                      num_kv_heads=self.nkv, head_dim=self.d, page_size=cache.page_size, window=self.window,
                                      scale=self.scale, part_o=part_o, part_ml=part_ml, single_rows=step.decode_only,
                                      merge=step.extras.get(key + "_joins") if n_joins else None, n_merge=n_joins)
        else:
            ops.attention_talking(q, pages, attn, gate, step.positions, step.req_of_token, block_table, self.mix, self.slopes,
                                  window=self.window, scale=self.scale, **sizes)
        ops.linear(attn, self.w_o, out)
        ws.release(mark)
