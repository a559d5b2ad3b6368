"""Arrangements of a layer's parts.

"prenorm":  x += m * mixer(norm_a(x));  x += m * feed_forward(norm_b(x))
(src/model/qwen.cpp:300-318, where m = 1; ``residual_mult`` in the arrangement's
constants gives another m).  Each addition is carried as a pending ``delta``
and performed, in float, inside the norm kernel that reads the sum next.

Where the parts on both sides of a norm say they can (``fuses_norm``) and the norm can be
split (``Norm.split``), no norm kernel runs: the product that ends the branch before the
norm adds its result to the residual stream, multiplies by the gain and leaves the rows'
sums of squares, and the product after the norm applies the factor (ops.ResidualNorm,
ops.RowScale).  That holds for the norm inside the layer and for the one the next layer
starts with.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Block, NormedInput, ScaledAddition, pending_mult, register_block, workspace_piece
from .mlp import NoFeedForward


@register_block("prenorm")
class PreNormBlock(Block):
    """``residual_mult`` (the arrangement's constant, 1 when absent) multiplies what both sublayers add to the stream; the
    product joins in one float multiply-add inside the norm kernel that reads the sum next.  With a factor other than 1
    the products' norm epilogues are not used.  A layer whose feed-forward is "none" has only the first line."""

    def __init__(self, params=None, **parts):
        super().__init__(params=params, **parts)
        self.mult = float(self.params.get("residual_mult", 1.0))
        self.has_ff = not isinstance(self.feed_forward, NoFeedForward)

    def _left(self):
        return True if self.mult == 1.0 else ScaledAddition(self.mult)

    def accepts_prenormed(self, n_tokens):
        if self.mult != 1.0 or not self.has_ff:
            return None
        return self.mixer_norm.split() if self.mixer.fuses_norm(n_tokens) else None

    def workspace_bytes(self, n_tokens, n_reqs, hidden, dtype):
        own = 2 * workspace_piece((n_tokens, hidden), dtype) \
            + workspace_piece((ops.sumsq_parts(hidden), n_tokens), torch.float32)
        return own + super().workspace_bytes(n_tokens, n_reqs, hidden, dtype)

    def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None):
        mark = ws.mark()
        n, hidden = residual.shape
        h = ws.take((n, hidden), delta.dtype)
        mixed = ws.take((n, hidden), delta.dtype)
        if isinstance(pending, ops.RowScale):
            x, scale_kw = delta, {"x_scale": pending}
        else:
            came = pending_mult(pending)               # norms of other makes know no factor; they are asked only for one
            self.mixer_norm.forward(residual, delta if pending else None, h, **({} if came == 1.0 else {"mult": came}))
            x, scale_kw = h, {}
        if not self.has_ff:
            self.mixer.forward(x, delta, step, cache, writes_cache, ws, **scale_kw)
            ws.release(mark)
            return self._left()
        inner = self.feed_forward_norm.split()
        if (self.mult != 1.0 or inner is None or carry is None
                or not (self.mixer.fuses_norm(n) and self.feed_forward.fuses_norm(n))):
            self.mixer.forward(x, mixed, step, cache, writes_cache, ws, **scale_kw)
            self.feed_forward_norm.forward(residual, mixed, h, **({} if self.mult == 1.0 else {"mult": self.mult}))
            self.feed_forward.forward(h, delta, step, ws)
            ws.release(mark)
            return self._left()
        # the mixer's last product ends its branch: residual += ..., mixed = residual * gain
        sumsq = ws.take((ops.sumsq_parts(hidden), n), torch.float32)
        ends = ops.ResidualNorm(residual, inner[0], sumsq, inner[1])
        self.mixer.forward(x, mixed, step, cache, writes_cache, ws, fuse=ends, **scale_kw)
        after = next_block.accepts_prenormed(n) if next_block is not None else None
        if after is None:
            self.feed_forward.forward(mixed, delta, step, ws, x_scale=ends.scale())
            ws.release(mark)
            return True
        # the feed-forward's last product does the same for the norm the next layer starts with
        came_in = pending.sumsq.data_ptr() if isinstance(pending, ops.RowScale) else None
        out_sumsq = carry[1] if came_in == carry[0].data_ptr() else carry[0]
        ends_layer = ops.ResidualNorm(residual, after[0], out_sumsq, after[1])
        self.feed_forward.forward(mixed, delta, step, ws, x_scale=ends.scale(), fuse=ends_layer)
        ws.release(mark)
        return ends_layer.scale()


@register_block("shift_gate_postnorm")
class ShiftGatePostNormBlock(Block):
    """Sublayers that read the residual stream itself and are normed on the way back:

        x += m * mixer_norm(mixer(shift(x)) * sigmoid(mixer_gate(x)))
        x += m * feed_forward_norm(feed_forward(x) * sigmoid(feed_forward_gate(x)))

    ``shift`` (a TokenShift) changes only what the mixer reads; the gates read the unshifted rows.
    ``m`` is the arrangement's constant ``residual_mult``.  Gate, norm and addition of a sublayer are one
    kernel (Norm.add_normed), which also hands the new rows to the next sublayer in the compute type.  A
    layer whose feed-forward is "none" has only the first line (its gate and norm slots are "none" too).
    The float32 path reads the residual stream directly; nothing is rounded on the way."""

    SLOTS = {"shift": "token_shift", "mixer": "mixer", "mixer_gate": "gate", "mixer_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_gate": "gate", "feed_forward_norm": "norm"}

    def __init__(self, params=None, **parts):
        super().__init__(params=params, **parts)
        self.mult = float(self.params.get("residual_mult", 1.0))
        self.has_ff = not isinstance(self.feed_forward, NoFeedForward)

    def workspace_bytes(self, n_tokens, n_reqs, hidden, dtype):
        return 4 * workspace_piece((n_tokens, hidden), dtype) + super().workspace_bytes(n_tokens, n_reqs, hidden, dtype)

    def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None, state=None):
        if isinstance(pending, ops.RowScale):
            raise ValueError("shift_gate_postnorm takes the residual stream as it is")
        if pending:
            residual.add_(delta)                  # an arrangement before this one left its last addition to its successor
        if state is None:
            raise ValueError("shift_gate_postnorm needs the state layer of its token shift (LayerCall.state)")
        mark = ws.mark()
        n, hidden = residual.shape
        dtype = delta.dtype
        exact = dtype == torch.float32
        shifted = ws.take((n, hidden), dtype)
        plain = None if exact else ws.take((n, hidden), dtype)
        self.shift.forward(residual, shifted, plain, step, state)
        x = residual if exact else plain
        pre = ws.take((n, hidden), dtype)
        y = ws.take((n, hidden), dtype)
        self.mixer_gate.forward(x, pre)
        self.mixer.forward(shifted, y, step, cache, writes_cache, ws)
        self.mixer_norm.add_normed(y, pre, self.mixer_gate.bias, residual, plain if self.has_ff else None, self.mult)
        if self.has_ff:
            self.feed_forward_gate.forward(x, pre)
            self.feed_forward.forward(x, y, step, ws)
            self.feed_forward_norm.add_normed(y, pre, self.feed_forward_gate.bias, residual, None, self.mult)
        ws.release(mark)
        return False


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and after each sublayer, and a learned factor per coordinate on what joins the stream:

        x += mixer_scale * mixer_post_norm(mixer(mixer_norm(x)))
        x += feed_forward_scale * feed_forward_post_norm(feed_forward(feed_forward_norm(x)))

    The factor is folded into the post norm's gain at first use (Norm.folded).  Post norm, addition and the norm
    before the next sublayer are one kernel (ops.norm_residual_norm): the one after the mixer prepares the
    feed-forward's input, the one after the feed-forward the next layer's, when that layer is of this arrangement
    too (NormedInput).  The residual stream is float32 throughout.  A layer whose feed-forward is "none" has only
    the first line."""

    SLOTS = {"mixer": "mixer", "feed_forward": "feed_forward",
             "mixer_norm": "norm", "mixer_post_norm": "norm", "mixer_scale": "scale",
             "feed_forward_norm": "norm", "feed_forward_post_norm": "norm", "feed_forward_scale": "scale"}

    def __init__(self, params=None, **parts):
        super().__init__(params=params, **parts)
        self.has_ff = not isinstance(self.feed_forward, NoFeedForward)
        self._gains = None

    def _folded(self):
        if self._gains is None:
            self._gains = (self.mixer_post_norm.folded(self.mixer_scale.vector),
                           self.feed_forward_post_norm.folded(self.feed_forward_scale.vector) if self.has_ff else None,
                           self.feed_forward_norm.folded(None) if self.has_ff else None)
        return self._gains

    def accepts_normed(self, n_tokens):
        return self.mixer_norm.folded(None)

    def workspace_bytes(self, n_tokens, n_reqs, hidden, dtype):
        return 2 * workspace_piece((n_tokens, hidden), dtype) + super().workspace_bytes(n_tokens, n_reqs, hidden, dtype)

    def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None):
        if isinstance(pending, ops.RowScale):
            raise ValueError("sandwich_norm takes the residual stream as it is")
        mark = ws.mark()
        n, hidden = residual.shape
        post_mixer, post_ff, pre_ff = self._folded()
        y = ws.take((n, hidden), delta.dtype)
        if isinstance(pending, NormedInput):
            h = delta
        else:
            h = ws.take((n, hidden), delta.dtype)
            self.mixer_norm.forward(residual, delta if pending else None, h)
        self.mixer.forward(h, y, step, cache, writes_cache, ws)
        after = next_block.accepts_normed(n) if next_block is not None else None
        if self.has_ff:
            ops.norm_residual_norm(y, post_mixer[0], residual, post_mixer[1], next_gain=pre_ff[0], next_out=h, next_eps=pre_ff[1])
            self.feed_forward.forward(h, y, step, ws)
            last = post_ff
        else:
            last = post_mixer
        if after is None:
            ops.norm_residual_norm(y, last[0], residual, last[1])
            ws.release(mark)
            return False
        ops.norm_residual_norm(y, last[0], residual, last[1], next_gain=after[0], next_out=delta, next_eps=after[1])
        ws.release(mark)
        return NormedInput()


@register_block("hyper_prenorm")
class HyperConnectionBlock(Block):
    """Pre-norm sublayers on a residual stream kept as several copies x_1 .. x_s (hyper-connections):

        u = sum_s read_1[s] x_s;  y = mixer(mixer_norm(u));         x_t <- sum_s mix_1[s, t] x_s + write_1[t] y
        u = sum_s read_2[s] x_s;  y = feed_forward(feed_forward_norm(u));  x_t <- sum_s mix_2[s, t] x_s + write_2[t] y

    ``mixer_streams`` / ``feed_forward_streams`` (family "stream_mixing") hold the coefficients; with the "plain" kind
    this is the ordinary pre-norm layer on one stream.  ``residual`` is float32 [streams, n, hidden] (the model class
    "stream_decoder" makes it).  The join of a sublayer's result, the read of the sublayer that follows and its norm
    are one kernel (ops.stream_join), also across layers of this arrangement (NormedInput).  A layer whose feed-forward
    is "none" has only the first line.  The norms are any norm with ``forward_streams`` (parts/norm.py "layernorm")."""

    SLOTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
             "mixer_streams": "stream_mixing", "feed_forward_streams": "stream_mixing"}

    def __init__(self, params=None, **parts):
        super().__init__(params=params, **parts)
        self.has_ff = not isinstance(self.feed_forward, NoFeedForward)
        if self.has_ff and self.mixer_streams.streams != self.feed_forward_streams.streams:
            raise ValueError("hyper_prenorm: both sublayers must see the same number of streams")
        self.streams = self.mixer_streams.streams

    def stream_input(self):
        """(coefficients, norm) with which this block reads the streams first."""
        return self.mixer_streams.read, self.mixer_norm

    def workspace_bytes(self, n_tokens, n_reqs, hidden, dtype):
        return 2 * workspace_piece((n_tokens, hidden), dtype) + super().workspace_bytes(n_tokens, n_reqs, hidden, dtype)

    def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None):
        if residual.dim() != 3 or residual.shape[0] != self.streams:
            raise ValueError(f"hyper_prenorm: the residual stream must be [{self.streams}, tokens, hidden]; the model "
                             "class 'stream_decoder' makes it so")
        if pending is not False and not isinstance(pending, NormedInput):
            raise ValueError("hyper_prenorm takes the streams as they are, or its own normed input")
        mark = ws.mark()
        n, hidden = residual.shape[1:]
        y = ws.take((n, hidden), delta.dtype)
        if isinstance(pending, NormedInput):
            h = delta
        else:
            h = ws.take((n, hidden), delta.dtype)
            self.mixer_norm.forward_streams(residual, self.mixer_streams.read, h)
        self.mixer.forward(h, y, step, cache, writes_cache, ws)
        last = self.mixer_streams
        if self.has_ff:
            fs, fn = self.feed_forward_streams, self.feed_forward_norm
            ops.stream_join(residual, y, last.mix, last.write, fn.eps, next_coef=fs.read, next_w=fn.weight, next_b=fn.bias, next_out=h)
            self.feed_forward.forward(h, y, step, ws)
            last = fs
        if isinstance(next_block, HyperConnectionBlock) and next_block.streams == self.streams:
            coef, norm = next_block.stream_input()
            ops.stream_join(residual, y, last.mix, last.write, norm.eps, next_coef=coef, next_w=norm.weight, next_b=norm.bias,
                            next_out=delta)
            ws.release(mark)
            return NormedInput()
        ops.stream_join(residual, y, last.mix, last.write)
        ws.release(mark)
        return False
