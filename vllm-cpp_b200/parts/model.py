"""A decoder put together from a ModelSpec: embedding, layers in their run order,
final norm, output product.

Flow of one step (src/model/qwen.cpp:291-328): ids -> embedding -> for each entry
of the run order, the layer's block on the residual stream -> final norm ->
lm_head.  Differences from the reference: the residual additions happen inside
the norm kernels; only the rows whose logits are wanted go through the final norm
and the output product (the reference computes logits for every token, :321-325);
the output matrix is the embedding table when ``tie_word_embeddings`` is set and a
tensor of its own otherwise (the reference overwrites the table with an untied
lm_head, :228-233,279-281).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..config.model_spec import ModelSpec
from ..csrc import ops
from .base import BLOCKS, FAMILIES, NORMS, ParamSpec, StepContext, Workspace, ScaledAddition, build_part, pending_mult
# importing the modules registers the built-in parts
from . import (attention as _attention, biased_attention as _biased, block as _block, gate as _gate,  # noqa: F401
               latent_attention as _latent, linear_attention as _linear, mlp as _mlp, moe as _moe, norm as _norm,
               gated_recurrence as _gated_recurrence, parallel as _parallel, position as _position, scale as _scale,
               shift as _shift, sink_attention as _sink_attention, streams as _streams, talking_attention as _talking)

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


MODEL_CLASSES: Dict[str, type] = {}


def register_model_class(name: str):
    """Registers a DecoderModel subclass under the name a ModelSpec's ``model_class`` gives."""
    def deco(cls):
        MODEL_CLASSES[name] = cls
        return cls
    return deco


def build_model(spec: ModelSpec, dtype: torch.dtype, device) -> "DecoderModel":
    if spec.model_class not in MODEL_CLASSES:
        raise ValueError(f"unknown model class {spec.model_class!r}; registered: {sorted(MODEL_CLASSES)}")
    return MODEL_CLASSES[spec.model_class](spec, dtype, device)


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.hidden, self.vocab = spec.hidden_size, spec.vocab_size
        ctx = {"dtype": dtype, "device": device}
        self.blocks = []
        for i, ls in enumerate(spec.layers):
            if ls.block not in BLOCKS:
                raise ValueError(f"layer {i}: unknown block arrangement {ls.block!r}; registered: {sorted(BLOCKS)}")
            arrangement = BLOCKS[ls.block]
            if set(ls.parts) != set(arrangement.SLOTS):
                raise ValueError(f"layer {i}: arrangement {ls.block!r} takes the parts {sorted(arrangement.SLOTS)}, "
                                 f"the layer names {sorted(ls.parts)}")
            built = {slot: build_part(FAMILIES[family], family, ls.parts[slot], **ctx)
                     for slot, family in arrangement.SLOTS.items()}
            params = getattr(ls, "block_params", None)
            self.blocks.append(arrangement(params=params, **built) if params else arrangement(**built))
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, **ctx)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self._check_cache_sharing()

    # ------------------------------------------------------------------ cache
    def cache_specs(self) -> List[object]:
        """The cache need of every cache layer, in order (PagedKVSpec, StateSpec or None)."""
        specs: List[object] = [None] * self.spec.num_cache_layers
        for call in self.spec.run_order:
            if call.writes_cache:
                specs[call.cache] = self.blocks[call.layer].cache_spec()
            if call.state >= 0:
                specs[call.state] = self.blocks[call.layer].state_spec()
        return specs

    def _check_cache_sharing(self) -> None:
        specs = self.cache_specs()
        for i, call in enumerate(self.spec.run_order):
            if not call.writes_cache:
                own = self.blocks[call.layer].cache_spec()
                if own != specs[call.cache]:
                    raise ValueError(f"run_order[{i}]: layer {call.layer} needs {own} but reads cache "
                                     f"{call.cache} of kind {specs[call.cache]}")
            if (call.state >= 0) != (self.blocks[call.layer].state_spec() is not None):
                raise ValueError(f"run_order[{i}]: layer {call.layer} " + (
                    "keeps no state but is given a state layer" if call.state >= 0 else
                    "keeps per-request state; its entry must name a cache layer for it (LayerCall.state)"))

    # ---------------------------------------------------------------- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every tensor of the model under its checkpoint name."""
        s = self.spec
        out = {s.embed_name: ParamSpec((self.vocab, self.hidden))}
        for ls, blk in zip(s.layers, self.blocks):
            for slot, part in blk.parts.items():
                for local, ps in part.param_specs().items():
                    out[ls.names[slot] + local] = ps
        for local, ps in self.final_norm.param_specs().items():
            out[s.final_norm_prefix + local] = ps
        if not s.tie_word_embeddings:
            out[s.lm_head_name] = ParamSpec((self.vocab, self.hidden))
        return out

    def placement(self, role: str) -> torch.dtype:
        return self.dtype if role == "matrix" else torch.float32

    def load_params(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint name -> device tensor in the role's type (see weights/loader.py)."""
        s = self.spec
        self.embed = tensors[s.embed_name].contiguous()
        self.lm_head = self.embed if s.tie_word_embeddings else tensors[s.lm_head_name].contiguous()
        for ls, blk in zip(s.layers, self.blocks):
            for slot, part in blk.parts.items():
                prefix = ls.names[slot]
                part.load_params({local: tensors[prefix + local] for local in part.param_specs()})
        self.final_norm.load_params({local: tensors[s.final_norm_prefix + local]
                                     for local in self.final_norm.param_specs()})

    def prepare_products(self, tune: bool = True, image_budget: Optional[int] = None) -> None:
        """Decide which product kernel runs for which shape and make the weights' tile images (parts/tuning.py)."""
        from .tuning import prepare_products
        prepare_products(self, tune, image_budget)

    def tensors(self) -> List[torch.Tensor]:
        """Every device tensor of the model once (a tied output matrix is the embedding table)."""
        seen, out = set(), []
        parts = [p for blk in self.blocks for p in blk.parts.values()] + [self.final_norm]
        for t in [self.embed, self.lm_head] + [t for p in parts for t in p.tensors()]:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                out.append(t)
        return out

    def tile_images(self) -> List[torch.Tensor]:
        """The pre-tiled images of weight matrices that exist now (see prepare_products)."""
        mats = [(self.lm_head, 0)] + [pw for blk in self.blocks for p in blk.parts.values() for pw in p.product_weights()]
        imgs = [ops.tiled_weights_of(w, bool(g)) for w, g in mats if w is not None]
        return [i for i in imgs if i is not None]

    def weight_bytes(self) -> int:
        """Bytes of the matrices a decode step reads once (embedding rows excluded unless tied)."""
        total = 0
        for blk in self.blocks:
            for part in blk.parts.values():
                for v, _ in part.product_weights():
                    total += v.numel() * v.element_size()
        total += self.lm_head.numel() * self.lm_head.element_size()
        return total

    # -------------------------------------------------------------------- run
    def forward(self, step: StepContext, caches: List[object], ws: Workspace,
                logits: torch.Tensor) -> torch.Tensor:
        """Runs the step's tokens; fills and returns logits[:n_logit_rows] (float32 [rows, vocab])."""
        n = step.n_tokens
        residual = ws.take(self.residual_shape(n), torch.float32)
        delta = ws.take((n, self.hidden), self.dtype)
        carry = ws.take((2, ops.sumsq_parts(self.hidden), n), torch.float32)
        self.embed_tokens(step, residual)
        pending = False                 # what delta holds: see Block.forward
        order = self.spec.run_order
        for i, call in enumerate(order):
            pending = self.before_call(i, residual, delta, pending, step, ws)
            following = self.blocks[order[i + 1].layer] if i + 1 < len(order) and not self.interrupts(i + 1) else None
            extra = {"state": caches[call.state]} if call.state >= 0 else {}
            pending = self.blocks[call.layer].forward(residual, delta, pending, step, caches[call.cache],
                                                      call.writes_cache, ws, next_block=following, carry=carry, **extra)
        has_delta = bool(pending)
        m = step.n_logit_rows
        out = logits[:m]
        if m:
            normed = ws.take((m, self.hidden), self.dtype)
            mult = pending_mult(pending)
            self.final_rows(residual, delta if has_delta else None, normed, step, **({} if mult == 1.0 else {"mult": mult}))
            self.head(normed, out)
        return out

    # Places an architecture may differ at without touching its layers; a subclass registered with
    # register_model_class overrides them (and ModelSpec.model_class names it).
    def residual_shape(self, n_tokens: int):
        """Shape of the float32 residual stream of a step (what the blocks receive as ``residual``)."""
        return (n_tokens, self.hidden)

    def final_rows(self, residual: torch.Tensor, delta: Optional[torch.Tensor], normed: torch.Tensor, step: StepContext,
                   mult: float = 1.0) -> None:
        """normed = the model's final norm of the rows whose logits are wanted (``delta``: an addition still pending, which
        joins times ``mult``)."""
        self.final_norm.forward(residual, delta, normed, step.logit_rows, **({} if mult == 1.0 else {"mult": mult}))

    def interrupts(self, i: int) -> bool:
        """True if the model does something of its own to the residual stream right before entry ``i`` of the run order
        (``before_call``): the block before it then may not prepare that entry's input."""
        return False

    def before_call(self, i: int, residual: torch.Tensor, delta: torch.Tensor, pending, step: StepContext, ws: Workspace):
        """Called before entry ``i`` of the run order with what the entry before left (see Block.forward for ``pending``);
        returns the ``pending`` the entry's block receives.  The plain decoder does nothing here."""
        return pending

    def embed_tokens(self, step: StepContext, residual: torch.Tensor) -> None:
        """residual[t] = the embedding of token t in float32 (src/kernels/embedding_kernel.cu:20-28: no scaling)."""
        ops.embedding(self.embed, step.token_ids, residual)

    def head(self, normed: torch.Tensor, out: torch.Tensor) -> None:
        """out [rows, vocab] (float32) = logits of the normed rows (src/model/qwen.cpp:325: a product, no bias)."""
        ops.linear(normed, self.lm_head, out)

    def workspace_bytes(self, n_tokens: int, n_reqs: int, n_logit_rows: int) -> int:
        """Most bytes ``forward`` takes from the workspace for a step of this size: its own buffers plus the
        largest need of any block (each piece rounded up as Workspace.take rounds)."""
        el = torch.empty((), dtype=self.dtype).element_size()
        r = lambda b: (b + 255) // 256 * 256
        rows = 1
        for d in self.residual_shape(n_tokens)[:-1]:
            rows *= d
        own = r(rows * self.hidden * 4) + r(n_tokens * self.hidden * el) \
            + r(2 * ops.sumsq_parts(self.hidden) * n_tokens * 4) + r(n_logit_rows * self.hidden * el) \
            + self.own_workspace_bytes(n_tokens)
        return own + max((blk.workspace_bytes(n_tokens, n_reqs, self.hidden, self.dtype) for blk in self.blocks), default=0)


    def own_workspace_bytes(self, n_tokens: int) -> int:
        """What a model class takes from the workspace beside the plain decoder's buffers."""
        return 0


MODEL_CLASSES["decoder"] = DecoderModel


@register_model_class("scaled_embedding_decoder")
class ScaledEmbeddingDecoderModel(DecoderModel):
    """A decoder whose residual stream starts as  embedding * ``embedding_scale``  (ModelSpec.model_params)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.embedding_scale = float(spec.model_params.get("embedding_scale", 1.0))

    def embed_tokens(self, step, residual):
        ops.embedding(self.embed, step.token_ids, residual, scale=self.embedding_scale)


@register_model_class("scaled_sinusoid_decoder")
class ScaledSinusoidDecoderModel(DecoderModel):
    """A decoder whose residual stream starts as  embedding * ``embedding_scale`` + a sinusoidal position
    vector: entry 2i is sin(p f_i), entry 2i + 1 is cos(p f_i), f_i = ``position_base``^(-2i / width), p the
    token's position in its request.  The f_i are computed once in double and rounded; the angle is their
    float product with the position (ModelSpec.model_params gives the two constants)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.model_params
        self.embedding_scale = float(p.get("embedding_scale", 1.0))
        base = float(p.get("position_base", 10000.0))
        i = np.arange((self.hidden + 1) // 2, dtype=np.float64)
        self.inv_freq = torch.from_numpy(np.power(base, -2.0 * i / self.hidden).astype(np.float32)).to(device)

    def tensors(self):
        return super().tensors() + [self.inv_freq]

    def embed_tokens(self, step, residual):
        ops.embedding_sinusoid(self.embed, step.token_ids, step.positions, self.inv_freq, residual, self.embedding_scale)


@register_model_class("stream_decoder")
class StreamDecoderModel(DecoderModel):
    """A decoder whose residual stream is ``streams`` copies of the embedding (ModelSpec.model_params), which its
    layers read and rejoin with coefficients of their own (parts/block.py "hyper_prenorm"); the final norm reads the
    sum of the copies.  ``streams`` 1 is one plain residual stream."""

    def __init__(self, spec, dtype, device):
        self.streams = int(spec.model_params.get("streams", 1))
        self.logit_scale = float(spec.model_params.get("logit_scale", 1.0))     # on the float32 logits, after the product
        super().__init__(spec, dtype, device)
        if not hasattr(self.final_norm, "forward_streams"):
            raise ValueError("stream_decoder: the final norm must read several streams (forward_streams)")
        for i, blk in enumerate(self.blocks):
            if getattr(blk, "streams", None) != self.streams:
                raise ValueError(f"stream_decoder: layer {i} does not take {self.streams} streams")
        self._ones = None if torch.device(device).type == "meta" else torch.ones(self.streams, dtype=torch.float32, device=device)

    def tensors(self):
        return super().tensors() + ([self._ones] if self._ones is not None else [])

    def residual_shape(self, n_tokens):
        return (self.streams, n_tokens, self.hidden)

    def embed_tokens(self, step, residual):
        for s in range(self.streams):
            ops.embedding(self.embed, step.token_ids, residual[s])

    def head(self, normed, out):
        super().head(normed, out)
        if self.logit_scale != 1.0:
            ops.scaled_sum(out, out, out, self.logit_scale, 0.0)

    def final_rows(self, residual, delta, normed, step):
        if delta is not None:
            raise ValueError("stream_decoder: its layers leave no addition pending")
        self.final_norm.forward_streams(residual, self._ones, normed, step.logit_rows)


@register_model_class("reentrant_decoder")
class ReentrantDecoderModel(DecoderModel):
    """A decoder that re-makes its residual stream from the stream itself and the embedding output x0 at given places of
    the run order:  x <- W [x ; x0]  with one matrix W [width, 2 * width] (x's columns first), right before each entry
    that ``ModelSpec.model_params["reentries"]`` lists (the first layer of every pass of a looped run of layers).  The
    tensor's name is ``model_params["reentry_tensor"]``.  An addition still pending is made first, in float; x and x0
    enter the product in the compute type and the result is the new float32 stream.  x0 is kept for the step."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.model_params
        self.reentries = frozenset(int(i) for i in p.get("reentries", ()))
        self.reentry_tensor = str(p.get("reentry_tensor", "reentry"))
        bad = [i for i in self.reentries if not 0 <= i < len(spec.run_order)]
        if bad:
            raise ValueError(f"reentrant_decoder: reentries {bad} are no entries of the run order")
        self.w_reentry: Optional[torch.Tensor] = None
        self._pair = None                      # [x | x0] of the step in the compute type, the product's input
        self._have_x0 = False

    def param_specs(self):
        out = super().param_specs()
        if self.reentries:
            out[self.reentry_tensor] = ParamSpec((self.hidden, 2 * self.hidden))
        return out

    def load_params(self, tensors):
        super().load_params(tensors)
        if self.reentries:
            self.w_reentry = tensors[self.reentry_tensor].contiguous()

    def tensors(self):
        return super().tensors() + ([self.w_reentry] if self.w_reentry is not None else [])

    def weight_bytes(self):
        extra = len(self.reentries) * self.w_reentry.numel() * self.w_reentry.element_size() if self.w_reentry is not None else 0
        return super().weight_bytes() + extra

    def own_workspace_bytes(self, n_tokens):
        el = torch.empty((), dtype=self.dtype).element_size()
        return (n_tokens * 2 * self.hidden * el + 255) // 256 * 256 if self.reentries else 0

    def forward(self, step, caches, ws, logits):
        self._pair = ws.take((step.n_tokens, 2 * self.hidden), self.dtype) if self.reentries else None
        self._have_x0 = False
        return super().forward(step, caches, ws, logits)

    def interrupts(self, i):
        return i in self.reentries

    def before_call(self, i, residual, delta, pending, step, ws):
        if self.reentries and not self._have_x0:
            # called first before entry 0, when the stream still is the embedding output: its rows in the compute type
            # are the right half of the product's input for the whole step
            ops.cast_rows(residual, None, 1.0, self._pair[:, self.hidden:])
            self._have_x0 = True
        if i not in self.reentries:
            return pending
        if pending is not False and pending is not True and not isinstance(pending, ScaledAddition):
            raise ValueError("reentrant_decoder: the block before a reentry must leave the stream or an addition to it")
        ops.cast_rows(residual, delta if pending else None, pending_mult(pending), self._pair[:, :self.hidden])
        ops.linear(self._pair, self.w_reentry, residual)
        return False
