"""Lutodra: a decoder on a residual stream kept as several copies (hyper-connections), whose layers mix tokens by a
real-gated linear recurrent unit, by the gated delta rule or by softmax attention with a sink, with dense or routed
feed-forwards, and of which a run of layers may be walked several times over; typed configuration and its description
as parts.

config.json names the design in ``architecture`` and gives every size and constant:

    vocab, width, norm.eps, streams (absent: one plain residual stream), logit_scale (absent: 1),
    loop = {start, stop, times} (absent: every layer once): layers start .. stop - 1 run ``times`` times in a row,
    layers[i] = {type: "rglru",         mixer: {width, blocks, conv},
                 type: "channel_delta", mixer: {heads, kv_heads, dim, vdim, conv},
                 type: "attention",     mixer: {heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling: {factor, low, high, original}}},
                 mlp: null | {kind: "dense", ff} | {kind: "moe", expert: {ff}, router: {experts, top, scale, groups: {count, keep}}}}

Layer i's tensors are ``l<i>.*``: ``norm1`` / ``norm1.b`` and ``hc1.in`` / ``hc1.out`` / ``hc1.mix`` around the mixer
``mix.*``, ``norm2`` / ``norm2.b`` and ``hc2.*`` around the feed-forward ``mlp.*``; outside the layers ``embed``,
``final.norm`` / ``final.norm.b`` and ``head``.  Every pass of a looped layer has cache and state of its own.  The inner
widths of the delta mixer's low-rank products come from the tensors alone.  What the design fixes (the gate constant 8
of the recurrent unit, 1e-6 in the unit norms, silu and sigmoid gates, a group's score as the sum of its two best, 1e-20
in the weights' sum) is named here or in the parts.  The reference has no model of this kind (src/core/engine.cpp:26-28).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

from ..config.engine_config import ConfigError
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture

MAX_POSITIONS = 1 << 22          # no position table bounds a request; the cache does first
RGLRU_GATE_CONSTANT = 8.0        # log a = -8 r softplus(lam)
GROUP_SCORE_TOP = 2              # a group of experts is scored by the sum of its two largest scores
ROUTE_SUM_EPS = 1e-20            # weights = scores / (their sum + 1e-20)
MIXERS = ("rglru", "channel_delta", "attention")


@dataclass
class LutodraLayer:
    kind: str
    mixer: dict
    mlp: Optional[dict] = None


@dataclass
class LutodraConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]           # None: one plain residual stream, no mixing tensors
    logit_scale: float
    loop: Optional[dict]
    layers: List[LutodraLayer] = field(default_factory=list)

    def run_order(self) -> List[int]:
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, k = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * k + list(range(b, n))

    @classmethod
    def from_dict(cls, cfg: dict) -> "LutodraConfig":
        problems: List[str] = []

        def number(d, key, where, integer=False, positive=True, default=None):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None:
                if default is not None:
                    return default
                problems.append(f"missing {where}'{key}'")
                return 1
            ok = isinstance(v, int) if integer else isinstance(v, (int, float))
            if isinstance(v, bool) or not ok:
                problems.append(f"{where}'{key}' must be {'an integer' if integer else 'a number'}, got {v!r}")
                return 1
            if positive and not v > 0:
                problems.append(f"{where}'{key}' must be positive, got {v!r}")
                return 1
            return v

        def integers(d, where, keys):
            return {k: number(d, k, where, integer=True) for k in keys}

        vocab = number(cfg, "vocab", "", integer=True)
        width = number(cfg, "width", "", integer=True)
        eps = float(number(cfg.get("norm"), "eps", "norm."))
        streams = None if cfg.get("streams") is None else number(cfg, "streams", "", integer=True)
        logit_scale = float(number(cfg, "logit_scale", "", positive=False, default=1.0))
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            problems.append("'layers' must be a non-empty list")
            raw_layers = []
        layers: List[LutodraLayer] = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"layers[{i}] must be an object with a 'mixer'")
                continue
            kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
            if kind == "rglru":
                mixer = integers(m, mw, ("width", "blocks", "conv"))
                if mixer["width"] % mixer["blocks"]:
                    problems.append(f"{mw}width {mixer['width']} is no multiple of blocks {mixer['blocks']}")
            elif kind == "channel_delta":
                mixer = integers(m, mw, ("heads", "dim", "vdim", "conv"))
                mixer["kv_heads"] = mixer["heads"] if m.get("kv_heads") is None else number(m, "kv_heads", mw, integer=True)
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{mw}heads {mixer['heads']} is no multiple of kv_heads {mixer['kv_heads']}")
            elif kind == "attention":
                mixer = integers(m, mw, ("heads", "dim", "vdim"))
                mixer["kv_heads"] = mixer["heads"] if m.get("kv_heads") is None else number(m, "kv_heads", mw, integer=True)
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{mw}heads {mixer['heads']} is no multiple of kv_heads {mixer['kv_heads']}")
                mixer["scale"] = float(number(m, "scale", mw))
                rot = m.get("rot")
                if rot is None:
                    mixer["rot"] = None
                else:
                    r = {"base": float(number(rot, "base", mw + "rot.")), "dims": number(rot, "dims", mw + "rot.", integer=True)}
                    if r["dims"] % 2 or r["dims"] > mixer["dim"]:
                        problems.append(f"{mw}rot.dims {r['dims']} must be even and at most dim {mixer['dim']}")
                    sc = rot.get("scaling") if isinstance(rot, dict) else None
                    r["scaling"] = None if sc is None else {k: float(number(sc, k, mw + "rot.scaling.", positive=(k != "low")))
                                                            for k in ("factor", "low", "high", "original")}
                    mixer["rot"] = r
            else:
                problems.append(f"{where}type {kind!r} is not a mixer of this design (known: {MIXERS})")
                continue
            mlp, checked = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    problems.append(f"{where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not a "
                                    "feed-forward of this design (known: 'dense', 'moe')")
                elif mlp["kind"] == "dense":
                    checked = {"kind": "dense", "ff": number(mlp, "ff", where + "mlp.", integer=True)}
                else:
                    ex, ro = mlp.get("expert"), mlp.get("router")
                    rw = where + "mlp.router."
                    checked = {"kind": "moe", "ff": number(ex, "ff", where + "mlp.expert.", integer=True),
                               "experts": number(ro, "experts", rw, integer=True), "top": number(ro, "top", rw, integer=True),
                               "scale": float(number(ro, "scale", rw, default=1.0))}
                    gr = ro.get("groups") if isinstance(ro, dict) else None
                    checked["groups"] = 1 if gr is None else number(gr, "count", rw + "groups.", integer=True)
                    checked["keep"] = 1 if gr is None else number(gr, "keep", rw + "groups.", integer=True)
                    if checked["experts"] % checked["groups"] or checked["keep"] > checked["groups"]:
                        problems.append(f"{rw}groups: {checked['experts']} experts in {checked['groups']} equal groups of which {checked['keep']} stay")
                    elif checked["top"] > checked["experts"] // checked["groups"] * checked["keep"]:
                        problems.append(f"{rw}top {checked['top']} exceeds what the {checked['keep']} groups that stay hold")
            layers.append(LutodraLayer(kind, mixer, checked))
        loop = cfg.get("loop")
        if loop is not None:
            lw = "loop."
            loop = {"start": number(loop, "start", lw, integer=True, positive=False), "stop": number(loop, "stop", lw, integer=True),
                    "times": number(loop, "times", lw, integer=True)}
            if not 0 <= loop["start"] <= loop["stop"] <= len(raw_layers):
                problems.append(f"loop runs layers {loop['start']} .. {loop['stop']} - 1 of {len(raw_layers)}")
        if problems:
            raise ConfigError("Lutodra config.json: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, eps=eps, streams=streams, logit_scale=logit_scale, loop=loop, layers=layers)


def lutodra_model_spec(c: LutodraConfig) -> ModelSpec:
    layers, absent = [], []
    norm = lambda: PartSpec("layernorm", {"size": c.width, "eps": c.eps, "tensor_name": ""})
    mixing = lambda: PartSpec("plain") if c.streams is None else PartSpec("learned", {"streams": c.streams})
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.kind == "rglru":
            mixer = PartSpec("rglru", {"hidden_size": c.width, "width": m["width"], "blocks": m["blocks"], "taps": m["conv"],
                                       "gate_constant": RGLRU_GATE_CONSTANT})
        elif layer.kind == "channel_delta":
            mixer = PartSpec("gated_delta", {"hidden_size": c.width, "num_heads": m["heads"], "num_qk_heads": m["kv_heads"],
                                             "head_dim": m["dim"], "v_head_dim": m["vdim"], "taps": m["conv"], "eps": c.eps})
        else:
            rot = m["rot"]
            position = PartSpec("none") if rot is None else PartSpec("scaled_rope", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                                                                     "pairing": "half", "scaling": rot["scaling"]})
            mixer = PartSpec("sink_attention", {"hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                                                "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"], "eps": c.eps,
                                                "position": position})
        mlp = layer.mlp
        if mlp is None:
            ff = PartSpec("none")
            absent += [p + "norm2", p + "norm2.b", p + "hc2.in", p + "hc2.out", p + "hc2.mix"]      # a file may still hold them
        elif mlp["kind"] == "dense":
            ff = PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": mlp["ff"], "activation": "silu",
                                        "tensor_names": ("gate", "up", "down")})
        else:
            ff = PartSpec("routed_experts", {"hidden_size": c.width, "expert_size": mlp["ff"], "num_experts": mlp["experts"],
                                             "num_identity": 0, "top": mlp["top"], "limit": float("inf"), "activation": "silu",
                                             "score": "sigmoid", "correction": False, "groups": mlp["groups"],
                                             "keep_groups": mlp["keep"], "group_top": GROUP_SCORE_TOP, "normalize": True,
                                             "sum_eps": ROUTE_SUM_EPS, "route_scale": mlp["scale"]})
        has_ff = mlp is not None
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=ff, mixer_norm=norm(), feed_forward_norm=norm() if has_ff else PartSpec("none"),
            mixer_streams=mixing(), feed_forward_streams=mixing() if has_ff else PartSpec("plain"),
            block="hyper_prenorm",
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1", "feed_forward_norm": p + "norm2",
                   "mixer_streams": p + "hc1.", "feed_forward_streams": p + "hc2."},
        ))
    # every pass of a looped layer is an entry of the run order with a cache layer of its own
    order = [LayerCall(layer=li, cache=n) for n, li in enumerate(c.run_order())]
    # logits = head x * logit_scale.  A power of two commutes with every rounding, so it rides in the final norm for nothing;
    # any other factor multiplies the float32 logits themselves, after the product (folded into the norm it would be rounded
    # to the activations' type with x)
    mantissa, _ = math.frexp(c.logit_scale)
    in_norm = mantissa == 0.5
    params = {"streams": c.streams or 1}
    if not in_norm:
        params["logit_scale"] = c.logit_scale
    return ModelSpec(
        architecture="Lutodra",
        hidden_size=c.width,
        vocab_size=c.vocab,
        layers=layers,
        run_order=order,
        final_norm=PartSpec("layernorm", {"size": c.width, "eps": c.eps, "tensor_name": "", "out_scale": c.logit_scale if in_norm else 1.0}),
        tie_word_embeddings=False,
        max_position_embeddings=MAX_POSITIONS,
        embed_name="embed",
        final_norm_prefix="final.norm",
        lm_head_name="head",
        ignored_tensors=absent,
        init_std=0.05,
        init_gain_std=0.05,
        model_class="stream_decoder",
        model_params=params,
    )


@register_architecture("Lutodra", "lutodra")
def build_lutodra(config: dict):
    typed = LutodraConfig.from_dict(config)
    return typed, lutodra_model_spec(typed)
