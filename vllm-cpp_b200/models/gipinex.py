"""Gipinex: a pre-norm decoder whose residual branches carry a constant factor, whose layers mix tokens by attention
with talking heads and a distance bias or by latent attention with one rotated key part, with dense or routed
feed-forwards of a clamped activation, and of which a run of layers may be walked several times over, the stream being
re-made from itself and the embedding output at the start of every pass; typed configuration and its description as parts.

config.json names the design in ``architecture`` and gives every size and constant:

    vocab, width, norm.eps, residual_mult,
    loop = {start, stop, times} (absent: every layer once): layers start .. stop - 1 run ``times`` times in a row,
    layers[i] = {type: "attention",        mixer: {heads, kv_heads, dim, vdim, scale},
                 type: "latent_attention", mixer: {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}},
                 mlp: null | {kind: "dense", ff, limit}
                           | {kind: "moe", expert: {ff, limit}, router: {experts, top}, shared: null | {ff, limit}}}

Layer i's tensors are ``l<i>.*``: ``norm1`` before the mixer ``mix.*``, ``norm2`` before the feed-forward ``mlp.*``;
outside the layers ``embed`` (also the output matrix), ``final.norm`` and ``loop.in`` [width, 2 width], the matrix that
re-makes the stream from [x ; embedding output] before the first layer of every pass.  Every pass of a looped layer has a
cache of its own.  The norms' gains are stored around zero.  What the design fixes (the span 8 of the distance slopes,
1.702 in the activation, the sigmoid gates) is named here or in the parts.  The reference has no model of this kind
(src/core/engine.cpp:26-28).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..config.engine_config import ConfigError
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture

MAX_POSITIONS = 1 << 22          # no position table bounds a request; the cache does first
SLOPE_SPAN = 8.0                 # slope of head h of H: 2^(-8 (h + 1) / H)
SWISH_ALPHA = 1.702              # g * sigmoid(1.702 g)
MIXERS = ("attention", "latent_attention")


@dataclass
class GipinexLayer:
    kind: str
    mixer: dict
    mlp: Optional[dict] = None


@dataclass
class GipinexConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    loop: Optional[dict]
    layers: List[GipinexLayer] = field(default_factory=list)

    def run_order(self):
        """[(layer, this entry starts a pass of the looped run)] in the order the layers run."""
        n = len(self.layers)
        if not self.loop:
            return [(i, False) for i in range(n)]
        a, b, k = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, False) for i in range(a)]
        for _ in range(k):
            order += [(i, i == a) for i in range(a, b)]
        return order + [(i, False) for i in range(b, n)]

    @classmethod
    def from_dict(cls, cfg: dict) -> "GipinexConfig":
        problems: List[str] = []

        def number(d, key, where, integer=False, positive=True):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None:
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

        def gated(d, where):
            return {"ff": number(d, "ff", where, integer=True), "limit": float(number(d, "limit", where))}

        vocab = number(cfg, "vocab", "", integer=True)
        width = number(cfg, "width", "", integer=True)
        eps = float(number(cfg.get("norm"), "eps", "norm."))
        mult = float(number(cfg, "residual_mult", "", positive=False))
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            problems.append("'layers' must be a non-empty list")
            raw_layers = []
        layers: List[GipinexLayer] = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"layers[{i}] must be an object with a 'mixer'")
                continue
            kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
            if kind == "attention":
                mixer = integers(m, mw, ("heads", "dim", "vdim"))
                mixer["kv_heads"] = mixer["heads"] if m.get("kv_heads") is None else number(m, "kv_heads", mw, integer=True)
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{mw}heads {mixer['heads']} is no multiple of kv_heads {mixer['kv_heads']}")
                if mixer["vdim"] != mixer["dim"]:
                    problems.append(f"{mw}vdim {mixer['vdim']} differs from dim {mixer['dim']}, but the values are the keys")
                mixer["scale"] = float(number(m, "scale", mw))
            elif kind == "latent_attention":
                mixer = integers(m, mw, ("heads", "dim", "vdim", "kv_rank", "q_rank"))
                mixer["rot_dim"] = number(m, "rot_dim", mw, integer=True, positive=False)
                mixer["scale"] = float(number(m, "scale", mw))
                if mixer["rot_dim"]:
                    rot = m.get("rot")
                    mixer["rot"] = {"base": float(number(rot, "base", mw + "rot.")), "dims": number(rot, "dims", mw + "rot.", integer=True)}
                    if mixer["rot"]["dims"] != mixer["rot_dim"] or mixer["rot_dim"] % 2 or mixer["rot_dim"] < 0:
                        problems.append(f"{mw}rot.dims {mixer['rot']['dims']} must be rot_dim {mixer['rot_dim']}, an even number")
                else:
                    mixer["rot"] = None
            else:
                problems.append(f"{where}type {kind!r} is not a mixer of this design (known: {MIXERS})")
                continue
            mlp, checked = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    problems.append(f"{where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not a "
                                    "feed-forward of this design (known: 'dense', 'moe')")
                elif mlp["kind"] == "dense":
                    checked = dict(gated(mlp, where + "mlp."), kind="dense")
                else:
                    ro, rw = mlp.get("router"), where + "mlp.router."
                    checked = {"kind": "moe", "expert": gated(mlp.get("expert"), where + "mlp.expert."),
                               "experts": number(ro, "experts", rw, integer=True), "top": number(ro, "top", rw, integer=True),
                               "shared": None if mlp.get("shared") is None else gated(mlp["shared"], where + "mlp.shared.")}
                    if checked["top"] > checked["experts"]:
                        problems.append(f"{rw}top {checked['top']} exceeds the {checked['experts']} experts")
            layers.append(GipinexLayer(kind, mixer, checked))
        loop = cfg.get("loop")
        if loop is not None:
            lw = "loop."
            loop = {"start": number(loop, "start", lw, integer=True, positive=False), "stop": number(loop, "stop", lw, integer=True),
                    "times": number(loop, "times", lw, integer=True)}
            if not 0 <= loop["start"] < loop["stop"] <= len(raw_layers):
                problems.append(f"loop runs layers {loop['start']} .. {loop['stop']} - 1 of {len(raw_layers)}")
        if problems:
            raise ConfigError("Gipinex config.json: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=mult, loop=loop, layers=layers)


def gipinex_model_spec(c: GipinexConfig) -> ModelSpec:
    layers, absent = [], []
    norm = lambda: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor_name": "", "unit_offset": True})
    names = ("gate", "up", "down")

    def clamped(d, biases):
        return PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": d["ff"], "activation": "clamped_swish",
                                      "limit": d["limit"], "alpha": SWISH_ALPHA, "biases": biases, "tensor_names": names})

    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.kind == "attention":
            mixer = PartSpec("talking_heads_attention", {"hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                                                         "head_dim": m["dim"], "scale": m["scale"], "eps": c.eps,
                                                         "slope_span": SLOPE_SPAN})
        else:
            rot = m["rot"]
            position = PartSpec("none") if rot is None else PartSpec("scaled_rope", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                                                                     "pairing": "interleaved", "scaling": None})
            mixer = PartSpec("rotary_latent_attention", {"hidden_size": c.width, "num_heads": m["heads"], "head_dim": m["dim"],
                                                         "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"],
                                                         "q_rank": m["q_rank"], "scale": m["scale"], "eps": c.eps, "gate": "head",
                                                         "position": position})
        mlp = layer.mlp
        if mlp is None:
            ff = PartSpec("none")
            absent.append(p + "norm2")                    # a file may still hold it
        elif mlp["kind"] == "dense":
            ff = clamped(mlp, True)
        else:
            # the ``top`` largest logits, softmax over those alone: softmax scores, the chosen divided by their sum
            ff = PartSpec("routed_experts", {"hidden_size": c.width, "expert_size": mlp["expert"]["ff"], "num_experts": mlp["experts"],
                                             "num_identity": 0, "top": mlp["top"], "limit": mlp["expert"]["limit"],
                                             "alpha": SWISH_ALPHA, "activation": "clamped_swish", "score": "softmax",
                                             "correction": False, "normalize": True, "router_bias": True,
                                             "shared": None if mlp["shared"] is None else clamped(mlp["shared"], False)})
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=ff, mixer_norm=norm(), feed_forward_norm=norm() if mlp is not None else PartSpec("none"),
            block="prenorm", block_params={"residual_mult": c.residual_mult},
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1", "feed_forward_norm": p + "norm2"},
        ))
    # every pass of a looped layer is an entry of the run order with a cache layer of its own
    run = c.run_order()
    order = [LayerCall(layer=li, cache=n) for n, (li, _) in enumerate(run)]
    return ModelSpec(
        architecture="Gipinex",
        hidden_size=c.width,
        vocab_size=c.vocab,
        layers=layers,
        run_order=order,
        final_norm=PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor_name": "", "unit_offset": True}),
        tie_word_embeddings=True,
        max_position_embeddings=MAX_POSITIONS,
        embed_name="embed",
        final_norm_prefix="final.norm",
        ignored_tensors=absent,
        init_std=0.05,
        init_gain_std=0.05,
        model_class="reentrant_decoder",
        model_params={"reentries": [n for n, (_, enters) in enumerate(run) if enters], "reentry_tensor": "loop.in"},
    )


@register_architecture("Gipinex", "gipinex")
def build_gipinex(config: dict):
    typed = GipinexConfig.from_dict(config)
    return typed, gipinex_model_spec(typed)
