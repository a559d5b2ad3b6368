"""The Gipinex design without a GPU: its configuration reader, its description as parts, the tensors it declares, the
run order of a looped run of layers with a cache layer per pass and the places where the stream is re-made, and the
plain implementation's own consistency (the routing rule, the rotation, causality)."""
import numpy as np
import pytest
import torch

import plain_gipinex as plain


def att(heads, kv_heads, dim, scale, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}, "mlp": mlp}


def lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, limit=1.5, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(layers, width=64, vocab=200, loop=None, mult=0.8, eps=1e-5):
    cfg = {"architecture": "Gipinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


SAMPLE = config([att(6, 2, 16, 0.3, mlp=moe(24, 5, 2, shared=(40, 1.0))),
                 lat(3, 16, 8, 24, 40, 20, 0.2, 5000.0, mlp=dense(96, 3.0)),
                 att(4, 4, 8, 0.5, mlp=None),
                 lat(2, 8, 4, 8, 16, 12, 0.3, mlp=moe(16, 3, 3))], loop=(1, 3, 3), mult=0.6)


def test_config_is_read_and_described_as_parts():
    from vllm_cpp_b200.config.registry import resolve_architecture
    typed, spec = resolve_architecture(SAMPLE)
    assert (typed.width, typed.vocab, typed.eps, typed.residual_mult) == (64, 200, 1e-5, 0.6)
    assert [l.kind for l in typed.layers] == ["attention", "latent_attention", "attention", "latent_attention"]
    assert [i for i, _ in typed.run_order()] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e for _, e in typed.run_order()] == [False, True, False, True, False, True, False, False]
    assert typed.layers[0].mlp["shared"] == {"ff": 40, "limit": 1.0} and typed.layers[3].mlp["shared"] is None
    assert spec.model_class == "reentrant_decoder"
    assert spec.model_params == {"reentries": [1, 3, 5], "reentry_tensor": "loop.in"}
    assert [l.block for l in spec.layers] == ["prenorm"] * 4 and all(l.block_params == {"residual_mult": 0.6} for l in spec.layers)
    assert [l.mixer.kind for l in spec.layers] == ["talking_heads_attention", "rotary_latent_attention"] * 2
    assert spec.layers[1].mixer.params["position"].params == {"theta": 5000.0, "rotary_dim": 8, "pairing": "interleaved", "scaling": None}
    assert spec.layers[0].mixer.params["slope_span"] == 8.0
    ff = spec.layers[0].feed_forward
    assert ff.kind == "routed_experts" and ff.params["router_bias"] and ff.params["normalize"] and ff.params["score"] == "softmax"
    assert ff.params["shared"].kind == "gated_mlp" and ff.params["shared"].params["biases"] is False
    assert spec.layers[1].feed_forward.params["biases"] is True and spec.layers[1].feed_forward.params["alpha"] == 1.702
    assert spec.layers[2].feed_forward.kind == "none" and spec.layers[2].feed_forward_norm.kind == "none"
    assert spec.tie_word_embeddings
    # every pass of a looped layer has a cache layer of its own
    assert [(c.layer, c.cache) for c in spec.run_order] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (1, 5), (2, 6), (3, 7)]
    assert resolve_architecture(SAMPLE, "gipinex")[1].architecture == "Gipinex"


def test_tensors_declared_are_the_design_s():
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.model import build_model
    for cfg in (SAMPLE, config([lat(2, 8, 4, 8, 16, 12, 0.3, mlp=dense(20))], width=24, vocab=50)):
        _, spec = resolve_architecture(cfg)
        model = build_model(spec, torch.float32, "meta")
        declared = {k: tuple(v.shape) for k, v in model.param_specs().items()}
        assert declared == plain.tensor_shapes(cfg)
    assert "loop.in" not in declared                       # no loop, no such tensor


def test_cache_layers_of_a_looped_model():
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.base import PagedKVSpec
    from vllm_cpp_b200.parts.model import build_model
    _, spec = resolve_architecture(SAMPLE)
    specs = build_model(spec, torch.bfloat16, "meta").cache_specs()
    assert len(specs) == 8
    assert specs[0] == PagedKVSpec(2, 16, 0) and specs[2] == specs[4] == PagedKVSpec(4, 8, 0)
    assert specs[1] == specs[3] == specs[5] == PagedKVSpec(1, 48, 0, planes=1)      # latent and rotated key part in one row
    assert specs[7] == PagedKVSpec(1, 20, 0, planes=1)


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "no multiple"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["loop"].update(stop=7), "loop runs"),
    (lambda c: c["norm"].pop("eps"), "norm.'eps'"),
])
def test_what_the_reader_refuses(change, message):
    import copy
    from vllm_cpp_b200.config.engine_config import ConfigError
    from vllm_cpp_b200.models.gipinex import GipinexConfig
    cfg = copy.deepcopy(SAMPLE)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        GipinexConfig.from_dict(cfg)


def test_plain_routing_rule():
    rng = np.random.default_rng(0)
    h, w, b = rng.standard_normal((7, 12)), rng.standard_normal((6, 12)), rng.standard_normal(6)
    ids, wts = plain.route(h, w, b, 3)
    z = h @ w.T + b
    for t in range(7):
        assert set(ids[t]) == set(np.argsort(-z[t])[:3])
        e = np.exp(z[t, ids[t]])
        assert np.allclose(wts[t], e / e.sum()) and abs(wts[t].sum() - 1) < 1e-12
    assert np.allclose(plain.route(h, w, b, 1)[1], 1.0)


def test_plain_rotation_and_causality():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 3, 8))
    y = plain.rotate_pairs(x, np.arange(5.0), 100.0, 8)
    assert np.allclose(y[0], x[0]) and np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
    a = 3 * 100.0 ** (-2.0 / 8)
    assert np.allclose(y[3, 1, 2], x[3, 1, 2] * np.cos(a) - x[3, 1, 3] * np.sin(a))
    assert np.allclose(y[3, 1, 3], x[3, 1, 3] * np.cos(a) + x[3, 1, 2] * np.sin(a))
    # a later token changes nothing before it; the slopes fall from head to head
    cfg = config([att(4, 2, 8, 0.4, mlp=dense(16)), lat(2, 8, 4, 8, 16, 12, 0.3, mlp=moe(8, 3, 2, shared=(8, 1.0)))], width=16, vocab=30, loop=(0, 2, 2))
    w = plain.random_weights(cfg, 3)
    ids = rng.integers(0, 30, size=12).tolist()
    assert np.allclose(plain.forward(cfg, w, ids)[:8], plain.forward(cfg, w, ids[:8]))
    s = plain.head_slopes(4)
    assert np.allclose(s, [0.25, 0.0625, 2.0 ** -6, 2.0 ** -8])
