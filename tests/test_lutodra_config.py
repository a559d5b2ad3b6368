"""The Lutodra design without a GPU: its configuration reader, its description as parts, the tensors it declares, the
run order of a looped stretch of layers with a cache layer per pass, the rescaled rotation frequencies and the plain
implementation's own consistency (a recurrence cut anywhere, the router's rule)."""
import numpy as np
import pytest
import torch

import plain_lutodra as plain


def rglru(width, blocks, conv=4, mlp=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv=4, mlp=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def att(heads, kv_heads, dim, vdim, scale, rotation, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation},
            "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale=1.0, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(layers, width=64, vocab=200, streams=2, loop=None, logit_scale=1.0, eps=1e-5):
    cfg = {"architecture": "Lutodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale != 1.0:
        cfg["logit_scale"] = logit_scale
    return cfg


SAMPLE = config([att(4, 2, 16, 24, 0.2, rot(8, 5000.0, (8.0, 1.0, 3.0, 64)), mlp=dense(96)),
                 rglru(48, 3, conv=3, mlp=moe(40, 6, 2, 2.5, groups=(3, 2))),
                 delta(4, 2, 16, 8, conv=2, mlp=None),
                 rglru(80, 1, conv=5, mlp=moe(24, 3, 3))], streams=3, loop=(1, 3, 3), logit_scale=0.5)


def test_config_is_read_and_described_as_parts():
    from vllm_cpp_b200.config.registry import resolve_architecture
    typed, spec = resolve_architecture(SAMPLE)
    assert (typed.width, typed.vocab, typed.eps, typed.streams, typed.logit_scale) == (64, 200, 1e-5, 3, 0.5)
    assert [l.kind for l in typed.layers] == ["attention", "rglru", "channel_delta", "rglru"]
    assert typed.run_order() == [0, 1, 2, 1, 2, 1, 2, 3]
    assert typed.layers[1].mlp == {"kind": "moe", "ff": 40, "experts": 6, "top": 2, "scale": 2.5, "groups": 3, "keep": 2}
    assert typed.layers[3].mlp["groups"] == 1 and typed.layers[3].mlp["keep"] == 1 and typed.layers[3].mlp["scale"] == 1.0
    assert spec.model_class == "stream_decoder" and spec.model_params == {"streams": 3}
    assert [l.block for l in spec.layers] == ["hyper_prenorm"] * 4
    assert [l.mixer.kind for l in spec.layers] == ["sink_attention", "rglru", "gated_delta", "rglru"]
    assert spec.layers[0].mixer.params["position"].kind == "scaled_rope"
    assert spec.layers[0].mixer.params["position"].params["scaling"] == {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 64.0}
    assert spec.layers[2].feed_forward.kind == "none" and spec.layers[2].feed_forward_streams.kind == "plain"
    assert spec.layers[1].feed_forward.params["keep_groups"] == 2 and spec.layers[1].feed_forward.params["group_top"] == 2
    assert spec.layers[1].mixer.params["gate_constant"] == 8.0
    assert spec.final_norm.params["out_scale"] == 0.5
    # every pass of a looped layer has a cache layer of its own
    assert [(c.layer, c.cache) for c in spec.run_order] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (1, 5), (2, 6), (3, 7)]
    assert resolve_architecture(SAMPLE, "lutodra")[1].architecture == "Lutodra"


def test_where_the_logit_scale_goes():
    """A power of two rides in the final norm (it commutes with every rounding); any other factor multiplies the
    float32 logits after the product."""
    from vllm_cpp_b200.config.registry import resolve_architecture
    for scale, in_norm in ((0.5, True), (4.0, True), (1.0, True), (3.0, False), (0.37, False)):
        _, spec = resolve_architecture(config([rglru(8, 1)], width=8, vocab=9, logit_scale=scale))
        assert spec.final_norm.params["out_scale"] == (scale if in_norm else 1.0)
        assert spec.model_params.get("logit_scale", 1.0) == (1.0 if in_norm else scale)


def test_what_a_config_may_leave_out():
    """No ``streams``: one plain residual stream without mixing tensors; no ``loop``: every layer once; no rotation,
    no scaling, no groups."""
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.model import build_model
    cfg = config([att(3, 3, 8, 8, 0.3, None, mlp=dense(32)), att(2, 1, 16, 8, 0.25, rot(16), mlp=None)], streams=None)
    typed, spec = resolve_architecture(cfg)
    assert typed.streams is None and typed.loop is None and typed.run_order() == [0, 1]
    assert spec.layers[0].mixer.params["position"].kind == "none" and spec.layers[1].mixer.params["position"].params["scaling"] is None
    assert spec.layers[0].mixer_streams.kind == "plain" and spec.model_params == {"streams": 1}
    declared = build_model(spec, torch.float32, "meta").param_specs()
    assert set(declared) == set(plain.tensor_shapes(cfg))
    assert not any(".hc" in name for name in declared)


def test_every_fault_of_a_config_is_named():
    from vllm_cpp_b200.config.engine_config import ConfigError
    from vllm_cpp_b200.config.registry import resolve_architecture
    bad = config([{"type": "conv", "mixer": {}}, rglru(50, 4), delta(3, 2, 8, 8), att(2, 2, 8, 8, 0.0, rot(6)),
                  att(2, 2, 8, 8, 0.1, rot(12)), dict(rglru(8, 1), mlp={"kind": "sparse"}), dict(rglru(8, 1), mlp=moe(8, 6, 5, groups=(3, 2))),
                  dict(rglru(8, 1), mlp=moe(8, 6, 1, groups=(4, 2)))], loop=(2, 9, 2))
    del bad["vocab"]
    with pytest.raises(ConfigError) as e:
        resolve_architecture(bad)
    msg = str(e.value)
    for piece in ("missing 'vocab'", "'conv' is not a mixer", "width 50 is no multiple of blocks 4", "heads 3 is no multiple of kv_heads 2",
                  "'scale' must be positive", "rot.dims 12 must be even and at most dim 8", "'sparse' is not a feed-forward",
                  "top 5 exceeds", "6 experts in 4 equal groups", "loop runs layers 2 .. 9 - 1 of 8"):
        assert piece in msg, (piece, msg)


def test_declared_tensors_are_the_design_s():
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.model import build_model
    _, spec = resolve_architecture(SAMPLE)
    model = build_model(spec, torch.bfloat16, "meta")
    declared = model.param_specs()
    want = plain.tensor_shapes(SAMPLE, rank=5)
    assert set(declared) == set(want)
    for name, shape in want.items():
        assert declared[name].fits(shape), (name, declared[name].shape, shape)
    # the inner widths of the low-rank products are free: the checkpoint's tensors give them
    assert declared["l2.mix.a1"].shape == (-1, 64) and declared["l2.mix.a1"].fits((11, 64)) and not declared["l2.mix.a1"].fits((11, 63))
    assert declared["l2.mix.g2"].shape == (32, -1)
    assert declared["l1.mlp.router"].role == "bias" and declared["l0.mix.sink"].role == "bias"       # held in float32
    assert declared["l1.hc2.mix"].shape == (3, 3) and declared["l0.hc1.in"].shape == (3,)
    assert "l2.norm2" not in declared and "l2.hc2.in" not in declared                                # no feed-forward there
    assert "l2.norm2" in spec.ignored_tensors                                                        # a file may still hold them


def test_state_and_pages_of_every_pass():
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.base import CompositeSpec, PagedKVSpec, StateSpec
    from vllm_cpp_b200.parts.model import build_model
    _, spec = resolve_architecture(SAMPLE)
    specs = build_model(spec, torch.float32, "meta").cache_specs()
    assert len(specs) == 8
    assert specs[0] == PagedKVSpec(2, 24, 0)                          # rows of max(dim, vdim) elements, no window
    assert specs[1] == specs[3] == specs[5] == StateSpec((3, 48), torch.float32)      # the state and conv - 1 inputs
    assert specs[2] == specs[4] == CompositeSpec((StateSpec((4, 16, 8), torch.float32), StateSpec((1, 2 * 2 * 16 + 4 * 8), torch.float32)))
    assert specs[7] == StateSpec((5, 80), torch.float32)
    cm = CacheManager(specs, 16, 6, 2, torch.float32, None)
    assert len(cm.paged) == 1 and sorted(g.layers for g in cm.state) == [[1, 3, 5], [2, 4, 6], [2, 4, 6], [7]]      # slots grouped by shape
    cm.add_request("a")
    cm.reserve("a", 40)
    cm.commit("a", 40)
    assert cm.num_free_pages() == 3
    cm.free_request("a")
    assert cm.num_free_pages() == 6


@pytest.mark.parametrize("dims,base,scaling", [(8, 5000.0, (8.0, 1.0, 3.0, 64)), (32, 1e6, (6.0, 1.0, 3.0, 1024)), (16, 100.0, (2.0, 0.5, 8.0, 32)),
                                                (64, 10000.0, (32.0, 1.0, 4.0, 8192)), (4, 3.0, None)])
def test_rescaled_frequencies(dims, base, scaling):
    """All three branches of the rescaling by wavelength occur and agree with the plain rule."""
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts.base import POSITION_ENCODINGS, build_part
    r = rot(dims, base, scaling)
    want = plain.rotary_frequencies(r)
    part = build_part(POSITION_ENCODINGS, "position encoding",
                      PartSpec("scaled_rope", {"theta": base, "rotary_dim": dims, "pairing": "half", "scaling": r.get("scaling")}),
                      dtype=torch.float32, device="cpu")
    assert np.allclose(part.inv_freq.numpy(), want, rtol=1e-6, atol=0)
    if scaling and dims >= 32:
        plainf = base ** (-2.0 * np.arange(dims // 2) / dims)
        ratio = want / plainf
        assert np.isclose(ratio, 1.0).any() and np.isclose(ratio, 1.0 / scaling[0]).any()
        assert ((ratio > 1.0 / scaling[0] + 1e-9) & (ratio < 1 - 1e-9)).any()


def test_plain_recurrences_do_not_depend_on_the_cut():
    """The plain implementation itself: a mixer over a whole sequence equals the same mixer over a prefix (causality),
    and its router obeys the group rule."""
    rng = np.random.default_rng(0)
    cfg = config([rglru(24, 2, conv=3, mlp=None), delta(2, 1, 8, 12, conv=4, mlp=None)], width=20, vocab=50)
    w = plain.random_weights(cfg, 1)
    ids = rng.integers(0, 50, size=30).tolist()
    full = plain.forward(cfg, w, ids)
    assert np.allclose(full[:17], plain.forward(cfg, w, ids[:17]), atol=1e-12)
    r = {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    wr = {"x.router": rng.standard_normal((8, 20))}
    h = rng.standard_normal((40, 20))
    chosen, wts = plain.route(wr, "x.", r, h)
    s = plain.sigmoid(h @ wr["x.router"].T)
    for t in range(40):
        gs = s[t].reshape(4, 2).sum(axis=1)
        kept = set(np.argsort(-gs)[:2].tolist())
        assert {c // 2 for c in chosen[t]} <= kept and len(set(chosen[t])) == 3
        assert np.isclose(wts[t].sum(), 2.0)


def test_random_weights_mode_fills_free_sizes(tmp_path):
    from vllm_cpp_b200.weights.random_init import write_random_model
    from vllm_cpp_b200.weights.safetensors_io import SafetensorsFile
    write_random_model(str(tmp_path), SAMPLE, seed=3, dtype="bfloat16")
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert tuple(f.shape("l2.mix.a1")) == (32, 64) and tuple(f.shape("l2.mix.a2")) == (64, 32)
    assert tuple(f.shape("l1.hc1.mix")) == (3, 3)
    m = f.tensor("l1.hc1.mix").float()
    assert abs(float(m.diagonal().mean()) - 1.0) < 0.2 and abs(float((m - torch.diag(m.diagonal())).mean())) < 0.2
