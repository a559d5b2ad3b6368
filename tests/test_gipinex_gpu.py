"""The Gipinex design on the GPU against the plain implementation of plain_gipinex.py: each mechanism alone (the clamped
activation with biases, the norm that takes a scaled addition, experts chosen by logit with a bias and a shared expert,
attention with talking heads and a distance bias under every cut with a key that matters hundreds of tokens back, latent
attention with its shared rotated key part), then whole models under every way of cutting the work, the stream after
every layer run, greedy generation through the engine's entry point and the replay program.  Configurations and weights
are made here."""
import json
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import plain_gipinex as plain
from helpers import MEAN_TOL, TOL, Replayer
from test_gipinex_config import att, config, dense, lat, moe

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# a looped run that starts after the first layer, three query heads per kv head, latent sizes with odd factors, a layer
# without feed-forward, experts with and without a shared one
CFG_A = config([att(6, 2, 32, 0.3, mlp=dense(96, 1.5)),
                lat(3, 24, 8, 16, 40, 28, 0.25, 300.0, mlp=moe(40, 6, 2, 1.0, shared=(56, 2.0))),
                att(4, 4, 16, 0.5, mlp=None),
                lat(5, 8, 16, 12, 24, 36, 0.35, 1e5, mlp=moe(24, 3, 1, 3.0))], width=64, vocab=200, loop=(1, 3, 2), mult=0.6)
# no loop, an odd vocabulary and widths with odd factors, one kv head, every expert chosen, a multiplier above one
CFG_B = config([lat(2, 40, 4, 20, 72, 10, 0.2, 50.0, mlp=moe(16, 3, 3, 2.0, shared=(24, 0.8))),
                att(5, 1, 24, 0.4, mlp=dense(50, 4.0)),
                att(2, 2, 64, 0.125, mlp=moe(20, 4, 2, 1.2))], width=72, vocab=301, mult=1.25, eps=1e-6)
# the whole model walked three times over, heads that run on the tensor cores in bfloat16 (64 and 128 wide), a latent
# row of 128 with its rotated part
CFG_C = config([att(8, 4, 64, 0.125, mlp=dense(80, 2.0)), lat(4, 32, 32, 32, 96, 48, 0.15, 1e4, mlp=moe(32, 4, 2, 1.0, shared=(48, 1.0))),
                att(2, 1, 128, 0.09, mlp=None)], width=96, vocab=97, loop=(0, 3, 3), mult=0.5)
CONFIGS = {"A": (CFG_A, 16), "B": (CFG_B, 32), "C": (CFG_C, 16)}
SHARP = {"float32": 3.0, "bfloat16": 1.0}
MARGIN = {"float32": 2e-5, "bfloat16": 6e-3}        # routing decisions closer than this are left to rounding


def compare(got, want, dtype, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    scale = np.abs(want).max()
    rows = np.abs(got - want).max(axis=1) / scale
    assert rows.max() <= TOL[dtype], f"{what}: worst row {rows.max():.3e} of the largest logit at row {int(rows.argmax())}"
    assert np.abs(got - want).mean() <= MEAN_TOL[dtype] * scale, f"{what}: mean error {np.abs(got - want).mean() / scale:.3e}"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def stored(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy().astype(np.float64)


def make_weights(cfg, seed, dtype):
    w = plain.random_weights(cfg, seed, sharp=SHARP[dtype], decisive_routing=dtype == "bfloat16")
    return plain.round_to_bf16(w) if dtype == "bfloat16" else w


def ids_of(cfg, w, n, seed, dtype):
    """Token ids whose routing decisions in the plain implementation all have a clear margin."""
    for k in range(40):
        ids = np.random.default_rng(seed * 1000 + k).integers(0, cfg["vocab"], size=n).tolist()
        if plain.routing_margin(cfg, w, ids) > MARGIN[dtype]:
            return ids
    raise AssertionError("no token sequence with clear routing found")


def build(tmp_path, name, dtype, num_pages, seed=1, max_seqs=4, graphs=False, cfg_page=None):
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    cfg, page = cfg_page or CONFIGS[name]
    weights = make_weights(cfg, seed, dtype)
    folder = str(tmp_path / f"gipinex_{name}_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=num_pages, max_num_seqs=max_seqs,
                        max_model_len=num_pages * page, max_num_batched_tokens=1024, use_cuda_graphs=graphs)
    model, cache, runner = factory.build(ecfg)
    return cfg, weights, folder, cache, runner


def run_mixer(mixer, x, schedule, page=16, pages=40, max_len=600, max_seqs=2):
    """Feeds the rows x[request] through ``mixer`` as ``schedule`` cuts them ([(request, tokens), ...] per step) on the
    engine's cache manager and step packing; a request that has had all its rows is freed, so later requests take its
    slot and pages.  Returns request -> rows."""
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import ModelRunner, StepEntry
    from vllm_cpp_b200.parts.base import Workspace
    cache = CacheManager([mixer.cache_spec()], page, pages, max_seqs, mixer.dtype, "cuda")
    fake = types.SimpleNamespace(vocab=100, blocks=[types.SimpleNamespace(parts={"mixer": mixer})], final_norm=None,
                                 spec=types.SimpleNamespace(max_position_embeddings=max_len))
    runner = ModelRunner(fake, cache, 1024, max_seqs, max_len, torch.device("cuda", 0))
    ws = Workspace("cuda")
    at = {r: 0 for r in x}
    got = {r: [] for r in x}
    for entries in schedule:
        for r, _ in entries:
            if r not in cache.requests:
                cache.add_request(r)
        step = runner._prepare([StepEntry(r, [0] * n, []) for r, n in entries])
        rows = dev(np.concatenate([x[r][at[r]: at[r] + n] for r, n in entries]), mixer.dtype)
        out = torch.empty_like(rows)
        ws.reset()
        mixer.forward(rows, out, step, runner.views[0], True, ws)
        o, t0 = out.float().cpu().numpy(), 0
        for r, n in entries:
            got[r].append(o[t0: t0 + n])
            t0 += n
            at[r] += n
            cache.commit(r, n)
            if at[r] == len(x[r]):
                cache.free_request(r)
    ops.check_status()
    assert all(at[r] == len(x[r]) for r in x), "the schedule does not feed every row"
    return {r: np.concatenate(got[r]) for r in x}


def load_part(part, weights, prefix, dtype):
    part.load_params({local: dev(np.asarray(weights[prefix + local], dtype=np.float32),
                                 DT[dtype] if ps.role == "matrix" else torch.float32) for local, ps in part.param_specs().items()})


# four requests of unequal length on two slots: portions of changing size beside single tokens, the second pair taking the
# slots and pages that the first pair gave back; a long prompt whose last tokens come one by one
LENGTHS = {"a": 37, "b": 5, "c": 64, "d": 18}
SCHEDULE = [[("a", 1), ("b", 3)], [("b", 2), ("a", 2)], [("a", 17)], [("a", 16)], [("a", 1), ("c", 30)], [("c", 1), ("d", 2)],
            [("c", 33), ("d", 15)], [("d", 1)]]


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter,biases", [(40, True), (64, False), (7, True)])
def test_clamped_activation(dtype, inter, biases):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(inter)
    n, limit = 9, 1.3
    gu = stored(2 * rng.standard_normal((n, 2 * inter)), dtype)
    b = (0.5 * rng.standard_normal(2 * inter)).astype(np.float32) if biases else None
    out = torch.empty((n, inter), dtype=DT[dtype], device="cuda")
    ops.clamped_swish_mul(dev(gu, DT[dtype]), None if b is None else dev(b), out, limit=limit, alpha=1.702)
    g, u = gu[:, :inter] + (0 if b is None else b[:inter]), gu[:, inter:] + (0 if b is None else b[inter:])
    g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
    want = g * plain.sigmoid(1.702 * g) * (u + 1)
    assert (np.minimum(gu[:, :inter], limit) != gu[:, :inter]).any() and (np.abs(gu[:, inter:]) > limit).any()
    assert np.abs(out.float().cpu().numpy() - want).max() <= (2e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [72, 2500])
def test_norm_takes_a_scaled_addition(dtype, width):
    """residual += m * delta in float, then the norm with a gain stored around zero; also on gathered rows."""
    from vllm_cpp_b200.parts.norm import RMSNorm
    rng = np.random.default_rng(width)
    n, eps, m = 5, 1e-5, 0.7
    x = rng.standard_normal((n, width)).astype(np.float32)
    d = stored(rng.standard_normal((n, width)), dtype)
    w = (0.2 * rng.standard_normal(width)).astype(np.float32)
    norm = RMSNorm(width, eps, DT[dtype], "cuda", tensor_name="", unit_offset=True)
    norm.load_params({"": dev(w)})
    want_x = x.astype(np.float64) + m * d
    want = plain.offset_norm(want_x, w.astype(np.float64), eps)
    tol = 3e-6 if dtype == "float32" else 1e-2
    xd, out = dev(x), torch.empty((n, width), dtype=DT[dtype], device="cuda")
    norm.forward(xd, dev(d, DT[dtype]), out, mult=m)
    assert np.abs(xd.cpu().numpy() - want_x).max() <= 3e-6 * np.abs(want_x).max()
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    rows = torch.tensor([3, 0, 3], dtype=torch.int32, device="cuda")
    xd, out = dev(x), torch.empty((3, width), dtype=DT[dtype], device="cuda")
    norm.forward(xd, dev(d, DT[dtype]), out, rows, mult=m)
    assert np.array_equal(xd.cpu().numpy(), x)
    assert np.abs(out.float().cpu().numpy() - want[[3, 0, 3]]).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,ff,experts,top,shared", [(13, 48, 24, 5, 2, (40, 0.9)), (70, 64, 64, 16, 4, None), (3, 40, 8, 3, 3, (8, 2.0)),
                                                           (200, 72, 20, 7, 1, (16, 1.0))])
def test_experts_chosen_by_logit_with_a_shared_expert(dtype, n, width, ff, experts, top, shared):
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.moe import RoutedExperts
    mlp = moe(ff, experts, top, 1.1, shared=shared)
    cfg = config([att(2, 1, 8, 0.3, mlp=mlp)], width=width)
    w = plain.random_weights(cfg, n, std=0.3)
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    rng = np.random.default_rng(n + 1)
    h = stored(rng.standard_normal((n, width)), dtype)
    sh = None if shared is None else PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": shared[0], "activation": "clamped_swish",
                                                            "limit": shared[1], "tensor_names": ("gate", "up", "down")})
    part = RoutedExperts(width, ff, experts, 0, top, 1.1, DT[dtype], "cuda", activation="clamped_swish", score="softmax", correction=False,
                         normalize=True, router_bias=True, shared=sh)
    load_part(part, w, "l0.mlp.", dtype)
    out = torch.empty((n, width), dtype=DT[dtype], device="cuda")
    part.forward(dev(h, DT[dtype]), out, None, Workspace("cuda"))
    margins = []
    want = plain.routed_ff(h, w, "l0.mlp.", mlp, margins)
    z = h @ w["l0.mlp.router"].T + w["l0.mlp.router.b"]
    ranked = -np.sort(-z, axis=-1)
    clear = np.ones(n, bool) if top == experts else (ranked[:, top - 1] - ranked[:, top]) > MARGIN[dtype]
    assert clear.sum() >= n * 0.7
    err = np.abs(out.float().cpu().numpy() - want)[clear].max()
    assert err <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), err


def talking_mixer(dtype, width, H, G, d, scale, window=0):
    from vllm_cpp_b200.parts.talking_attention import TalkingHeadsAttention
    return TalkingHeadsAttention(width, H, G, d, scale, 1e-5, DT[dtype], "cuda", window=window)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,page", [(8, 2, 64, 16), (4, 4, 128, 32), (12, 4, 64, 16), (6, 3, 16, 16), (3, 1, 40, 32), (20, 5, 32, 16), (1, 1, 64, 16)])
def test_talking_heads_under_every_cut(dtype, H, G, d, page):
    """Unequal requests in portions and single tokens on two slots and few pages, against each request whole."""
    width = 48
    layer = att(H, G, d, 0.9 / np.sqrt(d))
    cfg = config([layer], width=width)
    w = plain.random_weights(cfg, H * d, std=0.2)
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    mixer = talking_mixer(dtype, width, H, G, d, layer["mixer"]["scale"])
    load_part(mixer, w, "l0.mix.", dtype)
    rng = np.random.default_rng(d)
    x = {r: stored(rng.standard_normal((n, width)), dtype) for r, n in LENGTHS.items()}
    got = run_mixer(mixer, x, SCHEDULE, page=page, pages=160 // page)
    for r in x:
        want = plain.talking_attention(x[r], w, "l0.mix.", layer["mixer"], 1e-5)
        err = np.abs(got[r] - want).max() / np.abs(want).max()
        assert err <= (2e-5 if dtype == "float32" else 2.5e-2), (r, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,planted_at,cut", [(8, 2, 64, 3, "whole"), (8, 2, 64, 15, "decode"), (4, 1, 128, 16, "portions"),
                                                  (5, 5, 24, 0, "decode"), (16, 8, 64, 31, "portions")])
def test_a_key_far_back_that_the_last_heads_see(dtype, H, G, d, planted_at, cut):
    """Keys are projected by the matrix of the last query head of their group (the smallest slope) behind a rotation R of the
    input, and the row at ``planted_at`` (a page's edge, the first token, the middle of a page) is the last row turned
    back by R: its key is the last row's query, no other key is.  Hundreds of tokens later the heads with small slopes
    still give it most of their weight, so a key that is lost, misplaced or read from another page shows."""
    width, n, scale = 40, 421, (10.0 if d >= 64 else 16.0) / d
    layer = att(H, G, d, scale)
    cfg = config([layer], width=width)
    w = plain.random_weights(cfg, d + planted_at, std=0.3)
    turn = np.linalg.qr(np.random.default_rng(2).standard_normal((width, width)))[0]
    wq = w["l0.mix.q"].reshape(H, d, width)
    w["l0.mix.k"] = np.concatenate([wq[(g + 1) * (H // G) - 1] @ turn for g in range(G)])
    w["l0.mix.talk"] = np.eye(H) + 0.05 * np.random.default_rng(1).standard_normal((H, H))
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    rng = np.random.default_rng(7)
    x = rng.standard_normal((n, width))
    x[planted_at] = x[-1] @ turn
    x = stored(x, dtype)
    want = plain.talking_attention(x, w, "l0.mix.", layer["mixer"], 1e-5)
    moved = x.copy()
    moved[planted_at] = x[planted_at + 1]
    other = plain.talking_attention(moved, w, "l0.mix.", layer["mixer"], 1e-5)
    assert np.abs(want[-1] - other[-1]).max() > 0.2 * np.abs(want[-1]).max()         # the planted key decides the last row
    mixer = talking_mixer(dtype, width, H, G, d, scale)
    load_part(mixer, w, "l0.mix.", dtype)
    sched = {"whole": [[("r", n)]], "decode": [[("r", n - 40)]] + [[("r", 1)]] * 40,
             "portions": [[("r", 200)], [("r", 2)], [("r", 187)], [("r", 31)], [("r", 1)]]}[cut]
    got = run_mixer(mixer, {"r": x}, sched, pages=30)["r"]
    err = np.abs(got - want).max(axis=1) / np.abs(want).max()
    assert err.max() <= (3e-5 if dtype == "float32" else 3e-2), (int(err.argmax()), err.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,window", [(4, 2, 64, 24), (3, 3, 16, 7), (2, 1, 32, 1)])
def test_the_part_s_window(dtype, H, G, d, window):
    """The part may be given a window (this design gives none): a query sees the last ``window`` keys, its own included; the
    plain implementation is run on every row's visible keys alone."""
    width, n = 32, 90
    layer = att(H, G, d, 2.0 / np.sqrt(d))
    w = plain.random_weights(config([layer], width=width), window, std=0.3)
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    mixer = talking_mixer(dtype, width, H, G, d, layer["mixer"]["scale"], window=window)
    load_part(mixer, w, "l0.mix.", dtype)
    x = stored(np.random.default_rng(3).standard_normal((n, width)), dtype)
    got = run_mixer(mixer, {"r": x}, [[("r", 50)], [("r", 2)], [("r", 30)]] + [[("r", 1)]] * 8)["r"]
    for t in (0, 1, window - 1, window, window + 1, 49, 50, 51, 81, 82, 89):
        lo = max(0, t - window + 1)
        want = plain.talking_attention(x[lo: t + 1], w, "l0.mix.", layer["mixer"], 1e-5)[-1]
        assert np.abs(got[t] - want).max() <= (2e-5 if dtype == "float32" else 2.5e-2) * max(1e-3, np.abs(want).max()), t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dim,rot,vd,rank,q_rank,page", [(4, 32, 16, 24, 48, 40, 16), (8, 64, 32, 64, 96, 64, 16), (1, 8, 2, 8, 10, 6, 32),
                                                            (3, 16, 64, 8, 64, 16, 16), (16, 24, 8, 40, 56, 30, 16)])
def test_latent_attention_under_every_cut(dtype, H, dim, rot, vd, rank, q_rank, page):
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts.latent_attention import RotaryLatentAttention
    width, base = 56, 700.0
    layer = lat(H, dim, rot, vd, rank, q_rank, 1.5 / np.sqrt(dim + rot), base)
    w = plain.random_weights(config([layer], width=width), H + rank, std=0.25, sharp=2.0 if dtype == "float32" else 1.0)
    if dtype == "bfloat16":
        w = plain.round_to_bf16(w)
    pos = PartSpec("scaled_rope", {"theta": base, "rotary_dim": rot, "pairing": "interleaved", "scaling": None})
    mixer = RotaryLatentAttention(width, H, dim, rot, vd, rank, q_rank, layer["mixer"]["scale"], 1e-5, pos, DT[dtype], "cuda", gate="head")
    load_part(mixer, w, "l0.mix.", dtype)
    rng = np.random.default_rng(rank)
    x = {r: stored(rng.standard_normal((n, width)), dtype) for r, n in dict(LENGTHS, c=300).items()}
    sched = [s if i != 6 else [("c", 269), ("d", 15)] for i, s in enumerate(SCHEDULE)]
    got = run_mixer(mixer, x, sched, page=page, pages=640 // page)
    for r in x:
        want = plain.latent_attention(x[r], w, "l0.mix.", layer["mixer"], 1e-5)
        err = np.abs(got[r] - want).max() / np.abs(want).max()
        assert err <= (3e-5 if dtype == "float32" else 3e-2), (r, err)


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_the_first_tokens(tmp_path, name, dtype):
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 16)
    rp = Replayer(runner, cache)
    for n in (1, 2, 3, 47, 130):
        ids = ids_of(cfg, w, n, n, dtype)
        rp.step([(f"r{n}", ids, range(n))], end=[f"r{n}"])
        compare(rp.logits_of(f"r{n}", range(n)), plain.forward(cfg, w, ids), dtype, f"{name} whole {n}")
    assert cache.num_free_pages() == 16


def test_the_stream_after_every_layer_run(tmp_path):
    """The residual stream after each run of a layer (a looped layer counts every time), with what the layer still has
    pending added as the next kernel would add it; float32."""
    from vllm_cpp_b200.parts.base import pending_mult
    cfg, w, _, cache, runner = build(tmp_path, "A", "float32", 8)
    ids = ids_of(cfg, w, 40, 2, "float32")
    _, want = plain.forward(cfg, w, ids, return_layers=True)
    seen = []
    for blk in runner.model.blocks:
        def wrapped(residual, delta, *a, _inner=blk.forward, **k):
            pending = _inner(residual, delta, *a, **k)
            x = residual.double().cpu().numpy()
            seen.append(x + pending_mult(pending) * delta.double().cpu().numpy() if pending else x)
            return pending
        blk.forward = wrapped
    rp = Replayer(runner, cache)
    rp.step([("r", ids, [39])], end=["r"])
    assert len(seen) == len(plain.run_order(cfg)) == want.shape[0]
    for i, (g, t) in enumerate(zip(seen, want)):
        assert np.abs(g - t).max() <= 2e-5 * np.abs(t).max(), f"layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prefill_against_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """The same tokens as one portion and one by one (over many pages) give the same logits."""
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 24)
    n = 170
    ids = ids_of(cfg, w, n, 7, dtype)
    want = plain.forward(cfg, w, ids)
    rp = Replayer(runner, cache)
    rp.step([("p", ids, range(n))], end=["p"])
    compare(rp.logits_of("p", range(n)), want, dtype, f"{name} prefill")
    rp.step([("d", ids[:9], range(9))])
    for t in range(9, n):
        rp.step([("d", ids[t: t + 1], [0])])
    cache.free_request("d")
    compare(rp.logits_of("d", range(n)), want, dtype, f"{name} decode")
    a, b = rp.logits_of("p", range(n)), rp.logits_of("d", range(n))
    assert np.abs(a - b).max() <= (2e-5 if dtype == "float32" else 4e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_down_to_two_tokens(tmp_path, name, dtype):
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 24)
    n = 150
    ids = ids_of(cfg, w, n, 9, dtype)
    want = plain.forward(cfg, w, ids)
    for k, sizes in enumerate(([2] * 75, [5, 2, 31, 2, 17, 64, 3, 26], [16, 16, 1, 15, 33, 2, 67], [149, 1])):
        assert sum(sizes) == n
        rp, t = Replayer(runner, cache), 0
        for s in sizes:
            rp.step([(f"c{k}", ids[t: t + s], range(s))])
            t += s
        cache.free_request(f"c{k}")
        compare(rp.logits_of(f"c{k}", range(n)), want, dtype, f"{name} portions {sizes[:4]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_requests_together_on_few_pages(tmp_path, name, dtype):
    """Up to three live requests of unequal length, portions beside single tokens, on so few pages and slots that both
    are used again by later requests; every request's logits are those it has alone."""
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 28, max_seqs=3)
    rng = np.random.default_rng(3)
    lengths = {"a": 90, "b": 3, "c": 140, "d": 33, "e": 64, "f": 1, "g": 120}
    ids = {r: ids_of(cfg, w, n, 40 + i, dtype) for i, (r, n) in enumerate(lengths.items())}
    want = {r: plain.forward(cfg, w, ids[r]) for r in ids}
    rp = Replayer(runner, cache)
    waiting, live, at = list(lengths), [], {}
    slots_seen = []
    while waiting or live:
        while waiting and len(live) < 3:
            r = waiting.pop(0)
            live.append(r)
            at[r] = 0
        entries, end = [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 40 else rng.choice([1, 2, 7, 16, 29])))
            entries.append((r, ids[r][at[r]: at[r] + s], range(s)))
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        rp.step(entries, end=[])
        slots_seen += [cache.slot(r) for r, _, _ in entries]
        for r in end:
            cache.free_request(r)
            compare(rp.logits_of(r, range(lengths[r])), want[r], dtype, f"{name} mixed {r}")
            live.remove(r)
    assert cache.num_free_pages() == 28 and len(set(slots_seen)) == 3


# larger layers: talking heads of 128 and 64 on the tensor cores (the second with more than eight heads), a latent row of
# 128 and one of 192, experts in tiles
CFG_WIDE = config([att(8, 2, 128, 0.09, mlp=moe(192, 8, 2, 2.0, shared=(256, 1.0))),
                   lat(8, 64, 32, 64, 96, 128, 0.1, 1e5, mlp=dense(640, 2.0)),
                   att(12, 6, 64, 0.125, mlp=dense(512, 1.0)),
                   lat(6, 48, 64, 48, 128, 96, 0.1, 1e4, mlp=moe(128, 4, 1, 1.0))], width=384, vocab=700, loop=(1, 3, 2), mult=0.7)


def test_bfloat16_beside_float32_at_larger_sizes(tmp_path):
    """The same (bfloat16-valued) weights through the float32 engine, which the small configurations anchor to the plain
    implementation, and through the bfloat16 engine: a prompt of 450 tokens in two portions, then single tokens, beside
    a second request."""
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    w = plain.round_to_bf16(plain.random_weights(CFG_WIDE, 3, std=0.05, sharp=1.0, decisive_routing=True))
    rng = np.random.default_rng(5)
    ids = {"a": rng.integers(0, 700, size=480).tolist(), "b": rng.integers(0, 700, size=70).tolist()}
    steps = [[("a", 300)], [("a", 150), ("b", 40)]] + [[("a", 1), ("b", 1)]] * 30
    got = {}
    for dtype in ("float32", "bfloat16"):
        folder = str(tmp_path / dtype)
        plain.write_model_folder(folder, CFG_WIDE, w, store="BF16" if dtype == "bfloat16" else "F32")
        ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=16, num_gpu_blocks=48, max_num_seqs=2, max_model_len=768,
                            max_num_batched_tokens=512, use_cuda_graphs=False)
        _, cache, runner = factory.build(ecfg)
        rp, at = Replayer(runner, cache), {"a": 0, "b": 0}
        for step in steps:
            rp.step([(r, ids[r][at[r]: at[r] + n], range(n)) for r, n in step])
            for r, n in step:
                at[r] += n
        got[dtype] = {r: rp.logits_of(r, range(at[r])) for r in ids}
        del runner, cache
    for r in ids:
        compare(got["bfloat16"][r], got["float32"][r], "bfloat16", f"larger sizes {r}")


@pytest.mark.parametrize("dtype,name,pages", [("float32", "A", 24), ("bfloat16", "C", 24), ("float32", "B", 5)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name, pages):
    """LLM.generate: the scheduler cuts the prompts under a small token budget, decode steps are captured and replayed;
    every generated token is the plain implementation's best, or within rounding of it.  On 5 pages requests are
    preempted and fed again from their first token."""
    from vllm_cpp_b200 import LLM, SamplingParams
    cfg, page = CONFIGS[name]
    weights = make_weights(cfg, 5, dtype)
    folder = str(tmp_path / f"gen_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    llm = LLM(folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=3, max_model_len=pages * page,
              max_num_batched_tokens=48)
    prompts = [np.random.default_rng(500 + n).integers(0, cfg["vocab"], size=n).tolist() for n in (3, 41, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True))
    if pages < 24:
        assert llm.engine.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        assert len(o) == 30
        seq = list(p)
        for tok in o:
            if plain.routing_margin(cfg, weights, seq) < MARGIN[dtype]:
                break                                  # from a routing decision that rounding can turn on, nothing is compared
            logits = plain.forward(cfg, weights, seq)[-1]
            best = plain.greedy(logits)
            gap = (logits[best] - logits[tok]) / np.abs(logits).max()
            assert tok == best or gap < (1e-3 if dtype == "float32" else 5e-2), (dtype, len(p), tok, best, gap)
            seq.append(tok)


def random_gipinex_config(rng):
    """Sizes with odd factors, the two mixers in any order, every kind of feed-forward or none, with and without a loop."""
    width = int(rng.choice([36, 50, 64, 90, 104, 136]))
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        pick = rng.random()
        mlp = None if pick < 0.2 else dense(int(rng.integers(20, 160)), float(rng.uniform(0.5, 4))) if pick < 0.6 else None
        if pick >= 0.6:
            experts = int(rng.integers(1, 9))
            mlp = moe(int(rng.integers(8, 60)), experts, int(rng.integers(1, experts + 1)), float(rng.uniform(0.5, 3)),
                      shared=(int(rng.integers(8, 60)), float(rng.uniform(0.5, 3))) if rng.random() < 0.6 else None)
        if rng.random() < 0.5:
            g = int(rng.integers(1, 4))
            layers.append(att(g * int(rng.integers(1, 5)), g, int(rng.choice([8, 16, 24, 64, 128])), float(rng.uniform(0.1, 0.4)), mlp=mlp))
        else:
            layers.append(lat(int(rng.integers(1, 7)), int(rng.choice([8, 12, 32])), int(rng.choice([2, 4, 16])), int(rng.choice([8, 12, 64])),
                              int(rng.choice([10, 24, 48, 64])), int(rng.choice([6, 16, 40])), float(rng.uniform(0.1, 0.4)),
                              float(rng.choice([10.0, 500.0, 1e4, 1e6])), mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a + 1, n + 1)), int(rng.integers(1, 4)))
    return config(layers, width=width, vocab=int(rng.integers(40, 500)), loop=loop, mult=float(rng.choice([1.0, 0.5, 0.7, 1.3])),
                  eps=float(rng.choice([1e-5, 1e-6, 1e-4])))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [4, 27, 21, 22])
def test_the_replay_program_on_configurations_drawn_at_random(tmp_path, seed, dtype):
    """bin/trace_run on a model folder of a configuration drawn at random, under a schedule of portions and single tokens of
    three requests on a pool made for the tokens that are live; the logits are the plain implementation's."""
    rng = np.random.default_rng(seed)
    cfg = random_gipinex_config(rng)
    w = make_weights(cfg, seed, dtype)
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    plain.write_model_folder(folder, cfg, w, store="BF16" if dtype == "bfloat16" else "F32")
    lengths = {"a": 70, "b": 9, "c": 131}
    ids = {r: ids_of(cfg, w, n, seed + i, dtype) for i, (r, n) in enumerate(lengths.items())}
    steps, at, live, waiting, k = [], {}, [], list(lengths), 0
    while waiting or live:
        while waiting and len(live) < 2:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        entries, end = [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 50 else rng.choice([1, 2, 5, 16, 40])))
            entries.append({"id": r, "tokens": ids[r][at[r]: at[r] + s], "want": list(range(s))})
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        steps.append({"step": k, "entries": entries, "end": end})
        live = [r for r in live if r not in end]
        k += 1
    repo = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    p = subprocess.run([sys.executable, os.path.join(repo, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                        "--max-tokens", "384"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(k)]
    rows = {r: [] for r in lengths}
    for s in steps:
        got = np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        i = 0
        for e in s["entries"]:
            rows[e["id"]].append(got[i: i + len(e["want"])])
            i += len(e["want"])
    for r in lengths:
        compare(np.concatenate(rows[r]), plain.forward(cfg, w, ids[r]), dtype, f"seed {seed} request {r}")
