"""The Lutodra design on the GPU against the plain implementation of plain_lutodra.py: each mechanism alone (the
streams' join and norm, the short convolution, both recurrent mixers under every cut with slots used again, a key
written into the delta rule's state hundreds of tokens before it is asked for, attention with its sink, head norms,
partial rescaled rotation and gate, the router with groups), then whole models under every way of cutting the work and
greedy generation through the engine's entry point, the replay program and the command line.  Configurations and
weights are made here."""
import json
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import plain_lutodra as plain
from helpers import MEAN_TOL, TOL, Replayer
from test_lutodra_config import att, config, delta, dense, moe, rglru, rot

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# three streams, a looped stretch that starts after the first layer, key and value sizes that differ, three query heads
# per kv head, two delta heads per key head, convolutions of 2, 3 and 5 taps, a recurrent width that is not the model's,
# groups of experts of which some stay, a rotation of part of a head with all three branches of the rescaling
CFG_A = config([rglru(48, 3, conv=3, mlp=dense(96)),
                att(6, 2, 32, 16, 0.3, rot(16, 300.0, (8.0, 1.0, 3.0, 48)), mlp=moe(40, 8, 3, 2.0, groups=(4, 2))),
                delta(4, 2, 16, 24, conv=2, mlp=moe(24, 3, 1)),
                rglru(96, 1, conv=5, mlp=moe(16, 6, 2, 0.7, groups=(2, 1))),
                att(2, 2, 64, 64, 0.125, rot(64, 10000.0), mlp=dense(72))], width=64, vocab=200, streams=3, loop=(1, 3, 2),
               logit_scale=0.5)
# one stream with mixing tensors, widths with odd factors, an odd vocabulary, no loop, a layer without feed-forward, every
# expert chosen, one kv head, attention without rotation, a convolution of one tap, one delta head with many key channels
CFG_B = config([att(4, 1, 24, 40, 0.4, None, mlp=moe(16, 3, 3, 1.0)),
                delta(1, 1, 72, 8, conv=1, mlp=None),
                rglru(72, 4, conv=2, mlp=dense(50)),
                delta(5, 5, 8, 12, conv=4, mlp=dense(56)),
                att(5, 5, 16, 16, 0.25, rot(8, 50.0, (2.0, 0.5, 8.0, 16)), mlp=moe(20, 4, 2, 1.5, groups=(2, 2)))],
               width=72, vocab=301, streams=1, eps=1e-6)
# a plain residual stream (no ``streams`` key), the whole model walked three times over
CFG_C = config([delta(2, 1, 16, 16, conv=3, mlp=dense(40)), att(2, 1, 16, 24, 0.3, rot(4, 20.0), mlp=None),
                rglru(40, 2, conv=4, mlp=moe(24, 4, 2, 1.0, groups=(4, 3)))], width=40, vocab=97, streams=None, loop=(0, 3, 3))
CONFIGS = {"A": (CFG_A, 16), "B": (CFG_B, 32), "C": (CFG_C, 16)}
SHARP = {"float32": 3.0, "bfloat16": 1.0}
MARGIN = {"float32": 2e-5, "bfloat16": 6e-3}        # routing decisions closer than this are left to rounding


def compare(got, want, dtype, what=""):
    """Rows of logits against the plain implementation's.  float32: every row within TOL of the largest logit.
    bfloat16: the mean error within MEAN_TOL, and every row within TOL but for one row in fifty (at least one), which
    may reach twice that: a delta-rule head's result is normed by itself, and where its terms nearly cancel the norm
    multiplies the rounding of the projections by the inverse of what is left."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    scale = np.abs(want).max()
    rows = np.abs(got - want).max(axis=1) / scale
    over = int((rows > TOL[dtype]).sum())
    allowed = 0 if dtype == "float32" else max(1, len(rows) // 50)
    assert over <= allowed and rows.max() <= 2 * TOL[dtype], (
        f"{what}: {over} of {len(rows)} rows over {TOL[dtype]:.0e} of the largest logit, worst {rows.max():.3e} at row {int(rows.argmax())}")
    assert np.abs(got - want).mean() <= MEAN_TOL[dtype] * scale, f"{what}: mean error {np.abs(got - want).mean() / scale:.3e}"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def stored(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy().astype(np.float64)


def make_weights(cfg, seed, dtype):
    # bfloat16 rounds the routers' inputs: there a constant coordinate decides who is chosen (the router's own test and
    # the float32 runs cover choices that follow the input)
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
    folder = str(tmp_path / f"lutodra_{name}_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=num_pages, max_num_seqs=max_seqs,
                        max_model_len=num_pages * page, max_num_batched_tokens=1024, use_cuda_graphs=graphs)
    model, cache, runner = factory.build(ecfg)
    return cfg, weights, folder, cache, runner


def mixer_harness(mixer, page, pages, max_len, max_seqs=3):
    """The engine's cache manager and step packing around one mixer: steps come out of ModelRunner._prepare."""
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    cache = CacheManager([mixer.cache_spec()], page, pages, max_seqs, mixer.dtype, "cuda")
    fake = types.SimpleNamespace(vocab=100, blocks=[types.SimpleNamespace(parts={"mixer": mixer})], final_norm=None,
                                 spec=types.SimpleNamespace(max_position_embeddings=max_len))
    return cache, ModelRunner(fake, cache, 1024, max_seqs, max_len, torch.device("cuda", 0))


def run_mixer(mixer, x, schedule, page=16, pages=40, max_len=600, max_seqs=2, width_out=None):
    """Feeds the rows x[request] through ``mixer`` as ``schedule`` cuts them ([(request, tokens), ...] per step); a
    request that has had all its rows is freed, so later requests take its slot and pages.  Returns request -> rows."""
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import StepEntry
    from vllm_cpp_b200.parts.base import Workspace
    cache, runner = mixer_harness(mixer, page, pages, max_len, max_seqs)
    ws = Workspace("cuda")
    dtype = mixer.dtype
    at = {r: 0 for r in x}
    got = {r: [] for r in x}
    slots = []
    for entries in schedule:
        for r, _ in entries:
            if r not in cache.requests:
                cache.add_request(r)
        step = runner._prepare([StepEntry(r, [0] * n, []) for r, n in entries])
        rows = dev(np.concatenate([x[r][at[r]: at[r] + n] for r, n in entries]), dtype)
        out = torch.empty((rows.shape[0], width_out or rows.shape[1]), dtype=dtype, device="cuda")
        ws.reset()
        mixer.forward(rows, out, step, runner.views[0], True, ws)
        o, t0 = out.float().cpu().numpy(), 0
        for r, n in entries:
            got[r].append(o[t0: t0 + n])
            t0 += n
            at[r] += n
            cache.commit(r, n)
            slots.append(cache.slot(r))
            if at[r] == len(x[r]):
                cache.free_request(r)
    ops.check_status()
    assert all(at[r] == len(x[r]) for r in x), "the schedule does not feed every row"
    return {r: np.concatenate(got[r]) for r in x}, slots


# four requests of unequal length on two slots: portions of changing size beside single tokens, the second pair
# taking the slots (with their stale numbers) that the first pair gave back
LENGTHS = {"a": 37, "b": 5, "c": 64, "d": 18}
SCHEDULE = [[("a", 1), ("b", 3)], [("b", 2), ("a", 2)], [("a", 17)], [("a", 16)], [("a", 1), ("c", 30)], [("c", 1), ("d", 2)],
            [("c", 33), ("d", 15)], [("d", 1)]]


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,width,with_next", [(1, 72, True), (2, 72, False), (3, 2500, True), (8, 320, True), (2, 64, True)])
def test_streams_join_and_norm(dtype, S, width, with_next):
    """x_t <- sum_s mix[s, t] x_s + out[t] y for all streams at once (from, to: a transposed matrix shows), the read of
    the next sublayer through its layer norm with bias, and the model's last norm on gathered rows with its factor."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(S * width)
    n, eps = 6, 3e-6
    x = rng.standard_normal((S, n, width)).astype(np.float32) + 0.5
    y = stored(2 * rng.standard_normal((n, width)), dtype)
    mix = (np.eye(S) + 0.4 * rng.standard_normal((S, S))).astype(np.float32)
    out_c, in_c = (1 + 0.3 * rng.standard_normal(S)).astype(np.float32), rng.standard_normal(S).astype(np.float32)
    w, b = (1 + 0.2 * rng.standard_normal(width)).astype(np.float32), (0.3 * rng.standard_normal(width)).astype(np.float32)
    xd = dev(x)
    nxt = torch.empty((n, width), dtype=DT[dtype], device="cuda") if with_next else None
    ops.stream_join(xd, dev(y, DT[dtype]), dev(mix), dev(out_c), eps, next_coef=dev(in_c) if with_next else None,
                    next_w=dev(w) if with_next else None, next_b=dev(b) if with_next else None, next_out=nxt)
    want = np.stack([sum(mix[s, t] * x[s].astype(np.float64) for s in range(S)) + out_c[t] * y for t in range(S)])
    assert np.abs(xd.cpu().numpy() - want).max() <= 3e-6 * np.abs(want).max()
    if S > 1:
        wrong = np.stack([sum(mix[t, s] * x[s].astype(np.float64) for s in range(S)) + out_c[t] * y for t in range(S)])
        assert np.abs(wrong - want).max() > 0.1
    if with_next:
        u = sum(in_c[t] * want[t] for t in range(S))
        want2 = plain.layer_norm(u, w, b, eps)
        assert np.abs(nxt.float().cpu().numpy() - want2).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want2).max()
    rows = np.array([4, 0, 4], dtype=np.int32)
    last = torch.empty((3, width), dtype=DT[dtype], device="cuda")
    ops.stream_norm(xd, dev(np.ones(S, dtype=np.float32)), dev(w), dev(b), last, eps, dev(rows), 1.7)
    want3 = 1.7 * plain.layer_norm(want.sum(axis=0), w, b, eps)[rows]
    assert np.abs(last.float().cpu().numpy() - want3).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want3).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,J,act,biases", [(40, 4, "silu", False), (130, 2, "none", True), (8, 1, "silu", False), (300, 8, "none", True),
                                             (64, 3, "silu", True)])
def test_short_convolution_under_every_cut(dtype, C, J, act, biases):
    """The last column of the taps is the current token's; the J - 1 inputs before a portion come from the request's
    slot, zeros before the start; a portion shorter than J - 1 keeps part of what the slot held."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(C + J)
    taps = rng.standard_normal((C, J)).astype(np.float32)
    pb = rng.standard_normal(C).astype(np.float32) if biases else None
    cb = rng.standard_normal(C).astype(np.float32) if biases else None
    x = {r: stored(rng.standard_normal((n, C)), dtype) for r, n in LENGTHS.items()}
    want = {}
    for r in x:
        y = plain.causal_conv(x[r] + (pb if biases else 0.0), taps.astype(np.float64), cb)
        want[r] = plain.silu(y) if act == "silu" else y
    state = torch.full((2, max(J - 1, 1) + 1, C), 9.0, device="cuda")[:, 1:]       # a strided view, as a slot with more rows gives
    free, slot, at, got = [1, 0], {}, {r: 0 for r in x}, {r: [] for r in x}
    for step in SCHEDULE:
        for r, _ in step:
            if r not in slot:
                slot[r] = free.pop()
                state[slot[r]].zero_()
        rows = np.concatenate([x[r][at[r]: at[r] + n] for r, n in step])
        wide = dev(np.concatenate([np.zeros((len(rows), 3)), rows], axis=1), DT[dtype])       # a column slice of a wider buffer
        out = torch.empty((len(rows), C), dtype=torch.float32, device="cuda")
        q_start = dev(np.cumsum([0] + [n for _, n in step]).astype(np.int32))
        ops.causal_conv(wide[:, 3:], dev(taps), state, out, q_start, dev(np.array([slot[r] for r, _ in step], dtype=np.int32)), len(step),
                        max(n for _, n in step), pre_bias=None if pb is None else dev(pb), bias=None if cb is None else dev(cb), act=act)
        o, t0 = out.cpu().numpy(), 0
        for r, n in step:
            got[r].append(o[t0: t0 + n])
            t0 += n
            at[r] += n
            if at[r] == LENGTHS[r]:
                free.append(slot.pop(r))
    for r in x:
        g = np.concatenate(got[r])
        assert np.abs(g - want[r]).max() <= 3e-6 * np.abs(want[r]).max(), (r, int(np.abs(g - want[r]).max(axis=1).argmax()))
    if J > 1:
        flipped = plain.causal_conv(x["a"] + (pb if biases else 0.0), taps[:, ::-1].astype(np.float64), cb)
        assert np.abs((plain.silu(flipped) if act == "silu" else flipped) - want["a"]).max() > 0.1


def part_weights(w, p, dtype, float_names=()):
    """The tensors ``p*`` of a plain weight dictionary as a part's load_params wants them: matrices in the run's type,
    vectors, taps and what ``float_names`` lists in float32."""
    out = {}
    for name, a in w.items():
        if name.startswith(p):
            short = name[len(p):]
            small = a.ndim == 1 or short.endswith("conv") or short in float_names or short.endswith(".b") and a.ndim <= 2 and short != "b"
            out[short] = dev(np.asarray(a, dtype=np.float32), torch.float32 if small else DT[dtype])
    return out


def rows_close(got, want, tol, what):
    scale = np.abs(want).max()
    err = np.abs(got - want).max(axis=1)
    assert np.isfinite(got).all() and err.max() <= tol * scale, (
        f"{what}: first wrong token {int(np.argmax(err > tol * scale))}, error {err.max():.3e} of {scale:.3e}")


LONG = {"a": 37, "b": 5, "c": 64, "d": 18, "e": 260}
LONG_SCHEDULE = SCHEDULE + [[("e", 131)], [("e", 2)]] + [[("e", 1)]] * 120 + [[("e", 7)]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,width,blocks,taps", [(40, 48, 3, 3), (64, 64, 1, 4), (24, 130, 2, 1), (72, 96, 96, 5), (32, 192, 4, 2)])
def test_real_gated_linear_recurrence(dtype, hidden, width, blocks, taps):
    """The whole mixer through the cache manager's slots: unequal requests, portions cut anywhere beside single tokens,
    slots given back and taken again, 120 single tokens in a row; a recurrent width that is not the model's, one block,
    blocks of one channel, one tap."""
    from vllm_cpp_b200.parts.gated_recurrence import RealGatedLinearRecurrence
    cfg = config([rglru(width, blocks, conv=taps)], width=hidden, vocab=10)
    w = plain.random_weights(cfg, hidden + width)
    w = plain.round_to_bf16(w) if dtype == "bfloat16" else w
    p, m = "l0.mix.", cfg["layers"][0]["mixer"]
    mixer = RealGatedLinearRecurrence(hidden, width, blocks, taps, DT[dtype], "cuda", gate_constant=plain.RGLRU_C)
    mixer.load_params(part_weights(w, p, dtype))
    rng = np.random.default_rng(taps)
    x = {r: stored(rng.standard_normal((n, hidden)), dtype) for r, n in LONG.items()}
    got, slots = run_mixer(mixer, x, LONG_SCHEDULE)
    assert len(set(slots)) == 2
    for r in x:
        rows_close(got[r], plain.rglru_mixer(w, p, m, x[r]), 2e-5 if dtype == "float32" else 2.5e-2, f"rglru {r}")
    # the state matters: the same rows from an empty state at a cut give another result
    want = plain.rglru_mixer(w, p, m, x["e"])
    assert np.abs(plain.rglru_mixer(w, p, m, x["e"][131:]) - want[131:])[:4].max() > 0.02 * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,H,G,dk,dv,taps", [(40, 4, 2, 16, 24, 2), (64, 1, 1, 72, 8, 1), (48, 5, 5, 8, 12, 4), (32, 6, 2, 32, 32, 3),
                                                   (64, 2, 1, 128, 64, 4)])
def test_gated_delta_rule_mixer(dtype, hidden, H, G, dk, dv, taps):
    """As above for the delta rule: several heads on one key head, one head of many key channels, key and value sizes
    that differ, low-rank products whose inner width the tensors give (5 here)."""
    from vllm_cpp_b200.parts.gated_recurrence import GatedDeltaRule
    cfg = config([delta(H, G, dk, dv, conv=taps)], width=hidden, vocab=10, eps=2e-6)
    w = plain.random_weights(cfg, H * dk + dv, rank=5)
    w = plain.round_to_bf16(w) if dtype == "bfloat16" else w
    p, m = "l0.mix.", cfg["layers"][0]["mixer"]
    mixer = GatedDeltaRule(hidden, H, G, dk, dv, taps, 2e-6, DT[dtype], "cuda")
    mixer.load_params(part_weights(w, p, dtype))
    assert mixer.rank_a == 5 and mixer.rank_g == 5
    rng = np.random.default_rng(dk)
    x = {r: stored(rng.standard_normal((n, hidden)), dtype) for r, n in LONG.items()}
    got, slots = run_mixer(mixer, x, LONG_SCHEDULE)
    assert len(set(slots)) == 2
    for r in x:
        want = plain.channel_delta_mixer(w, p, m, x[r], 2e-6)
        if dtype == "float32":
            rows_close(got[r], want, 3e-5, f"delta {r}")
        else:
            # a head's result is normed by itself: where it nearly cancels, rounding of the projections is multiplied
            err = np.abs(got[r] - want).max(axis=1) / np.abs(want).max()
            assert np.isfinite(got[r]).all() and np.median(err) <= 1.5e-2 and (err > 5e-2).mean() <= 0.03, (r, err.max(), int(err.argmax()))


@pytest.mark.parametrize("H,G,dk,dv,planted_at,cut", [(2, 1, 16, 8, 0, 250), (4, 2, 32, 16, 3, 7), (1, 1, 64, 64, 17, 300), (3, 3, 8, 40, 1, 2)])
def test_a_key_written_long_before_it_is_asked_for(H, G, dk, dv, planted_at, cut):
    """The recurrence itself with chosen inputs: one early token writes a value under a key direction that no later key
    touches and whose channel hardly decays; four hundred tokens later, across a cut of the prompt, single tokens, and a
    second request beside it, a query along that direction reads the value back.  A state that is dropped, zeroed, or
    written to the neighbour's slot gives nothing there."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(dk + dv)
    n = 420
    q = rng.standard_normal((n, G, dk))
    k = rng.standard_normal((n, G, dk))
    v = rng.standard_normal((n, H, dv))
    k[:, :, 0] = 0.0
    k[planted_at] = 0.0
    k[planted_at, :, 0] = 3.0
    v[planted_at] = 5.0 * np.sign(rng.standard_normal((H, dv)))
    q[400:] = 0.0
    q[400:, :, 0] = 2.0
    beta_pre = rng.standard_normal((n, H))
    beta_pre[planted_at] = 8.0
    decay_pre = rng.standard_normal((n, H, dk))
    decay_pre[:, :, 0] = -30.0                      # softplus -> 0: the planted channel keeps what it holds
    a_log, dt_bias = 0.3 * rng.standard_normal(H), 0.1 * rng.standard_normal((H, dk))
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    q, k, v, beta_pre, decay_pre, a_log, dt_bias = map(f32, (q, k, v, beta_pre, decay_pre, a_log, dt_bias))
    unit = lambda z: z / np.sqrt((z * z).sum(axis=-1, keepdims=True) + plain.UNIT_EPS)
    g = np.exp(-np.exp(a_log)[None, :, None] * plain.softplus(decay_pre + dt_bias))
    want = np.stack([plain.gated_delta_rule(unit(q[:, h // (H // G)]) * dk ** -0.5, unit(k[:, h // (H // G)]), v[:, h], g[:, h],
                                            plain.sigmoid(beta_pre[:, h])) for h in range(H)], axis=1)
    assert np.abs(want[400:]).min() > 0.5          # the planted value is what the late queries read
    state = torch.full((3, H, dk, dv), 7.0, device="cuda")
    state[1].zero_()
    state[2].zero_()
    other = {name: dev(np.asarray(rng.standard_normal(a[:1].shape), dtype=np.float32)) for name, a in
             (("q", q), ("k", k), ("v", v), ("b", beta_pre), ("d", decay_pre))}
    got = np.zeros((n, H, dv))
    portions = [cut, 400 - cut - 10] + [1] * 20 + [10]
    assert sum(portions) == n
    t = 0
    for s in portions:
        # the other request (slot 2) stands first in the batch with one token, this one (slot 1) second
        pack = lambda a, name: torch.cat([other[name].reshape(1, -1), dev(np.asarray(a[t: t + s], dtype=np.float32)).reshape(s, -1)]).contiguous()
        out = torch.empty((s + 1, H * dv), device="cuda")
        ops.gated_delta_scan(pack(q, "q"), pack(k, "k"), pack(v, "v"), pack(beta_pre, "b"), pack(decay_pre, "d"), dev(np.float32(a_log)),
                             dev(np.float32(dt_bias).reshape(-1)), state, out, dev(np.array([0, 1, s + 1], dtype=np.int32)),
                             dev(np.array([2, 1], dtype=np.int32)), 2, num_heads=H, num_qk_heads=G, q_scale=dk ** -0.5,
                             unit_eps=plain.UNIT_EPS, max_q_len=s)
        got[t: t + s] = out[1:].cpu().numpy().reshape(s, H, dv)
        t += s
    ops.check_status()
    assert float(state[0].min()) == 7.0             # nobody's slot is left alone
    rows_close(got.reshape(n, -1), want.reshape(n, -1), 3e-5, "planted key")


@pytest.mark.parametrize("dtype,H,G,dk,dv,rotation,page,plain_kernel", [
    ("float32", 4, 2, 32, 16, rot(16, 300.0, (8.0, 1.0, 3.0, 48)), 16, True), ("float32", 3, 3, 24, 40, None, 16, True),
    ("float32", 2, 1, 8, 8, rot(8, 20.0), 32, True), ("bfloat16", 6, 2, 64, 64, rot(32, 1e4, (5.0, 1.0, 3.0, 128)), 16, False),
    ("bfloat16", 6, 2, 64, 64, rot(32, 1e4, (5.0, 1.0, 3.0, 128)), 16, True), ("bfloat16", 2, 1, 128, 128, rot(128, 1e5), 32, False),
    ("bfloat16", 20, 1, 64, 64, None, 16, False), ("bfloat16", 4, 4, 128, 128, rot(64, 500.0), 16, False),
    ("bfloat16", 8, 2, 64, 64, rot(32, 2e4, (3.0, 1.0, 2.0, 64)), 16, False), ("bfloat16", 16, 8, 128, 128, rot(16, 30.0), 32, False),
    ("bfloat16", 5, 1, 48, 80, rot(24, 50.0, (2.0, 0.5, 8.0, 16)), 16, True), ("float32", 8, 8, 16, 16, rot(2, 7.0), 16, True)])
def test_attention_with_a_sink_and_a_planted_key(dtype, H, G, dk, dv, rotation, page, plain_kernel):
    """The mixer itself (its products are identities, so its input rows are q, k, v and the gate's logits) through the
    cache manager's pages, two requests, portions beside single tokens across page borders.  Request "a" has one key
    near its start that the queries of its last tokens point at (in the coordinates that no rotation turns): a key far
    away, among hundreds, carries most of their weight.  The sinks are as large as the largest scores, so a sink that is
    left out, scaled, or counted per key shows; every head has its own.  bfloat16 heads of 64 and 128 run the tensor-core
    kernels (a portion's tiles, single tokens in splits that are merged) unless the case asks for the plain one."""
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts import model as _registers_every_part  # noqa: F401
    from vllm_cpp_b200.parts.sink_attention import SinkAttention
    rng = np.random.default_rng(dk * H + dv)
    T, scale, eps, far = 330, 0.3, 1e-5, 6
    o0, o1, o2 = H * dk, H * dk + G * dk, H * dk + G * dk + G * dv
    width = max(o2 + H, H * dv)
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": scale, "rot": rotation}
    position = PartSpec("none") if rotation is None else PartSpec("scaled_rope", {
        "theta": rotation["base"], "rotary_dim": rotation["dims"], "pairing": "half", "scaling": rotation.get("scaling")})
    att_ = SinkAttention(width, H, G, dk, dv, scale, eps, position, DT[dtype], "cuda")
    # normed rows have unit mean square: peaked scores in 32-bit, milder ones where the normed rows are rounded to 16 bits
    sharp = (1.6 if dtype == "float32" else 1.0) / np.sqrt(scale)
    eye = np.eye(width)
    p = "x."
    w = {p + "q": eye[:o0], p + "k": eye[o0:o1], p + "v": eye[o1:o2], p + "g": eye[o2: o2 + H], p + "o": eye[:, : H * dv],
         p + "q.norm": stored((1 + 0.1 * rng.standard_normal(dk)) * sharp / dk ** 0.25, "bfloat16"),
         p + "k.norm": stored((1 + 0.1 * rng.standard_normal(dk)) * sharp / dk ** 0.25, "bfloat16"),
         p + "sink": stored(4.0 + 2.0 * rng.standard_normal(H), "bfloat16")}
    att_.load_params(part_weights(w, p, dtype))
    if plain_kernel:
        att_._tensor_core_path = lambda: False
    else:
        assert att_._tensor_core_path()
    x = {r: rng.standard_normal((n, width)) for r, n in (("a", T), ("b", 90))}
    unrot = slice(rotation["dims"] if rotation else 0, dk) if (rotation is None or rotation["dims"] < dk) else None
    if unrot is not None:
        d = np.zeros(dk)
        d[unrot] = 3.0 * np.sign(rng.standard_normal(dk)[unrot])
        for g in range(G):
            x["a"][far, o0 + g * dk: o0 + (g + 1) * dk] += 2 * d
        for h in range(H):
            x["a"][300:, h * dk: (h + 1) * dk] += d
    x = {r: stored(a, dtype) for r, a in x.items()}
    # the oracle gets the rounding of the normed, rotated rows only through the weights: bfloat16 runs compare loosely
    want = {r: plain.attention_mixer(w, p, m, x[r], eps) for r in x}
    w_no_sink = dict(w)
    w_no_sink[p + "sink"] = np.full(H, -50.0)
    assert np.abs(plain.attention_mixer(w_no_sink, p, m, x["a"], eps) - want["a"]).max() > 0.1 * np.abs(want["a"]).max()
    if unrot is not None:
        blind = x["a"].copy()
        blind[far, o1:o2] = 0.0                        # the far key's value: the late tokens' results rest on it
        late = np.abs(plain.attention_mixer(w, p, m, blind, eps) - want["a"])[300:, : H * dv]
        assert np.median(late.max(axis=1)) > 0.1 * np.abs(want["a"]).max()
    steps = [[("a", 70), ("b", 3)], [("b", 80), ("a", 1)], [("a", 200), ("b", 1)], [("a", 2), ("b", 2)]] + [[("a", 1), ("b", 1)]] * 4 \
        + [[("a", 1)]] * 40 + [[("a", 13)]]
    got, _ = run_mixer(att_, x, steps, page=page, pages=2 * (-(-T // page)) + 2, max_len=T + page, max_seqs=3, width_out=width)
    for r in x:
        rows_close(got[r][:, : H * dv], want[r][:, : H * dv], 3e-5 if dtype == "float32" else 3e-2, f"attention {r}")


@pytest.mark.parametrize("dtype,H,G,d,window,page", [("float32", 2, 1, 16, 21, 16), ("bfloat16", 4, 2, 64, 33, 16), ("bfloat16", 2, 2, 128, 24, 32),
                                                     ("float32", 3, 3, 8, 1, 16)])
def test_the_part_s_window_with_a_sink(dtype, H, G, d, window, page):
    """The part takes a window (no layer of this design has one): position i sees the last ``window`` keys.  Every
    key leans towards the queries' direction, some more than others, so that a key more or fewer at the window's far edge
    moves the result beyond rounding (the plain implementation with a window one off says by how much); the sink stays in
    the denominator."""
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts import model as _registers_every_part  # noqa: F401
    from vllm_cpp_b200.parts.sink_attention import SinkAttention
    rng = np.random.default_rng(window)
    T, scale, eps = 150, 0.3, 1e-5
    o0, o1, o2 = H * d, H * d + G * d, H * d + 2 * G * d
    width = o2 + H
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": scale, "rot": None, "window": window}
    part = SinkAttention(width, H, G, d, d, scale, eps, PartSpec("none"), DT[dtype], "cuda", window=window)
    eye, p = np.eye(width), "x."
    gain = stored(np.full(d, (1.5 if dtype == "float32" else 1.0) / np.sqrt(scale) / d ** 0.25), "bfloat16")
    w = {p + "q": eye[:o0], p + "k": eye[o0:o1], p + "v": eye[o1:o2], p + "g": eye[o2:], p + "o": eye[:, : H * d],
         p + "q.norm": gain, p + "k.norm": gain, p + "sink": stored(2.0 + rng.standard_normal(H), "bfloat16")}
    part.load_params(part_weights(w, p, dtype))
    x = {r: rng.standard_normal((n, width)) for r, n in (("a", T), ("b", 70))}
    direction = 2.0 * np.sign(rng.standard_normal(d))
    for r in x:
        for t in range(len(x[r])):                       # every key carries the direction, one in five strongly
            for g in range(G):
                x[r][t, o0 + g * d: o0 + (g + 1) * d] += direction * (1.0 + 1.0 * ((len(x[r]) - t) % 5))
        for h in range(H):
            x[r][:, h * d: (h + 1) * d] += direction
    x = {r: stored(a, dtype) for r, a in x.items()}
    want = {r: plain.attention_mixer(w, p, m, x[r], eps) for r in x}
    for other in (window + 1, max(window - 1, 1)) if window > 1 else (2,):
        off = plain.attention_mixer(w, p, dict(m, window=other), x["a"], eps)
        assert np.abs(off - want["a"]).max() > 0.03 * np.abs(want["a"]).max()
    steps = [[("a", 40), ("b", 3)], [("b", 60), ("a", 1)], [("a", 70), ("b", 1)]] + [[("a", 1), ("b", 1)]] * 6 + [[("a", 1)]] * 20 + [[("a", 13)]]
    got, _ = run_mixer(part, x, steps, page=page, pages=2 * (-(-T // page)) + 2, max_len=T + page, max_seqs=3, width_out=width)
    for r in x:
        rows_close(got[r][:, : H * d], want[r][:, : H * d], 3e-5 if dtype == "float32" else 3e-2, f"window {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,ff,experts,top,groups,scale", [(9, 72, 40, 6, 2, (3, 2), 2.5), (150, 64, 24, 3, 3, None, 1.0),
                                                                 (33, 80, 16, 8, 3, (4, 2), 0.5), (700, 48, 20, 15, 4, (3, 1), 1.25),
                                                                 (40, 40, 8, 4, 1, (4, 4), 1.0), (64, 32, 16, 16, 2, (2, 1), 3.0),
                                                                 (50, 48, 16, 6, 2, (6, 3), 1.0)])
def test_experts_routed_by_sigmoid_scores_within_groups(dtype, n, width, ff, experts, top, groups, scale):
    """Scores are sigmoids; a group counts by the sum of its two best; only experts of the groups that stay can be
    chosen; weights are the chosen scores over their sum, times the scale.  Also: no groups, every group kept, every
    expert chosen, one expert chosen, groups of two (whose score is then their whole sum)."""
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.moe import RoutedExperts
    rng = np.random.default_rng(n + experts)
    p = "x."
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    w = {p + "router": stored(4 * rng.standard_normal((experts, width)) / np.sqrt(width), "bfloat16")}
    for e in range(experts):
        w[f"{p}e{e}.gate"] = stored(2 * rng.standard_normal((ff, width)) / np.sqrt(width), dtype)
        w[f"{p}e{e}.up"] = stored(2 * rng.standard_normal((ff, width)) / np.sqrt(width), dtype)
        w[f"{p}e{e}.down"] = stored(rng.standard_normal((width, ff)) / np.sqrt(ff), dtype)
    h = stored(rng.standard_normal((n, width)), dtype)
    margins = []
    want = plain.moe_ff(w, p, mlp, h, margins)
    per_token = np.asarray(margins).reshape(-1, n).min(axis=0) if margins else np.full(n, 1.0)
    clear = per_token > 1e-4
    assert clear.sum() > 0.9 * n
    if groups and groups[1] < groups[0] and experts // groups[0] > 1:        # groups of one only restate the order of the scores
        free = plain.moe_ff(w, p, {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}, h)
        assert np.abs(free - want).max() > 0.05 * np.abs(want).max()          # the groups decide something here
    g, k = groups or (1, 1)
    part = RoutedExperts(width, ff, experts, 0, top, float("inf"), DT[dtype], "cuda", activation="silu", score="sigmoid", correction=False,
                         groups=g, keep_groups=k, group_top=plain.GROUP_SCORE_TOP, normalize=True, sum_eps=plain.WEIGHT_SUM_EPS,
                         route_scale=scale)
    part.load_params(part_weights(w, p, dtype, float_names=("router",)))
    out = torch.empty((n, width), dtype=DT[dtype], device="cuda")
    part.forward(dev(h, DT[dtype]), out, None, Workspace("cuda"))
    got = out.float().cpu().numpy()
    err = np.abs(got - want)[clear].max()
    assert err <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), err


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


def test_the_streams_after_every_layer_run(tmp_path):
    """The sum of the streams after each run of a layer (a looped layer counts every time), float32."""
    cfg, w, _, cache, runner = build(tmp_path, "A", "float32", 8)
    ids = ids_of(cfg, w, 40, 2, "float32")
    _, want = plain.forward(cfg, w, ids, return_layers=True)
    seen = []
    for blk in runner.model.blocks:
        def wrapped(residual, *a, _inner=blk.forward, **k):
            result = _inner(residual, *a, **k)
            seen.append(residual.float().sum(dim=0).cpu().numpy())
            return result
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


# larger layers: heads of 128 and 64, a delta rule with 128 key channels, recurrent widths above the model's, experts
# in tiles, portions that run in pieces
CFG_WIDE = config([rglru(512, 8, conv=4, mlp=dense(640)),
                   att(8, 2, 128, 128, 0.09, rot(64, 1e5, (8.0, 1.0, 4.0, 256)), mlp=moe(192, 8, 2, 2.0, groups=(4, 2))),
                   delta(4, 2, 128, 64, conv=4, mlp=moe(128, 4, 1)),
                   att(6, 6, 64, 64, 0.125, rot(64, 1e4), mlp=dense(512)),
                   rglru(384, 3, conv=4, mlp=None)], width=384, vocab=700, streams=4, loop=(2, 4, 2), logit_scale=1.5)


def test_bfloat16_beside_float32_at_larger_sizes(tmp_path):
    """The same (bfloat16-valued) weights through the float32 engine, which the small configurations anchor to the plain
    implementation, and through the bfloat16 engine: a prompt of 450 tokens in two portions, then single tokens, beside
    a second request."""
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    w = plain.round_to_bf16(plain.random_weights(CFG_WIDE, 3, sharp=1.0, decisive_routing=True))
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


@pytest.mark.parametrize("dtype,name,pages", [("float32", "A", 24), ("bfloat16", "A", 24), ("float32", "B", 5), ("float32", "C", 24)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name, pages):
    """LLM.generate: the scheduler cuts the prompts under a small token budget, decode steps are captured and replayed;
    every generated token is the plain implementation's best, or within rounding of it.  On 5 pages requests are
    preempted and fed again from their first token: their state slots start from zero again."""
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


def random_lutodra_config(rng):
    """Sizes with odd factors, the three mixers in any order, every kind of feed-forward or none, with and without
    streams, loop, rotation, rescaling and groups.  (Value heads of a delta mixer have eight channels and more: a head's
    result is normed by itself, and the norm of three or four channels is too often nearly zero.)"""
    width = int(rng.choice([36, 50, 64, 90, 104, 136]))
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        pick = rng.random()
        mlp = None if pick < 0.2 else dense(int(rng.integers(20, 160))) if pick < 0.6 else None
        if pick >= 0.6:
            count = int(rng.choice([1, 2, 3]))
            per = int(rng.integers(2 if count > 1 else 1, 5))
            keep = int(rng.integers(1, count + 1))
            mlp = moe(int(rng.integers(8, 60)), count * per, int(rng.integers(1, per * keep + 1)), float(rng.uniform(0.5, 3)),
                      groups=(count, keep) if count > 1 or rng.random() < 0.5 else None)
        kind = rng.integers(0, 3)
        if kind == 0:
            blocks = int(rng.choice([1, 2, 3, 5]))
            layers.append(rglru(blocks * int(rng.integers(3, 40)), blocks, conv=int(rng.integers(1, 6)), mlp=mlp))
        elif kind == 1:
            g = int(rng.integers(1, 4))
            layers.append(delta(g * int(rng.integers(1, 4)), g, int(rng.choice([4, 8, 12, 16, 40, 72])), int(rng.choice([8, 16, 33, 64])),
                                conv=int(rng.integers(1, 6)), mlp=mlp))
        else:
            g = int(rng.integers(1, 4))
            dk = int(rng.choice([8, 16, 24, 64]))
            dims = int(rng.choice([0, 2, dk // 2, dk]))
            scaling = None if rng.random() < 0.4 else (float(rng.uniform(1.5, 16)), float(rng.uniform(0.5, 1.5)), float(rng.uniform(2, 8)),
                                                       int(rng.choice([8, 32, 128, 1024])))
            layers.append(att(g * int(rng.integers(1, 4)), g, dk, int(rng.choice([8, 12, 64])), float(rng.uniform(0.1, 0.4)),
                              rot(dims, float(rng.choice([10.0, 500.0, 1e4, 1e6])), scaling) if dims else None, mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a + 1, n + 1)), int(rng.integers(1, 4)))
    return config(layers, width=width, vocab=int(rng.integers(40, 500)), streams=[None, 1, 2, 3, 4][int(rng.integers(0, 5))], loop=loop,
                  logit_scale=float(rng.choice([1.0, 0.25, 3.0])), eps=float(rng.choice([1e-5, 1e-6, 1e-4])))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [4, 27, 21, 22, 25])
def test_the_replay_program_on_configurations_drawn_at_random(tmp_path, seed, dtype):
    """bin/trace_run as a user calls it, on a configuration drawn at random, under a schedule drawn at random: JSON
    lines in, <step>.f32 files and 'done' lines out; a pool of as many tokens as live requests hold, four slots."""
    rng = np.random.default_rng(seed)
    cfg = random_lutodra_config(rng)
    weights = make_weights(cfg, seed, dtype)
    folder = str(tmp_path / "model")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    lengths = {f"q{i}": int(n) for i, n in enumerate(rng.choice([1, 2, 30, 77, 150, 64], size=6))}
    ids = {r: ids_of(cfg, weights, n, seed * 100 + i, dtype) for i, (r, n) in enumerate(lengths.items())}
    waiting, live, at, lines, asked = list(lengths), [], {}, [], []
    most = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        most = max(most, sum(-(-lengths[r] // 64) * 64 for r in live))
        entries, end, rows = [], [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 50 else rng.choice([1, 2, 3, 16, 37, 64])))
            want = sorted(set(int(x) for x in rng.integers(0, s, size=min(s, 3))))
            entries.append({"id": r, "tokens": ids[r][at[r]: at[r] + s], "want": want})
            rows += [(r, at[r] + x) for x in want]
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        lines.append({"step": len(lines), "entries": entries, "end": end})
        asked.append(rows)
        live = [r for r in live if r not in end]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    want = {r: plain.forward(cfg, weights, ids[r]) for r in ids}
    got_rows, want_rows = [], []
    for i, rows in enumerate(asked):
        if rows:
            got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape[0] == len(rows), f"step {i}: {got.shape[0]} rows written, {len(rows)} asked for"
            got_rows.append(got)
            want_rows.append(np.stack([want[r][t] for r, t in rows]))
    compare(np.concatenate(got_rows), np.concatenate(want_rows), dtype, f"seed {seed}: {cfg['layers']}")


def test_command_line_and_sampling_options(tmp_path):
    """python -m vllm_cpp_b200.engine.cli on a Lutodra folder, the architecture taken from config.json or named by
    --arch: greedy ids are the plain implementation's; seeded sampling gives ids of the vocabulary, the same when asked again."""
    cfg, page = CONFIGS["B"]
    weights = make_weights(cfg, 8, "float32")
    folder = str(tmp_path / "cli_model")
    plain.write_model_folder(folder, cfg, weights, store="F32")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = ids_of(cfg, weights, 21, 3, "float32")
    base = [sys.executable, "-m", "vllm_cpp_b200.engine.cli", "--model", folder, "--dtype", "float32", "--block-size", str(page),
            "--num-gpu-blocks", "24", "--max-num-seqs", "2", "--max-model-len", "128", "--max-num-batched-tokens", "64", "--ignore-eos",
            "--prompt-ids", ",".join(map(str, prompt))]
    env = dict(os.environ, PYTHONPATH=root)

    def run(extra):
        p = subprocess.run(base + extra, capture_output=True, text=True, timeout=600, env=env, cwd=root)
        assert p.returncode == 0, p.stderr[-3000:]
        return [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]

    greedy = run(["--max-tokens", "6", "--temperature", "0"])
    seq = list(prompt)
    for tok in greedy:
        logits = plain.forward(cfg, weights, seq)[-1]
        assert tok == plain.greedy(logits) or (logits.max() - logits[tok]) / np.abs(logits).max() < 1e-3
        seq.append(tok)
    options = ["--arch", "lutodra", "--max-tokens", "12", "--temperature", "0.9", "--top-k", "20", "--top-p", "0.9",
               "--repetition-penalty", "1.2", "--sample-seed", "5"]
    drawn = run(options)
    assert len(drawn) == 12 and all(0 <= t < cfg["vocab"] for t in drawn)
    assert run(options) == drawn
