"""A plain, slow implementation of the Gipinex design in numpy (float64), one function per mechanism, written from
the design's equations.  It shares no code with the engine: the tests compare the engine with it.

The design.  A pre-norm decoder on one residual stream: x += m * mixer(norm_a(x)), x += m * ff(norm_b(x)), the norms
RMS norms whose gain is stored around zero (1 + w), m a constant of the model.  A run of layers may be walked several
times with the same weights (every pass has a cache of its own); right before the first layer of each such pass the
stream is re-made from itself and the embedding output x0:  x <- W_in [x ; x0].  The model's output is the norm of the
stream times the embedding table.  Mixers:

  "attention"         grouped-query softmax attention without rotation and without a value projection: the values are
                      the unnormed key projection, while scores are taken between q and k divided by their root mean square
                      per head.  A score is scale * q_i . k_j - slope_h * (i - j) with slope_h = 2^(-8 (h + 1) / H); the
                      scores of the H heads at (i, j) are then mixed by an H x H matrix before the softmax.  The
                      concatenated heads are gated coordinate by coordinate by sigmoid(W_g x).
  "latent_attention"  queries through a normed low-rank row; one normed low-rank row per token of which every head's keys
                      (the part without rotation) and values are projections, and one rotated key part that all heads
                      share (pairs 2i, 2i + 1); one sigmoid gate per head.

Feed-forwards: a dense gated one with biases and a clamped activation, or routed experts of the same form without
biases (the ``top`` largest router logits, softmax over those alone) plus a shared expert that every token takes.
"""
import json
import math
import os
import struct

import numpy as np

SWISH_ALPHA = 1.702
SLOPE_LOG2_SPAN = 8.0           # slope_h = 2^(-8 (h + 1) / H)


# ------------------------------------------------------------- files
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif meta["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: type {meta['dtype']}")
        out[name] = a.astype(np.float64).reshape(meta["shape"])
    return out


def read_model_folder(path):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(path, "model.safetensors"))


def round_to_bf16(weights):
    out = {}
    for k, v in weights.items():
        u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        out[k] = u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(v))
    return out


def write_model_folder(path, cfg, weights, store="F32"):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, w in weights.items():
        a = np.ascontiguousarray(w, dtype=np.float32)
        if store == "BF16":
            u = a.view(np.uint32).astype(np.uint64)
            raw = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype("<u2")).tobytes()
        else:
            raw = a.astype("<f4").tobytes()
        header[name] = {"dtype": store, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


# ------------------------------------------------------------- shapes and random weights
def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration has."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        H = m["heads"]
        if layer["type"] == "attention":
            G = m.get("kv_heads") or H
            out.update({p + "mix.q": (H * m["dim"], W), p + "mix.k": (G * m["dim"], W), p + "mix.talk": (H, H),
                        p + "mix.g": (H * m["vdim"], W), p + "mix.o": (W, H * m["vdim"])})
        else:
            out.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],),
                        p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],),
                        p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]),
                        p + "mix.g": (H, W), p + "mix.o": (W, H * m["vdim"])})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            for nm, shape in (("gate", (mlp["ff"], W)), ("up", (mlp["ff"], W)), ("down", (W, mlp["ff"]))):
                out[p + "mlp." + nm] = shape
                out[p + "mlp." + nm + ".b"] = shape[:1]
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            out[p + "mlp.router"] = (E, W)
            out[p + "mlp.router.b"] = (E,)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def random_weights(cfg, seed, std=0.08, gain_std=0.1, sharp=1.0, decisive_routing=False):
    """Normal weights; norm gains around zero; the mixing matrix of the heads near the identity; the projections of
    queries and keys times ``sharp`` (peaked attention, so that a wrong key shows).  ``decisive_routing``: the routers'
    biases lie far apart and their matrices are small, so that no rounding of a router's input turns a choice."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".")[-1]
        if name.endswith("norm1") or name.endswith("norm2") or name == "final.norm":
            w = rng.normal(0.0, gain_std, shape)
        elif tail == "norm":                     # the latents' norms: plain gains
            w = 1.0 + rng.normal(0.0, gain_std, shape)
        elif tail == "talk":
            w = np.eye(shape[0]) + rng.normal(0.0, 0.15, shape)
        elif name.endswith("router.b"):
            w = rng.permutation(shape[0]) * 0.7 if decisive_routing else rng.normal(0.0, 0.3, shape)
        elif name.endswith("mlp.router") and decisive_routing:
            w = rng.normal(0.0, 0.02 * std, shape)
        elif tail == "b":
            w = rng.normal(0.0, std, shape)
        else:
            w = rng.normal(0.0, std, shape)
            if name.endswith((".mix.q", ".mix.uq", ".mix.k", ".mix.uk")):
                w = w * sharp
        out[name] = w
    return out


# ------------------------------------------------------------- mechanisms
def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def clamped_swish_ff(h, w_gate, w_up, w_down, limit, b_gate=None, b_up=None, b_down=None):
    """down(g * sigmoid(1.702 g) * (u + 1)) with g cut off above ``limit`` and u on both sides."""
    g = h @ w_gate.T + (0.0 if b_gate is None else b_gate)
    u = h @ w_up.T + (0.0 if b_up is None else b_up)
    g = np.minimum(g, limit)
    u = np.clip(u, -limit, limit)
    return (g * sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ w_down.T + (0.0 if b_down is None else b_down)


def route(h, w_router, b_router, top, margins=None):
    """(chosen experts [n, top], their weights): the ``top`` largest logits, softmax over those alone.  ``margins``
    (a list) receives the smallest gap between a chosen logit and the best one left out."""
    z = h @ w_router.T + b_router
    if margins is not None and top < z.shape[-1]:
        ranked = -np.sort(-z, axis=-1)
        margins.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, order, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return order, e / e.sum(axis=-1, keepdims=True)


def routed_ff(h, weights, p, mlp, margins=None):
    ids, wts = route(h, weights[p + "router"], weights[p + "router.b"], mlp["router"]["top"], margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wts[t]):
            q = f"{p}e{int(e)}."
            out[t] += a * clamped_swish_ff(h[t:t + 1], weights[q + "gate"], weights[q + "up"], weights[q + "down"],
                                           mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_swish_ff(h, weights[p + "shared.gate"], weights[p + "shared.up"], weights[p + "shared.down"],
                                mlp["shared"]["limit"])
    return out


def feed_forward(h, weights, p, mlp, margins=None):
    if mlp["kind"] == "dense":
        return clamped_swish_ff(h, weights[p + "gate"], weights[p + "up"], weights[p + "down"], mlp["limit"],
                                weights[p + "gate.b"], weights[p + "up.b"], weights[p + "down.b"])
    return routed_ff(h, weights, p, mlp, margins)


def head_slopes(H):
    return np.array([2.0 ** (-SLOPE_LOG2_SPAN * (h + 1) / H) for h in range(H)])


def talking_attention(h, weights, p, m, eps):
    """One request, whole: h [n, width] -> [n, width]."""
    n = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads") or H
    q = (h @ weights[p + "q"].T).reshape(n, H, d)
    k = (h @ weights[p + "k"].T).reshape(n, G, d)
    v = k                                           # the unnormed key projection doubles as the value
    qn, kn = rms(q, eps), rms(k, eps)
    pos = np.arange(n)
    dist = pos[:, None] - pos[None, :]              # i - j
    s = np.empty((H, n, n))
    slopes = head_slopes(H)
    for a in range(H):
        s[a] = (qn[:, a] @ kn[:, a // (H // G)].T) * m["scale"] - slopes[a] * dist
    s = np.einsum("ab,bij->aij", weights[p + "talk"], s)
    s = np.where(dist[None] >= 0, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    w = w / w.sum(axis=-1, keepdims=True)
    o = np.empty((n, H, dv))
    for a in range(H):
        o[:, a] = w[a] @ v[:, a // (H // G), :dv]
    o = o.reshape(n, H * dv) * sigmoid(h @ weights[p + "g"].T)
    return o @ weights[p + "o"].T


def rotate_pairs(x, positions, base, dims):
    """Pairs (2i, 2i + 1) of the first ``dims`` coordinates of the last axis turned by position * base^(-2i / dims).
    x: [n, ..., D]; positions: [n]."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = positions[:, None] * base ** (-2.0 * i / dims)                 # [n, dims / 2]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h, weights, p, m, eps):
    """One request, whole, keys and values formed per head as the equations say."""
    n = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n, dtype=np.float64)
    cq = rms(h @ weights[p + "dq"].T, eps) * weights[p + "dq.norm"]
    q = (cq @ weights[p + "uq"].T).reshape(n, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"])
    kv = h @ weights[p + "dkv"].T
    c = rms(kv[:, :rank], eps) * weights[p + "dkv.norm"]
    k_rot = rotate_pairs(kv[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])          # [n, r], shared by the heads
    k_plain = (c @ weights[p + "uk"].T).reshape(n, H, d)
    v = (c @ weights[p + "uv"].T).reshape(n, H, dv)
    gate = sigmoid(h @ weights[p + "g"].T)                                  # [n, H]
    mask = pos[:, None] >= pos[None, :]
    o = np.empty((n, H, dv))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        w = np.exp(s)
        w = w / w.sum(axis=-1, keepdims=True)
        o[:, a] = (w @ v[:, a]) * gate[:, a:a + 1]
    return o.reshape(n, H * dv) @ weights[p + "o"].T


MIXERS = {"attention": talking_attention, "latent_attention": latent_attention}


def run_order(cfg):
    """[(layer, enters a pass)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, k = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(a)]
    for _ in range(k):
        out += [(i, i == a) for i in range(a, b)]
    return out + [(i, False) for i in range(b, n)]


def forward(cfg, weights, ids, return_layers=False, margins=None):
    """Logits [n, vocab] of one request's tokens, all at once."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = weights["embed"][np.asarray(ids)]
    x = x0.copy()
    after = []
    for li, enters in run_order(cfg):
        if enters:
            x = np.concatenate([x, x0], axis=-1) @ weights["loop.in"].T
        layer, p = cfg["layers"][li], f"l{li}."
        x = x + m * MIXERS[layer["type"]](offset_norm(x, weights[p + "norm1"], eps), weights, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + m * feed_forward(offset_norm(x, weights[p + "norm2"], eps), weights, p + "mlp.", layer["mlp"], margins)
        after.append(x.copy())
    logits = offset_norm(x, weights["final.norm"], eps) @ weights["embed"].T
    return (logits, np.stack(after)) if return_layers else logits


def routing_margin(cfg, weights, ids):
    """The smallest gap, over all routed layers and tokens, between a chosen router logit and the best one left out."""
    margins = []
    forward(cfg, weights, ids, margins=margins)
    return min(margins) if margins else math.inf


def greedy(logits):
    return int(np.argmax(logits))
