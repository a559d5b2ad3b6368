"""A plain, slow implementation of the Lutodra design in numpy (float64), one function per mechanism, written from
the design's equations.  It shares no code with the engine: the tests compare the engine with it.

The design.  A decoder whose residual stream is ``streams`` copies x_1 .. x_s of the embedding (hyper-connections).
Sublayer q of a layer reads u = sum_s in_q[s] x_s through a layer norm with gain and bias, and its result y joins
every stream at once: x_t <- sum_s mix_q[s, t] x_s + out_q[t] y.  The model's output is the layer norm of the sum of
the streams, a product with ``head`` and a constant.  A run of layers may be walked several times over with the
same weights (every pass has state and cache of its own).  Mixers:

  "attention"      grouped-query softmax attention; queries and keys RMS-normed per head (one gain vector for all
                   heads), rotated on their first ``rot.dims`` coordinates (pairs i, i + dims / 2; frequencies
                   base^(-2i/dims), rescaled by wavelength), scores scaled by a given constant, a learned logit per head
                   in the softmax's denominator that has no value, a sigmoid gate per head on the result
  "rglru"          two branches of ``width``: gelu_tanh(W_y h + b) and a causal convolution of (W_x h + b); gates from
                   block-diagonal products of the convolved branch; S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with
                   a_t = exp(-8 r_t softplus(lam)); result W_o (S_t * y_t)
  "channel_delta"  the gated delta rule: q, k, v through short causal convolutions and silu, q and k made unit vectors,
                   a decay per head and key channel, S <- g S; S += k (beta (v - S^T k))^T; o = S^T q, then an RMS norm
                   per head, a sigmoid gate from a low-rank product, W_o

Feed-forwards: SwiGLU, or routed experts with sigmoid scores, groups of neighbouring experts of which only the best
may be chosen from (a group's score: the sum of its two largest), weights divided by their sum and scaled.
"""
import json
import math
import os
import struct

import numpy as np

GROUP_SCORE_TOP = 2
WEIGHT_SUM_EPS = 1e-20
UNIT_EPS = 1e-6
RGLRU_C = 8.0


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
    for name in sorted(weights):
        a = np.ascontiguousarray(weights[name], dtype=np.float32)
        raw = (a.view(np.uint32) >> 16).astype("<u2").tobytes() if store == "BF16" else a.astype("<f4").tobytes()
        header[name] = {"dtype": store, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))


# ------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(z, eps):
    """z divided by its root mean square over the last axis, eps inside the root."""
    return z / np.sqrt((z * z).mean(axis=-1, keepdims=True) + eps)


def layer_norm(z, w, b, eps):
    d = z - z.mean(axis=-1, keepdims=True)
    return d / np.sqrt((d * d).mean(axis=-1, keepdims=True) + eps) * w + b


def causal_conv(x, taps, bias=None):
    """y[t, c] = sum_j taps[c, j] x[t - (J - 1) + j, c] (+ bias[c]); rows before the first are zero."""
    n, J = x.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((J - 1, x.shape[1])), x], axis=0)
    y = np.zeros_like(x)
    for j in range(J):
        y += padded[j: j + n] * taps[:, j]
    return y if bias is None else y + bias


# ------------------------------------------------------------- mixers
def rglru_mixer(w, p, m, h):
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    bs = W // B
    r, i = np.empty_like(u), np.empty_like(u)
    for b in range(B):
        sl = slice(b * bs, (b + 1) * bs)
        r[:, sl] = sigmoid(u[:, sl] @ w[p + "ra"][b].T + w[p + "ra.b"][b])
        i[:, sl] = sigmoid(u[:, sl] @ w[p + "ri"][b].T + w[p + "ri.b"][b])
    a = np.exp(-RGLRU_C * r * softplus(w[p + "lam"]))
    S = np.zeros(W)
    out = np.empty_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S * y[t]
    return out @ w[p + "o"].T


def gated_delta_rule(q, k, v, g, beta):
    """One head.  q, k, g: [n, dk]; v: [n, dv]; beta: [n].  S starts at zero."""
    n, dk = q.shape
    S = np.zeros((dk, v.shape[1]))
    o = np.empty_like(v)
    for t in range(n):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def channel_delta_mixer(w, p, m, h, eps):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(n, G, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(n, G, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(n, H, dv)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + UNIT_EPS) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ w[p + "b"].T)                                              # [n, H]
    pre = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * softplus(pre).reshape(n, H, dk))
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(n, H, dv)
    out = np.empty((n, H, dv))
    for head in range(H):
        kv = head // (H // G)
        o = gated_delta_rule(q[:, kv], k[:, kv], v[:, head], g[:, head], beta[:, head])
        out[:, head] = rms_unit(o, eps) * w[p + "norm"] * gate[:, head]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def rotary_frequencies(rot):
    dims = rot["dims"]
    f = rot["base"] ** (-2.0 * np.arange(dims // 2) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
        out = np.empty_like(f)
        for i, fi in enumerate(f):
            wl = 2.0 * math.pi / fi
            if wl < orig / high:
                out[i] = fi
            elif wl > orig / low:
                out[i] = fi / factor
            else:
                s = (orig / wl - low) / (high - low)
                out[i] = (1.0 - s) * fi / factor + s * fi
        f = out
    return f


def rotate(x, positions, freqs):
    """x: [n, heads, d]; the first 2 * len(freqs) coordinates of every head are rotated, pair (i, i + len(freqs))."""
    half = len(freqs)
    ang = positions[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half: 2 * half]
    out = x.copy()
    out[..., :half] = a * c - b * s
    out[..., half: 2 * half] = b * c + a * s
    return out


def attention_mixer(w, p, m, h, eps, positions=None):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    positions = np.arange(n, dtype=np.float64) if positions is None else positions
    q = rms_unit((h @ w[p + "q"].T).reshape(n, H, dk), eps) * w[p + "q.norm"]
    k = rms_unit((h @ w[p + "k"].T).reshape(n, G, dk), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    if m.get("rot"):
        f = rotary_frequencies(m["rot"])
        q, k = rotate(q, positions, f), rotate(k, positions, f)
    gate = sigmoid(h @ w[p + "g"].T)                                              # [n, H]
    out = np.empty((n, H, dv))
    causal = np.tril(np.ones((n, n), dtype=bool))
    if m.get("window"):                       # position i sees j with i - window < j <= i (not of this design; the part offers it)
        causal &= ~np.tril(np.ones((n, n), dtype=bool), -int(m["window"]))
    for head in range(H):
        kv = head // (H // G)
        s = np.where(causal, (q[:, head] @ k[:, kv].T) * m["scale"], -np.inf)
        sink = w[p + "sink"][head]
        top = np.maximum(s.max(axis=1, keepdims=True), sink)
        e = np.exp(s - top)
        out[:, head] = (e @ v[:, kv]) / (e.sum(axis=1, keepdims=True) + np.exp(sink - top)) * gate[:, head: head + 1]
    return out.reshape(n, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------- feed-forwards
def gated_ff(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(w, p, r, h, margins=None):
    """(chosen [n, top], weights [n, top]).  ``margins`` collects how far each decision is from turning."""
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ w[p + "router"].T)
    allowed = np.ones_like(s, dtype=bool)
    groups = r.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        per = E // count
        parts = np.sort(s.reshape(-1, count, per), axis=-1)
        gs = parts[..., -GROUP_SCORE_TOP:].sum(axis=-1)                           # [n, count]
        order = np.argsort(-gs, axis=-1, kind="stable")
        kept = np.zeros_like(gs, dtype=bool)
        np.put_along_axis(kept, order[:, :keep], True, axis=-1)
        allowed = np.repeat(kept, per, axis=-1)
        if margins is not None and keep < count:
            sg = np.sort(gs, axis=-1)
            margins.extend((sg[:, count - keep] - sg[:, count - keep - 1]).tolist())
    masked = np.where(allowed, s, -np.inf)
    order = np.argsort(-masked, axis=-1, kind="stable")
    chosen = order[:, :top]
    if margins is not None and top < allowed.sum(axis=-1).min():
        sm = np.take_along_axis(masked, order, axis=-1)
        margins.extend((sm[:, top - 1] - sm[:, top]).tolist())
    wts = np.take_along_axis(s, chosen, axis=-1)
    wts = wts / (wts.sum(axis=-1, keepdims=True) + WEIGHT_SUM_EPS) * r["scale"]
    return chosen, wts


def moe_ff(w, p, mlp, h, margins=None):
    chosen, wts = route(w, p, mlp["router"], h, margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], wts[t]):
            out[t] += a * gated_ff(w, f"{p}e{e}.", h[t: t + 1])[0]
    return out


# ------------------------------------------------------------- the model
def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    body = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + body * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, w, tokens, return_layers=False, margins=None):
    """Logits [n, vocab] of one request's tokens (and, asked for, the sum of the streams after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)]
    s = cfg.get("streams")
    x = [x0.copy() for _ in range(s or 1)]
    seen = []
    for li in run_order(cfg):
        layer, p = cfg["layers"][li], f"l{li}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if sub == "mlp" and layer.get("mlp") is None:
                continue
            if s:
                u = sum(w[f"{p}hc{q}.in"][i] * x[i] for i in range(s))
            else:
                u = x[0]
            hn = layer_norm(u, w[f"{p}norm{q}"], w[f"{p}norm{q}.b"], eps)
            if sub == "mixer":
                kind, m = layer["type"], layer["mixer"]
                if kind == "attention":
                    y = attention_mixer(w, p + "mix.", m, hn, eps)
                elif kind == "rglru":
                    y = rglru_mixer(w, p + "mix.", m, hn)
                elif kind == "channel_delta":
                    y = channel_delta_mixer(w, p + "mix.", m, hn, eps)
                else:
                    raise ValueError(kind)
            else:
                mlp = layer["mlp"]
                y = gated_ff(w, p + "mlp.", hn) if mlp["kind"] == "dense" else moe_ff(w, p + "mlp.", mlp, hn, margins)
            if s:
                mix, out = w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"]
                x = [sum(mix[i, t] * x[i] for i in range(s)) + out[t] * y for t in range(s)]
            else:
                x = [x[0] + y]
        seen.append(sum(x))
    final = layer_norm(sum(x), w["final.norm"], w["final.norm.b"], eps)
    logits = final @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, np.stack(seen)) if return_layers else logits


def greedy(logits_row):
    return int(np.argmax(logits_row))


def routing_margin(cfg, w, tokens):
    margins = []
    forward(cfg, w, tokens, margins=margins)
    return min(margins) if margins else math.inf


# ------------------------------------------------------------ random models
DEFAULT_RANK = 8


def tensor_shapes(cfg, rank=DEFAULT_RANK):
    D, V = cfg["width"], cfg["vocab"]
    s = cfg.get("streams")
    shapes = {"embed": (V, D), "head": (V, D), "final.norm": (D,), "final.norm.b": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            shapes[f"{p}norm{q}"] = (D,)
            shapes[f"{p}norm{q}.b"] = (D,)
            if s:
                shapes[f"{p}hc{q}.in"] = (s,)
                shapes[f"{p}hc{q}.out"] = (s,)
                shapes[f"{p}hc{q}.mix"] = (s, s)
        x = p + "mix."
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({x + "q": (H * dk, D), x + "k": (G * dk, D), x + "v": (G * dv, D), x + "q.norm": (dk,), x + "k.norm": (dk,),
                           x + "sink": (H,), x + "g": (H, D), x + "o": (D, H * dv)})
        elif layer["type"] == "rglru":
            W, B, J = m["width"], m["blocks"], m["conv"]
            shapes.update({x + "y": (W, D), x + "y.b": (W,), x + "x": (W, D), x + "x.b": (W,), x + "conv": (W, J), x + "conv.b": (W,),
                           x + "ra": (B, W // B, W // B), x + "ra.b": (B, W // B), x + "ri": (B, W // B, W // B), x + "ri.b": (B, W // B),
                           x + "lam": (W,), x + "o": (D, W)})
        else:
            H, G, dk, dv, J = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            shapes.update({x + "q": (G * dk, D), x + "q.conv": (G * dk, J), x + "k": (G * dk, D), x + "k.conv": (G * dk, J),
                           x + "v": (H * dv, D), x + "v.conv": (H * dv, J), x + "b": (H, D), x + "A_log": (H,), x + "norm": (dv,),
                           x + "a1": (rank, D), x + "a2": (H * dk, rank), x + "dt_bias": (H * dk,), x + "g1": (rank, D),
                           x + "g2": (H * dv, rank), x + "o": (D, H * dv)})
        mlp = layer.get("mlp")
        f = p + "mlp."
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            shapes.update({f + "gate": (mlp["ff"], D), f + "up": (mlp["ff"], D), f + "down": (D, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{f}e{e}.gate": (ff, D), f"{f}e{e}.up": (ff, D), f"{f}e{e}.down": (D, ff)})
            shapes[f + "router"] = (mlp["router"]["experts"], D)
    return shapes


def static_levels(rng, router, floor=0.04):
    """Router levels (one logit per expert, in an order drawn at random) whose decisions between groups and between
    experts all have a clear margin in score space."""
    E, top = router["experts"], router["top"]
    step = min(0.35, 5.0 / E)
    for _ in range(200):
        c = rng.permutation((np.arange(E) - (E - 1) / 2.0) * step + rng.uniform(-0.1, 0.1, E) * step)
        margins = []
        route({"x.router": c[:, None]}, "x.", router, np.ones((1, 1)), margins)
        if not margins or min(margins) > floor:
            return c
    raise AssertionError("no router levels with clear margins found")


def random_weights(cfg, seed, sharp=1.0, rank=DEFAULT_RANK, decisive_routing=False):
    """Weights that keep the residual stream of order one and make every mechanism matter: peaked attention (``sharp``
    scales the query and key gains), sinks around the scores' size, decays spread between fast and slow, mixing
    matrices near the identity with visible off-diagonal parts, biases that are not zero.  ``decisive_routing``: the
    routers' inputs get a coordinate that is always 1 (gain 0, bias 1 in the norm before) and the routers read mostly
    that, every expert at a level of its own, so that no rounding of the input turns a choice (for 16-bit runs; what
    follows the input is covered by the 32-bit runs and the router's own test)."""
    rng = np.random.default_rng(seed)
    D = cfg["width"]
    w = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        fan_in = shape[-1] if len(shape) > 1 else D
        if leaf.startswith("norm") and leaf.endswith(".b") or name == "final.norm.b":
            a = 0.1 * rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf.endswith("hc1.in") or leaf.endswith("hc2.in"):
            a = 1.0 / shape[0] + 0.3 * rng.standard_normal(shape)
        elif leaf.endswith(".out"):
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif leaf.endswith(".mix") and "hc" in leaf:
            a = np.eye(shape[0]) + 0.25 * rng.standard_normal(shape)
        elif leaf in ("mix.q.norm", "mix.k.norm"):
            a = (1.0 + 0.1 * rng.standard_normal(shape)) * sharp
        elif leaf == "mix.sink":
            a = rng.standard_normal(shape) * 2.0
        elif leaf == "mix.norm":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf in ("mix.conv", "mix.q.conv", "mix.k.conv", "mix.v.conv"):
            a = rng.standard_normal(shape) * 0.5
        elif leaf in ("mix.y.b", "mix.x.b", "mix.conv.b", "mix.ra.b", "mix.ri.b"):
            a = 0.3 * rng.standard_normal(shape)
        elif leaf == "mix.lam":
            a = rng.uniform(-4.0, 0.5, shape)
        elif leaf == "mix.A_log":
            a = rng.uniform(-3.0, 0.5, shape)
        elif leaf == "mix.dt_bias":
            a = rng.uniform(-3.0, 0.0, shape)
        elif leaf in ("mix.ra", "mix.ri"):
            a = rng.standard_normal(shape) * (1.5 / math.sqrt(shape[-1]))
        elif leaf == "mlp.router":
            a = rng.standard_normal(shape) * (2.0 / math.sqrt(D))
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / math.sqrt(fan_in)
        w[name] = a.astype(np.float64)
    if decisive_routing:
        for i, layer in enumerate(cfg["layers"]):
            mlp = layer.get("mlp")
            if mlp and mlp["kind"] == "moe":
                w[f"l{i}.norm2"][0], w[f"l{i}.norm2.b"][0] = 0.0, 1.0
                r = 0.01 / math.sqrt(D) * rng.standard_normal((mlp["router"]["experts"], D))
                r[:, 0] = static_levels(rng, mlp["router"])
                w[f"l{i}.mlp.router"] = r
    return w
