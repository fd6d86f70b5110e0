"""Plain, slow restatement of the Kotutar decoder: the oracle of its tests.

Whole sequences, no cache, one function per mechanism, NumPy float64.  It
shares no code with the product package: it reads config.json itself and takes
another algebraic route where there is one (keys and values are made per head
from the latent, nothing is carried into the latent space).

Notation.  x: rows of the residual stream [n, width].  rms(v) = v /
sqrt(mean(v^2) + eps).  A layer: x += rms(mixer(rms(x) w1)) w1b, then x +=
rms(ff(rms(x) w2)) w2b.  Looped layers: the stretch start..stop-1 runs `times`
times in a row, every pass opened by x = W_in [x; e] with e the embedding rows.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np

from plain_qwen2 import read_safetensors

_erf = np.vectorize(math.erf, otypes=[np.float64])


def load(folder):
    """(weights as float64 arrays by name, config.json as a dict)."""
    folder = Path(folder)
    return read_safetensors(folder / "model.safetensors"), json.loads((folder / "config.json").read_text())


def rms(v, w=None, eps=1e-6):
    y = v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def turn_pairs(v, positions, base, dims):
    """Neighbouring pairs (2i, 2i+1), i < dims/2, of the last axis of v [n, ..., d]
    turned by positions[n] * base^(-2i/dims); the other dimensions pass."""
    out = np.array(v, dtype=np.float64, copy=True)
    for i in range(dims // 2):
        a = np.asarray(positions, dtype=np.float64) * float(base) ** (-2.0 * i / dims)
        c, s = np.cos(a), np.sin(a)
        while c.ndim < v.ndim - 1:
            c, s = c[..., None], s[..., None]
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_queries(x, w, p, m, eps):
    """q [n, heads, dim + rot_dim] before the rotation."""
    cq = rms(x @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    return (cq @ w[p + "uq"].T).reshape(len(x), m["heads"], m["dim"] + m["rot_dim"])


def latent_rows(x, w, p, m, eps):
    """(c [n, kv_rank] normed, shared key part [n, rot_dim] before the rotation)."""
    both = x @ w[p + "dkv"].T
    return rms(both[:, : m["kv_rank"]], w[p + "dkv.norm"], eps), both[:, m["kv_rank"] :]


def softmax_with_sink(scores, sink):
    """scores [n, n] masked with -inf; one more term exp(sink) in the denominator."""
    top = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - top)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))


def latent_attention(x, positions, w, p, m, eps, window=None):
    n, H, d, r, vd = len(x), m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = latent_queries(x, w, p, m, eps)
    c, kr = latent_rows(x, w, p, m, eps)
    qr = turn_pairs(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"])
    kr = turn_pairs(kr, positions, m["rot"]["base"], m["rot"]["dims"])
    keys = (c @ w[p + "uk"].T).reshape(n, H, d)
    values = (c @ w[p + "uv"].T).reshape(n, H, vd)
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = j <= i
    if window:
        seen &= j > i - window
    heads = []
    for h in range(H):
        s = (q[:, h, :d] @ keys[:, h].T + qr[:, h] @ kr.T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        sink = w[p + "sink"][h] if p + "sink" in w else -np.inf
        heads.append(softmax_with_sink(s, sink) @ values[:, h])
    return np.concatenate(heads, axis=-1) @ w[p + "o"].T


def dense_mlp(x, w, p, bias=True, act=gelu_erf):
    mid = x @ w[p + "up"].T + (w[p + "up.b"] if bias else 0.0)
    return act(mid) @ w[p + "down"].T + (w[p + "down.b"] if bias else 0.0)


def router(x, w, p, top):
    """(chosen experts [n, top], their weights [n, top]): sigmoid scores, the largest first, not renormalised."""
    s = 1.0 / (1.0 + np.exp(-(x @ w[p + "router"].T)))
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def router_margin(x, w, p, top):
    """Per token: how far the last chosen expert's score lies above the best one not chosen (inf when
    all are chosen).  Where it is within rounding, reduced precision may choose otherwise."""
    s = -np.sort(-1.0 / (1.0 + np.exp(-(x @ w[p + "router"].T))), axis=-1)
    return s[:, top - 1] - s[:, top] if top < s.shape[1] else np.full(len(x), np.inf)


def routed_mlp(x, w, p, f, margins=None):
    chosen, weight = router(x, w, p, f["router"]["top"])
    if margins is not None:
        margins.append(router_margin(x, w, p, f["router"]["top"]))
    out = np.zeros_like(x)
    for t in range(len(x)):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += dense_mlp((g * x[t])[None], w, p + f"e{e}.", bias=False)[0]  # the weight multiplies the expert's input
    if f.get("shared"):
        gate = 1.0 / (1.0 + np.exp(-(x @ w[p + "shared.sg"].T)))
        out += gate * dense_mlp(x, w, p + "shared.", bias=False)
    return out


def run_order(cfg):
    """(layer, opens a pass) in running order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    return [(i, False) for i in range(a)] + [(i, i == a) for _ in range(loop["times"]) for i in range(a, b)] + [(i, False) for i in range(b, n)]


def layer(x, positions, w, i, cfg, margins=None):
    eps, p, spec = cfg["norm"]["eps"], f"l{i}.", cfg["layers"][i]
    x = x + rms(latent_attention(rms(x, w[p + "norm1"], eps), positions, w, p + "mix.", spec["mixer"], eps), w[p + "norm1b"], eps)
    f = spec["mlp"]
    if f is not None:
        inner = rms(x, w[p + "norm2"], eps)
        y = routed_mlp(inner, w, p + "mlp.", f, margins) if f["kind"] == "moe" else dense_mlp(inner, w, p + "mlp.")
        x = x + rms(y, w[p + "norm2b"], eps)
    return x


def forward(ids, w, cfg, rows=None, stream=None, margins=None):
    """Logits [n or len(rows), vocab]; ``stream`` (a list) collects x after every layer run, ``margins``
    (a list) the router margins [n] of every run of a routed layer."""
    positions = np.arange(len(ids))
    e = w["embed"][np.asarray(ids)]
    x = e.copy()
    for i, opens in run_order(cfg):
        if opens:
            x = np.concatenate([x, e], axis=-1) @ w["loop.in"].T
        x = layer(x, positions, w, i, cfg, margins)
        if stream is not None:
            stream.append(x.copy())
    x = rms(x, w["final.norm"], cfg["norm"]["eps"])
    if rows is not None:
        x = x[list(rows)]
    return x @ w["head"].T


def sure_prefix(margins, n, least=0.05):
    """How many leading positions of a sequence of n tokens precede its first close call of a router: up
    to there reduced precision must choose the same experts (a position depends on none after it)."""
    if not margins:
        return n
    close = np.nonzero(np.min(np.stack(margins), axis=0) < least)[0]
    return int(close[0]) if len(close) else n


def greedy(ids, n_new, w, cfg):
    seq, out = list(ids), []
    for _ in range(n_new):
        tok = int(np.argmax(forward(seq, w, cfg, rows=[len(seq) - 1])[0]))
        out.append(tok)
        seq.append(tok)
    return out
