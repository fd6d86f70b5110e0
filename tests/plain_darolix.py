"""Darolix, plain and slow: NumPy float64, one whole sequence at a time, no
cache and no state (every position is computed from the whole prefix), one
function per mechanism.  It shares nothing with the package: it reads
config.json as a dict and model.safetensors with its own few lines."""
import json
import struct
from pathlib import Path

import numpy as np


def load(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    meta = json.loads(raw[8 : 8 + n])
    data = raw[8 + n :]
    w = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = m["data_offsets"]
        if m["dtype"] == "BF16":
            arr = (np.frombuffer(data[lo:hi], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif m["dtype"] == "F32":
            arr = np.frombuffer(data[lo:hi], dtype="<f4").astype(np.float64)
        else:
            raise ValueError(m["dtype"])
        w[name] = arr.reshape(m["shape"])
    return w, cfg


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def embedding(table, ids, scale, base=10000.0, first_position=0):
    width = table.shape[1]
    pos = np.arange(first_position, first_position + len(ids), dtype=np.float64)[:, None]
    out = table[np.asarray(ids)] * scale
    for i in range((width + 1) // 2):
        angle = pos[:, 0] * base ** (-2.0 * i / width)
        out[:, 2 * i] += np.sin(angle)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] += np.cos(angle)
    return out


def short_convolution(u, taps_w, bias):
    """u [T, C]; taps_w [C, taps], the last column multiplies the token itself; zeros before the start; silu."""
    T, taps = u.shape[0], taps_w.shape[1]
    out = np.zeros_like(u)
    for t in range(T):
        acc = bias.copy()
        for lag in range(taps):
            if t - lag >= 0:
                acc = acc + taps_w[:, taps - 1 - lag] * u[t - lag]
        out[t] = silu(acc)
    return out


def scalar_decay_recurrence(x, B, C, dt, a_log, d_skip, groups):
    """x [T, H, P], B/C [T, G, N], dt [T, H] (already positive): y [T, H, P]."""
    T, H, P = x.shape
    N = B.shape[2]
    y = np.zeros((T, H, P))
    for h in range(H):
        g = h // (H // groups)
        S = np.zeros((N, P))
        rate = np.exp(a_log[h])
        for t in range(T):
            S = np.exp(-rate * dt[t, h]) * S + dt[t, h] * B[t, g][:, None] * x[t, h][None, :]
            y[t, h] = C[t, g] @ S + d_skip[h] * x[t, h]
    return y


def channel_decay_recurrence(q, k, v, alpha):
    """q/k/alpha [T, H, N], v [T, H, P]: o [T, H, P] with S_t = alpha_t[:, None] * S + k_t v_t^T."""
    T, H, N = q.shape
    o = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        S = np.zeros((N, v.shape[2]))
        for t in range(T):
            S = alpha[t, h][:, None] * S + k[t, h][:, None] * v[t, h][None, :]
            o[t, h] = q[t, h] @ S
    return o


def state_space_mixer(m, w, pre, h, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ w[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner : 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N :]
    xbc = short_convolution(xbc, w[pre + "conv"], w[pre + "conv.b"])
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner : inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N :].reshape(T, G, N)
    y = scalar_decay_recurrence(x, B, C, softplus(dt + w[pre + "dt_bias"]), w[pre + "A_log"], w[pre + "D"], G)
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def capped_attention(q, k, v, scale, softcap):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; scores capped by softcap * tanh(. / softcap) when softcap > 0."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[: i + 1, g]
    return out


def query_temperature(positions, coef, every):
    return 1.0 + coef * np.log(np.floor((positions + 1) / every) + 1.0)


def left_branch(m, w, pre, h, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w[pre + "q"].T).reshape(T, H, d), eps)
    k = unit_rms((h @ w[pre + "k"].T).reshape(T, G, d), eps)
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    if m.get("q_temp"):
        q = q * query_temperature(np.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    return capped_attention(q, k, v, m["scale"], m.get("softcap", 0.0)).reshape(T, H * dv) @ w[pre + "o"].T


def right_branch(m, w, pre, h, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, d) / np.sqrt(d)
    k = (h @ w[pre + "k"].T).reshape(T, H, d)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = (1.0 / (1.0 + np.exp(-z))) ** (1.0 / m["tau"])
    o = channel_decay_recurrence(q, k, v, alpha.reshape(T, H, d))
    o = (unit_rms(o, eps) * w[pre + "norm"]).reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def side_by_side(m, w, pre, h, eps):
    a = unit_rms(left_branch(m["left"], w, pre + "left.", h, eps), eps) * w[pre + "left.out"]
    b = unit_rms(right_branch(m["right"], w, pre + "right.", h, eps), eps) * w[pre + "right.out"]
    return (a + b) / 2.0


def route(h, router_w, correction, top):
    """(chosen [T, top], weights [T, top], margins [T]): margin = gap between the last chosen and the first not chosen choice score."""
    z = h @ router_w.T
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s = s / s.sum(axis=1, keepdims=True)
    pick = s + correction
    order = np.argsort(-pick, axis=1, kind="stable")
    chosen = order[:, :top]
    sc = np.take_along_axis(s, chosen, axis=1)
    sorted_pick = np.take_along_axis(pick, order, axis=1)
    margin = sorted_pick[:, top - 1] - sorted_pick[:, top] if pick.shape[1] > top else np.full(len(h), np.inf)
    return chosen, sc / (sc.sum(axis=1, keepdims=True) + 1e-20), margin


def experts_mixture(f, w, pre, h, margins=None):
    E, top = f["router"]["experts"], f["router"]["top"]
    chosen, weight, margin = route(h, w[pre + "router"], w[pre + "correction"], top)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            if e >= E:  # an identity expert
                out[t] += g * h[t]
            else:
                p = pre + f"e{e}."
                out[t] += g * ((silu(h[t] @ w[p + "gate"].T) * (h[t] @ w[p + "up"].T)) @ w[p + "down"].T)
    return out


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for k in range(loop["times"]):
        order += [(i, k > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(ids, w, cfg, streams=None, margins=None):
    """Logits [T, vocab]; ``streams`` collects the residual stream after every layer run, ``margins`` every router's margins."""
    eps = cfg["norm"]["eps"]
    e = embedding(w["embed"], ids, cfg.get("embedding", {}).get("scale", 1.0))
    x = e.copy()
    for i, again in run_order(cfg):
        layer = cfg["layers"][i]
        if again:
            x = x + e
        h = unit_rms(x, eps) * w[f"l{i}.norm1"]
        if layer["type"] == "mamba2":
            y = state_space_mixer(layer["mixer"], w, f"l{i}.mix.", h, eps)
        else:
            y = side_by_side(layer["mixer"], w, f"l{i}.mix.", h, eps)
        if layer.get("mlp"):
            y = y + experts_mixture(layer["mlp"], w, f"l{i}.mlp.", h, margins)
        x = x + y
        if streams is not None:
            streams.append(x.copy())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T


def greedy(ids, n_new, w, cfg):
    seq, out = list(ids), []
    for _ in range(n_new):
        tok = int(np.argmax(forward(seq, w, cfg)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def sure_prefix(margins, n, least=0.02):
    """How many leading positions come before the first close call of any router (a margin below ``least``)."""
    if not margins:
        return n
    close = np.min(np.stack(margins), axis=0) < least
    return int(np.argmax(close)) if close.any() else n
