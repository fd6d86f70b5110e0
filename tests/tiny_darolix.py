"""The tests' own small Darolix configurations and weights.

Sizes differ between the configurations and from layer to layer: inner sizes
unlike the width, one and several groups, state sizes that are no power of
two, key and value sizes that differ, as many key/value heads as query heads
and fewer, with and without a cap of the scores and a query temperature, one
and several experts per token, with and without identity experts, layers
without a feed-forward, loops that start at the first layer and later, one
pass, and no loop.  Weights are drawn here: matrices N(0, gain / sqrt(inputs))
so that scores, router logits, decays and gates are of order one."""
import json
from pathlib import Path

import numpy as np
import torch


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def pair(heads, kv_heads, dim, vdim, scale, softcap, q_temp, r_heads, r_dim, r_vdim, tau):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        left["softcap"] = softcap
    if q_temp:
        left["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau}}


def moe(experts, identity, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # a loop over layers 1..2, twice; inner 120 unlike the width; three norm parts; a cap low enough to bend scores; temperature steps every 4 tokens
    "A": {"architecture": "Darolix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [layer("parallel", pair(6, 3, 16, 24, 0.3, 5.0, (0.5, 4), 3, 16, 40, 4.0), moe(5, 2, 3, 40)),
                     layer("mamba2", mamba(5, 24, 16, 1, 3, 3), moe(5, 2, 3, 40)),
                     layer("parallel", pair(2, 1, 24, 8, 0.2, 0.0, None, 2, 8, 8, 9.0), None),
                     layer("mamba2", mamba(4, 8, 40, 4, 2, 1), moe(3, 0, 1, 24))]},
    # no loop; a width that is no multiple of 8; as many key/value heads as heads; no identity experts; two taps
    "B": {"architecture": "Darolix", "vocab": 157, "width": 100, "norm": {"eps": 3e-6}, "embedding": {"scale": 1.0},
          "layers": [layer("mamba2", mamba(6, 12, 24, 3, 2, 2), moe(7, 0, 2, 24)),
                     layer("parallel", pair(5, 5, 12, 12, 0.25, 30.0, (0.2, 7), 5, 20, 4, 1.0), moe(4, 3, 4, 16))]},
    # three passes from the first layer; sizes in multiples of 64 that the tensor-core kernels take
    "C": {"architecture": "Darolix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3}, "loop": {"start": 0, "stop": 1, "times": 3},
          "layers": [layer("parallel", pair(4, 2, 64, 64, 0.125, 20.0, (0.3, 16), 2, 64, 64, 16.0), moe(4, 1, 2, 64)),
                     layer("mamba2", mamba(4, 64, 64, 2, 4, 2), moe(4, 1, 2, 64))]},
    # head sizes of 128 and of 32 for keys and values alike (the tensor-core attention kernels, capped and not), pages of 64
    "D": {"architecture": "Darolix", "vocab": 190, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
          "layers": [layer("parallel", pair(2, 1, 128, 128, 0.09, 8.0, (0.4, 32), 1, 32, 16, 3.0), moe(3, 1, 2, 32)),
                     layer("parallel", pair(4, 4, 32, 32, 0.2, 0.0, None, 2, 16, 32, 8.0), None),
                     layer("mamba2", mamba(2, 16, 8, 1, 4, 1), moe(3, 1, 2, 32))]},
}


def tensor_shapes(cfg, decay_rank=8):
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,), "head": (cfg["vocab"], w)}
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        shapes[p + "norm1"] = (w,)
        if spec["type"] == "mamba2":
            inner, bc = m["heads"] * m["vdim"], m["groups"] * m["state"]
            shapes.update({p + "mix.in": (2 * inner + 2 * bc + m["heads"], w), p + "mix.conv": (inner + 2 * bc, m["conv"]), p + "mix.conv.b": (inner + 2 * bc,),
                           p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],), p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (w, inner)})
        else:
            lo, r = m["left"], m["right"]
            shapes.update({p + "mix.left.q": (lo["heads"] * lo["dim"], w), p + "mix.left.k": (lo["kv_heads"] * lo["dim"], w), p + "mix.left.v": (lo["kv_heads"] * lo["vdim"], w),
                           p + "mix.left.o": (w, lo["heads"] * lo["vdim"]), p + "mix.left.out": (w,), p + "mix.right.out": (w,),
                           p + "mix.right.q": (r["heads"] * r["dim"], w), p + "mix.right.k": (r["heads"] * r["dim"], w), p + "mix.right.v": (r["heads"] * r["vdim"], w),
                           p + "mix.right.g": (r["heads"] * r["vdim"], w), p + "mix.right.o": (w, r["heads"] * r["vdim"]), p + "mix.right.norm": (r["vdim"],),
                           p + "mix.right.a1": (decay_rank + i, w), p + "mix.right.a2": (r["heads"] * r["dim"], decay_rank + i), p + "mix.right.a2.b": (r["heads"] * r["dim"],)})
        f = spec["mlp"]
        if f is not None:
            routed = f["router"]["experts"] + f["router"].get("identity", 0)
            shapes.update({p + "mlp.router": (routed, w), p + "mlp.correction": (routed,)})
            for e in range(f["router"]["experts"]):
                shapes.update({p + f"mlp.e{e}.gate": (f["expert"]["ff"], w), p + f"mlp.e{e}.up": (f["expert"]["ff"], w), p + f"mlp.e{e}.down": (w, f["expert"]["ff"])})
    return shapes


def weights(cfg, seed):
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm", "norm1", "out", "D"):
            v = 1.0 + 0.1 * rng.standard_normal(shape)
        elif last == "A_log":
            v = np.log(rng.uniform(0.3, 4.0, size=shape))
        elif last == "dt_bias":
            v = rng.uniform(-3.0, 0.5, size=shape)
        elif last == "correction":
            v = 0.05 * rng.standard_normal(shape)
        elif last == "b":
            v = (2.0 if name.endswith("a2.b") else 0.0) + 0.3 * rng.standard_normal(shape)
        elif last == "conv":
            v = rng.standard_normal(shape) / np.sqrt(shape[-1])
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            gain = 2.0 if last in ("router", "a2") else 1.0
            v = gain * rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v)).to(torch.bfloat16)
    return out


def write(folder, name, seed=0):
    from alofa_b200.weights.safetensors_io import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = CONFIGS[name]
    (folder / "config.json").write_text(json.dumps(cfg, indent=1) + "\n")
    write_safetensors(folder / "model.safetensors", weights(cfg, seed), {"format": "pt"})
    return folder


def tokens(name, n, seed=0):
    rng = np.random.default_rng(9000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], size=n)]
