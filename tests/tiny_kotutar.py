"""The tests' own small Kotutar configurations and weights.

Sizes differ from one configuration to the next and within one (every layer
has a mixer of its own): heads above and below one kernel block's eight, value
size unlike key size, one and several experts per token, with and without a
shared expert, layers without a feed-forward, loops from the first layer, one
pass and several, and no loop at all.  The weights are drawn here, not by the
package: matrices N(0, gain / sqrt(inputs)) so that scores, router logits and
gates are of order one (N(0, 0.02) would make every softmax flat and hide a
wrong key or position), norm weights 1 + N(0, 0.1), sinks N(0, 1)."""
import json
from pathlib import Path

import numpy as np
import torch


def mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim},
            "scale": scale if scale is not None else 1.0 / np.sqrt(dim + rot_dim)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mix, mlp):
    return {"type": "latent_attention", "mixer": mix, "mlp": mlp}


CONFIGS = {
    # loop over layers 0..1 twice; 3 heads; value size above key size; two experts per token
    "A": {"architecture": "Kotutar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [layer(mixer(3, 24, 8, 40, 48, 40, 1e4), dense(136)), layer(mixer(3, 24, 8, 40, 48, 40, 1e4), moe(5, 2, 56, 72)),
                     layer(mixer(2, 16, 16, 8, 24, 56, 300.0, 0.31), None)]},
    # no loop; 10 heads (two blocks of heads per token); an odd width; experts without a shared one; top 3
    "B": {"architecture": "Kotutar", "vocab": 157, "width": 100, "norm": {"eps": 3e-6},
          "layers": [layer(mixer(10, 8, 4, 12, 20, 28, 5e5), moe(7, 3, 24)), layer(mixer(10, 8, 4, 12, 20, 28, 5e5), dense(64))]},
    # one pass of a loop over the last layer (mixed in once); sizes the tensor-core products take (multiples of 64)
    "C": {"architecture": "Kotutar", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 2, "times": 1},
          "layers": [layer(mixer(4, 32, 32, 32, 64, 64, 1e4), moe(4, 1, 64, 64)), layer(mixer(4, 32, 32, 32, 64, 64, 1e4), dense(256))]},
}


def tensor_shapes(cfg):
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,), "head": (cfg["vocab"], w)}
    if cfg.get("loop"):
        shapes["loop.in"] = (w, 2 * w)
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        shapes.update({p + "norm1": (w,), p + "norm1b": (w,), p + "mix.dq": (m["q_rank"], w), p + "mix.dq.norm": (m["q_rank"],),
                       p + "mix.uq": (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"]), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], w),
                       p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (m["heads"] * m["dim"], m["kv_rank"]), p + "mix.uv": (m["heads"] * m["vdim"], m["kv_rank"]),
                       p + "mix.sink": (m["heads"],), p + "mix.o": (w, m["heads"] * m["vdim"])})
        f = spec["mlp"]
        if f is None:
            continue
        shapes.update({p + "norm2": (w,), p + "norm2b": (w,)})
        if f["kind"] == "dense":
            shapes.update({p + "mlp.up": (f["ff"], w), p + "mlp.up.b": (f["ff"],), p + "mlp.down": (w, f["ff"]), p + "mlp.down.b": (w,)})
        else:
            shapes[p + "mlp.router"] = (f["router"]["experts"], w)
            for e in range(f["router"]["experts"]):
                shapes.update({p + f"mlp.e{e}.up": (f["expert"]["ff"], w), p + f"mlp.e{e}.down": (w, f["expert"]["ff"])})
            if f.get("shared"):
                shapes.update({p + "mlp.shared.up": (f["shared"]["ff"], w), p + "mlp.shared.down": (w, f["shared"]["ff"]), p + "mlp.shared.sg": (1, w)})
    return shapes


def weights(cfg, seed):
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm") or ".norm" in name.split(".")[-1] or name.split(".")[-1].startswith("norm"):
            v = 1.0 + 0.1 * rng.standard_normal(shape)
        elif name.endswith("sink"):
            v = rng.standard_normal(shape)
        elif name.endswith(".b"):
            v = 0.1 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            gain = 2.0 if name.endswith(("router", "sg", "uq", "uk")) else 1.0
            v = gain * rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(v).to(torch.bfloat16)
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
    rng = np.random.default_rng(7000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], size=n)]
