"""Kotutar: a decoder whose layers are listed one by one in config.json.

Every layer is a latent-attention mixer followed (optionally) by a dense or a
routed feed-forward, each sublayer with a norm before it and a norm after it;
a stretch of layers may run several times in a row with the same weights
(``loop``), every pass with caches of its own and preceded by a projection
that mixes the embedding output back into the residual stream.  This file only
reads the architecture's config keys and describes the model as a
:class:`~alofa_b200.config.spec.ModelSpec`; the parts it names live in
:mod:`alofa_b200.parts` and know nothing about Kotutar.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``layers[i].type`` / ``.mixer`` (``heads, dim, rot_dim, vdim, kv_rank, q_rank,
scale, rot.base, rot.dims``) / ``.mlp`` (null, ``{kind: dense, ff}`` or ``{kind:
moe, router: {experts, top}, expert: {ff}, shared: {ff}}``), and ``loop``
(``start, stop, times``; absent: every layer runs once, nothing is mixed in).
Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..config.json_reader import Keys
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..errors import AlofaError

NAME = "Kotutar"
# positions are counted in fp32 by the rotation kernels: exact up to 2^24
MAX_POSITION = 1 << 24


@dataclass
class LatentMixerConfig:
    heads: int
    dim: int  # unrotated query/key dimensions per head
    rot_dim: int  # rotated query/key dimensions per head (the key part is shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass
class MlpConfig:
    kind: str  # "dense" or "moe"
    ff: int = 0  # dense: the hidden size; moe: the hidden size of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0  # 0: no shared expert


@dataclass
class KotutarLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MlpConfig]


@dataclass
class KotutarConfig:
    vocab: int
    width: int
    eps: float
    layers: list = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0  # 0 with start == stop: no loop

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def validate(self, origin: str = "") -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("parse", what, f"{detail} config={origin}")

        need(self.vocab > 0, "vocab must be positive", f"vocab={self.vocab}")
        need(self.width > 0, "width must be positive", f"width={self.width}")
        need(self.eps > 0, "norm.eps must be positive", f"eps={self.eps}")
        need(len(self.layers) > 0, "layers must not be empty", "layers=[]")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            need(layer.type == "latent_attention", "unknown layer type", f"layers[{i}].type={layer.type}")
            need(min(m.heads, m.dim + m.rot_dim, m.vdim, m.kv_rank, m.q_rank) > 0, "mixer sizes must be positive", f"layers[{i}].mixer={m}")
            need(m.dim >= 0 and m.rot_dim >= 0, "mixer sizes must not be negative", f"layers[{i}].mixer={m}")
            need(0 <= m.rot_dims <= m.rot_dim and m.rot_dims % 2 == 0, "rot.dims must be even and at most rot_dim", f"layers[{i}] rot.dims={m.rot_dims} rot_dim={m.rot_dim}")
            need(m.rot_base > 0, "rot.base must be positive", f"layers[{i}] rot.base={m.rot_base}")
            if layer.mlp is not None:
                f = layer.mlp
                need(f.kind in ("dense", "moe"), "unknown mlp kind", f"layers[{i}].mlp.kind={f.kind}")
                need(f.ff > 0, "ff must be positive", f"layers[{i}].mlp ff={f.ff}")
                if f.kind == "moe":
                    need(0 < f.top <= f.experts, "router.top must lie in [1, experts]", f"layers[{i}] top={f.top} experts={f.experts}")
                    need(f.shared_ff >= 0, "shared.ff must not be negative", f"layers[{i}] shared.ff={f.shared_ff}")
        if self.has_loop or self.loop_times:
            need(0 <= self.loop_start < self.loop_stop <= len(self.layers), "loop must name a stretch of layers", f"start={self.loop_start} stop={self.loop_stop}")
            need(self.loop_times >= 1, "loop.times must be at least 1", f"times={self.loop_times}")


def _object(obj: dict, key: str, origin: str) -> dict:
    value = obj.get(key)
    if not isinstance(value, dict):
        raise AlofaError("parse", "config key must be an object", f"key={key} config={origin}")
    return value


def _read_mixer(obj: dict, origin: str) -> LatentMixerConfig:
    k = Keys(obj, origin)
    rot = Keys(_object(obj, "rot", origin), origin)
    rot_dim = k.integer("rot_dim")
    return LatentMixerConfig(
        heads=k.integer("heads"), dim=k.integer("dim"), rot_dim=rot_dim, vdim=k.integer("vdim"), kv_rank=k.integer("kv_rank"),
        q_rank=k.integer("q_rank"), scale=k.number("scale"), rot_base=rot.number("base"), rot_dims=rot.integer("dims", rot_dim),
    )


def _read_mlp(obj, origin: str) -> Optional[MlpConfig]:
    if obj is None:
        return None
    if not isinstance(obj, dict):
        raise AlofaError("parse", "mlp must be an object or null", f"config={origin}")
    kind = Keys(obj, origin).string("kind")
    if kind == "moe":
        router = Keys(_object(obj, "router", origin), origin)
        shared = obj.get("shared")
        return MlpConfig("moe", Keys(_object(obj, "expert", origin), origin).integer("ff"), router.integer("experts"), router.integer("top"),
                         Keys(shared, origin).integer("ff") if isinstance(shared, dict) else 0)
    return MlpConfig(kind, Keys(obj, origin).integer("ff"))


def read_config(obj: dict, origin: str) -> KotutarConfig:
    k = Keys(obj, origin)
    layers = obj.get("layers")
    if not isinstance(layers, list):
        raise AlofaError("parse", "config key must be a list", f"key=layers config={origin}")
    cfg = KotutarConfig(vocab=k.integer("vocab"), width=k.integer("width"), eps=Keys(_object(obj, "norm", origin), origin).number("eps"))
    for i, entry in enumerate(layers):
        if not isinstance(entry, dict):
            raise AlofaError("parse", "a layer must be an object", f"layers[{i}] config={origin}")
        cfg.layers.append(KotutarLayer(Keys(entry, origin).string("type"), _read_mixer(_object(entry, "mixer", origin), origin), _read_mlp(entry.get("mlp"), origin)))
    if isinstance(obj.get("loop"), dict):
        loop = Keys(obj["loop"], origin)
        cfg.loop_start, cfg.loop_stop, cfg.loop_times = loop.integer("start"), loop.integer("stop"), loop.integer("times")
    cfg.validate(origin)
    return cfg


def to_json(cfg: KotutarConfig) -> dict:
    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale,
                 "rot": {"base": m.rot_base, "dims": m.rot_dims}}
        mlp = None
        if layer.mlp is not None and layer.mlp.kind == "moe":
            f = layer.mlp
            mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.ff}}
            if f.shared_ff:
                mlp["shared"] = {"ff": f.shared_ff}
        elif layer.mlp is not None:
            mlp = {"kind": layer.mlp.kind, "ff": layer.mlp.ff}
        layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
    out = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "layers": layers}
    if cfg.has_loop:
        out["loop"] = {"start": cfg.loop_start, "stop": cfg.loop_stop, "times": cfg.loop_times}
    return out


def run_order(cfg: KotutarConfig) -> list:
    """(layer index, first of a pass) in the order the layers run."""
    n = len(cfg.layers)
    if not cfg.has_loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(cfg.loop_start)]
    for _ in range(cfg.loop_times):
        order += [(i, i == cfg.loop_start) for i in range(cfg.loop_start, cfg.loop_stop)]
    return order + [(i, False) for i in range(cfg.loop_stop, n)]


def build_spec(cfg: KotutarConfig) -> ModelSpec:
    width = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        rotary = PartSpec("rotary_interleaved", {"dims": m.rot_dims, "base": m.rot_base})
        mixer = PartSpec(
            "latent_attention",
            {"hidden_size": width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank,
             "scale": m.scale, "eps": cfg.eps, "sink": True, "window": None, "position": rotary},
            prefix=p + "mix.",
        )
        norm = lambda name: PartSpec("rmsnorm", {"size": width, "eps": cfg.eps, "weight_name": name}, prefix=p)
        params = {"mixer": mixer, "mixer_norm": norm("norm1"), "mixer_post_norm": norm("norm1b"), "feed_forward": None}
        f = layer.mlp
        if f is not None:
            if f.kind == "moe":
                params["feed_forward"] = PartSpec(
                    "routed_experts",
                    {"hidden_size": width, "experts": f.experts, "top": f.top, "expert_ff": f.ff, "shared_ff": f.shared_ff, "activation": "gelu_erf",
                     "score": "sigmoid", "renormalize": False, "weight_on_input": True, "shared_gate": True},
                    prefix=p + "mlp.",
                )
            else:
                params["feed_forward"] = PartSpec("mlp", {"hidden_size": width, "intermediate_size": f.ff, "activation": "gelu_erf", "bias": True}, prefix=p + "mlp.")
            params["feed_forward_norm"] = norm("norm2")
            params["feed_forward_post_norm"] = norm("norm2b")
        layers.append(LayerSpec(PartSpec("sandwich_residual", params, prefix=p)))
    order = run_order(cfg)
    run = []
    if cfg.has_loop:
        mix_in = len(layers)  # the projection that brings the embedding output back in: a block of its own, run before every pass
        layers.append(LayerSpec(PartSpec("embedding_mix_in", {"hidden_size": width, "weight_name": "loop.in"})))
    for layer, first in order:
        if first:
            run.append(RunEntry(mix_in))
        run.append(RunEntry(layer))
    spec = ModelSpec(
        architecture=NAME, hidden_size=width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": width, "weight_name": "embed"}),
        layers=layers, run=run,
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": cfg.eps, "weight_name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": width, "tied_to": None, "weight_name": "head"}),
    )
    spec.validate()
    return spec


register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)
