"""Darolix: a decoder whose layers, listed one by one in config.json, each have
ONE norm whose output a mixer and a routed feed-forward read side by side
(``h += mixer(norm(h)) + ff(norm(h))``).  The mixer is a state-space layer
(``mamba2``) or a softmax attention and a gated linear attention run side by
side (``parallel``); the feed-forward is a mixture of gated experts with a
softmax router, a stored correction of the choice and experts that are the
identity.  The embedding is scaled and gets a sinusoidal position vector; a
stretch of layers may run several times in a row with the same weights
(``loop``), every pass with caches and states of its own, the embedding output
added to the stream before every pass but the first.  This file only reads
the architecture's config keys and describes the model as a
:class:`~alofa_b200.config.spec.ModelSpec`; the parts it names live in
:mod:`alofa_b200.parts` and know nothing about Darolix.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``layers[i].type`` (``mamba2`` | ``parallel``),
``layers[i].mixer`` (mamba2: ``heads, vdim, state, groups, conv,
norm_groups``; parallel: ``left`` = ``heads, kv_heads, dim, vdim, scale,
softcap, q_temp.coef, q_temp.every`` and ``right`` = ``heads, dim, vdim,
tau``), ``layers[i].mlp`` (null or ``{kind: moe, router: {experts, top,
identity}, expert: {ff}}``) and ``loop`` (``start, stop, times``).
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..config.json_reader import Keys
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..errors import AlofaError

NAME = "Darolix"
MAX_POSITION = 1 << 24  # positions are fp32 in the embedding's angles: whole numbers are exact up to here
SINUSOID_BASE = 10000.0
RENORM_EPS = 1e-20


@dataclass
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass
class LeftConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0  # 0: scores are not capped
    q_temp_coef: float = 0.0  # 0: no query temperature
    q_temp_every: int = 1


@dataclass
class RightConfig:
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass
class MoeConfig:
    experts: int
    top: int
    ff: int
    identity: int = 0


@dataclass
class DarolixLayer:
    type: str
    mixer: object  # StateSpaceConfig, or (LeftConfig, RightConfig)
    mlp: Optional[MoeConfig]


@dataclass
class DarolixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: list = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def validate(self, origin: str = "") -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("parse", what, f"{detail} config={origin}")

        need(self.vocab > 0 and self.width > 0, "vocab and width must be positive", f"vocab={self.vocab} width={self.width}")
        need(self.eps > 0, "norm.eps must be positive", f"eps={self.eps}")
        need(len(self.layers) > 0, "layers must not be empty", "layers=[]")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "mamba2":
                need(min(m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups) > 0, "mixer sizes must be positive", f"layers[{i}].mixer={m}")
                need(m.heads % m.groups == 0, "groups must divide heads", f"layers[{i}].mixer={m}")
                need((m.heads * m.vdim) % m.norm_groups == 0, "norm_groups must divide heads * vdim", f"layers[{i}].mixer={m}")
            else:
                left, right = m
                need(min(left.heads, left.kv_heads, left.dim, left.vdim) > 0 and left.heads % left.kv_heads == 0, "left: kv_heads must divide heads",
                     f"layers[{i}].mixer.left={left}")
                need(left.softcap >= 0 and left.q_temp_every > 0, "left: softcap must not be negative, q_temp.every positive", f"layers[{i}].mixer.left={left}")
                need(min(right.heads, right.dim, right.vdim) > 0 and right.tau > 0, "right: sizes and tau must be positive", f"layers[{i}].mixer.right={right}")
            f = layer.mlp
            if f is not None:
                need(f.experts > 0 and f.ff > 0 and f.identity >= 0, "router.experts and expert.ff must be positive", f"layers[{i}].mlp={f}")
                need(0 < f.top <= f.experts + f.identity, "router.top must lie in [1, experts + identity]", f"layers[{i}].mlp={f}")
        if self.has_loop or self.loop_times:
            need(0 <= self.loop_start < self.loop_stop <= len(self.layers), "loop must name a stretch of layers", f"start={self.loop_start} stop={self.loop_stop}")
            need(self.loop_times >= 1, "loop.times must be at least 1", f"times={self.loop_times}")


def _object(obj: dict, key: str, origin: str) -> dict:
    value = obj.get(key)
    if not isinstance(value, dict):
        raise AlofaError("parse", "config key must be an object", f"key={key} config={origin}")
    return value


def _read_mixer(kind: str, obj: dict, origin: str):
    if kind == "mamba2":
        k = Keys(obj, origin)
        return StateSpaceConfig(k.integer("heads"), k.integer("vdim"), k.integer("state"), k.integer("groups"), k.integer("conv"), k.integer("norm_groups", 1))
    if kind == "parallel":
        lo = _object(obj, "left", origin)
        k = Keys(lo, origin)
        left = LeftConfig(k.integer("heads"), k.integer("kv_heads"), k.integer("dim"), k.integer("vdim"), k.number("scale"),
                          float(lo["softcap"]) if lo.get("softcap") else 0.0)
        if isinstance(lo.get("q_temp"), dict):
            qt = Keys(lo["q_temp"], origin)
            left.q_temp_coef, left.q_temp_every = qt.number("coef"), qt.integer("every")
        k = Keys(_object(obj, "right", origin), origin)
        return left, RightConfig(k.integer("heads"), k.integer("dim"), k.integer("vdim"), k.number("tau"))
    raise AlofaError("parse", "unknown layer type", f"type={kind} config={origin}")


def _read_mlp(obj, origin: str) -> Optional[MoeConfig]:
    if obj is None:
        return None
    if not isinstance(obj, dict):
        raise AlofaError("parse", "mlp must be an object or null", f"config={origin}")
    kind = Keys(obj, origin).string("kind")
    if kind != "moe":
        raise AlofaError("parse", "unknown mlp kind", f"kind={kind} config={origin}")
    router = Keys(_object(obj, "router", origin), origin)
    return MoeConfig(router.integer("experts"), router.integer("top"), Keys(_object(obj, "expert", origin), origin).integer("ff"), router.integer("identity", 0))


def read_config(obj: dict, origin: str) -> DarolixConfig:
    k = Keys(obj, origin)
    layers = obj.get("layers")
    if not isinstance(layers, list):
        raise AlofaError("parse", "config key must be a list", f"key=layers config={origin}")
    emb = obj.get("embedding")
    cfg = DarolixConfig(vocab=k.integer("vocab"), width=k.integer("width"), eps=Keys(_object(obj, "norm", origin), origin).number("eps"),
                        embedding_scale=Keys(emb, origin).number("scale") if isinstance(emb, dict) and "scale" in emb else 1.0)
    for i, entry in enumerate(layers):
        if not isinstance(entry, dict):
            raise AlofaError("parse", "a layer must be an object", f"layers[{i}] config={origin}")
        kind = Keys(entry, origin).string("type")
        cfg.layers.append(DarolixLayer(kind, _read_mixer(kind, _object(entry, "mixer", origin), origin), _read_mlp(entry.get("mlp"), origin)))
    if isinstance(obj.get("loop"), dict):
        loop = Keys(obj["loop"], origin)
        cfg.loop_start, cfg.loop_stop, cfg.loop_times = loop.integer("start"), loop.integer("stop"), loop.integer("times")
    cfg.validate(origin)
    return cfg


def to_json(cfg: DarolixConfig) -> dict:
    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        if layer.type == "mamba2":
            mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv, "norm_groups": m.norm_groups}
        else:
            left, right = m
            lo = {"heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim, "vdim": left.vdim, "scale": left.scale}
            if left.softcap:
                lo["softcap"] = left.softcap
            if left.q_temp_coef:
                lo["q_temp"] = {"coef": left.q_temp_coef, "every": left.q_temp_every}
            mixer = {"left": lo, "right": {"heads": right.heads, "dim": right.dim, "vdim": right.vdim, "tau": right.tau}}
        f = layer.mlp
        mlp = None if f is None else {"kind": "moe", "router": {"experts": f.experts, "top": f.top, "identity": f.identity}, "expert": {"ff": f.ff}}
        layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
    out = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "embedding": {"scale": cfg.embedding_scale}, "layers": layers}
    if cfg.has_loop:
        out["loop"] = {"start": cfg.loop_start, "stop": cfg.loop_stop, "times": cfg.loop_times}
    return out


def run_order(cfg: DarolixConfig) -> list:
    """(layer index, opens a pass after the first) in the order the layers run."""
    n = len(cfg.layers)
    if not cfg.has_loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(cfg.loop_start)]
    for k in range(cfg.loop_times):
        order += [(i, k > 0 and i == cfg.loop_start) for i in range(cfg.loop_start, cfg.loop_stop)]
    return order + [(i, False) for i in range(cfg.loop_stop, n)]


def build_spec(cfg: DarolixConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "mamba2":
            mixer = PartSpec("state_space", {"hidden_size": width, "heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                                             "norm_groups": m.norm_groups, "eps": eps}, prefix=p + "mix.")
        else:
            left, right = m
            attention = PartSpec("normed_attention", {"hidden_size": width, "heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim, "vdim": left.vdim,
                                                      "scale": left.scale, "softcap": left.softcap, "qk_norm": True, "eps": eps, "q_temp_coef": left.q_temp_coef,
                                                      "q_temp_every": left.q_temp_every, "window": None}, prefix=p + "mix.left.")
            linear = PartSpec("gated_linear_attention", {"hidden_size": width, "heads": right.heads, "dim": right.dim, "vdim": right.vdim, "tau": right.tau,
                                                         "eps": eps}, prefix=p + "mix.right.")
            mixer = PartSpec("side_by_side", {"hidden_size": width, "eps": eps, "names": ["left", "right"], "branches": [attention, linear]}, prefix=p + "mix.")
        ff = None
        f = layer.mlp
        if f is not None:
            ff = PartSpec("routed_experts", {"hidden_size": width, "experts": f.experts, "top": f.top, "expert_ff": f.ff, "identity": f.identity, "gated": True,
                                             "activation": "silu", "score": "softmax", "correction": True, "renormalize": True, "renorm_eps": RENORM_EPS,
                                             "weight_on_input": False}, prefix=p + "mlp.")
        norm = PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "norm1"}, prefix=p)
        layers.append(LayerSpec(PartSpec("parallel_residual", {"norm": norm, "mixer": mixer, "feed_forward": ff}, prefix=p)))
    run = []
    again = len(layers)
    if any(first for _, first in run_order(cfg)):
        layers.append(LayerSpec(PartSpec("embedding_add", {})))  # a block of its own, run before every pass but the first
    for layer, first in run_order(cfg):
        if first:
            run.append(RunEntry(again))
        run.append(RunEntry(layer))
    spec = ModelSpec(
        architecture=NAME, hidden_size=width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": width, "weight_name": "embed", "scale": cfg.embedding_scale,
                                               "sinusoid_base": SINUSOID_BASE}),
        layers=layers, run=run,
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": width, "tied_to": None, "weight_name": "head"}),
    )
    spec.validate()
    return spec


register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)
