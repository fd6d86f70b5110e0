"""Kotutar without a GPU: the configuration reader, the run list that a loop
expands to, tensor names and shapes, the seeded random model, and the plain
implementation's own algebra (the latent-space route that the kernels take
gives the scores and outputs of the per-head route)."""
import json

import numpy as np
import pytest

import plain_kotutar as plain
import tiny_kotutar as tiny
from alofa_b200.config.registry import get_architecture, read_model_config
from alofa_b200.errors import AlofaError
from alofa_b200.parts.base import PagedRows
from alofa_b200.parts.model import Model, expected_tensors


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("kotutar")
    return {name: tiny.write(base / name, name, seed=i) for i, name in enumerate(tiny.CONFIGS)}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_is_read_and_written_back(folders, name):
    arch, cfg = read_model_config(folders[name])
    assert arch.name == "Kotutar"
    assert arch.to_json(cfg) == json.loads(json.dumps(tiny.CONFIGS[name]))
    assert cfg.width == tiny.CONFIGS[name]["width"] and len(cfg.layers) == len(tiny.CONFIGS[name]["layers"])


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_tensor_names_and_shapes(folders, name):
    arch, cfg = read_model_config(folders[name])
    got = {n: tuple(s.shape) for n, s in expected_tensors(arch.build_spec(cfg)).items()}
    assert got == tiny.tensor_shapes(tiny.CONFIGS[name])


def test_run_list_of_a_loop():
    arch = get_architecture("Kotutar")
    raw = json.loads(json.dumps(tiny.CONFIGS["A"]))
    spec = arch.build_spec(arch.read_config(raw, "test"))
    mix_in = len(raw["layers"])
    assert [e.layer for e in spec.run] == [mix_in, 0, 1, mix_in, 0, 1, 2]  # a pass opens with the mix-in, also the first
    assert plain.run_order(raw) == [(0, True), (1, False), (0, True), (1, False), (2, False)]
    raw["loop"] = {"start": 1, "stop": 3, "times": 3}
    spec = arch.build_spec(arch.read_config(raw, "test"))
    assert [e.layer for e in spec.run] == [0, mix_in, 1, 2, mix_in, 1, 2, mix_in, 1, 2]
    assert all(e.cache is None for e in spec.run)  # every run of a layer has a cache of its own
    del raw["loop"]
    spec = arch.build_spec(arch.read_config(raw, "test"))
    assert [e.layer for e in spec.run] == [0, 1, 2] and "loop.in" not in expected_tensors(spec)


def test_caches_are_rows_of_latent_width():
    import torch
    from alofa_b200.parts.base import Runtime

    arch = get_architecture("Kotutar")
    spec = arch.build_spec(arch.read_config(tiny.CONFIGS["A"], "test"))
    plan = Model(spec, Runtime(torch.device("cpu"), torch.float32)).cache_plan()
    widths = [plan[i].width if plan[i] is not None else None for i in sorted(plan)]
    assert widths == [None, 56, 56, None, 56, 56, 40] and all(isinstance(s, PagedRows) for s in plan.values() if s is not None)


@pytest.mark.parametrize("broken", [
    lambda c: c["layers"][0]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=9),
    lambda c: c.update(loop={"start": 2, "stop": 1, "times": 1}),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c.pop("norm"),
])
def test_bad_configs_are_refused(broken):
    raw = json.loads(json.dumps(tiny.CONFIGS["A"]))
    broken(raw)
    arch = get_architecture("Kotutar")
    with pytest.raises(AlofaError) as err:
        arch.read_config(raw, "test")
    assert err.value.code == "parse"


def test_random_model_folder(tmp_path):
    """The package's seeded random mode writes a folder of this architecture
    that the plain reader takes."""
    from alofa_b200.weights.random_init import write_random_model

    arch = get_architecture("Kotutar")
    folder = write_random_model(tmp_path / "m", "Kotutar", arch.read_config(tiny.CONFIGS["B"], "test"), seed=3)
    w, cfg = plain.load(folder)
    assert {n: v.shape for n, v in w.items()} == tiny.tensor_shapes(tiny.CONFIGS["B"])
    assert np.isfinite(plain.forward(tiny.tokens("B", 9), w, cfg)).all()


def test_latent_space_route_equals_per_head_route(folders):
    """(Wuk_h^T q_h) . c = q_h . (Wuk_h c), and Wuv_h (sum_j p_j c_j) = sum_j p_j (Wuv_h c_j)."""
    w, cfg = plain.load(folders["A"])
    m, eps, p = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], "l0.mix."
    rng = np.random.default_rng(0)
    x = rng.standard_normal((11, cfg["width"]))
    pos = np.arange(11)
    want = plain.latent_attention(x, pos, w, p, m, eps)
    H, d, r, vd, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = plain.latent_queries(x, w, p, m, eps)
    c, key_part = plain.latent_rows(x, w, p, m, eps)
    rows = np.concatenate([c, plain.turn_pairs(key_part, pos, m["rot"]["base"], m["rot"]["dims"])], axis=-1)
    heads = []
    for h in range(H):
        qa = np.concatenate([q[:, h, :d] @ w[p + "uk"][h * d : (h + 1) * d], plain.turn_pairs(q[:, h, d:], pos, m["rot"]["base"], m["rot"]["dims"])], axis=-1)
        s = np.where(np.tril(np.ones((11, 11), bool)), qa @ rows.T * m["scale"], -np.inf)
        heads.append((plain.softmax_with_sink(s, w[p + "sink"][h]) @ rows[:, :kr]) @ w[p + "uv"][h * vd : (h + 1) * vd].T)
    np.testing.assert_allclose(np.concatenate(heads, axis=-1) @ w[p + "o"].T, want, rtol=1e-9, atol=1e-9)


def test_the_sink_only_takes_weight_away():
    s = np.array([[0.3, -np.inf, -np.inf], [0.1, 0.9, -np.inf], [2.0, -1.0, 0.5]])
    without = plain.softmax_with_sink(s, -np.inf)
    np.testing.assert_allclose(without.sum(-1), 1.0)
    with_sink = plain.softmax_with_sink(s, 1.5)
    np.testing.assert_allclose(with_sink.sum(-1), np.exp(s).sum(-1) / (np.exp(s).sum(-1) + np.exp(1.5)))
    np.testing.assert_allclose(with_sink / with_sink.sum(-1, keepdims=True), without)
