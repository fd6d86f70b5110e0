"""Darolix without a GPU: config.json is read into a typed configuration and back, the model description
names the parts, tensors and run list that the plain implementation's weights and layer order have, and
the plain implementation itself has the properties the engine is held to (a position depends on its
prefix alone; the recurrences can be carried from token to token)."""
import json

import numpy as np
import pytest

import plain_darolix as plain
import tiny_darolix as tiny
from alofa_b200.config.registry import get_architecture, read_model_config
from alofa_b200.errors import AlofaError
from alofa_b200.parts.base import PagedKV, SlotState
from alofa_b200.parts.model import Model, expected_tensors
from alofa_b200.parts.base import Runtime
from alofa_b200.weights.loader import shape_fits


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("darolix")
    return {name: tiny.write(base / name, name, seed=i) for i, name in enumerate(tiny.CONFIGS)}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_is_read_and_written_back(folders, name):
    arch, cfg = read_model_config(folders[name])
    assert arch.name == "Darolix"
    assert arch.to_json(cfg) == tiny.CONFIGS[name]


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_the_description_names_the_tensors_and_the_order_of_the_plain_implementation(folders, name):
    import torch

    arch, cfg = read_model_config(folders[name])
    spec = arch.build_spec(cfg)
    want = tiny.tensor_shapes(tiny.CONFIGS[name])
    got = expected_tensors(spec)
    assert set(got) == set(want)
    assert all(shape_fits(want[n], got[n].shape) for n in want)
    # the run list: the layers in plain's order, a block that adds the embedding output before every pass but the first
    blocks = [spec.layers[e.layer].block.kind for e in spec.run]
    order = plain.run_order(tiny.CONFIGS[name])
    assert [b for b in blocks if b == "parallel_residual"] == ["parallel_residual"] * len(order)
    assert blocks.count("embedding_add") == sum(1 for _, again in order if again)
    layers_run = [e.layer for e in spec.run if spec.layers[e.layer].block.kind == "parallel_residual"]
    assert layers_run == [i for i, _ in order]
    # every run owns caches of its own: pages for the attention, state slots for the recurrences
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32))
    plan = model.cache_plan()
    for idx, entry in enumerate(spec.run):
        kind = spec.layers[entry.layer].block.kind
        if kind == "embedding_add":
            assert plan[idx] is None
            continue
        layer = tiny.CONFIGS[name]["layers"][entry.layer]
        if layer["type"] == "mamba2":
            m = layer["mixer"]
            words = m["heads"] * m["vdim"] * m["state"] + (m["conv"] - 1) * (m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"])
            assert plan[idx] == SlotState((words,))
        else:
            lo, r = layer["mixer"]["left"], layer["mixer"]["right"]
            assert plan[idx] == (PagedKV(lo["kv_heads"], lo["dim"], None, lo["vdim"]), SlotState((r["heads"] * r["dim"] * r["vdim"],)))


def test_bad_configs_are_refused(tmp_path):
    arch = get_architecture("Darolix")
    good = json.loads(json.dumps(tiny.CONFIGS["A"]))
    for change in (lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][1]["mixer"].update(groups=2),
                   lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), lambda c: c["layers"][0]["mlp"]["router"].update(top=8),
                   lambda c: c["loop"].update(stop=9), lambda c: c["layers"][0]["mlp"].update(kind="dense"), lambda c: c.pop("width")):
        bad = json.loads(json.dumps(good))
        change(bad)
        with pytest.raises(AlofaError):
            arch.read_config(bad, "test")


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_positions_depend_on_their_prefix_alone(folders, name):
    w, cfg = plain.load(folders[name])
    ids = tiny.tokens(name, 40, seed=3)
    whole = plain.forward(ids, w, cfg)
    for n in (1, 2, 17, 39):
        assert np.abs(plain.forward(ids[:n], w, cfg) - whole[:n]).max() < 1e-9


def test_plain_recurrences_can_be_carried():
    """The two recurrences written as a carried state give what the whole-sequence functions give."""
    rng = np.random.default_rng(0)
    T, H, N, P = 11, 2, 5, 3
    q, k, alpha = rng.standard_normal((T, H, N)), rng.standard_normal((T, H, N)), rng.uniform(0.5, 1.0, (T, H, N))
    v = rng.standard_normal((T, H, P))
    whole = plain.channel_decay_recurrence(q, k, v, alpha)
    S = np.zeros((H, N, P))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        assert np.abs(np.einsum("hn,hnp->hp", q[t], S) - whole[t]).max() < 1e-12
    u, taps_w, bias = rng.standard_normal((T, 4)), rng.standard_normal((4, 3)), rng.standard_normal(4)
    conv = plain.short_convolution(u, taps_w, bias)
    assert np.abs(conv[0] - plain.silu(bias + taps_w[:, 2] * u[0])).max() < 1e-12
    assert np.abs(conv[5] - plain.silu(bias + taps_w[:, 2] * u[5] + taps_w[:, 1] * u[4] + taps_w[:, 0] * u[3])).max() < 1e-12


def test_plain_router_uses_the_correction_for_the_choice_only():
    h = np.eye(3)
    router = np.array([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0]])
    chosen, weight, _ = plain.route(h[:1], router, np.array([0.0, 0.0, 5.0]), 2)
    s = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    assert chosen.tolist() == [[2, 0]]
    assert np.allclose(weight[0], [s[2] / (s[2] + s[0]), s[0] / (s[2] + s[0])])
