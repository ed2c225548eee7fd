"""Host-side tests of the Pozirax architecture: its configuration, its layout of parts and its order of runs, and the
plain implementation's own consistency (a sequence cut anywhere gives what the whole gives)."""

from __future__ import annotations

import copy

import numpy as np
import pytest

import plain_pozirax as pp


def test_the_architecture_is_registered_and_declares_the_tensors_of_the_format():
    from borrowed_compute_b200.architectures import architecture_names
    from borrowed_compute_b200.engine.model import model_for_config

    assert "Pozirax" in architecture_names()
    for name in ("A", "B"):
        cfg = pp.SMALL[name]
        typed, model = model_for_config(cfg)
        declared = model.expected_tensors()
        shapes = pp.tensor_shapes(cfg)
        assert set(declared) == set(shapes)
        assert all(tuple(declared[n].shape) == tuple(shapes[n]) for n in shapes)
        runs = [(r.layer, None if r.enter is None else r.enter[1]) for r in model.spec.schedule]
        assert runs == pp.layer_runs(cfg)


def test_every_run_of_a_looped_layer_has_memory_of_its_own():
    from borrowed_compute_b200.engine.model import model_for_config

    _, model = model_for_config(pp.SMALL["A"])
    needs, states, memory_of = model.memory_needs()
    assert len(needs) == 8 and all(m is None for m in memory_of)
    more = model.more_state_needs()
    assert sorted(more[0]) == ["mixer.right", "mixer.right.conv"] and more[1] == {}
    assert needs[0] is not None and needs[0].window == 9 and needs[1] is None and states[1] is not None


def test_the_rank_comes_from_the_tensors_when_the_file_leaves_it_out():
    from borrowed_compute_b200.config import ConfigError
    from borrowed_compute_b200.engine.model import model_for_config

    cfg = copy.deepcopy(pp.SMALL["B"])
    cfg["layers"][0]["mixer"].pop("rank")
    with pytest.raises(ConfigError, match="rank"):
        model_for_config(cfg)
    typed, _ = model_for_config(cfg, {"l0.mix.a1": (4, 80)})
    assert typed.layers[0].mixer.rank == 4


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=66), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=2), "groups"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=7), "norm_groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=10), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c.update(loop={"start": 1, "stop": 5, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c.update(width=0), "width"),
])
def test_configuration_errors_name_the_key(change, match):
    from borrowed_compute_b200.config import ConfigError
    from borrowed_compute_b200.config.pozirax import PoziraxConfig

    cfg = copy.deepcopy(pp.SMALL["B"])
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        PoziraxConfig.from_dict(cfg)


def test_defaults_of_keys_that_a_file_may_leave_out():
    from borrowed_compute_b200.config.pozirax import PoziraxConfig

    cfg = copy.deepcopy(pp.SMALL["B"])
    cfg.pop("logit_softcap")
    cfg.pop("embedding")
    left = cfg["layers"][1]["mixer"]["left"]
    for key in ("kv_heads", "vdim", "mask", "rot"):
        left.pop(key)
    typed = PoziraxConfig.from_dict(cfg)
    a = typed.layers[1].mixer.left
    assert typed.logit_softcap == 0.0 and typed.embedding_scale == 1.0 and typed.loop is None
    assert (a.kv_heads, a.vdim, a.window, a.rot_dims) == (a.heads, a.dim, 0, 0)


def test_the_plain_mixers_carry_their_state_across_a_cut():
    cfg = pp.SMALL["A"]
    w = {n: pp.f64(a) for n, a in pp.make_weights(cfg, 3).items()}
    h = np.random.default_rng(0).standard_normal((23, cfg["width"]))
    eps = cfg["norm"]["eps"]
    whole, _ = pp.gla_mixer(h, w, "l1.mix.", cfg["layers"][1]["mixer"], eps)
    first, state = pp.gla_mixer(h[:9], w, "l1.mix.", cfg["layers"][1]["mixer"], eps)
    second, _ = pp.gla_mixer(h[9:], w, "l1.mix.", cfg["layers"][1]["mixer"], eps, state)
    assert np.abs(np.concatenate([first, second]) - whole).max() < 1e-12
    m = cfg["layers"][0]["mixer"]["right"]
    whole, _ = pp.state_space_mixer(h, w, "l0.mix.right.", m, eps)
    first, state = pp.state_space_mixer(h[:1], w, "l0.mix.right.", m, eps)
    second, _ = pp.state_space_mixer(h[1:], w, "l0.mix.right.", m, eps, state)
    assert np.abs(np.concatenate([first, second]) - whole).max() < 1e-12


def test_the_plain_router_breaks_ties_by_index_and_keeps_the_scores_as_weights():
    router = np.array([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0], [2.0, 0.0]])
    chosen, weight = pp.route(np.array([[1.0, 0.5]]), router, 3)
    assert chosen.tolist() == [[3, 0, 1]]
    assert np.allclose(weight, pp.sigmoid(np.array([[2.0, 1.0, 1.0]])))
