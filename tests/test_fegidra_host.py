"""Host-side checks of the Fegidra architecture: its config.json reader, the layout of parts and tensor
names it gives, sizes filled in from tensor shapes, the cache's bookkeeping for chunked attention, and
the plain implementation's own consistency (a recurrence continued from its state, the chunk mask)."""

from __future__ import annotations

import copy

import numpy as np
import pytest

import plain_fegidra as pf


def test_config_is_read_layer_by_layer():
    from borrowed_compute_b200.config import ConfigError, FegidraConfig
    from borrowed_compute_b200.config.fegidra import AttentionMixerConfig, DeltaMixerConfig

    c = FegidraConfig.from_dict(pf.SMALL["Q"])
    assert (c.vocab, c.width, c.taps, c.norm_eps) == (160, 48, 5, 1e-6)
    assert [type(l.mixer) for l in c.layers] == [AttentionMixerConfig, DeltaMixerConfig, AttentionMixerConfig]
    assert [l.ff for l in c.layers] == [80, 0, 40]
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.rot_dims, a.rot_base, a.scale) == (3, 1, 16, 48, 64, 16, 500.0, 0.35)
    assert c.layers[2].mixer.kv_heads == 3 and c.layers[1].mixer == DeltaMixerConfig(3, 24, 5)
    for path, value, word in ((("width",), None, "width"), (("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "decay_rank"), None, "decay_rank"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mlp", "kind"), "experts", "kind"),
                              (("norm",), None, "norm.eps"), (("layers", 0, "mixer", "heads"), 2.5, "heads")):
        bad = copy.deepcopy(pf.SMALL["Q"])
        d = bad
        for k in path[:-1]:
            d = d[k]
        if value is None:
            del d[path[-1]]
        else:
            d[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            FegidraConfig.from_dict(bad)


def test_layout_names_every_tensor_and_sizes_come_from_shapes():
    from borrowed_compute_b200.architectures import resolve
    from borrowed_compute_b200.config import ConfigError
    from borrowed_compute_b200.engine.model import model_for_config

    cfg = pf.SMALL["P"]
    assert resolve(cfg).name == "Fegidra"
    w = pf.make_weights(cfg, 1)
    typed, model = model_for_config(cfg)
    expected = model.expected_tensors()
    assert {n: tuple(s.shape) for n, s in expected.items()} == {n: a.shape for n, a in w.items()}
    assert expected["l0.mix.w2"].role == "vector" and expected["l1.mix.q.b"].role == "vector" and expected["l0.mlp.up"].role == "matrix"
    bare = copy.deepcopy(cfg)
    for L in bare["layers"]:
        L["mixer"].pop("decay_rank", None)
    with pytest.raises(ConfigError, match="decay_rank"):
        model_for_config(bare)
    typed2, _ = model_for_config(bare, {n: a.shape for n, a in w.items()})
    assert typed2 == typed
    # A layer without feed-forward has neither its tensors nor its norm.
    _, q = model_for_config(pf.SMALL["Q"])
    names = set(q.expected_tensors())
    assert "l1.norm1" in names and "l1.canon1" in names and not any(n.startswith("l1.mlp.") for n in names)
    assert q.expected_tensors()["l1.norm2"].optional, "the norm of the branch that is left out is tolerated, not asked for"
    needs, states, _ = q.memory_needs()
    assert needs[0].planes == ((1, 16), (1, 48)) and needs[0].chunk == 64 and needs[1] is None
    assert tuple(states[1].shape) == (3, 24, 24) and states[0] is None
    assert [sorted(m) for m in q.more_state_needs()] == [["conv"]] * 3 and tuple(q.more_state_needs()[0]["conv"].shape) == (4, 48)


def test_chunked_groups_let_whole_chunks_go():
    from borrowed_compute_b200.cache.slots import PAGE, GroupPlan, SlotTable

    t = SlotTable(n_slots=2, n_pages=8, max_seq=1024, groups=[GroupPlan(), GroupPlan(chunk=96), GroupPlan(chunk=64)])
    s = t.acquire()
    t.reserve(s, 200, 200)          # a prompt's first row sees from position 0: nothing can go yet
    t.commit(s, 200)
    assert [sum(p >= 0 for p in t.tables[g][s]) for g in range(3)] == [4, 4, 4]
    t.reserve(s, 201, 1)            # position 200 lies in the chunk from 192: pages before 192 // 64 = 3 go
    t.commit(s, 201)
    assert [sum(p >= 0 for p in t.tables[g][s]) for g in range(3)] == [4, 1, 1]
    for n in range(202, 290):
        t.reserve(s, n, 1)
        t.commit(s, n)
        t.check()
    # position 288 opens the chunk of 96 from 288 (page 4) and lies in the chunk of 64 from 256 (page 4)
    assert [[i for i, p in enumerate(t.tables[g][s]) if p >= 0] for g in (1, 2)] == [[4], [4]]
    assert t.pools[1].available == 7 and t.pools[0].available == 8 - 5
    t.release(s)
    t.check()
    assert all(pool.available == 8 for pool in t.pools)


def test_plain_recurrence_continues_from_its_state():
    rng = np.random.default_rng(0)
    T, D = 20, 6
    r, k, v = (rng.standard_normal((T, D)) for _ in range(3))
    decay, rate = rng.uniform(0.5, 1.0, (T, D)), rng.uniform(0, 1, (T, D))
    whole, S = pf.delta_rule_states(r, k, v, decay, rate)
    a, Sa = pf.delta_rule_states(r[:7], k[:7], v[:7], decay[:7], rate[:7])
    b, Sb = pf.delta_rule_states(r[7:], k[7:], v[7:], decay[7:], rate[7:], Sa)
    assert np.allclose(np.concatenate([a, b]), whole, atol=1e-12) and np.allclose(S, Sb, atol=1e-12)
    # One step by hand: from S = 0 the state is k v^T and the output v (k . r).
    o, S1 = pf.delta_rule_states(r[:1], k[:1], v[:1], decay[:1], rate[:1])
    assert np.allclose(S1, np.outer(k[0], v[0])) and np.allclose(o[0], v[0] * (k[0] @ r[0]))


def test_plain_masks_and_convolution():
    ok = pf.visible(7, 3)
    assert ok[2].tolist() == [True, True, True, False, False, False, False] and ok[3].tolist() == [False, False, False, True, False, False, False]
    assert pf.visible(4, 0).sum() == 10
    h = np.arange(10.0).reshape(5, 2)
    out = pf.short_conv_residual(h, np.array([[1.0, 0.0, 0.0], [0.0, 0.0, 2.0]]))     # channel 0: two back; channel 1: itself, twice
    assert out[:, 0].tolist() == [0.0, 2.0, 4.0 + 0.0, 6.0 + 2.0, 8.0 + 4.0] and out[:, 1].tolist() == [3.0, 9.0, 15.0, 21.0, 27.0]
    x = np.array([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]])
    y = pf.rotate(x, [1], 4, 100.0)
    assert np.allclose(y[0, 0, 4:], [5.0, 6.0]) and np.allclose(y[0, 0, 0], 1 * np.cos(1.0) - 3 * np.sin(1.0)) and np.allclose(y[0, 0, 3], 4 * np.cos(0.1) + 2 * np.sin(0.1))
