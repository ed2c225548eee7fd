"""The Fegidra decoder on the engine against the plain implementation (plain_fegidra.py):
each new mechanism alone through its kernels, then whole models through the engine's step
function, cache, scheduler and entry points: whole prompts, token-by-token decoding,
portions down to two tokens, unequal batches, slots and pages used again, the edges of
chunks and pages, the first tokens, long decoding, and greedy generation.

float32 engines are held to the float64 oracle tightly (1e-4 (1 + max|score|)); bfloat16 engines to the
same oracle on the same (bfloat16-valued) weights within 6e-2 (1 + max|score|): these models put cubes
under a norm and sharp gates after every product, and three or four such layers showed single scores
up to 2.8e-2 (1 + max) off by rounding alone, evenly over rows.  What the bfloat16 runs are for, a
wrong key, edge or state in the bfloat16 kernels, moves scores by ten times the allowance in the
tests whose weights are made for it."""

from __future__ import annotations

import copy
import json
import math
import os

import numpy as np
import pytest

import plain_fegidra as pf
from conftest import BF16_TOL, F32_TOL

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def tol(dtype, ref):
    return (F32_TOL if dtype == "float32" else 2 * BF16_TOL) * (1.0 + float(np.abs(ref).max()))


def close(got, ref, dtype, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} against {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    worst = np.abs(got - ref).max(axis=-1)
    assert worst.max() <= tol(dtype, ref), f"{what}: row {int(worst.argmax())} differs by {worst.max():.4g} (allowed {tol(dtype, ref):.4g})"


def tokens_for(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def engine_for(cfg, weights, dtype, **kw):
    from borrowed_compute_b200.engine import Engine

    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_slots", 6)
    kw.setdefault("max_seq", 512)
    return Engine.from_tensors(cfg, {n: torch.from_numpy(np.ascontiguousarray(a)) for n, a in weights.items()}, dtype=dtype, **kw)


_made = {}


def small(name, dtype, sharp=False):
    """(engine, config, weights) of one of the two small models; ``sharp`` makes single keys matter:
    attention four times as pointed, delta-rule decays close to one (a long memory)."""
    key = (name, dtype, sharp)
    if key not in _made:
        cfg = pf.SMALL[name]
        w = pf.make_weights(cfg, seed=11 if name == "P" else 12)
        if sharp:
            for n in w:
                if n.endswith(("q.norm", "k.norm")):
                    w[n] = pf.bf16_round(w[n] * 2.0)
                if n.endswith("mix.w0"):
                    w[n] = pf.bf16_round(w[n] - 4.0)
        _made[key] = (engine_for(cfg, w, dtype), cfg, w)
    return _made[key]


def run_whole(eng, toks):
    from borrowed_compute_b200.engine import StepEntry

    s = eng.acquire()
    out = eng.step([StepEntry(s, toks, tuple(range(len(toks))))]).cpu().numpy()
    eng.release(s)
    return out


def run_cut(eng, toks, cuts):
    """The same tokens in portions of the given sizes (the rest one token at a time)."""
    from borrowed_compute_b200.engine import StepEntry

    s, at, rows = eng.acquire(), 0, []
    for n in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        part = toks[at:at + n]
        rows.append(eng.step([StepEntry(s, part, tuple(range(len(part))))]).cpu().numpy())
        at += len(part)
    eng.release(s)
    return np.concatenate(rows)


# ------------------------------------------------------------------ each mechanism alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_short_convolution_whole_and_in_portions(dtype, taps):
    from borrowed_compute_b200 import ops

    rng, E, dev = np.random.default_rng(taps), 72, "cuda:0"
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    kernel = rng.standard_normal((E, taps)).astype(np.float32)
    lens = [9, 1, 14]                                               # three sequences in slots 2, 0, 3
    slots = [2, 0, 3]
    hs = [pf.bf16_round(rng.standard_normal((n, E))) for n in lens]
    ref = [pf.short_conv_residual(pf.f64(h), pf.f64(kernel)) for h in hs]
    tail = torch.zeros((4, max(taps - 1, 1), E), dtype=td, device=dev)
    tail[1] = 7.0                                                   # a slot nobody uses keeps what it holds
    got = [[] for _ in lens]
    for portion in ([4, 1, 2], [1, 0, 1], [2, 0, 9], [2, 0, 2]):    # rows each sequence brings, step by step
        live = [i for i, n in enumerate(portion) if n > 0]
        done = [sum(len(g) for g in got[i]) for i in range(3)]
        h = torch.from_numpy(np.concatenate([hs[i][done[i]:done[i] + portion[i]] for i in live])).to(dev, td)
        seq_rows = torch.tensor(np.concatenate([[0], np.cumsum([portion[i] for i in live])]), dtype=torch.int32, device=dev)
        seq_slot = torch.tensor([slots[i] for i in live] + [-1], dtype=torch.int32, device=dev)[:len(live)]
        out = torch.zeros_like(h)
        t = tail if taps > 1 else tail[:, :0]
        ops.short_conv(h, torch.from_numpy(np.ascontiguousarray(kernel.T)).to(dev), t, seq_rows, seq_slot, out, len(live), max(portion[i] for i in live))
        o = out.float().cpu().numpy()
        at = 0
        for i in live:
            got[i].append(o[at:at + portion[i]])
            at += portion[i]
    for i in range(3):
        close(np.concatenate(got[i]), ref[i], dtype, f"sequence {i}")
    assert float(tail[1].float().min()) == 7.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [0, 1, 3, 4])
def test_two_norms_with_one_statistic_and_the_convolution_riding_along(dtype, taps):
    """out1 = conv(norm(x) w1), out2 = norm(x) w2 for single rows of three sequences, six steps in a row,
    against the plain norm and the plain convolution over each sequence's rows."""
    from borrowed_compute_b200 import ops

    rng, E, dev, eps = np.random.default_rng(taps + 20), 200, "cuda:0", 1e-5
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    w1, w2 = (rng.uniform(0.5, 1.5, E).astype(np.float32) for _ in range(2))
    kernel = rng.standard_normal((E, max(taps, 1))).astype(np.float32)
    xs = rng.standard_normal((6, 3, E)).astype(np.float32) * np.array([0.1, 1.0, 30.0], dtype=np.float32)[None, :, None]
    slots = [3, 0, 1]
    tail = torch.zeros((4, max(taps - 1, 1), E), dtype=td, device=dev)
    got1, got2 = [], []
    for step in range(6):
        x = torch.from_numpy(xs[step]).to(dev)
        out1, out2 = torch.empty((4, E), dtype=td, device=dev), torch.empty((4, E), dtype=td, device=dev)
        xx = torch.cat([x, torch.ones((1, E), device=dev)])          # a padding row (slot -1) after the three
        row_slot = torch.tensor(slots + [-1], dtype=torch.int32, device=dev)
        if taps:
            ops.norm_pair(xx, torch.from_numpy(w1).to(dev), torch.from_numpy(w2).to(dev), out1, out2, eps, torch.from_numpy(np.ascontiguousarray(kernel.T)).to(dev),
                          tail if taps > 1 else tail[:, :0], row_slot)
        else:
            ops.norm_pair(xx, torch.from_numpy(w1).to(dev), torch.from_numpy(w2).to(dev), out1, out2, eps)
        got1.append(out1[:3].float().cpu().numpy())
        got2.append(out2[:3].float().cpu().numpy())
    got1, got2 = np.stack(got1), np.stack(got2)
    for i in range(3):
        h = pf.rms_norm(pf.f64(xs[:, i]), w1, eps)
        if dtype == "bfloat16":
            h = pf.f64(pf.bf16_round(h))                            # the convolution reads the rounded norm
        close(got1[:, i], pf.short_conv_residual(h, pf.f64(kernel)) if taps else h, dtype, f"sequence {i}, first output")
        close(got2[:, i], pf.rms_norm(pf.f64(xs[:, i]), w2, eps), dtype, f"sequence {i}, second output")
    assert float(tail[2].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [4, 6, 200, 201, 8192, 8196, 14336, 16388, 32768, 32772, 40001])
def test_polynorm(dtype, width):
    """Rows of every kind of width: no multiple of four (one value at a time), rows a block of 256, of 512 or of
    1,024 threads keeps in registers, and rows too wide for that (two passes over memory)."""
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(3)
    z = (rng.standard_normal((5, width)) * np.array([[0.1], [1.0], [3.0], [10.0], [1.0]])).astype(np.float32)
    coef = np.array([0.7, -0.4, 0.2, 0.05], dtype=np.float32)
    out = torch.full((5, width), 9.0, dtype=torch.float32 if dtype == "float32" else torch.bfloat16, device="cuda:0")
    ops.polynorm(torch.from_numpy(z).cuda(), torch.from_numpy(coef).cuda(), out, 1e-5)
    close(out.float().cpu().numpy(), pf.polynorm(pf.f64(z), coef, 1e-5), dtype)


def test_polynorm_behind_a_product_that_is_still_writing():
    """The activation right behind the product that makes its input, linked by programmatic dependent launch, many
    times over: no load of the input may run ahead of the wait for the product."""
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts import products

    rng = np.random.default_rng(4)
    x = torch.from_numpy(rng.standard_normal((64, 256)).astype(np.float32)).cuda().bfloat16()
    w = torch.from_numpy((rng.standard_normal((320, 256)) / 16).astype(np.float32)).cuda().bfloat16()
    coef = torch.tensor([0.7, -0.4, 0.2, 0.05], device="cuda:0")
    ref = pf.polynorm(pf.f64(x.float().cpu().numpy()) @ pf.f64(w.float().cpu().numpy()).T, coef.cpu().numpy(), 1e-5)
    z = torch.empty((64, 320), dtype=torch.float32, device="cuda:0")
    out = torch.empty((64, 320), dtype=torch.float32, device="cuda:0")
    for _ in range(50):
        z.fill_(1e4)                        # what an early load would see
        products.linear(x, w, z, products.EPI_STORE_F32)
        ops.polynorm(z, coef, out, 1e-5)
        close(out.cpu().numpy(), ref, "float32", "behind the product")


@pytest.mark.parametrize("heads,dim,rank", [(2, 8, 3), (3, 24, 5), (1, 32, 16), (2, 64, 7), (1, 128, 4)])
def test_delta_rule_kernels(heads, dim, rank):
    """prepare + scan + finish against the recurrence written out, for head sizes on both sides of every
    register tiling, in one piece and continued from the state in pieces of 1, 2 and 17 rows, with a
    sequence beside it and a padding sequence in the batch."""
    from borrowed_compute_b200 import ops

    rng, dev, f32 = np.random.default_rng(dim), "cuda:0", torch.float32
    HD, T, eps = heads * dim, 45, 1e-5
    lens, slots = [T, 6], [1, 3]
    proj = [rng.standard_normal((n, 5 * HD + rank)).astype(np.float32) * 1.5 for n in lens]
    w2 = rng.standard_normal((HD, rank)).astype(np.float32)
    w0 = rng.uniform(-5, 1, HD).astype(np.float32)          # some decays near one, some well below
    a_b = rng.uniform(-1, 1, HD).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, HD).astype(np.float32)

    def plain(p):
        p = pf.f64(p)
        r, k, v, g, a = (p[:, i * HD:(i + 1) * HD] for i in range(5))
        decay = np.exp(-pf.DECAY_SCALE * pf.sigmoid(np.tanh(p[:, 5 * HD:]) @ pf.f64(w2).T + w0))
        rate = pf.sigmoid(a + a_b)
        o = np.zeros_like(r)
        for h in range(heads):
            s = slice(h * dim, (h + 1) * dim)
            o[:, s] = pf.over_rms(pf.delta_rule_states(r[:, s], k[:, s], v[:, s], decay[:, s], rate[:, s])[0], eps)
        return o * nw * pf.sigmoid(g)

    ref = [plain(p) for p in proj]
    for cuts in ([T], [1, 2, 17, 25]):
        state = torch.zeros((4, heads, dim, dim), dtype=f32, device=dev)
        state[0] = 3.0
        got, at = [[], []], [0, 0]
        for step, n0 in enumerate(cuts):
            portion = [n0, lens[1] if step == 0 else 0]
            live = [i for i in range(2) if portion[i] > 0]
            p = torch.from_numpy(np.concatenate([proj[i][at[i]:at[i] + portion[i]] for i in live])).to(dev)
            rows = p.shape[0]
            seq_rows = torch.tensor(list(np.concatenate([[0], np.cumsum([portion[i] for i in live])])) + [rows], dtype=torch.int32, device=dev)
            seq_slot = torch.tensor([slots[i] for i in live] + [-1], dtype=torch.int32, device=dev)       # the last one is padding
            decay, unit, removal, o = (torch.empty((rows, HD), dtype=f32, device=dev) for _ in range(4))
            dots = torch.empty((rows, heads, 2), dtype=f32, device=dev)
            ops.delta_prepare(p, torch.from_numpy(np.ascontiguousarray(w2.T)).to(dev), torch.from_numpy(w0).to(dev), torch.from_numpy(a_b).to(dev), decay, unit,
                              removal, dots, heads, dim, pf.DECAY_SCALE, pf.KEY_EPS)
            ops.delta_scan(p, decay, unit, removal, dots, state, seq_rows, seq_slot, o, len(live) + 1, heads, dim)
            y = torch.empty((rows, HD), dtype=f32, device=dev)
            ops.delta_finish(o, p, 3 * HD, torch.from_numpy(nw).to(dev), y, heads, dim, eps)
            y, r0 = y.cpu().numpy(), 0
            for i in live:
                got[i].append(y[r0:r0 + portion[i]])
                r0 += portion[i]
                at[i] += portion[i]
        for i in range(2):
            close(np.concatenate(got[i]), ref[i], "float32", f"cuts {cuts}, sequence {i}")
        assert float(state[0].min()) == 3.0 and float(state[2].abs().max()) == 0.0, "slots of no sequence keep what they hold"


# --------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole_prompt(name, dtype):
    eng, cfg, w = small(name, dtype)
    for n in (1, 2, 3, 7, 150):                 # shorter than the convolution, and across chunks and pages
        toks = tokens_for(n, n, cfg["vocab"])
        close(run_whole(eng, toks), pf.logits(cfg, w, toks), dtype, f"{n} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_decoding_token_by_token_after_a_prompt(name, dtype):
    """A prompt, then 140 single tokens through the captured decode step: over two chunk edges, two page
    edges, with keys that matter far back (sharp weights).  And from the very first token on."""
    eng, cfg, w = small(name, dtype, sharp=True)
    toks = tokens_for(5, 190, cfg["vocab"])
    ref = pf.logits(cfg, w, toks)
    close(run_cut(eng, toks, [50]), ref, dtype, "prompt of 50")
    close(run_cut(eng, toks[:70], []), ref[:70], dtype, "from the first token")


@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_of_a_prompt(name):
    eng, cfg, w = small(name, "float32", sharp=True)
    toks = tokens_for(6, 200, cfg["vocab"])
    ref = pf.logits(cfg, w, toks)
    whole = run_whole(eng, toks)
    close(whole, ref, "float32")
    for cuts in ([2, 2, 3, 33, 24, 64, 2, 70], [39, 1, 1, 23, 64, 72], [64, 64, 64, 8], [199, 1]):
        got = run_cut(eng, toks, cuts)
        close(got, ref, "float32", f"portions {cuts}")
        assert np.abs(got - whole).max() <= 2e-5 * (1 + np.abs(ref).max()), f"portions {cuts} differ from the whole prompt beyond rounding"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    """Four prompts of 1, 2, 70 and 131 tokens start together, decode together, and end at different steps."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small("P", dtype, sharp=True)
    lens, more = [1, 2, 70, 131], [30, 3, 12, 20]
    seqs = [tokens_for(40 + i, n + m, cfg["vocab"]) for i, (n, m) in enumerate(zip(lens, more))]
    refs = [pf.logits(cfg, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([StepEntry(s, q[:n], tuple(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy()
    got, at = [], 0
    for n in lens:
        got.append([out[at:at + n]])
        at += n
    for step in range(max(more)):
        live = [i for i in range(4) if step < more[i]]
        out = eng.step([StepEntry(slots[i], [seqs[i][lens[i] + step]], (0,)) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
        for i in range(4):
            if step + 1 == more[i]:
                eng.release(slots[i])
    for i in range(4):
        close(np.concatenate(got[i]), refs[i], dtype, f"sequence {i}")
    assert eng.cache.slots.live() == []


def test_single_rows_in_one_launch_or_three_give_the_same_bits():
    """Steps of single rows run the delta rule as one launch; the three kernels of a prompt step must give the
    same bits, and so must a prompt cut anywhere (float32: every sum's order depends on the row alone)."""
    from borrowed_compute_b200.parts import delta_rule

    eng, cfg, w = small("Q", "float32")
    toks = tokens_for(77, 90, cfg["vocab"])
    one = run_cut(eng, toks, [40])
    graphs, eng.use_graphs, delta_rule.split_steps = eng.use_graphs, False, True
    try:
        three = run_cut(eng, toks, [40])
    finally:
        eng.use_graphs, delta_rule.split_steps = graphs, False
    assert np.array_equal(one, three)
    assert np.array_equal(one, run_cut(eng, toks, [7, 2, 60, 1, 1, 19]))


def test_slots_and_pages_used_again():
    """A cache of four pages and two slots: every request takes the slot and pages the last one gave back;
    state, convolution tails and pages must start clean."""
    cfg = pf.SMALL["Q"]
    w = pf.make_weights(cfg, 12)
    eng = engine_for(cfg, w, "float32", max_tokens=256, max_slots=2, max_seq=256)
    for i, n in enumerate([130, 3, 200, 64, 65]):
        toks = tokens_for(70 + i, n, cfg["vocab"])
        cut = max(1, n - 5)
        close(run_cut(eng, toks, [cut]), pf.logits(cfg, w, toks), "float32", f"request {i}")
        eng.cache.slots.check()
    # Attention that only sees its chunk lets whole chunks go: after a prompt of 200 positions in chunks of 64,
    # the next single token (in the chunk from 192) leaves one page held a group.
    from borrowed_compute_b200.engine import StepEntry
    s = eng.acquire()
    eng.step([StepEntry(s, tokens_for(1, 200, cfg["vocab"]), (199,))])
    eng.step([StepEntry(s, [5], (0,))])
    held = [sum(1 for p in eng.cache.slots.tables[g][s] if p >= 0) for g in range(len(eng.cache.groups))]
    assert held and max(held) == 1, held
    eng.release(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim", [(16, 8), (32, 16), (64, 64)])
def test_one_key_that_matters_at_every_edge(dtype, dim, vdim):
    """One attention layer whose scores are made so that a single key stands out: the marked token's key is
    large and every query looks for it.  Queries just inside its chunk must find it, queries just outside
    must not, in a prompt and when decoded; the positions lie at a page's edge (64) and off it.  The sizes
    take the one-warp-a-row kernel and the tensor-core tiles."""
    chunk = 48
    cfg = {"architecture": "Fegidra", "vocab": 32, "width": 32, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
           "layers": [pf.attention_layer(2, 1, dim, vdim, chunk, 4, 10000.0, 1.0, None)]}
    w = pf.make_weights(cfg, 5)
    w["l0.canon1"][:] = 0.0                                      # the mixer reads the norm's output as it is
    w["l0.mix.q.b"][:] = 0.0
    w["l0.mix.k.b"][:] = 0.0
    w["l0.mix.q.b"][8:12] = 6.0                                  # both heads ask for dimensions 8..11 (not rotated)
    w["l0.mix.q.b"][dim + 8:dim + 12] = 6.0
    marked = 7
    w["embed"][marked] = pf.bf16_round(w["embed"][marked] * 0 + np.sign(w["l0.mix.k"][8:12].sum(0)) * 3)
    eng = engine_for(cfg, w, dtype, max_tokens=512, max_slots=2, max_seq=256)
    for at in (0, 47, 48, 63, 64, 95, 100):                      # where the marked token stands
        toks = [t if t != marked else 8 for t in tokens_for(at, 150, 32)]
        toks[at] = marked
        ref = pf.logits(cfg, w, toks)
        inside, outside = min(149, (at // chunk + 1) * chunk - 1), min(149, (at // chunk + 1) * chunk)
        assert np.abs(ref[inside] - ref[outside]).max() > 5 * tol(dtype, ref), "the marked key does not stand out in the plain model"
        close(run_whole(eng, toks), ref, dtype, f"marked at {at}, prompt")
        close(run_cut(eng, toks, [max(1, at)]), ref, dtype, f"marked at {at}, decoded")


def test_tiles_against_rows_in_bfloat16():
    """The tensor-core tiles and the one-warp-a-row kernel on the same bfloat16 cache: prompts, portions and
    single rows agree within the rounding of the weights P to bfloat16."""
    from borrowed_compute_b200.parts import attention_kv

    eng, cfg, w = small("P", "bfloat16", sharp=True)
    toks = tokens_for(33, 170, cfg["vocab"])
    tiles = run_cut(eng, toks, [100, 30])
    attention_kv.force_rows = True
    try:
        rows = run_cut(eng, toks, [100, 30])
    finally:
        attention_kv.force_rows = False
    assert np.abs(tiles - rows).max() <= 0.5 * tol("bfloat16", rows)


def test_prompts_on_tcgen05_tiles():
    """Heads of 64 with values of 64, and of 128 with values of 64: prompts and portions take the tcgen05 kernel
    under the chunk mask (chunks of 100 cut pages and query tiles), single rows the mma.sync tiles; against the
    oracle, and against the same steps with every prompt kept on the mma.sync tiles."""
    from borrowed_compute_b200.parts import attention_kv

    cfg = {"architecture": "Fegidra", "vocab": 80, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 2}, "layers": [
        pf.attention_layer(6, 2, 64, 64, 100, 16, 10000.0, 0.125, 96), pf.delta_layer(2, 16, 4, None),
        pf.attention_layer(4, 4, 128, 64, 100, 64, 10000.0, 0.09, 96)]}
    w = pf.make_weights(cfg, 21)
    for n in w:
        if n.endswith(("q.norm", "k.norm")):
            w[n] = pf.bf16_round(w[n] * 2.0)
    eng = engine_for(cfg, w, "bfloat16")
    toks = tokens_for(34, 330, cfg["vocab"])
    ref = pf.logits(cfg, w, toks)
    tc = run_cut(eng, toks, [150, 99, 2, 60])
    close(tc, ref, "bfloat16", "tcgen05 prompts")
    attention_kv.force_tiles = True
    try:
        tiles = run_cut(eng, toks, [150, 99, 2, 60])
    finally:
        attention_kv.force_tiles = False
    assert np.abs(tc - tiles).max() <= 0.5 * tol("bfloat16", ref)


def test_a_far_key_in_the_delta_state():
    """One delta-rule layer with decays close to one: a token 300 positions back still shapes the output;
    decoding from the carried state must agree with the whole prompt."""
    cfg = {"architecture": "Fegidra", "vocab": 32, "width": 32, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
           "layers": [pf.delta_layer(2, 16, 4, 40)]}
    w = pf.make_weights(cfg, 9)
    w["l0.mix.w0"] = pf.bf16_round(w["l0.mix.w0"] - 12.0)       # decays within 1e-5 of one
    w["l0.mix.a.b"] = pf.bf16_round(w["l0.mix.a.b"] - 5.0)      # and little is removed
    toks = tokens_for(2, 330, 32)
    other = list(toks)
    other[3] = (toks[3] + 1) % 32
    ref = pf.logits(cfg, w, toks)
    assert np.abs(ref[-1] - pf.logits(cfg, w, other)[-1]).max() > 1e-2, "the early token is forgotten in the plain model"
    eng = engine_for(cfg, w, "float32", max_tokens=512, max_slots=2, max_seq=384)
    close(run_cut(eng, toks, [300]), ref, "float32")
    close(run_cut(eng, toks, [64, 2, 200]), ref, "float32")


def drawn_config(seed):
    """A configuration drawn from sizes that no other test uses: widths and vocabularies that are no multiple of 8,
    heads of 4 to 128 channels, values wider and narrower than keys, chunks from 1 to beyond the sequence, 1 to 9
    taps, layers without feed-forward, attention without rotation or without chunks, any order of layers."""
    rng = np.random.default_rng(seed)
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        ff = None if rng.random() < 0.2 else int(rng.choice([16, 40, 52, 96, 130, 256]))
        if rng.random() < 0.5:
            layers.append(pf.delta_layer(int(rng.choice([1, 2, 3, 5])), int(rng.choice([4, 8, 12, 16, 20, 32, 40, 64])), int(rng.choice([1, 3, 8, 16, 33])), ff))
            continue
        G = int(rng.choice([1, 2, 3]))
        D = int(rng.choice([8, 16, 24, 32, 40, 64, 128]))
        rot = min(int(rng.choice([0, 2, 4, 8, D])), D) // 2 * 2
        L = pf.attention_layer(G * int(rng.choice([1, 2, 3, 4])), G, D, int(rng.choice([4, 8, 16, 24, 32, 64, 128])),
                               int(rng.choice([1, 2, 7, 16, 33, 64, 65, 100, 128, 1000])), max(rot, 2), float(rng.choice([100.0, 10000.0, 1e6])),
                               float(rng.choice([0.05, 0.125, 0.3])), ff)
        if rot == 0:
            del L["mixer"]["rot"]
        if rng.random() < 0.15:
            del L["mixer"]["mask"]
        layers.append(L)
    cfg = {"architecture": "Fegidra", "vocab": int(rng.choice([17, 64, 100, 257])), "width": int(rng.choice([24, 40, 48, 64, 72, 100, 128, 136])),
           "norm": {"eps": float(rng.choice([1e-5, 1e-6, 1e-3]))}, "canon": {"taps": int(rng.choice([1, 2, 3, 4, 5, 7, 9]))}, "layers": layers}
    return cfg, rng


@pytest.mark.parametrize("seed", range(12))
def test_drawn_configurations_in_a_batch(seed):
    """Two or three unequal prompts of a drawn configuration start together and decode together, in float32."""
    from borrowed_compute_b200.engine import StepEntry

    cfg, rng = drawn_config(seed)
    w = pf.make_weights(cfg, 100 + seed)
    n = int(rng.integers(2, 4))
    lens, more = [int(rng.integers(1, 110)) for _ in range(n)], [int(rng.integers(1, 14)) for _ in range(n)]
    seqs = [tokens_for(seed * 10 + i, a + b, cfg["vocab"]) for i, (a, b) in enumerate(zip(lens, more))]
    eng = engine_for(cfg, w, "float32", max_tokens=1024, max_slots=3, max_seq=192)
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([StepEntry(s, q[:a], tuple(range(a))) for s, q, a in zip(slots, seqs, lens)]).cpu().numpy()
    got, at = [], 0
    for a in lens:
        got.append([out[at:at + a]])
        at += a
    for step in range(max(more)):
        live = [i for i in range(n) if step < more[i]]
        out = eng.step([StepEntry(slots[i], [seqs[i][lens[i] + step]], (0,)) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    for i in range(n):
        close(np.concatenate(got[i]), pf.logits(cfg, w, seqs[i]), "float32", f"{json.dumps(cfg)}: sequence {i}")


def test_greedy_generation_through_the_entry_point(tmp_path):
    """A folder whose config.json leaves the decay's inner width to the tensors' shapes, loaded by Local and by
    the command line; greedy tokens of a batch of unequal prompts against the plain loop."""
    import subprocess
    import sys

    from borrowed_compute_b200 import Local, Sampling
    from borrowed_compute_b200.weights.safetensors_io import write_safetensors
    from conftest import ROOT

    cfg = copy.deepcopy(pf.SMALL["P"])
    w = pf.make_weights(cfg, 11)
    for L in cfg["layers"]:
        L["mixer"].pop("decay_rank", None)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in w.items()})
    prompts = [tokens_for(90 + i, n, cfg["vocab"]) for i, n in enumerate([3, 45, 1])]
    want = [pf.generate(pf.SMALL["P"], w, p, 12) for p in prompts]
    model = Local.load(folder, dtype="float32", max_tokens=1024, max_slots=4, max_seq=128)
    out, stats = model.generate(prompts, 12, Sampling(), stop_ids=())
    assert out == want and stats.generated == 36
    assert model.engine.cache.slots.live() == []
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", folder, ";".join(",".join(map(str, p)) for p in prompts),
                          "--max-tokens", "12", "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in res.stdout.strip().splitlines()] == want
    model16 = Local.load(folder, dtype="bfloat16", max_tokens=1024, max_slots=4, max_seq=128)
    out16, _ = model16.generate(prompts, 12, Sampling(), stop_ids=())
    for p, o in zip(prompts, out16):
        seq = list(p) + list(o)
        ref = pf.logits(pf.SMALL["P"], w, seq[:-1])
        for i, t in enumerate(o):
            row = ref[len(p) - 1 + i]
            assert row.max() - row[t] <= 2 * tol("bfloat16", row), f"token {i} is not a greedy choice within rounding"


def test_a_cut_back_is_refused_unless_to_zero():
    from borrowed_compute_b200.config import CacheError
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small("P", "float32")
    toks = tokens_for(8, 30, cfg["vocab"])
    s = eng.acquire()
    eng.step([StepEntry(s, toks, ())])
    before = [t[s].clone() for t in eng.cache.all_state()]
    with pytest.raises(CacheError, match="per-sequence state"):
        eng.rollback(s, 20)
    assert eng.length(s) == 30 and all(torch.equal(a, t[s]) for a, t in zip(before, eng.cache.all_state()))
    eng.rollback(s, 0)
    got = eng.step([StepEntry(s, toks, tuple(range(30)))]).cpu().numpy()
    eng.release(s)
    close(got, pf.logits(cfg, w, toks), "float32")
