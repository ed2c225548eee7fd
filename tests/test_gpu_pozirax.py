"""The Pozirax decoder on the engine against the plain implementation (plain_pozirax.py): each new mechanism alone
through its kernels, then whole models through the engine's step function, cache, scheduler and entry points:
whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used again,
keys at the edges of windows and pages, far keys in the recurrent states, the first tokens, long decoding, and
greedy generation.

float32 engines are held to the float64 oracle tightly (1e-4 (1 + max|score|)).  bfloat16 engines are compared with
the oracle on token sequences for which every router chooses by a margin (rounding that flips a choice gives another,
equally valid output, and a comparison would say nothing), within 6e-2 (1 + max|score|)."""

from __future__ import annotations

import copy
import json
import math
import os

import numpy as np
import pytest

import plain_pozirax as pp
from conftest import BF16_TOL, F32_TOL

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
DEV = "cuda:0"


def tol(dtype, ref):
    return (F32_TOL if dtype == "float32" else 2 * BF16_TOL) * (1.0 + float(np.abs(ref).max()))


def close(got, ref, dtype, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} against {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    worst = np.abs(got - ref).reshape(got.shape[0], -1).max(axis=-1)
    assert worst.max() <= tol(dtype, ref), f"{what}: row {int(worst.argmax())} differs by {worst.max():.4g} (allowed {tol(dtype, ref):.4g})"


def tokens_for(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def engine_for(cfg, weights, dtype, **kw):
    from borrowed_compute_b200.engine import Engine

    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_slots", 6)
    kw.setdefault("max_seq", 512)
    return Engine.from_tensors(cfg, {n: torch.from_numpy(np.ascontiguousarray(a)) for n, a in weights.items()}, dtype=dtype, **kw)


_made = {}


def small(name, dtype):
    key = (name, dtype)
    if key not in _made:
        cfg = pp.SMALL[name]
        w = pp.make_weights(cfg, seed=21 if name == "A" else 22)
        _made[key] = (engine_for(cfg, w, dtype), cfg, w)
    return _made[key]


_decisive = {}


def decisive(name, n, seed):
    """Tokens and the oracle's scores for which every router of the small model chooses by a margin."""
    key = (name, n, seed)
    if key not in _decisive:
        cfg = pp.SMALL[name]
        _decisive[key] = pp.decisive_tokens(cfg, pp.make_weights(cfg, seed=21 if name == "A" else 22), n, seed, margin=0.03)
    return _decisive[key]


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

def scan_case(rng, H, N, P, groups, vector_decay, lens):
    """Inputs of the recurrence for sequences of the given lengths, and the oracle's outputs and last states."""
    rows = sum(lens)
    q = rng.standard_normal((rows, groups, N))
    k = rng.standard_normal((rows, groups, N))
    v = rng.standard_normal((rows, H, P))
    decay = rng.uniform(0.6, 1.0, (rows, H, N) if vector_decay else (rows, H))
    kscale = rng.uniform(0.1, 1.5, (rows, H))
    skip = rng.standard_normal(H)
    return q, k, v, decay, kscale, skip


def scan_oracle(q, k, v, decay, kscale, skip, out_scale, lens, H, N, P, groups, vector_decay):
    out, states, at = [], [], 0
    for n in lens:
        o, S = np.zeros((n, H, P)), np.zeros((H, N, P))
        for h in range(H):
            g = h // (H // groups)
            d = decay[at:at + n, h] if vector_decay else np.repeat(decay[at:at + n, h:h + 1], N, axis=1)
            oh, S[h] = pp.decayed_outer_scan(d, k[at:at + n, g] * kscale[at:at + n, h:h + 1], v[at:at + n, h], q[at:at + n, g])
            o[:, h] = out_scale * oh + skip[h] * v[at:at + n, h]
        out.append(o.reshape(n, H * P))
        states.append(S)
        at += n
    return out, states


@pytest.mark.parametrize("H,N,P,groups,vector_decay", [(4, 16, 16, 4, True), (6, 24, 5, 2, False), (2, 8, 48, 1, False), (3, 40, 20, 3, True),
                                                       (1, 130, 33, 1, True), (5, 1, 1, 5, False)])
def test_recurrence_whole_in_portions_and_in_slots_used_again(H, N, P, groups, vector_decay):
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(H * 100 + N)
    lens, slots = [37, 1, 12], [3, 0, 2]
    q, k, v, decay, kscale, skip = scan_case(rng, H, N, P, groups, vector_decay, lens)
    ref, ref_states = scan_oracle(q, k, v, decay, kscale, skip, 0.5, lens, H, N, P, groups, vector_decay)
    f32 = torch.float32
    # One wide tensor holds everything, as a fused projection would: columns q | k | v | decay | kscale.
    widths = [groups * N, groups * N, H * P, H * N if vector_decay else H, H]
    at = np.concatenate([[0], np.cumsum(widths)])
    packed = np.concatenate([a.reshape(sum(lens), -1) for a in (q, k, v, decay, kscale)], axis=1).astype(np.float32)
    starts = np.concatenate([[0], np.cumsum(lens)])
    state = torch.zeros((5, H, P, N), dtype=f32, device=DEV)
    state[1] = 3.0                                                   # a slot nobody uses keeps what it holds
    state[4] = float("nan")
    got = [[] for _ in lens]
    for portion in ([5, 1, 2], [1, 0, 1], [29, 0, 2], [2, 0, 7]):     # rows each sequence brings, step by step
        live = [i for i, n in enumerate(portion) if n > 0]
        done = [sum(len(g) for g in got[i]) for i in range(3)]
        x = dev(np.concatenate([packed[starts[i] + done[i]:starts[i] + done[i] + portion[i]] for i in live]))
        seq_rows = i32(np.concatenate([[0], np.cumsum([portion[i] for i in live])]))
        out = torch.full((x.shape[0], H * P), 7.0, dtype=f32, device=DEV)
        ops.linear_scan(x, int(at[0]), H // groups, x, int(at[1]), H // groups, x, int(at[2]), x, int(at[3]), vector_decay, x, int(at[4]),
                        dev(skip.astype(np.float32)), 0.5, state, seq_rows, i32([slots[i] for i in live]), out, len(live), H, N, P)
        o, r = out.cpu().numpy(), 0
        for i in live:
            got[i].append(o[r:r + portion[i]])
            r += portion[i]
    for i in range(3):
        close(np.concatenate(got[i]), ref[i], "float32", f"sequence {i}")
        close(state[slots[i]].cpu().numpy().transpose(0, 2, 1).reshape(1, -1), ref_states[i].reshape(1, -1), "float32", f"state {i}")
    assert torch.all(state[1] == 3.0) and torch.isnan(state[4]).all()
    # A slot that held another sequence, cleared as the cache does, gives the first sequence's results again; a
    # sequence whose slot is negative is skipped and its rows of the output stay.
    state[slots[1]].zero_()
    x = dev(packed[:lens[0]])
    out = torch.full((lens[0] + 2, H * P), 7.0, dtype=f32, device=DEV)
    xx = torch.cat([x, x[:2]])
    ops.linear_scan(xx, int(at[0]), H // groups, xx, int(at[1]), H // groups, xx, int(at[2]), xx, int(at[3]), vector_decay, xx, int(at[4]),
                    dev(skip.astype(np.float32)), 0.5, state, i32([0, lens[0], lens[0] + 2]), i32([slots[1], -1]), out, 2, H, N, P)
    close(out[:lens[0]].cpu().numpy(), ref[0], "float32", "a slot used again")
    assert torch.all(out[lens[0]:] == 7.0)


def test_a_far_key_stays_in_the_recurrent_state():
    """One key written at the first position with decays of one on its channel is read back 300 positions later by
    a query on that channel alone: the output is that position's value, whatever came between on other channels."""
    from borrowed_compute_b200 import ops

    H, N, P, T = 2, 16, 16, 301
    rng = np.random.default_rng(5)
    q, k = 0.01 * rng.standard_normal((T, H, N)), 0.01 * rng.standard_normal((T, H, N))
    v = rng.standard_normal((T, H, P))
    decay = rng.uniform(0.5, 0.9, (T, H, N))
    k[:, :, 3], q[:, :, 3], decay[:, :, 3] = 0.0, 0.0, 1.0
    k[0, :, 3], q[T - 1, :, 3] = 4.0, 5.0
    x = dev(np.concatenate([a.reshape(T, -1) for a in (q, k, v, decay)], axis=1).astype(np.float32))
    for cuts in ([T], [1, 63, 64, 1, 172], [299, 2]):
        state = torch.zeros((1, H, P, N), dtype=torch.float32, device=DEV)
        rows, at = [], 0
        for n in cuts:
            part = x[at:at + n].contiguous()
            out = torch.empty((n, H * P), dtype=torch.float32, device=DEV)
            ops.linear_scan(part, 0, 1, part, H * N, 1, part, 2 * H * N, part, 2 * H * N + H * P, True, None, 0, None, 1.0, state, i32([0, n]),
                            i32([0]), out, 1, H, N, P)
            rows.append(out.cpu().numpy())
            at += n
        last = np.concatenate(rows)[-1].reshape(H, P)
        assert np.abs(last - 20.0 * v[0]).max() < 0.05, f"cuts {cuts}: the far key is lost"


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_convolution_with_bias_and_silu_and_the_step_sizes(taps):
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(taps)
    C, H, lead = 44, 3, 7                                            # the projection has `lead` columns ahead of the channels
    kernel, bias = rng.standard_normal((C, taps)), rng.standard_normal(C)
    dt_bias, a_log = rng.standard_normal(H), rng.uniform(-2, 1, H)
    lens, slots = [40, 1, 11], [2, 0, 3]
    xs = [rng.standard_normal((n, lead + C + H)) for n in lens]
    ref = [pp.conv_silu(x[:, lead:lead + C], kernel, bias)[0] for x in xs]
    tail = torch.zeros((4, max(taps - 1, 1), C), dtype=torch.float32, device=DEV)
    tail[1] = 7.0
    got, got_dt = [[] for _ in lens], [[] for _ in lens]
    for portion in ([3, 1, 2], [1, 0, 1], [34, 0, 6], [2, 0, 2]):
        live = [i for i, n in enumerate(portion) if n > 0]
        done = [sum(len(g) for g in got[i]) for i in range(3)]
        proj = dev(np.concatenate([xs[i][done[i]:done[i] + portion[i]] for i in live]).astype(np.float32))
        xbc = torch.empty((proj.shape[0], C), dtype=torch.float32, device=DEV)
        dtda = torch.empty((proj.shape[0], 2 * H), dtype=torch.float32, device=DEV)
        ops.ssd_prepare(proj, lead, lead + C, dev(kernel.T.astype(np.float32)), dev(bias.astype(np.float32)), dev(dt_bias.astype(np.float32)),
                        dev(a_log.astype(np.float32)), tail, i32(np.concatenate([[0], np.cumsum([portion[i] for i in live])])),
                        i32([slots[i] for i in live]), xbc, dtda, len(live), max(portion))
        o, d, r = xbc.cpu().numpy(), dtda.cpu().numpy(), 0
        for i in live:
            got[i].append(o[r:r + portion[i]])
            got_dt[i].append(d[r:r + portion[i]])
            r += portion[i]
    for i in range(3):
        close(np.concatenate(got[i]), ref[i], "float32", f"sequence {i}")
        dt = pp.softplus(xs[i][:, lead + C:] + dt_bias)
        close(np.concatenate(got_dt[i]), np.concatenate([dt, np.exp(-np.exp(a_log) * dt)], axis=1), "float32", f"step sizes {i}")
    assert torch.all(tail[1] == 7.0)


def test_decay_of_gated_linear_attention_and_the_gated_norms():
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(9)
    rows, W, rank, lead = 13, 72, 10, 5
    proj = rng.standard_normal((rows, lead + rank)) * 3.0
    w2, b = rng.standard_normal((W, rank)), rng.uniform(-3, 6, W)
    z = proj[:, lead:] @ w2.T + b
    decay = torch.empty((rows, W), dtype=torch.float32, device=DEV)
    ops.gla_decay(dev(proj.astype(np.float32)), lead, dev(w2.T.astype(np.float32)), dev(b.astype(np.float32)), decay, 7.0)
    close(decay.cpu().numpy(), pp.sigmoid(z) ** (1.0 / 7.0), "float32", "decay")
    for parts, period, gate_first in ((6, 12, False), (3, 72, True), (1, 72, True), (72, 1, False)):
        y, gate = rng.standard_normal((rows, W)), rng.standard_normal((rows, lead + W))
        weight = rng.standard_normal(period)
        ref = 0.7 * pp.gated_part_norm(y, gate[:, lead:], weight, parts, 1e-5, gate_first)
        for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            out = torch.empty((rows, W), dtype=td, device=DEV)
            ops.gated_norm(dev(y.astype(np.float32)), dev(gate.astype(np.float32)), lead, dev(weight.astype(np.float32)), out, parts, 1e-5, gate_first, 0.7)
            close(out.float().cpu().numpy(), ref, dtype, f"{parts} parts, gate first {gate_first}")


def attention_case(rng, T, H, G, D, DV, sharp=None):
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, G, DV))
    if sharp is not None:
        row, key = sharp                  # one score of that row stands out by far in every head, if the row sees the key at all
        base = rng.standard_normal((G, D))
        q[row] = 3.0 * base.repeat(H // G, axis=0)
        k[key] = 2.0 * base
    return q, k, v


def run_attention(q, k, v, window, scale, dtype, cuts, kernel, H, G, D, DV, sink=True, out_scale=1.0):
    """q, k, v of one sequence through the cache and an attention kernel, in steps of the given sizes."""
    from borrowed_compute_b200 import ops

    td = torch.float32 if dtype == "float32" else torch.bfloat16
    T = q.shape[0]
    pages = -(-T // 64)
    table = torch.full((3, pages + 1), -1, dtype=torch.int32, device=DEV)
    order = list(range(pages))[::-1]                                    # pages in an order of their own
    table[1, :pages] = i32([p + 1 for p in order])
    k_cache = torch.full((pages + 2, G, 64, D), float("nan"), dtype=td, device=DEV)
    v_cache = torch.full((pages + 2, G, 64, DV), float("nan"), dtype=td, device=DEV)
    outs, at = [], 0
    for n in cuts:
        pos = np.arange(at, at + n)
        qkv = dev(np.concatenate([q[pos].reshape(n, -1), k[pos].reshape(n, -1), v[pos].reshape(n, -1)], axis=1).astype(np.float32))
        q_out = torch.empty((n, H * D), dtype=td, device=DEV)
        ops.qkv_prepare_heads(qkv, None, None, None, i32(pos), i32([1] * n), table, q_out, k_cache, v_cache, H, G, D, DV, 0, 1, 0.0)
        out = torch.empty((n, H * DV), dtype=td, device=DEV)
        if kernel == "split" and n == 1:
            for via_scratch in (False, True):                       # the splits' two ways of merging give the same
                ops.attention_decode(q_out, H * D, k_cache, v_cache, table, i32(pos), i32([1]), out, H, G, D, window=window, scale=scale,
                                     splits=2 if at >= 64 and window != 1 else 1, via_scratch=via_scratch, sink=sink, out_scale=out_scale)
        elif kernel == "tc" and n > 1:
            ops.attention_prefill(q_out, H * D, k_cache, v_cache, table, i32([0, n]), i32([1]), i32([at]), out, 1, n, H, G, D, window=window, scale=scale,
                                  use_tc=True, value_dim=DV, sink=sink, out_scale=out_scale)
        elif kernel == "rows":
            ops.attention_rows(q_out, H * D, k_cache, v_cache, table, i32(pos), i32([1] * n), out, H, G, D, window=window, scale=scale,
                               value_dim=DV, sink=sink, out_scale=out_scale)
        else:
            ops.attention_tiles(q_out, H * D, k_cache, v_cache, table, i32([0, n]), i32([1]), i32([at]), out, 1, n, H, G, D, DV, window=window,
                                scale=scale, sink=sink, out_scale=out_scale)
        outs.append(out.float().cpu().numpy())
        at += n
    return np.concatenate(outs).reshape(T, H, DV)


@pytest.mark.parametrize("dtype,kernel", [("float32", "rows"), ("bfloat16", "rows"), ("bfloat16", "tiles"), ("bfloat16", "tc"), ("bfloat16", "split")])
@pytest.mark.parametrize("window", [0, 1, 9, 64, 70])
def test_sink_attention_with_one_key_that_matters_at_every_edge(dtype, kernel, window):
    """A key just inside the window takes nearly all the weight, one just outside none; in a prompt and when the row is
    decoded alone; at a page's border; and a row whose scores are all very low gives nearly nothing (the sink).  The
    tcgen05 kernel takes prompts of heads of 64 or 128 (single rows go to the tiles there too); "split" sends single
    rows to the kernel that splits a row's positions over blocks (prompts to the tiles)."""
    H, G, D, DV, T, scale = {"tc": (4, 2, 128, 64, 150, 0.1), "split": (4, 2, 64, 64, 150, 0.15)}.get(kernel, (4, 2, 32, 16, 150, 0.2))
    rng = np.random.default_rng(window)
    row = 140
    edges = [row, row - 1, 128, 127, 0] if window == 0 else sorted({row - window + 1, row - window, max(row - window + 2, 0), row})
    for key in edges:
        if not 0 <= key <= row:
            continue
        q, k, v = attention_case(rng, T, H, G, D, DV, sharp=(row, key))
        if dtype == "bfloat16":
            q, k, v = pp.bf16_round(q), pp.bf16_round(k), pp.bf16_round(v)
        ref = pp.sink_softmax_attention(pp.f64(q), pp.f64(k), pp.f64(v), scale, window)
        seen = window == 0 or row - key < window
        assert (np.abs(ref[row] - v[key].repeat(H // G, axis=0)).max() < 0.1) == seen      # the case is what it is meant to be
        for cuts in ([T], [row, 1, T - row - 1], [64, 64, 12, 10]):
            got = run_attention(q, k, v, window, scale, dtype, cuts, kernel, H, G, D, DV)
            close(got.reshape(T, -1), ref.reshape(T, -1), dtype, f"key {key}, cuts {cuts}")
    q, k, v = attention_case(rng, 20, H, G, D, DV)
    low = rng.standard_normal((20, G, D))
    q_low, k_low = low.repeat(H // G, axis=1), -4.0 * low                                         # row 0 sees itself alone, far below the sink's 0
    ref = pp.sink_softmax_attention(q_low, k_low, v, 1.0, window)
    got = run_attention(q_low, k_low, v, window, 1.0, dtype, [20], kernel, H, G, D, DV)
    assert np.abs(ref[0]).max() < 1e-3
    close(got.reshape(20, -1), ref.reshape(20, -1), dtype, "the sink")
    got = run_attention(q, k, v, window, scale, dtype, [20], kernel, H, G, D, DV, sink=False, out_scale=0.5)
    plain = pp.sink_softmax_attention(q, k, v, scale, window)
    assert np.abs(got - 0.5 * plain).max() > 0.01                                              # without the sink the weights add up to one


@pytest.mark.parametrize("D,rot,pairing", [(32, 32, 1), (48, 16, 1), (20, 6, 1), (64, 32, 0), (16, 0, 1)])
def test_norm_of_single_heads_and_rotation_of_neighbours(D, rot, pairing):
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.rope import inverse_frequencies, rotary_table

    H, G, DV, n, base, eps = 5, 5, 12, 9, 1000.0, 1e-5
    rng = np.random.default_rng(D + rot)
    pos = np.array([0, 1, 2, 63, 64, 65, 200, 5, 130])
    x = rng.standard_normal((n, (H + G) * D + G * DV))
    wq, wk = rng.standard_normal(D), rng.standard_normal(D)
    q = pp.rms_norm(x[:, :H * D].reshape(n, H, D), wq, eps)
    k = pp.rms_norm(x[:, H * D:(H + G) * D].reshape(n, G, D), wk, eps)
    if pairing == 1:
        q, k = pp.rotate_pairs(q, pos, rot, base), pp.rotate_pairs(k, pos, rot, base)
    else:                                                                                        # dimension i with i + rot / 2
        def half(t):
            out = t.copy()
            for i in range(rot // 2):
                a = pos * base ** (-2.0 * i / rot)
                c, s = np.cos(a)[:, None], np.sin(a)[:, None]
                out[:, :, i], out[:, :, i + rot // 2] = t[:, :, i] * c - t[:, :, i + rot // 2] * s, t[:, :, i + rot // 2] * c + t[:, :, i] * s
            return out
        q, k = half(q), half(k)
    table = torch.full((2, 5), -1, dtype=torch.int32, device=DEV)
    table[1, :4] = i32([2, 0, 3, 1])
    cos_sin = None if rot == 0 else rotary_table(inverse_frequencies(rot, base, None), 256).to(DEV)
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        k_cache = torch.zeros((4, G, 64, D), dtype=td, device=DEV)
        v_cache = torch.zeros((4, G, 64, DV), dtype=td, device=DEV)
        q_out = torch.empty((n, H * D), dtype=td, device=DEV)
        ops.qkv_prepare_heads(dev(x.astype(np.float32)), dev(wq.astype(np.float32)), dev(wk.astype(np.float32)), cos_sin, i32(pos), i32([1] * n), table,
                              q_out, k_cache, v_cache, H, G, D, DV, rot, pairing, eps)
        close(q_out.float().cpu().numpy(), q.reshape(n, -1), dtype, "q")
        pages = [2, 0, 3, 1]
        got_k = np.stack([k_cache[pages[p // 64], :, p % 64].float().cpu().numpy() for p in pos])
        got_v = np.stack([v_cache[pages[p // 64], :, p % 64].float().cpu().numpy() for p in pos])
        close(got_k.reshape(n, -1), k.reshape(n, -1), dtype, "k")
        close(got_v.reshape(n, -1), x[:, (H + G) * D:], dtype, "v")


@pytest.mark.parametrize("E,top,ff,K,rows", [(5, 2, 24, 40, 77), (3, 3, 8, 16, 77), (9, 1, 70, 72, 77), (33, 4, 16, 24, 77), (5, 2, 16, 32, 150),
                                             (4, 2, 24, 40, 230), (3, 2, 24, 40, 600)])
def test_routed_experts(E, top, ff, K, rows):
    """The router's choices (ties to the lower index), the sort by expert, both products and the sum, against the
    plain loop; rows of no sequence choose nothing.  The rows an expert gets on average decide the tile of the
    tensor-core products: the cases reach tiles of 16, 32, 64, 128 and 256 sorted rows, and widths that only the
    CUDA-core products take."""
    from borrowed_compute_b200.parts.base import Runtime, StepContext
    from borrowed_compute_b200.parts.moe import RoutedExperts

    rng = np.random.default_rng(E)
    w = {"router": pp.bf16_round(rng.standard_normal((E, K)))}
    for e in range(E):
        w.update({f"e{e}.gate": pp.bf16_round(rng.standard_normal((ff, K)) / math.sqrt(K)), f"e{e}.up": pp.bf16_round(rng.standard_normal((ff, K)) / math.sqrt(K)),
                  f"e{e}.down": pp.bf16_round(rng.standard_normal((K, ff)) / math.sqrt(ff))})
    w.update({"shared.gate": pp.bf16_round(rng.standard_normal((12, K)) / 4), "shared.up": pp.bf16_round(rng.standard_normal((12, K)) / 4),
              "shared.down": pp.bf16_round(rng.standard_normal((K, 12)) / 4)})
    h = pp.bf16_round(rng.standard_normal((rows, K)))
    w["router"][1] = w["router"][0]                                   # two experts that always tie
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": 12}}
    ref = pp.moe_feed_forward(pp.f64(h), {n: pp.f64(a) for n, a in w.items()}, "", mlp)
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        part = RoutedExperts(K, E, top, ff, shared_size=12)
        part.load({n: dev(a, torch.float32 if n == "router" else td) for n, a in w.items()}, Runtime(torch.device(DEV), td))
        slot = np.zeros(rows + 3, dtype=np.int32)
        slot[rows:] = -1
        x = torch.cat([dev(h, td), torch.full((3, K), float("nan"), dtype=td, device=DEV)])
        residual = torch.ones((rows + 3, K), dtype=torch.float32, device=DEV)
        ctx = StepContext(rows=rows + 3, seqs=1, tokens=None, row_pos=None, row_slot=i32(slot), seq_rows=None, seq_slot=None, seq_start=None,
                          max_new=rows, max_total=rows, decode=False)
        part.forward(x, residual, ctx)
        out = residual.cpu().numpy()
        close(out[:rows] - 1.0, ref, dtype, "experts")
        # Alone, a row gives the same bits as in the batch.
        alone = torch.ones((1, K), dtype=torch.float32, device=DEV)
        ctx1 = StepContext(rows=1, seqs=1, tokens=None, row_pos=None, row_slot=i32([0]), seq_rows=None, seq_slot=None, seq_start=None, max_new=1,
                           max_total=1, decode=True)
        RoutedExperts.forward(part, x[40:41].contiguous(), alone, ctx1)
        if part.shared is None or dtype == "float32":
            assert torch.equal(alone[0], residual[40])


def test_scaled_embedding_soft_cap_and_the_mix_with_the_embedding():
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.base import Runtime
    from borrowed_compute_b200.parts.reentry import MixWithEmbedding

    rng = np.random.default_rng(3)
    V, E, rows = 37, 40, 11
    table = pp.bf16_round(rng.standard_normal((V, E)))
    toks = rng.integers(0, V, rows)
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        out = torch.empty((rows, E), dtype=torch.float32, device=DEV)
        ops.embed(dev(table, td), i32(toks), out, 6.5)
        assert np.array_equal(out.cpu().numpy(), table[toks] * np.float32(6.5))
        x, x0 = rng.standard_normal((rows, E)).astype(np.float32), rng.standard_normal((rows, E)).astype(np.float32)
        w_in, steps = pp.bf16_round(rng.standard_normal((E, 2 * E)) / 6), pp.bf16_round(rng.standard_normal((3, E)))
        part = MixWithEmbedding(E, 3)
        part.load({"in": dev(w_in, td), "step": dev(steps)}, Runtime(torch.device(DEV), td))
        for number in (0, 2):
            stream = dev(x)
            part.forward(stream, dev(x0), None, number)
            close(stream.cpu().numpy(), np.concatenate([pp.f64(x), pp.f64(x0)], axis=1) @ pp.f64(w_in).T + steps[number], dtype, f"pass {number}")
    scores = rng.standard_normal((5, 23)).astype(np.float32) * 40
    capped = dev(scores)
    ops.softcap(capped, 15.0)
    close(capped.cpu().numpy(), 15.0 * np.tanh(pp.f64(scores) / 15.0), "float32", "soft cap")


# ---------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_in_float32(name):
    eng, cfg, w = small(name, "float32")
    toks = tokens_for(3, 150, cfg["vocab"])
    close(run_whole(eng, toks), pp.forward(cfg, w, toks), "float32")


@pytest.mark.parametrize("name,n", [("A", 30), ("B", 90)])
def test_whole_prompt_and_decoding_in_bfloat16(name, n):
    eng, cfg, w = small(name, "bfloat16")
    toks, ref = decisive(name, n, 4)
    close(run_whole(eng, toks), ref, "bfloat16", "whole")
    close(run_cut(eng, toks, [n // 2]), ref, "bfloat16", "decoded")
    close(run_cut(eng, toks, [n - 9, 2, 3]), ref, "bfloat16", "portions")


@pytest.mark.parametrize("name", ["A", "B"])
def test_decoding_token_by_token_and_portions_in_float32(name):
    """Windows of 9, 70 and 130 positions pass over decoded tokens and over the borders of 64-token pages."""
    eng, cfg, w = small(name, "float32")
    toks = tokens_for(5, 210, cfg["vocab"])
    ref = pp.forward(cfg, w, toks)
    close(run_cut(eng, toks, [60]), ref, "float32", "decoded from 60")
    close(run_cut(eng, toks, [1]), ref, "float32", "decoded from the first token")
    for cuts in ([2, 2, 61, 63, 2, 64, 16], [129, 2, 7, 70, 2], [64, 64, 64, 18]):
        close(run_cut(eng, toks, cuts), ref, "float32", f"portions {cuts}")


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "B")])
def test_unequal_batch_against_each_alone(dtype, name):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small(name, dtype)
    lens = [1, 77, 3, 130] if dtype == "float32" else [1, 60, 3, 78]
    seqs = [tokens_for(40 + i, n + 12, cfg["vocab"]) if dtype == "float32" else decisive(name, n + 12, 40 + i)[0] for i, n in enumerate(lens)]
    alone = [run_cut(eng, s, [n]) for s, n in zip(seqs, lens)]
    slots = [eng.acquire() for _ in seqs]
    got = [[eng_rows] for eng_rows in np.split(
        eng.step([StepEntry(s, q[:n], tuple(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy(), np.cumsum(lens)[:-1])]
    for t in range(12):
        live = [i for i in range(4) if t < 12 - 3 * (i == 2)]             # one sequence ends earlier
        out = eng.step([StepEntry(slots[i], [seqs[i][lens[i] + t]], (0,)) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
        if t == 8:
            eng.release(slots[2])
    for i in (0, 1, 3):
        eng.release(slots[i])
    for i in range(4):
        mine = np.concatenate(got[i])
        if dtype == "float32":
            close(mine, pp.forward(cfg, w, seqs[i])[:len(mine)], "float32", f"sequence {i}")
        else:
            close(mine, decisive(name, lens[i] + 12, 40 + i)[1][:len(mine)], "bfloat16", f"sequence {i}")
        assert np.abs(mine - alone[i][:len(mine)]).max() <= (1e-5 if dtype == "float32" else 0.1), f"sequence {i} depends on the batch"


def test_slots_and_pages_used_again():
    from borrowed_compute_b200.engine import StepEntry

    cfg = pp.SMALL["B"]
    w = pp.make_weights(cfg, 22)
    eng = engine_for(cfg, w, "float32", max_tokens=448, max_slots=2, max_seq=320)
    first = None
    for turn in range(4):
        toks = tokens_for(60 + turn % 2, 200, cfg["vocab"])
        other = tokens_for(70 + turn, 100 + 20 * turn, cfg["vocab"])
        a, b = eng.acquire(), eng.acquire()
        eng.step([StepEntry(b, other, ())])
        got = eng.step([StepEntry(a, toks[:150], tuple(range(150)))]).cpu().numpy()
        eng.release(b)
        rest = [eng.step([StepEntry(a, [t], (0,))]).cpu().numpy() for t in toks[150:]]
        eng.release(a)
        got = np.concatenate([got] + rest)
        if turn < 2:
            close(got, pp.forward(cfg, w, toks), "float32", f"turn {turn}")
        if turn == 0:
            first = got
        if turn == 2:
            assert np.array_equal(got, first), "what a slot or a page held before shows"
    assert eng.cache.slots.live() == []


def test_long_decoding_and_the_first_tokens():
    eng, cfg, w = small("B", "float32")
    toks = tokens_for(8, 330, cfg["vocab"])
    ref = pp.forward(cfg, w, toks)
    close(run_cut(eng, toks, [3]), ref, "float32", "327 tokens decoded")
    for n in (1, 2, 3, 5):
        close(run_whole(eng, toks[:n]), ref[:n], "float32", f"the first {n}")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_drawn_configurations(seed):
    """Sizes drawn at random, among them values that make parts of the design equal or 1."""
    from borrowed_compute_b200.engine import StepEntry

    rng = np.random.default_rng(seed)
    pick = lambda *a: a[int(rng.integers(len(a)))]                        # noqa: E731
    layers = []
    for _ in range(int(rng.integers(1, 4))):
        if rng.random() < 0.5:
            mixer, kind = pp._gla(pick(1, 2, 3), pick(4, 8, 20), pick(4, 12, 16), pick(1.0, 3.0, 16.0), pick(1, 5)), "gla"
        else:
            heads, kv = pick((1, 1), (2, 2), (4, 2), (6, 1))
            dim = pick(8, 16, 24, 64)
            sheads, groups = pick((1, 1), (4, 2), (3, 3), (6, 1))
            svdim = pick(4, 8, 10)
            parts = pick(*[p for p in (1, 2, sheads) if (sheads * svdim) % p == 0])
            mixer = pp._pair(heads, kv, dim, pick(8, 16, dim), pick(0, 1, 5, 64, 100), pick(0, 2, dim), pick(100.0, 1e6), pick(0.1, 0.3), sheads, svdim,
                             pick(4, 16, 33), groups, parts, pick(1, 2, 4), pick(0.5, 1.0), pick(1.0, 1.5))
            kind = "parallel"
        mlp = None if rng.random() < 0.2 else pp._moe(pick(1, 2, 6), 1, pick(8, 20), pick(0, 8))
        if mlp is not None:
            mlp["router"]["top"] = int(rng.integers(1, mlp["router"]["experts"] + 1))
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Pozirax", "vocab": pick(50, 97), "width": pick(24, 40, 64), "norm": {"eps": pick(1e-5, 1e-6)},
           "embedding": {"scale": pick(1.0, 4.0)}, "logit_softcap": pick(None, 8.0), "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        cfg["loop"] = {"start": start, "stop": int(rng.integers(start + 1, len(layers) + 1)), "times": pick(1, 2, 3)}
    w = pp.make_weights(cfg, seed)
    eng = engine_for(cfg, w, "float32", max_tokens=1024, max_slots=4, max_seq=256)
    seqs = [tokens_for(seed * 10 + i, n, cfg["vocab"]) for i, n in enumerate([70, 5, 131])]
    slots = [eng.acquire() for _ in seqs]
    first = [30, 5, 129]
    out = eng.step([StepEntry(s, q[:n], tuple(range(n))) for s, q, n in zip(slots, seqs, first)]).cpu().numpy()
    got = [[a] for a in np.split(out, np.cumsum(first)[:-1])]
    got[0].append(eng.step([StepEntry(slots[0], seqs[0][30:68], tuple(range(38)))]).cpu().numpy())
    for t in range(2):
        out = eng.step([StepEntry(slots[0], [seqs[0][68 + t]], (0,)), StepEntry(slots[2], [seqs[2][129 + t]], (0,))]).cpu().numpy()
        got[0].append(out[:1])
        got[2].append(out[1:])
    refs = [pp.forward(cfg, w, q) for q in seqs]
    for i in range(3):
        close(np.concatenate(got[i]), refs[i], "float32", f"{json.dumps(cfg)}: sequence {i}")
    # The same sizes on the bfloat16 kernels: a router's choice may flip by rounding on a few rows (and, through a state,
    # on those after them), so most rows are held to the oracle, and all of them to being numbers.
    eng16 = engine_for(cfg, w, "bfloat16", max_tokens=1024, max_slots=4, max_seq=256)
    for i in (0, 2):
        got16 = run_cut(eng16, seqs[i], [first[i]])
        assert np.isfinite(got16).all()
        errors = np.abs(got16 - refs[i]).max(axis=-1)
        assert np.median(errors) <= tol("bfloat16", refs[i]), f"{json.dumps(cfg)}: sequence {i} in bfloat16, median error {np.median(errors):.3g}"


def test_the_trace_tool_replays_prompts_decoding_and_a_batch(tmp_path):
    """bin/trace_run on a folder of this design: whole prompts, single tokens after a prompt, and a batch of unequal
    requests that start together and end one after another, in float32 against the plain implementation."""
    import subprocess
    import sys

    from borrowed_compute_b200.weights.safetensors_io import write_safetensors
    from conftest import ROOT

    cfg = {"architecture": "Pozirax", "vocab": 301, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 7.0}, "logit_softcap": 25.0,
           "loop": {"start": 1, "stop": 4, "times": 2},
           "layers": [
               {"type": "parallel", "mixer": pp._pair(8, 2, 32, 32, 100, 32, 1e5, 0.2, 8, 16, 16, 4, 2, 4, 0.8, 1.2), "mlp": pp._moe(8, 2, 32, 64)},
               {"type": "gla", "mixer": pp._gla(2, 64, 64, 12.0, 8), "mlp": pp._moe(8, 2, 32, 64)},
               {"type": "gla", "mixer": pp._gla(4, 16, 48, 6.0, 8), "mlp": None},
               {"type": "parallel", "mixer": pp._pair(4, 4, 64, 64, 33, 64, 1e4, 0.15, 4, 32, 24, 1, 4, 3, 1.0, 0.6), "mlp": pp._moe(6, 1, 40, 0)},
               {"type": "gla", "mixer": pp._gla(1, 128, 32, 3.0, 16), "mlp": pp._moe(4, 4, 24, 24)},
           ]}
    w = pp.make_weights(cfg, 31)
    on_disk = copy.deepcopy(cfg)
    for layer in on_disk["layers"]:
        layer["mixer"].pop("rank", None)
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(on_disk, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in w.items()})
    a, b, c = (tokens_for(70 + i, n, cfg["vocab"]) for i, n in enumerate([150, 40, 9]))
    refs = {"a": pp.forward(cfg, w, a), "b": pp.forward(cfg, w, b), "c": pp.forward(cfg, w, c)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:120], "want": [0, 64, 119]}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "a", "tokens": [a[120 + i]], "want": [0]}], "end": ["a"] if i == 29 else []} for i in range(30)]
    steps.append({"step": 31, "entries": [{"id": "x", "tokens": a[:100], "want": [99]}, {"id": "y", "tokens": b[:30], "want": []},
                                          {"id": "z", "tokens": c[:5], "want": [4]}], "end": []})
    for i in range(10):
        live = [("x", a, 100), ("y", b, 30)] + ([("z", c, 5)] if i < 4 else [])
        steps.append({"step": 32 + i, "entries": [{"id": n, "tokens": [t[at + i]], "want": [0]} for n, t, at in live],
                      "end": (["z"] if i == 3 else []) + (["x", "y"] if i == 9 else [])})
    text = "".join(json.dumps(s) + "\n" for s in steps)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
                          "--max-tokens", "512"], input=text, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [line for line in res.stdout.splitlines() if line.startswith("done")] == [f"done {s['step']}" for s in steps]
    V = cfg["vocab"]
    read = lambda n: np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V)      # noqa: E731
    close(read(0), refs["a"][[0, 64, 119]], "float32", "the prompt")
    for i in range(30):
        close(read(1 + i), refs["a"][120 + i:121 + i], "float32", f"token {i} after the prompt")
    close(read(31), np.stack([refs["a"][99], refs["c"][4]]), "float32", "the batch's prompts")
    for i in range(10):
        want = [refs["a"][100 + i], refs["b"][30 + i]] + ([refs["c"][5 + i]] if i < 4 else [])
        close(read(32 + i), np.stack(want), "float32", f"the batch's token {i}")


def test_greedy_generation_through_the_entry_point(tmp_path):
    """A folder whose config.json leaves the decay's inner width to the tensors' shapes, loaded by Local and by the
    command line; greedy tokens of a batch of unequal prompts against the plain loop."""
    import subprocess
    import sys

    from borrowed_compute_b200 import Local, Sampling
    from borrowed_compute_b200.weights.safetensors_io import write_safetensors
    from conftest import ROOT

    cfg = copy.deepcopy(pp.SMALL["A"])
    w = pp.make_weights(cfg, 21)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in w.items()})
    prompts = [tokens_for(90 + i, n, cfg["vocab"]) for i, n in enumerate([3, 45, 1])]
    want = [pp.generate(pp.SMALL["A"], w, p, 10) for p in prompts]
    model = Local.load(folder, dtype="float32", max_tokens=1024, max_slots=4, max_seq=128)
    out, stats = model.generate(prompts, 10, Sampling(), stop_ids=())
    assert out == want and stats.generated == 30
    assert model.engine.cache.slots.live() == []
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", folder, ";".join(",".join(map(str, p)) for p in prompts),
                          "--max-tokens", "10", "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in res.stdout.strip().splitlines()] == want
    model16 = Local.load(folder, dtype="bfloat16", max_tokens=1024, max_slots=4, max_seq=128)
    out16, _ = model16.generate(prompts, 10, Sampling(), stop_ids=())
    assert all(len(o) == 10 and all(0 <= t < cfg["vocab"] for t in o) for o in out16)


def test_a_cut_back_is_refused_unless_to_zero():
    from borrowed_compute_b200.config import CacheError
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small("A", "float32")
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
    close(got, pp.forward(cfg, w, toks), "float32")
