"""A plain, slow restatement of the Pozirax decoder in NumPy float64, one function per
mechanism, written from the design's equations and sharing no code with the package.

Notation: X is [T, width] for one sequence of T tokens at positions 0 .. T-1; matrices are
[out, in] and applied as X @ W.T; `cfg` is the config.json dict, `w` maps tensor names to
arrays.  Every recurrent function takes the state it starts from and returns the state it
ends with, so that a test can cut a sequence anywhere.
"""

from __future__ import annotations

import math

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def bf16_round(a):
    """The nearest bfloat16 (ties to even) of every value, as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(a.shape)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def over_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return over_rms(x, eps) * weight


# ------------------------------------------------------------------------------ attention side

def rotate_pairs(x, positions, dims, base):
    """x: [T, heads, dim].  Dimension 2i turns with dimension 2i + 1 by position * base^(-2i/dims),
    for i < dims / 2; the other dimensions pass."""
    out = x.copy()
    for i in range(dims // 2):
        a = f64(positions) * base ** (-2.0 * i / dims)
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, window):
    """q: [T, H, D] at positions 0..T-1 against k [T, G, D], v [T, G, DV] of the same positions.
    Position i sees j with 0 <= i - j < window (window 0: every j <= i).  The weights are
    exp(s_j) / (1 + sum_j exp(s_j)): a sink of score 0 that has no value."""
    T, H, _ = q.shape
    G, DV = k.shape[1], v.shape[2]
    out = np.zeros((T, H, DV))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window > 0 else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(0.0, float(s.max()))
            e = np.exp(s - m)
            out[i, h] = (e / (math.exp(-m) + e.sum())) @ v[lo:i + 1, g]
    return out


def window_attention_mixer(h, w, p, m, eps, positions=None):
    """The left side of a 'parallel' mixer for a whole sequence.  m is the config's mixer.left."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    pos = np.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, DV)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate_pairs(q, pos, rot["dims"], rot["base"]), rotate_pairs(k, pos, rot["dims"], rot["base"])
    window = m["mask"]["size"] if m.get("mask") else 0
    o = sink_softmax_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * DV) @ w[p + "o"].T


# --------------------------------------------------------------------------- state-space side

def conv_silu(x, kernel, bias, before=None):
    """Causal convolution per channel, then silu.  x: [T, C]; kernel [C, taps], its last column is the
    current token's; `before` [taps - 1, C] are the inputs ahead of x (zeros at a sequence's start).
    Returns the outputs and the last taps - 1 inputs."""
    T, C = x.shape
    taps = kernel.shape[1]
    past = np.zeros((taps - 1, C)) if before is None else before
    full = np.concatenate([past, x], axis=0)
    out = np.zeros((T, C))
    for t in range(T):
        out[t] = bias + np.sum(kernel.T * full[t:t + taps], axis=0)
    return silu(out), full[full.shape[0] - (taps - 1):]


def decayed_outer_scan(decay, key, value, query, state=None):
    """One head of S_t = diag(decay_t) S_(t-1) + key_t value_t^T, out_t = S_t^T query_t.
    decay, key, query: [T, N] (a scalar decay is the same number in every channel); value: [T, P]."""
    T, N = key.shape
    P = value.shape[1]
    S = np.zeros((N, P)) if state is None else state.copy()
    out = np.zeros((T, P))
    for t in range(T):
        S = decay[t][:, None] * S + np.outer(key[t], value[t])
        out[t] = S.T @ query[t]
    return out, S


def gated_part_norm(y, gate, weight, parts, eps, gate_first):
    """y, gate: [T, W].  The row is cut into `parts` equal parts, each divided by its own root mean
    square and multiplied by `weight` (as wide as a part, or as the row); the gate silu(gate)
    multiplies before the norm (gate_first) or after it."""
    T, W = y.shape
    if gate_first:
        y = y * silu(gate)
    y = over_rms(y.reshape(T, parts, W // parts), eps).reshape(T, W)
    y = y * (np.tile(weight, parts) if weight.shape[0] != W else weight)
    return y if gate_first else y * silu(gate)


def state_space_mixer(h, w, p, m, eps, state=None):
    """The right side of a 'parallel' mixer.  m is the config's mixer.right; state = (S [heads, N, P], past
    inputs of the convolution [taps - 1, channels]) or None at a sequence's start."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    S0, past = (None, None) if state is None else state
    xbc, past = conv_silu(xbc, w[p + "conv"], w[p + "conv.b"], past)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = np.exp(-np.exp(w[p + "A_log"]) * dt)                       # [T, H]
    y = np.zeros((T, H, P))
    S = np.zeros((H, N, P))
    for a in range(H):
        g = a // (H // G)
        y[:, a], S[a] = decayed_outer_scan(np.repeat(decay[:, a:a + 1], N, axis=1), B[:, g] * dt[:, a:a + 1], x[:, a], C[:, g],
                                           None if S0 is None else S0[a])
        y[:, a] += w[p + "D"][a] * x[:, a]
    y = gated_part_norm(y.reshape(T, inner), z, w[p + "norm"], m["norm_groups"], eps, gate_first=True)
    return y @ w[p + "o"].T, (S, past)


def side_by_side_mixer(h, w, p, m, eps, state=None):
    """left_scale * attention + right_scale * state space, both reading h.  Whole sequences only on
    the attention side (it keeps no state here), so `state` serves tests of the right side alone."""
    left = window_attention_mixer(h, w, p + "left.", m["left"], eps)
    right, state = state_space_mixer(h, w, p + "right.", m["right"], eps, state)
    return m["left_scale"] * left + m["right_scale"] * right, state


# ------------------------------------------------------------------------ gated linear attention

def gla_mixer(h, w, p, m, eps, state=None):
    """q = W_q h / sqrt(dim), k, v; a decay per key channel sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b;
    S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; every head's o over its root mean square times
    a weight shared by the heads, then times silu(W_g h), then W_o."""
    T = h.shape[0]
    H, D, P = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D) / math.sqrt(D)
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, P)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = np.exp(-softplus(-z) / m["tau"]).reshape(T, H, D)          # sigmoid(z)^(1/tau)
    o = np.zeros((T, H, P))
    S = np.zeros((H, D, P))
    for a in range(H):
        o[:, a], S[a] = decayed_outer_scan(decay[:, a], k[:, a], v[:, a], q[:, a], None if state is None else state[a])
    y = gated_part_norm(o.reshape(T, H * P), h @ w[p + "g"].T, w[p + "norm"], H, eps, gate_first=False)
    return y @ w[p + "o"].T, S


# ------------------------------------------------------------------------------- feed-forward

def gated_expert(x, w, p):
    return (silu(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, router, top):
    """Scores sigmoid(W_router h); the `top` largest of a row (the lower index wins a tie), with
    their scores as weights, not renormalised."""
    s = sigmoid(h @ router.T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def route_margin(h, router, top):
    """The least distance, over the rows, between the last chosen expert's logit and the first one left out."""
    z = np.sort(h @ router.T, axis=-1)[:, ::-1]
    return float(np.min(z[:, top - 1] - z[:, top])) if top < z.shape[1] else math.inf


def moe_feed_forward(h, w, p, mlp, stats=None):
    """The sum over a row's chosen experts of expert(weight * h), plus a shared expert of h."""
    chosen, weight = route(h, w[p + "router"], mlp["router"]["top"])
    if stats is not None:
        stats["margin"] = min(stats.get("margin", math.inf), route_margin(h, w[p + "router"], mlp["router"]["top"]))
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            out[t] += gated_expert(s * h[t:t + 1], w, f"{p}e{int(e)}.")[0]
    if mlp.get("shared") is not None:
        out += gated_expert(h, w, p + "shared.")
    return out


# ----------------------------------------------------------------------------------- the model

def layer_runs(cfg):
    """The order in which layers run: (layer, pass number if it is the first layer of a pass else None)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, layers_out=None, stats=None):
    """Scores [T, vocab] of one whole sequence.  `layers_out` (a list) receives the stream after every run of a
    layer; `stats` (a dict) the least margin by which any router chose ("margin")."""
    w = {n: f64(a) for n, a in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    for i, t in layer_runs(cfg):
        if t is not None:
            x = np.concatenate([x, x0], axis=1) @ w["loop.in"].T + w["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "gla":
            mixed = gla_mixer(h, w, p + "mix.", layer["mixer"], eps)[0]
        elif layer["type"] == "parallel":
            mixed = side_by_side_mixer(h, w, p + "mix.", layer["mixer"], eps)[0]
        else:
            raise ValueError(layer["type"])
        ff = moe_feed_forward(h, w, p + "mlp.", layer["mlp"], stats) if layer.get("mlp") is not None else 0.0
        x = x + (mixed + ff)
        if layers_out is not None:
            layers_out.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits


def generate(cfg, w, prompt, n):
    """Greedy continuation (the lowest id among equal scores), recomputing the whole sequence a token."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]


def decisive_tokens(cfg, w, n, seed, margin=0.08):
    """n random tokens for which every router of the model chooses by at least `margin` at every position, so that
    rounding to bfloat16 cannot change a choice (a changed choice is another, equally valid, model output; a
    comparison with this implementation would say nothing).  Seeds are tried in turn."""
    for attempt in range(200):
        toks = [int(t) for t in np.random.default_rng(1000 * seed + attempt).integers(0, cfg["vocab"], n)]
        stats = {}
        ref = forward(cfg, w, toks, stats=stats)
        if stats.get("margin", math.inf) >= margin:
            return toks, ref
    raise RuntimeError("no decisive sequence found")


# ------------------------------------------------------------------- small models for the tests

def tensor_shapes(cfg):
    E, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, E), "final.norm": (E,), "head": (V, E)}
    if cfg.get("loop"):
        out["loop.in"] = (E, 2 * E)
        out["loop.step"] = (cfg["loop"]["times"], E)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (E,)
        if layer["type"] == "gla":
            H, D, P, rank = m["heads"], m["dim"], m["vdim"], m["rank"]
            out.update({p + "mix.q": (H * D, E), p + "mix.k": (H * D, E), p + "mix.v": (H * P, E), p + "mix.g": (H * P, E),
                        p + "mix.o": (E, H * P), p + "mix.norm": (P,), p + "mix.a1": (rank, E), p + "mix.a2": (H * D, rank),
                        p + "mix.a2.b": (H * D,)})
        else:
            a, s = m["left"], m["right"]
            H, G, D, DV = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            out.update({p + "mix.left.q": (H * D, E), p + "mix.left.k": (G * D, E), p + "mix.left.v": (G * DV, E),
                        p + "mix.left.q.norm": (D,), p + "mix.left.k.norm": (D,), p + "mix.left.o": (E, H * DV)})
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            out.update({p + "mix.right.in": (2 * inner + 2 * gn + s["heads"], E), p + "mix.right.conv": (inner + 2 * gn, s["conv"]),
                        p + "mix.right.conv.b": (inner + 2 * gn,), p + "mix.right.dt_bias": (s["heads"],), p + "mix.right.A_log": (s["heads"],),
                        p + "mix.right.D": (s["heads"],), p + "mix.right.norm": (inner,), p + "mix.right.o": (E, inner)})
        mlp = layer.get("mlp")
        if mlp is not None:
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (mlp["expert"]["ff"], E), f"{p}mlp.e{e}.up": (mlp["expert"]["ff"], E),
                            f"{p}mlp.e{e}.down": (E, mlp["expert"]["ff"])})
            out[p + "mlp.router"] = (mlp["router"]["experts"], E)
            if mlp.get("shared") is not None:
                f = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (f, E), p + "mlp.shared.up": (f, E), p + "mlp.shared.down": (E, f)})
    return out


def make_weights(cfg, seed):
    """Random bfloat16-valued weights with scales that keep every mechanism alive: decays spread between
    short and long memories, routers that do choose, norms near one."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last in ("norm", "norm1"):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif last == "A_log":
            a = rng.uniform(-3.0, 0.5, shape)
        elif last == "dt_bias":
            a = rng.uniform(-3.0, 0.0, shape)
        elif last == "D":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith("a2.b"):
            a = rng.uniform(1.0, 5.0, shape)
        elif name.endswith("conv.b"):
            a = 0.1 * rng.standard_normal(shape)
        elif name.endswith(".conv"):
            a = rng.standard_normal(shape) / math.sqrt(shape[1])
        elif name == "embed":
            a = rng.standard_normal(shape) / cfg["embedding"]["scale"]
        elif name == "loop.step":
            a = 0.1 * rng.standard_normal(shape)
        elif name == "loop.in":
            a = rng.standard_normal(shape) / math.sqrt(shape[1] / 2)
        elif name.endswith("router"):
            a = 2.0 * rng.standard_normal(shape) / math.sqrt(shape[1])
        else:
            a = rng.standard_normal(shape) / math.sqrt(shape[-1])
        w[name] = bf16_round(a)
    return w


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": None if not shared else {"ff": shared}}


def _gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _pair(heads, kv, dim, vdim, window, rot_dims, base, scale, sheads, svdim, state, groups, parts, taps, ls, rs):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window} if window else None,
            "rot": {"dims": rot_dims, "base": base} if rot_dims else None}
    right = {"heads": sheads, "vdim": svdim, "state": state, "groups": groups, "norm_groups": parts, "conv": taps}
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


# Two small models whose sizes share nothing that would hide a mix-up: keys and values of different
# widths, grouped heads, part of a head rotated, two and three experts a token, loops over other
# stretches of the layers, a layer without a feed-forward, a model without a loop.
SMALL = {
    "A": {"architecture": "Pozirax", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.0}, "logit_softcap": 20.0,
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [
              {"type": "parallel", "mixer": _pair(6, 2, 32, 16, 9, 16, 10000.0, 0.25, 6, 16, 16, 3, 3, 3, 0.7, 1.1), "mlp": _moe(5, 2, 48, 64)},
              {"type": "gla", "mixer": _gla(3, 16, 32, 8.0, 8), "mlp": _moe(7, 3, 32, 0)},
              {"type": "parallel", "mixer": _pair(4, 4, 16, 48, 70, 16, 500000.0, 0.3, 2, 32, 8, 1, 1, 2, 1.2, 0.5), "mlp": None},
              {"type": "gla", "mixer": _gla(2, 48, 16, 4.0, 24), "mlp": _moe(4, 1, 80, 32)},
          ]},
    "B": {"architecture": "Pozirax", "vocab": 157, "width": 80, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0}, "logit_softcap": 12.0,
          "layers": [
              {"type": "gla", "mixer": _gla(5, 8, 24, 2.0, 4), "mlp": _moe(3, 3, 40, 24)},
              {"type": "parallel", "mixer": _pair(2, 1, 64, 64, 130, 32, 100.0, 0.125, 5, 8, 24, 5, 5, 5, 1.0, 1.0), "mlp": _moe(9, 2, 16, 16)},
          ]},
}
