"""A plain, slow restatement of the Fegidra decoder in NumPy float64, one function per
mechanism, written from the design's equations and sharing no code with the package.

Notation: X is [T, width] for one sequence of T tokens at positions 0 .. T-1; matrices are
[out, in] and applied as X @ W.T; `cfg` is the config.json dict (delta-rule mixers carry
their `decay_rank`), `w` maps tensor names to arrays.
"""

from __future__ import annotations

import math

import numpy as np

KEY_EPS = 1e-6                      # under the root of a key's length
DECAY_SCALE = math.exp(-0.5)        # the decay is exp(-DECAY_SCALE * sigmoid(.))


def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def over_rms(x, eps):
    """Every row of x divided by its root mean square, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return over_rms(x, eps) * weight


def short_conv_residual(h, kernel):
    """h_t + sum_j kernel[:, j] * h_(t - taps + 1 + j), zeros before position 0."""
    T, taps = h.shape[0], kernel.shape[1]
    out = h.copy()
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += kernel[:, j] * h[src]
    return out


def delta_rule_states(r, k, v, decay, rate, state=None):
    """The recurrence of one head.  r, k, v, decay, rate: [T, D].  Returns the outputs [T, D]
    and the state [D, D] (key channel, value channel) after the last token."""
    T, D = k.shape
    S = np.zeros((D, D)) if state is None else state.copy()
    out = np.zeros((T, D))
    for t in range(T):
        u = k[t] / math.sqrt(float(np.sum(k[t] * k[t])) + KEY_EPS)
        seen = u @ S                                              # u^T S_(t-1), a row over value channels
        S = decay[t][:, None] * S - np.outer(rate[t] * u, seen) + np.outer(k[t], v[t])
        out[t] = S.T @ r[t]
    return out, S


def general_delta_mixer(h, w, p, heads, dim, eps):
    T = h.shape[0]
    r, k, v = (h @ w[p + n].T for n in ("r", "k", "v"))
    inner = np.tanh(h @ w[p + "w1"].T)
    decay = np.exp(-DECAY_SCALE * sigmoid(inner @ w[p + "w2"].T + w[p + "w0"]))
    rate = sigmoid(h @ w[p + "a"].T + w[p + "a.b"])
    o = np.zeros((T, heads * dim))
    for a in range(heads):
        s = slice(a * dim, (a + 1) * dim)
        o[:, s] = over_rms(delta_rule_states(r[:, s], k[:, s], v[:, s], decay[:, s], rate[:, s])[0], eps)
    return (o * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def rotate(x, positions, dims, base):
    """x: [T, heads, dim]; the first `dims` dimensions of each head turn by position * base^(-2i/dims),
    dimension i paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    lo, hi = x[..., :half], x[..., half:dims]
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


def visible(T, chunk):
    """[T, T] booleans: position i sees j <= i of its own chunk (chunk 0: no chunks)."""
    i = np.arange(T)
    ok = i[None, :] <= i[:, None]
    if chunk > 0:
        ok &= (i[None, :] // chunk) == (i[:, None] // chunk)
    return ok


def attention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    DV = m.get("vdim", D)
    q = rms_norm(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.norm"], eps).reshape(T, H, D)
    k = rms_norm(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.norm"], eps).reshape(T, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, DV)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, range(T), rot["dims"], rot["base"]), rotate(k, range(T), rot["dims"], rot["base"])
    scale = m.get("scale", 1.0 / math.sqrt(D))
    ok = visible(T, m["mask"]["size"] if m.get("mask") else 0)
    out = np.zeros((T, H, DV))
    for a in range(H):
        g = a // (H // G)
        s = np.where(ok, (q[:, a] @ k[:, g].T) * scale, -np.inf)
        e = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, a] = (e / e.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * DV) @ w[p + "o"].T


def polynorm(z, coef, eps):
    a, b, c, e = (float(x) for x in coef)
    return a * over_rms(z, eps) + b * over_rms(z * z, eps) + c * over_rms(z * z * z, eps) + e


def feed_forward(h, w, p, eps):
    return polynorm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def layer(x, cfg, w, i):
    L, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    if cfg.get("canon"):
        h = short_conv_residual(h, w[p + "canon1"])
    if L["type"] == "general_delta":
        mixed = general_delta_mixer(h, w, p + "mix.", L["mixer"]["heads"], L["mixer"]["dim"], eps)
    else:
        mixed = attention_mixer(h, w, p + "mix.", L["mixer"], eps)
    if L.get("mlp") is not None:
        mixed = mixed + feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", eps)
    return x + mixed


def logits(cfg, weights, tokens):
    """[T, vocab] float64: the scores after every token of one sequence."""
    w = {n: f64(a) for n, a in weights.items()}
    x = w["embed"][np.asarray(tokens, dtype=np.int64)]
    for i in range(len(cfg["layers"])):
        x = layer(x, cfg, w, i)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def generate(cfg, weights, prompt, n):
    """Greedy continuation (the lowest id among equal scores), recomputing the whole sequence a token."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(logits(cfg, weights, seq)[-1])))
    return seq[len(prompt):]


# ------------------------------------------------------------------------------ test models

def bf16_round(a):
    """float32 values rounded to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def make_weights(cfg, seed, std=None):
    """Seeded float32 weights by tensor name, every value a bfloat16 number, so that a folder
    stored in bfloat16 and the float64 arithmetic here start from the same numbers.  Spreads
    are chosen so that no mechanism sits in its linear range: projections of spread about 1
    a row, gates and decays away from 1/2, norm weights around 1."""
    rng = np.random.default_rng(seed)
    E = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return bf16_round(rng.standard_normal((rows, cols)) * (gain / math.sqrt(cols) if std is None else std))

    def vec(n, centre=1.0, spread=0.3):
        return bf16_round(centre + spread * rng.uniform(-1, 1, n))

    w = {"embed": bf16_round(rng.standard_normal((cfg["vocab"], E))), "final.norm": vec(E), "head": mat(cfg["vocab"], E, 2.0)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = vec(E)
        if cfg.get("canon"):
            w[p + "canon1"] = bf16_round(rng.standard_normal((E, cfg["canon"]["taps"])) * 0.4)
        if L["type"] == "general_delta":
            hd, rank = m["heads"] * m["dim"], m["decay_rank"]
            for n in ("r", "k", "v", "g", "a"):
                w[p + "mix." + n] = mat(hd, E, 1.5)
            w[p + "mix.a.b"] = vec(hd, 0.0, 1.0)
            w[p + "mix.w1"] = mat(rank, E, 1.5)
            w[p + "mix.w2"] = mat(hd, rank, 2.0)
            w[p + "mix.w0"] = vec(hd, 0.0, 1.5)
            w[p + "mix.norm"] = vec(hd)
            w[p + "mix.o"] = mat(E, hd)
        else:
            H, G, D = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
            DV = m.get("vdim", D)
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * D, E, 1.5), mat(G * D, E, 1.5), mat(G * DV, E, 1.5)
            w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"] = vec(H * D, 0.0, 0.5), vec(G * D, 0.0, 0.5), vec(G * DV, 0.0, 0.5)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(H * D, 1.0, 0.5), vec(G * D, 1.0, 0.5)
            w[p + "mix.o"] = mat(E, H * DV)
        if L.get("mlp") is not None:
            w[p + "norm2"] = vec(E)
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(L["mlp"]["ff"], E, 1.5), mat(E, L["mlp"]["ff"])
            w[p + "mlp.act"] = bf16_round(np.array([0.9, 0.5, 0.25, -0.1]) + 0.1 * rng.uniform(-1, 1, 4))
    return w


def delta_layer(heads, dim, rank, ff):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def attention_layer(heads, kv_heads, dim, vdim, chunk, rot_dims, base, scale, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                      "rot": {"dims": rot_dims, "base": base}, "scale": scale},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


# Two small models that differ in every size, in the order of their layers and in what is equal to what.
# P: delta first; heads 4 on 2 kv heads; keys 32 wide, values 16, 8 rotated dimensions; chunks of 40
#    (no multiple or divisor of the cache's pages of 64); 3 taps; feed-forward wider than the model.
SMALL_P = {"architecture": "Fegidra", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "layers": [
    delta_layer(2, 16, 8, 96), attention_layer(4, 2, 32, 16, 40, 8, 10000.0, 0.2, 96), delta_layer(2, 16, 8, 96),
    attention_layer(4, 2, 32, 16, 40, 8, 10000.0, 0.2, 96)]}
# Q: attention first; one kv head; keys 16 wide rotated whole, values 48 (wider than keys); chunks of 64
#    (exactly a page); 5 taps; a layer without feed-forward; delta heads of 24 (not a power of two); another eps.
SMALL_Q = {"architecture": "Fegidra", "vocab": 160, "width": 48, "norm": {"eps": 1e-6}, "canon": {"taps": 5}, "layers": [
    attention_layer(3, 1, 16, 48, 64, 16, 500.0, 0.35, 80), delta_layer(3, 24, 5, None), attention_layer(3, 3, 16, 48, 64, 16, 500.0, 0.35, 40)]}
SMALL = {"P": SMALL_P, "Q": SMALL_Q}
