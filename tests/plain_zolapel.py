"""A plain, slow Zolapel in float64 over whole sequences: the oracle of the tests.

One function per mechanism, written from the design's equations; it shares no code with the
engine.  ``rnd`` (identity by default) is applied where the bfloat16 path stores an activation, so
that the same functions give the bfloat16-stored model when handed a rounding function.

Notation: ``W`` width, ``H`` query heads, ``G`` key/value heads, ``D`` head size, ``p`` a token's
position in its sequence (from 0).

* layer: ``x += m * ls1 * mixer(LN1(x))``; ``x += m * ls2 * ff(LN2(x))`` (if the layer has a
  feed-forward); then the token's side input (if the model has one).
* LN: ``(x - mean) / sqrt(var + eps) * w + b`` (population variance).
* attention: ``q = W_q h``, ``k = W_k h``, values ``= k`` as projected; q and k RMS-normed per
  head (one weight vector of size D for all heads), then rotated: pair ``(2i, 2i+1)`` of the first
  ``dims`` channels by ``p * f_i``; ``score = q.k * scale`` over keys ``j`` with
  ``0 <= p - j < window``; softmax; head ``h``'s output times ``sigmoid(W_g h)_h``; ``W_o``.
* feed-forward: ``s = sigmoid(W_r h)``; the ``top`` largest; ``sum_e W_down relu(W_up (s_e h))^2``.
* side input of layer ``i``: ``e = E_side[token, i*d:(i+1)*d]``; ``g = gelu_tanh(W_gate x) * e``;
  ``y = W_proj g``; ``x += m * y / rms(y) * w``.
* loop: layers ``start..stop-1`` run ``times`` times; before pass ``t > 0`` the embedding output is
  added to ``x``; before every pass ``step[t]`` is added.
"""
from __future__ import annotations

import math

import numpy as np


def ident(a):
    return a


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotary_frequencies(dims: int, base: float, scaling=None):
    """``f_i = base^(-2i/dims)``; with ``scaling = {factor, low, high, original}`` the long
    wavelengths are stretched: kept below ``original/high``, divided by ``factor`` above
    ``original/low``, blended linearly in ``original / wavelength`` in between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / hi:
                pass
            elif wave > orig / lo:
                f = f / fac
            else:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    # positions and angles are 32-bit quantities in the engine: the frequency is rounded once
    return np.asarray(out, dtype=np.float32).astype(np.float64)


def rotate_pairs(x, positions, freqs):
    """``x [T, heads, D]``: channels ``(2i, 2i+1)`` for ``i < len(freqs)`` rotated by
    ``positions[t] * freqs[i]``; the rest pass."""
    out = x.copy()
    n = len(freqs)
    if n == 0:
        return out
    ang = (positions.astype(np.float32)[:, None] * freqs.astype(np.float32)[None, :]).astype(np.float64)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


def visible(T: int, window: int):
    """``[T, T]`` booleans: query ``i`` sees key ``j`` iff ``0 <= i - j < window`` (no window:
    every earlier key and itself)."""
    d = np.arange(T)[:, None] - np.arange(T)[None, :]
    return (d >= 0) & ((d < window) if window > 0 else True)


def attention(h, t, m, eps, rnd=ident):
    """``h [T, W]`` -> ``[T, W]``; ``t``: the mixer's tensors by short name; ``m``: its sizes."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = rnd(h @ t["q"].T).reshape(T, H, D)
    k = rnd(h @ t["k"].T).reshape(T, G, D)
    v = k.copy()                                        # the values are the keys as projected
    gate = sigmoid(h @ t["g"].T)                        # [T, H]
    pos = np.arange(T)
    rot = m.get("rot")
    freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else np.zeros(0)
    q = rnd(rotate_pairs(rms_norm(q, t["q.norm"], eps), pos, freqs))
    k = rnd(rotate_pairs(rms_norm(k, t["k.norm"], eps), pos, freqs))
    window = m["mask"]["size"] if m.get("mask") else 0
    out = np.zeros((T, H, D))
    see = visible(T, window)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = np.where(see, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(-1, keepdims=True)
        out[:, hd] = p @ v[:, g]
    out = rnd(rnd(out) * gate[:, :, None])
    return out.reshape(T, H * D) @ t["o"].T


def router(h, w_router, top: int):
    """-> ``(experts [T, top], weights [T, top])``: sigmoid scores, the ``top`` largest (lowest
    index among equals), the scores themselves as weights."""
    s = sigmoid(h @ w_router.T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def expert(h, up, down, rnd=ident):
    a = np.maximum(rnd(h @ up.T), 0.0) ** 2
    return rnd(a) @ down.T


def routed_ff(h, t, mlp, rnd=ident):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wgt = router(h, t["router"], top)
    out = np.zeros((h.shape[0], t["e0.down"].shape[0]))
    for n in range(h.shape[0]):
        for e, w in zip(idx[n], wgt[n]):
            out[n] += expert(rnd(w * h[n:n + 1]), t[f"e{e}.up"], t[f"e{e}.down"], rnd)[0]
    return out


def side_input(x, tokens, side_embed, layer: int, dim: int, t, m: float, eps, rnd=ident):
    e = side_embed[tokens, layer * dim:(layer + 1) * dim]
    g = rnd(gelu_tanh(rnd(rnd(x) @ t["gate"].T)) * e)
    y = g @ t["proj"].T
    return x + m * rms_norm(y, t["norm"], eps)


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x, tokens, i: int, tensors, cfg, rnd=ident):
    L = cfg["layers"][i]
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    p = f"l{i}."
    h = rnd(layer_norm(x, tensors[p + "norm1"], tensors[p + "norm1.b"], eps))
    x = x + m * tensors[p + "ls1"] * attention(h, sub(tensors, p + "mix."), L["mixer"], eps, rnd)
    if L.get("mlp") is not None:
        h = rnd(layer_norm(x, tensors[p + "norm2"], tensors[p + "norm2.b"], eps))
        x = x + m * tensors[p + "ls2"] * routed_ff(h, sub(tensors, p + "mlp."), L["mlp"], rnd)
    side = cfg.get("token_side")
    if side:
        x = side_input(x, tokens, tensors["side.embed"], i, side["dim"], sub(tensors, p + "side."),
                       m, eps, rnd)
    return x


def run_order(cfg):
    """The runs of a step as ``(layer, pass or None, first of its pass)``."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, None, False) for i in range(a)]
    for t in range(times):
        out += [(i, t, i == a) for i in range(a, b)]
    return out + [(i, None, False) for i in range(b, n)]


def forward(tokens, tensors, cfg, rnd=ident, want_layers: bool = False):
    """``tokens [T]`` of one sequence from position 0 -> logits ``[T, vocab]`` (and the stream
    after every run)."""
    tokens = np.asarray(tokens)
    x = tensors["embed"][tokens].astype(np.float64)
    emb = x.copy()
    streams = []
    for i, t, first in run_order(cfg):
        if first:
            if t > 0:
                x = x + emb
            x = x + tensors["loop.step"][t]
        x = layer(x, tokens, i, tensors, cfg, rnd)
        streams.append(x.copy())
    eps = cfg["norm"]["eps"]
    h = rnd(layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps))
    logits = h @ tensors["embed"].T
    return (logits, streams) if want_layers else logits


def bf16_round(a):
    """Round a float64 array to the nearest bfloat16 value (ties to even)."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)
