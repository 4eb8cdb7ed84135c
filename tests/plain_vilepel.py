"""A plain, slow Vilepel: every mechanism of the design as one function over a whole sequence,
in float64 on the CPU, written from the design's equations.  It shares no code with the engine
and is the oracle of the Vilepel tests.

Notation: ``h [T, width]`` is a sublayer's input (the residual stream itself), ``W`` a mapping
from tensor names (relative to the layer, as the weight file has them) to float64 tensors.
Linear weights are ``[out, in]``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def rotate_pairs(x, positions, base, dims):
    """Rotate the first ``dims`` channels of ``x [T, ..., D]``: channel ``2i`` with ``2i + 1`` by
    the angle ``p * base^(-2i/dims)``; the other channels pass."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F64)[:, None] * f[None, :]                  # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def gelu_sigmoid_glu(g, u, limit):
    """``min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)``."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, gate, up, down, limit):
    return gelu_sigmoid_glu(h @ gate.T, h @ up.T, limit) @ down.T


def routed_ff(h, W, m):
    """Mixture of experts: softmax over all experts, the ``top`` largest chosen, their scores as
    weights without renormalisation."""
    E, top = m["router"]["experts"], m["router"]["top"]
    limit = m["expert"]["limit"]
    s = torch.softmax(h @ W["mlp.router"].T, dim=-1)             # [T, E]
    _, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in idx[t].tolist():
            y = dense_ff(h[t:t + 1], W[f"mlp.e{e}.gate"], W[f"mlp.e{e}.up"], W[f"mlp.e{e}.down"],
                         limit)
            out[t] += s[t, e] * y[0]
    return out


def feed_forward(h, W, m):
    if m["kind"] == "dense":
        return dense_ff(h, W["mlp.gate"], W["mlp.up"], W["mlp.down"], m["limit"])
    if m["kind"] == "moe":
        return routed_ff(h, W, m)
    raise ValueError(m["kind"])


# ----------------------------------------------------------------------------- latent attention
def latent_attention(h, W, m, eps):
    """Queries per head ``[dim | rot_dim]``; keys and values rebuilt from one latent vector a
    token plus one rotated key part shared by the heads; sliding window; softmax."""
    T = h.shape[0]
    H, D, R, Vd, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W["mix.q"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    dkv = h @ W["mix.dkv"].T
    c = norm_plain(dkv[:, :C], W["mix.dkv.norm"], eps)            # [T, C]
    k_rot = dkv[:, C:]                                            # [T, R]
    rot = m["rot"]
    q_rot = rotate_pairs(q_rot, pos, rot["base"], rot["dims"])
    k_rot = rotate_pairs(k_rot, pos, rot["base"], rot["dims"])
    k_plain = (c @ W["mix.uk"].T).reshape(T, H, D)
    v = (c @ W["mix.uv"].T).reshape(T, H, Vd)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * Vd)
    return o @ W["mix.o"].T


# ----------------------------------------------------------------------------- channel delta
def short_conv_silu(x, w):
    """Causal convolution over time per channel (``w [channels, taps]``, last tap = the current
    token, zeros before the start), then SiLU."""
    T, taps = x.shape[0], w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j][None, :]
    return y * torch.sigmoid(y)


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def channel_delta(h, W, m, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ W["mix.q"].T, W["mix.q.conv"]).reshape(T, G, D)
    k = short_conv_silu(h @ W["mix.k"].T, W["mix.k.conv"]).reshape(T, G, D)
    v = short_conv_silu(h @ W["mix.v"].T, W["mix.v.conv"]).reshape(T, H, Vd)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ W["mix.b"].T)                        # [T, H]
    a = (h @ W["mix.a1"].T) @ W["mix.a2"].T + W["mix.dt_bias"]    # [T, H * D]
    rate = torch.exp(W["mix.A_log"]).reshape(1, H, 1)
    g = torch.exp(-rate * torch.nn.functional.softplus(a).reshape(T, H, D))
    out = torch.zeros(T, H, Vd, dtype=h.dtype)
    per = H // G
    for n in range(H):
        S = torch.zeros(D, Vd, dtype=h.dtype)
        qn, kn = q[:, n // per], k[:, n // per]
        for t in range(T):
            S = g[t, n][:, None] * S
            u = beta[t, n] * (v[t, n] - S.T @ kn[t])
            S = S + torch.outer(kn[t], u)
            out[t, n] = S.T @ qn[t]
    gate = torch.sigmoid((h @ W["mix.g1"].T) @ W["mix.g2"].T).reshape(T, H, Vd)
    o = unit_rms(out, eps) * W["mix.norm"] * gate
    return o.reshape(T, H * Vd) @ W["mix.o"].T


MIXERS = {"latent_attention": latent_attention, "channel_delta": channel_delta}


# ----------------------------------------------------------------------------- the model
def layer_tensors(weights, i):
    pre = f"l{i}."
    return {k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}


def forward(config, weights, tokens, want_layers=False):
    """Logits ``[T, vocab]`` of a whole sequence (and the residual stream after every layer
    run).  ``weights``: name -> tensor (any float dtype; used as float64)."""
    w64 = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w64["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    stream = []
    for i, layer in enumerate(config["layers"]):
        W = layer_tensors(w64, layer.get("weights_of", i))
        x = x + norm_around_zero(MIXERS[layer["type"]](x, W, layer["mixer"], eps), W["norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_around_zero(feed_forward(x, W, layer["mlp"]), W["norm2"], eps)
        stream.append(x.clone())
    logits = norm_around_zero(x, w64["final.norm"], eps) @ w64["head"].T
    return (logits, torch.stack(stream)) if want_layers else logits
