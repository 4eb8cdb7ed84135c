"""Gated delta rule with one decay per head and key channel.

``q = W_q h``, ``k = W_k h`` (``G`` kv heads of ``D``), ``v = W_v h`` (``H`` heads of ``Vd``); head
``n`` reads q/k head ``n // (H / G)``.  Each passes a short causal convolution over time per
channel and SiLU; q and k become unit vectors per head (q also times ``D^-1/2``).  ``beta =
sigmoid(W_b h)`` per head; decay ``g = exp(-exp(A_log_n) * softplus(W_a2 (W_a1 h) + dt_bias))``
per head and key channel.  Per head, token after token: ``S <- diag(g) S``; ``u = beta (v - S^T
k)``; ``S <- S + k u^T``; ``o = S^T q``.  ``o`` is RMS-normed per head (plain weight shared by the
heads), gated by ``sigmoid(W_g2 (W_g1 h))`` and projected by ``W_o``.

State per request (one fp32 row of a slot): ``S [H, D, Vd]``, then the last ``taps - 1`` inputs of
the convolutions ``[taps - 1, 2 G D + H Vd]``.  Decays, gates of the recurrence, unit norms and the
state are fp32 in both paths.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import delta
from .base import Mixer, StateSpec, TensorSpec, register_mixer


class ChannelDelta(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 v_dim: int, conv_taps: int, out_norm_eps: float = 1e-6,
                 decay_rank: int = -1, gate_rank: int = -1, prefix: str = "mix"):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.D, self.Vd, self.taps = int(key_dim), int(v_dim), int(conv_taps)
        self.eps = float(out_norm_eps)
        self.decay_rank, self.gate_rank = int(decay_rank), int(gate_rank)   # -1: the file's
        self.prefix = prefix + "." if prefix else ""
        self.channels = 2 * self.G * self.D + self.H * self.Vd
        self.state_floats = self.H * self.D * self.Vd
        self.conv_off = self.state_floats

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        H, G, D, Vd, W, t = self.H, self.G, self.D, self.Vd, self.hidden_size, self.taps
        ra, rg = self.decay_rank, self.gate_rank
        return [TensorSpec(self._n("q"), (G * D, W)), TensorSpec(self._n("q.conv"), (G * D, t), "f32"),
                TensorSpec(self._n("k"), (G * D, W)), TensorSpec(self._n("k.conv"), (G * D, t), "f32"),
                TensorSpec(self._n("v"), (H * Vd, W)),
                TensorSpec(self._n("v.conv"), (H * Vd, t), "f32"),
                TensorSpec(self._n("b"), (H, W)),
                TensorSpec(self._n("A_log"), (H,), "f32"),
                TensorSpec(self._n("norm"), (Vd,), "f32"),
                TensorSpec(self._n("a1"), (ra, W)), TensorSpec(self._n("a2"), (H * D, ra)),
                TensorSpec(self._n("dt_bias"), (H * D,), "f32"),
                TensorSpec(self._n("g1"), (rg, W)), TensorSpec(self._n("g2"), (H * Vd, rg)),
                TensorSpec(self._n("o"), (W, H * Vd))]

    def load(self, tensors, dtype, device):
        t = {k: tensors[self._n(k)] for k in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o",
                                              "q.conv", "k.conv", "v.conv", "A_log", "norm",
                                              "dt_bias")}
        ra, rg = t["a1"].shape[0], t["g1"].shape[0]
        if t["a2"].shape[1] != ra or t["g2"].shape[1] != rg:
            raise ValueError(f"{self.prefix}a1/a2 or g1/g2 disagree on their inner size")
        # one product for everything that reads h: q | k | v | a1 | g1 | b, rows padded to 8
        rows = [t["q"], t["k"], t["v"], t["a1"], t["g1"], t["b"]]
        n = sum(r.shape[0] for r in rows)
        pad = -n % 8
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=device))
        self.first = ops.Linear(torch.cat(rows, dim=0))
        self.a1_off = self.channels
        self.g1_off = self.a1_off + ra
        self.b_off = self.g1_off + rg
        self.ra, self.rg = ra, rg
        self.decay = ops.Linear(t["a2"], None, out_dtype=torch.float32)
        self.gate = ops.Linear(t["g2"])
        self.out = ops.Linear(t["o"], None, out_dtype=torch.float32)
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).float().contiguous()
        self.A_log = t["A_log"].float().contiguous()
        self.dt_bias = t["dt_bias"].float().contiguous()
        self.norm_w = t["norm"].float().contiguous()

    def cache_spec(self):
        return StateSpec((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, ctx, cache):
        H, G, D, Vd = self.H, self.G, self.D, self.Vd
        state = cache.state
        p = self.first(x)                                         # [T, q | k | v | a1 | g1 | b]
        a = self.decay(p[:, self.a1_off:self.a1_off + self.ra].contiguous())     # fp32 [T, H D]
        gate = self.gate(p[:, self.g1_off:self.g1_off + self.rg].contiguous())   # [T, H Vd]
        qn, kn, v, g, beta = delta.prepare(p, self.b_off, a, self.conv_w, self.dt_bias,
                                           self.A_log, state, ctx, H, G, D, Vd, self.taps,
                                           self.conv_off)
        o = delta.recurrence(qn, kn, v, g, beta, state, ctx)
        return self.out(delta.output(o, gate, self.norm_w, self.eps, ctx.dtype))


register_mixer("channel_delta", ChannelDelta)
