"""Latent attention: a token keeps one latent vector and one rotated key part for all heads.

``q = W_q h`` per head ``[D plain | R rotated]``; ``W_dkv h`` gives ``C + R`` channels: the first
``C``, RMS-normed with a plain weight, are the latent vector ``c``, the last ``R`` one rotated key
part shared by the heads.  A head's key is ``[W_uk c | rotated part]``, its value ``W_uv c``, the
score ``(q_plain . k_plain + q_rot . k_rot) * scale`` under a sliding window, softmax, and ``W_o``
on the joined heads.  Rotation: of the first ``rotary_dims`` channels of the rotated part, channel
``2i`` with ``2i + 1`` by the angle ``p * base^(-2i / rotary_dims)``.

Only ``c`` and the rotated part are cached (two planes of a paged cache).  The key up-projection
is folded into the query (``q_lat = W_uk^T q_plain``, a batched product over heads), the kernel
attends over ``[c | r]`` with values ``c``, and the value up-projection (a second batched product)
follows: keys and values of the heads are never formed.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops import latent
from .base import Mixer, PagedKVSpec, TensorSpec, register_mixer


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, nope_dim: int, rope_dim: int, v_dim: int,
                 kv_rank: int, scale: float, window: int = 0, rotary_dims: int | None = None,
                 rotary_base: float = 10000.0, latent_eps: float = 1e-6, prefix: str = "mix"):
        self.hidden_size, self.H = int(hidden_size), int(num_heads)
        self.D, self.R, self.Vd, self.C = int(nope_dim), int(rope_dim), int(v_dim), int(kv_rank)
        self.scale, self.window = float(scale), int(window)
        self.rot = int(self.R if rotary_dims is None else rotary_dims)
        if self.rot % 2 or self.rot > self.R:
            raise ValueError(f"{self.rot} rotated channels of {self.R}: must be even and fit")
        self.base, self.eps = float(rotary_base), float(latent_eps)
        self.prefix = prefix + "." if prefix else ""

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        H, D, R, Vd, C, W = self.H, self.D, self.R, self.Vd, self.C, self.hidden_size
        return [TensorSpec(self._n("q"), (H * (D + R), W)),
                TensorSpec(self._n("dkv"), (C + R, W)),
                TensorSpec(self._n("dkv.norm"), (C,), "f32"),
                TensorSpec(self._n("uk"), (H * D, C)),
                TensorSpec(self._n("uv"), (H * Vd, C)),
                TensorSpec(self._n("o"), (W, H * Vd))]

    def load(self, tensors, dtype, device):
        H, D, Vd, C = self.H, self.D, self.Vd, self.C
        self.q_dkv = ops.Linear(torch.cat([tensors[self._n("q")], tensors[self._n("dkv")]], dim=0))
        self.latent_w = tensors[self._n("dkv.norm")].float().contiguous()
        self.uk = tensors[self._n("uk")].view(H, D, C)                     # q_lat = q_plain @ uk[h]
        self.uv_t = tensors[self._n("uv")].view(H, Vd, C).transpose(1, 2)  # values = o_lat @ uv[h]^T
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        i = np.arange(self.rot // 2, dtype=np.float64)
        freq = np.power(np.float64(self.base), -2.0 * i / self.rot).astype(np.float32)
        self.freq = torch.from_numpy(freq).to(device)

    def cache_spec(self):
        return PagedKVSpec(1, self.C, self.window, planes=((1, self.C), (1, self.R)))

    def forward(self, x, ctx, cache):
        H, D, R, C = self.H, self.D, self.R, self.C
        T = x.shape[0]
        qd = self.q_dkv(x)                                        # [T, H (D + R) + C + R]
        c_pages, r_pages = cache.pages
        q_rot = latent.prepare(qd, H, D, R, C, self.rot, self.freq, self.latent_w, self.eps,
                               ctx.positions, cache.slot_mapping if cache.write else None,
                               c_pages, r_pages)
        q_plain = qd[:, :H * (D + R)].unflatten(1, (H, D + R))[:, :, :D].transpose(0, 1)
        q_lat = ops.bmm_f32_out(q_plain, self.uk)                 # [H, T, C] fp32
        o_lat = latent.attention(q_lat, q_rot, c_pages, r_pages, cache.block_table, ctx,
                                 cache.window, self.scale, cache.page_size)
        o = torch.bmm(o_lat, self.uv_t)                           # [H, T, Vd]
        return self.out(o.transpose(0, 1).reshape(T, H * self.Vd))


register_mixer("latent_attention", LatentAttention)
