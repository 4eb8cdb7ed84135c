"""Additions to the residual stream that are not a sublayer's output.

:class:`TokenSideInput` ends a layer: every layer reads its own slice of a second token table,
gates it by the stream, projects it back to the width and adds its RMS norm.
:class:`LoopEntry` starts a pass of a loop over some layers: the embedding output is added again
from the second pass on, and a learned vector per pass.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import prenorm
from .base import StreamInput, TensorSpec, register_stream_input


def _norm_args(then):
    fused = then.fused() if then is not None else None
    if fused is None:
        return {}
    kind, w, b, eps = fused
    return dict(norm=kind, norm_weight=w, norm_bias=b, norm_eps=eps)


class TokenSideInput(StreamInput):
    """``e = table[token, offset : offset + dim]``; ``g = gelu_tanh(W_gate x) * e``;
    ``y = W_proj g``; ``x' = x + mult * y / sqrt(mean(y^2) + eps) * w``.  ``table`` (``[vocab,
    total]``) is a tensor of the whole model; gate, projection and norm weight are the layer's."""

    wants_act = True

    def __init__(self, hidden_size: int, vocab_size: int, dim: int, offset: int, total: int,
                 eps: float, table_name: str = "/side.embed", prefix: str = "side"):
        self.H, self.V, self.dim = int(hidden_size), int(vocab_size), int(dim)
        self.offset, self.total, self.eps = int(offset), int(total), float(eps)
        if not (0 <= self.offset and self.offset + self.dim <= self.total):
            raise ValueError(f"columns {self.offset}..{self.offset + self.dim} lie outside a table "
                             f"of {self.total}")
        self.table_name = table_name
        self.prefix = prefix + "." if prefix else ""

    def tensor_specs(self):
        p = self.prefix
        return [TensorSpec(self.table_name, (self.V, self.total), "embedding"),
                TensorSpec(p + "gate", (self.dim, self.H)),
                TensorSpec(p + "proj", (self.H, self.dim)),
                TensorSpec(p + "norm", (self.H,), "norm32")]

    def load(self, tensors, dtype, device):
        p = self.prefix
        self.table = tensors[self.table_name]
        self.gate = ops.Linear(tensors[p + "gate"], None, out_dtype=torch.float32)
        self.proj = ops.Linear(tensors[p + "proj"], None, out_dtype=torch.float32)
        self.weight = tensors[p + "norm"].float().contiguous()

    def forward(self, x, act, ctx, mult, then=None):
        if act is None:
            act = x if self.table.dtype == torch.float32 else x.to(self.table.dtype)
        g = prenorm.token_gate(self.gate(act), ctx.token_ids, self.table, self.offset)
        x, _, n = prenorm.stream_update(x, ctx.dtype, y=self.proj(g), scale=self.weight, mult=mult,
                                        y_rms_eps=self.eps, **_norm_args(then))
        return x, n


class LoopEntry(StreamInput):
    """Entry ``n`` of a loop of ``times`` passes: ``x' = x + (embedding output if n > 0) +
    step[n]`` with ``step`` a tensor ``[times, width]`` of the whole model."""

    def __init__(self, hidden_size: int, times: int, name: str = "/loop.step"):
        self.H, self.times, self.name = int(hidden_size), int(times), name

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.times, self.H), "f32")]

    def load(self, tensors, dtype, device):
        self.step = tensors[self.name].float().contiguous()

    def enter(self, x, ctx, embedding_output, index):
        if not (0 <= index < self.times):
            raise ValueError(f"pass {index} of a loop of {self.times}")
        if x.dtype != torch.float32:
            x = x.float()
        emb = None
        if index > 0:
            emb = embedding_output if embedding_output.dtype == torch.float32 \
                else embedding_output.float()
        return prenorm.stream_update(x, ctx.dtype, add_full=emb, add_row=self.step[index])[0]


register_stream_input("token_side", TokenSideInput)
register_stream_input("loop_entry", LoopEntry)
