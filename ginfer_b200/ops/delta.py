"""Gated delta rule with a decay per key channel over per-request state
(``csrc/delta_rule.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream


def prepare(proj: torch.Tensor, b_off: int, a: torch.Tensor, conv_w: torch.Tensor,
            dt_bias: torch.Tensor, A_log: torch.Tensor, state: torch.Tensor, ctx, H: int, G: int,
            D: int, Vd: int, taps: int, conv_off: int):
    """``proj [T, >= 2 G D + H Vd + ...]``: the q | k | v projections first, the ``H`` beta columns
    at ``b_off``; ``a [T, H D]`` fp32: the decay's pre-activation.  Convolves (reading the slots'
    last inputs, and bringing them up to date afterwards), activates, normalises; returns fp32
    ``(q [T, G, D], k [T, G, D], v [T, H, Vd], g [T, H, D], beta [T, H])``."""
    _cuda(proj, a, conv_w, dt_bias, A_log, state)
    T = proj.shape[0]
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert a.dtype == torch.float32 and a.is_contiguous() and a.shape == (T, H * D)
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    ch = 2 * G * D + H * Vd
    assert conv_w.dtype == torch.float32 and conv_w.shape == (ch, taps) and conv_w.is_contiguous()
    dev = proj.device
    qn = torch.empty((T, G, D), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    v = torch.empty((T, H, Vd), dtype=torch.float32, device=dev)
    g = torch.empty((T, H, D), dtype=torch.float32, device=dev)
    beta = torch.empty((T, H), dtype=torch.float32, device=dev)
    f = _fn("delta_rule", "gf_delta_prepare",
            [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p] + [c_int] * 9 + [c_void_p] * 5 + [c_int, c_void_p],
            kernels=2)
    rc = f(_p(proj), proj.stride(0), int(b_off), _p(a), _p(conv_w), _p(dt_bias), _p(A_log),
           _p(state), _p(ctx.seq_of_token), _p(ctx.cu_seqlens_q), _p(ctx.slot_ids), T,
           ctx.num_seqs, H, G, D, Vd, taps, state.stride(0), int(conv_off), _p(qn), _p(kn), _p(v),
           _p(g), _p(beta), _code(proj.dtype), _stream())
    if rc == -3:
        raise ValueError("the delta-rule kernels need heads to be a multiple of kv heads and key "
                         f"sizes up to 256; got {H} heads, {G} kv heads, key size {D}")
    _ok(rc, "delta_prepare")
    return qn, kn, v, g, beta


def recurrence(qn, kn, v, g, beta, state: torch.Tensor, ctx) -> torch.Tensor:
    """Advance every request's state over its tokens of this step; returns ``o [T, H, Vd]`` fp32."""
    T, G, D = qn.shape
    H, Vd = v.shape[1], v.shape[2]
    o = torch.empty((T, H, Vd), dtype=torch.float32, device=qn.device)
    f = _fn("delta_rule", "gf_delta_recurrence",
            [c_void_p] * 8 + [c_int] * 6 + [c_void_p, c_void_p])
    rc = f(_p(qn), _p(kn), _p(v), _p(g), _p(beta), _p(state), _p(ctx.cu_seqlens_q),
           _p(ctx.slot_ids), ctx.num_seqs, H, G, D, Vd, state.stride(0), _p(o), _stream())
    if rc == -3:
        raise ValueError(f"the delta-rule recurrence takes key sizes up to 256, got {D}")
    _ok(rc, "delta_recurrence")
    return o


def output(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float,
           dtype: torch.dtype) -> torch.Tensor:
    """``o / rms(o) * w * sigmoid(gate)`` per head; ``[T, H Vd]`` in ``dtype``."""
    _cuda(o, gate, w)
    T, H, Vd = o.shape
    assert gate.stride(1) == 1 and gate.shape == (T, H * Vd) and gate.dtype == dtype
    assert w.dtype == torch.float32 and w.numel() == Vd
    out = torch.empty((T, H * Vd), dtype=dtype, device=o.device)
    f = _fn("delta_rule", "gf_delta_output",
            [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
             c_void_p])
    _ok(f(_p(o), _p(gate), gate.stride(0), _p(w), float(eps), _p(out), T, H, Vd, _code(dtype),
          _stream()), "delta_output")
    return out
