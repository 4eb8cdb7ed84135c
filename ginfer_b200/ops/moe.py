"""Routed feed-forward: routing, the plan of a step's (token, expert) pairs and the grouped
products, all on the device (``csrc/moe.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream, load_library

_tile_rows: dict = {}


def tile_rows(tensor_cores) -> int:
    """Rows of a tile of the plain kernel (``False``), of the ``mma.sync`` kernel (``True``), of
    the tcgen05 kernel (``"tcgen05"``) or of the kernel for a handful of pairs (``"few"``)."""
    if tensor_cores not in _tile_rows:
        if tensor_cores == "tcgen05":
            _tile_rows[tensor_cores] = int(load_library("gemm_prefill").gf_gemm_grouped_tile_rows())
        elif tensor_cores == "few":
            _tile_rows[tensor_cores] = int(load_library("moe").gf_moe_tile_rows(2))
        else:
            _tile_rows[tensor_cores] = int(load_library("moe").gf_moe_tile_rows(int(tensor_cores)))
    return _tile_rows[tensor_cores]


# From this many (token, expert) pairs on, the grouped products of the bf16 path run on the
# persistent tcgen05 kernel (csrc/gemm_prefill.cu, tiles of 128 rows x 256 columns, the rows brought
# into sorted order first); below it on the mma.sync kernel with its tiles of 64 rows, which is
# bound by the experts' weight bytes there.
TCGEN05_MIN_PAIRS = 1024
# Up to this many pairs (decode steps of few requests) the products run on the kernel that streams
# an expert's rows once for up to eight pairs; it keeps the rows in shared memory, which bounds the
# reduction size.
FEW_MAX_PAIRS = 16
FEW_MAX_K = 4096


def kernel_for(x: torch.Tensor, pairs: int, reductions, widths) -> object:
    """Which grouped-product kernel serves activations ``x`` with these reduction sizes and output
    widths: ``"tcgen05"``, ``"few"`` (a handful of pairs), ``True`` (``mma.sync``) or ``False``
    (plain)."""
    if not (on_tensor_cores(x.dtype, *reductions) and x.stride(0) % 8 == 0):
        return False
    if pairs >= TCGEN05_MIN_PAIRS and all(n % 8 == 0 for n in widths):
        return "tcgen05"
    if pairs <= FEW_MAX_PAIRS and max(reductions) <= FEW_MAX_K and all(n % 2 == 0 for n in widths):
        return "few"
    return True


def on_tensor_cores(dtype: torch.dtype, *reductions: int) -> bool:
    """Whether the grouped products of this dtype and these reduction sizes run on the tensor-core
    kernel (bf16, sizes that 16-byte copies can fetch) or on the plain one."""
    return dtype == torch.bfloat16 and all(k % 8 == 0 for k in reductions)


def route(logits: torch.Tensor, top: int, renormalize: bool, score: str = "softmax"):
    """fp32 ``logits [T, E]`` -> ``(experts [T, top] int32, weights [T, top] fp32)``: scores =
    softmax over all experts (``score="softmax"``) or each logit's sigmoid (``"sigmoid"``), the
    ``top`` largest, lowest index among equals."""
    if score not in ("softmax", "sigmoid"):
        raise ValueError(f"router scores are 'softmax' or 'sigmoid', not {score!r}")
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    T, E = logits.shape
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wgt = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    f = _fn("moe", "gf_moe_route", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p])
    rc = f(_p(logits), T, E, int(top), int(bool(renormalize)), int(score == "sigmoid"), _p(idx),
           _p(wgt), _stream())
    if rc == -3:
        raise ValueError(f"the router kernel takes up to 256 experts and 32 choices, got {E}, {top}")
    _ok(rc, "moe_route")
    return idx, wgt


class Plan:
    """Where every (token, choice) pair sits once the pairs are sorted by expert."""

    def __init__(self, idx: torch.Tensor, num_experts: int, tensor_cores=False):
        T, top = idx.shape
        self.tcgen05 = tensor_cores == "tcgen05"
        self.few = tensor_cores == "few"
        self.tensor_cores = bool(tensor_cores)
        rows = tile_rows(tensor_cores if isinstance(tensor_cores, str) else self.tensor_cores)
        P = T * top
        dev = idx.device
        self.pairs, self.top, self.num_experts = P, top, num_experts
        # every tile holds at least one pair, and every expert's last tile may be partly empty
        self.max_tiles = min(-(-P // rows) + num_experts, P)
        ints = torch.empty(num_experts + 1 + 2 * P + 2 * self.max_tiles + 1, dtype=torch.int32,
                           device=dev)
        at = 0

        def take(n):
            nonlocal at
            t = ints[at:at + n]
            at += n
            return t
        self.offsets, self.pos_of_pair, self.pair_of_pos = take(num_experts + 1), take(P), take(P)
        self.tile_expert, self.tile_row0 = take(self.max_tiles), take(self.max_tiles)
        self.num_tiles = take(1)
        f = _fn("moe", "gf_moe_plan", [c_void_p, c_int, c_int, c_int] + [c_void_p] * 7)
        rc = f(_p(idx), P, num_experts, rows, _p(self.offsets), _p(self.pos_of_pair),
               _p(self.pair_of_pos), _p(self.tile_expert), _p(self.tile_row0), _p(self.num_tiles),
               _stream())
        _ok(rc, "moe_plan")


def grouped_glu(x: torch.Tensor, w_gate_up: torch.Tensor, plan: Plan, limit: float, alpha: float,
                up_shift: float, act: torch.Tensor | None = None) -> torch.Tensor:
    """``x [T, K]``, ``w_gate_up [E, 2 F, K]`` (gate row, up row, ...) -> the activated gate/up
    product of every pair, in sorted order: ``[P, F]``.  ``act``: ``{limit, alpha, up_shift}`` as
    an fp32 tensor on the device, for the tcgen05 kernel, which reads them from memory."""
    _cuda(x, w_gate_up)
    E, N, K = w_gate_up.shape
    assert x.dtype == w_gate_up.dtype and x.stride(1) == 1 and x.shape[1] == K
    assert w_gate_up.is_contiguous()
    out = torch.empty((plan.pairs, N // 2), dtype=x.dtype, device=x.device)
    if plan.tcgen05:
        if act is None:      # (a caller inside a CUDA graph brings the three constants on the device)
            act = torch.tensor([limit, alpha, up_shift], dtype=torch.float32, device=x.device)
        if _grouped_tc(gather_rows(x, plan), w_gate_up, plan, out, 2, act=act):
            return out
        raise RuntimeError("the tcgen05 grouped product refused a shape its plan was made for")
    _gemm(x, w_gate_up, plan, out, 1, limit, alpha, up_shift)
    return out


def gather_rows(x: torch.Tensor, plan: Plan) -> torch.Tensor:
    """The tokens' rows in the order of the sorted pairs, ``[P, K]``."""
    K = x.shape[1]
    xs = torch.empty((plan.pairs, K), dtype=x.dtype, device=x.device)
    f = _fn("moe", "gf_moe_gather_rows", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                          c_void_p])
    _ok(f(_p(x), x.stride(0), _p(plan.pair_of_pos), plan.top, plan.pairs, K, _p(xs), _stream()),
        "moe_gather_rows")
    return xs


def _grouped_tc(a, w, plan: Plan, out, epi: int, act=None, row_w=None) -> bool:
    """The grouped product on the persistent tcgen05 kernel; ``False`` if it refuses the shape."""
    from .gemm_bf16 import _dev_state
    E, N, K = w.shape
    f = _fn("gemm_prefill", "gf_gemm_grouped",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p])
    rc = f(_p(a), a.stride(0), _p(w), E, N, K, _p(plan.tile_expert), _p(plan.tile_row0),
           _p(plan.offsets), _p(plan.num_tiles), plan.max_tiles, _p(plan.pair_of_pos), _p(row_w),
           _p(act), _p(out), out.stride(0), plan.pairs, int(epi),
           int(out.dtype == torch.float32), _p(_dev_state(a.device)["err"]), _stream())
    if rc == -6:
        return False
    _ok(rc, "gemm_grouped")
    return True


def grouped_relu2(x: torch.Tensor, w_up: torch.Tensor, plan: Plan, row_weights=None
                  ) -> torch.Tensor:
    """``x [T, K]``, ``w_up [E, F, K]`` -> ``relu(w * (x W^T))^2`` of every pair, in sorted order:
    ``[P, F]``; ``row_weights [T, top]`` fp32 gives each pair's ``w`` (the product of the row
    scaled by ``w``), ``None`` means 1."""
    _cuda(x, w_up, row_weights)
    E, N, K = w_up.shape
    assert x.dtype == w_up.dtype and x.stride(1) == 1 and x.shape[1] == K
    assert w_up.is_contiguous()
    if row_weights is not None:
        assert row_weights.dtype == torch.float32 and row_weights.is_contiguous()
        assert row_weights.numel() == plan.pairs
    out = torch.empty((plan.pairs, N), dtype=x.dtype, device=x.device)
    if plan.tcgen05:
        if _grouped_tc(gather_rows(x, plan), w_up, plan, out, 4, row_w=row_weights):
            return out
        raise RuntimeError("the tcgen05 grouped product refused a shape its plan was made for")
    _gemm(x, w_up, plan, out, 2, 0.0, 0.0, 0.0, row_weights)
    return out


def grouped_down(y: torch.Tensor, w_down: torch.Tensor, plan: Plan) -> torch.Tensor:
    """``y [P, F]`` (sorted pairs), ``w_down [E, N, F]`` -> ``[P, N]`` fp32."""
    _cuda(y, w_down)
    E, N, K = w_down.shape
    assert y.dtype == w_down.dtype and y.is_contiguous() and y.shape == (plan.pairs, K)
    out = torch.empty((plan.pairs, N), dtype=torch.float32, device=y.device)
    if plan.tcgen05:
        if _grouped_tc(y, w_down, plan, out, 0):
            return out
        raise RuntimeError("the tcgen05 grouped product refused a shape its plan was made for")
    _gemm(y, w_down, plan, out, 0, 0.0, 0.0, 0.0)
    return out


def _gemm(a, w, plan, out, first, limit, alpha, up_shift, row_w=None):
    f = _fn("moe", "gf_moe_gemm",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_float, c_float, c_void_p,
             c_int, c_int, c_void_p, c_int])
    _ok(f(_p(a), a.stride(0), _p(w), w.shape[1], w.shape[2], _p(plan.offsets),
          _p(plan.pair_of_pos), plan.top, _p(plan.tile_expert), _p(plan.tile_row0),
          _p(plan.num_tiles), plan.max_tiles, _p(out), int(first), float(limit), float(alpha),
          float(up_shift), _p(row_w), _code(a.dtype), 2 if plan.few else int(plan.tensor_cores),
          _stream(), plan.pairs),
        "moe_gemm")


def combine(y: torch.Tensor, plan: Plan, weights, num_tokens: int) -> torch.Tensor:
    """``out[t] = sum_k weights[t, k] * y[place of pair (t, k)]``, fp32 (``weights`` ``None``:
    the plain sum)."""
    N = y.shape[1]
    out = torch.empty((num_tokens, N), dtype=torch.float32, device=y.device)
    f = _fn("moe", "gf_moe_combine", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                      c_int, c_void_p])
    _ok(f(_p(y), _p(plan.pos_of_pair), _p(weights), num_tokens, plan.top, N, _p(out), 0,
          _stream()), "moe_combine")
    return out
