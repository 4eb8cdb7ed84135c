"""Typed configuration of the Zolapel design, read from its own ``config.json`` keys.

A Zolapel folder names its design under ``architecture``.  ``layers[i] = {"type": "attention",
"mixer": sizes and constants, "mlp": routed feed-forward or null}``; beside the layers ``width``,
``vocab``, ``norm.eps``, ``residual_mult``, ``token_side.dim`` (the width of every layer's slice
of the second token table; absent or null: no such input) and ``loop = {start, stop, times}``
(layers ``start .. stop-1`` run ``times`` times in a row, each pass with caches of its own;
absent or null: every layer once).  Every size and constant of a model comes from this object.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError
from .vilepel_config import _eos, _need, _plain, _positive_int

MIXER_KEYS = {"attention": ("heads", "kv_heads", "dim", "scale")}
_TOP_KEYS = ("architecture", "width", "vocab", "norm", "residual_mult", "token_side", "loop",
             "layers", "eos_token_id", "torch_dtype")


@dataclass(frozen=True)
class ZolapelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": _plain(self.mixer), "mlp": _plain(self.mlp)}


@dataclass(frozen=True)
class ZolapelConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    layers: tuple[ZolapelLayer, ...]
    side_dim: int = 0                                  # 0: no per-layer token input
    loop: tuple[int, int, int] | None = None           # (start, stop, times)
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZolapelConfig":
        width = _positive_int(_need(d, "width", "the model"), "width")
        vocab = _positive_int(_need(d, "vocab", "the model"), "vocab")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        mult = float(d.get("residual_mult", 1.0))
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known mixers are "
                                  f"{sorted(MIXER_KEYS)}")
            mixer = _need(L, "mixer", where)
            for k in MIXER_KEYS[kind]:
                _need(mixer, k, f"{where}.mixer")
            mlp = L.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r}: this design's "
                                      "feed-forward is 'moe' (or null for none)")
                ex = _need(mlp, "expert", f"{where}.mlp")
                _positive_int(_need(ex, "ff", f"{where}.mlp.expert"), f"{where}.mlp.expert.ff")
                ro = _need(mlp, "router", f"{where}.mlp")
                n = _positive_int(_need(ro, "experts", f"{where}.mlp.router"), "experts")
                top = _positive_int(_need(ro, "top", f"{where}.mlp.router"), "top")
                if top > n:
                    raise ConfigError(f"config.json: {where} chooses {top} of {n} experts")
            layers.append(ZolapelLayer(kind, mixer, mlp))
        side = d.get("token_side")
        side_dim = 0 if side is None else _positive_int(_need(side, "dim", "token_side"),
                                                        "token_side.dim")
        loop = d.get("loop")
        if loop is not None:
            loop = tuple(int(_need(loop, k, "loop")) for k in ("start", "stop", "times"))
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, residual_mult=mult,
                  layers=tuple(layers), side_dim=side_dim, loop=loop,
                  eos_token_ids=_eos(d.get("eos_token_id"), vocab),
                  torch_dtype=str(d.get("torch_dtype", "bfloat16")),
                  extra={k: v for k, v in d.items() if k not in _TOP_KEYS})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        if self.loop is not None:
            a, b, times = self.loop
            if not (0 <= a < b <= len(self.layers)) or times < 1:
                raise ConfigError(f"config.json: loop {self.loop} does not fit "
                                  f"{len(self.layers)} layers (0 <= start < stop <= layers, "
                                  "times >= 1)")
        for i, L in enumerate(self.layers):
            m = L.mixer
            for k in ("heads", "kv_heads", "dim"):
                _positive_int(m[k], f"layers[{i}].mixer.{k}")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: layers[{i}] has {m['heads']} heads for "
                                  f"{m['kv_heads']} kv heads")
            if m.get("vdim", m["dim"]) != m["dim"]:
                raise ConfigError(f"config.json: layers[{i}]: the values are the keys as "
                                  f"projected, so vdim ({m['vdim']}) must equal dim ({m['dim']})")
            if m.get("mask") is not None:            # no mask: every earlier token is seen
                _positive_int(_need(m["mask"], "size", f"layers[{i}].mixer.mask"), "mask.size")
            rot = m.get("rot")
            if rot is not None:                      # no rot: no rotation
                dims = _need(rot, "dims", f"layers[{i}].mixer.rot")
                if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 \
                        or dims > m["dim"]:
                    raise ConfigError(f"config.json: layers[{i}] rotates {dims!r} of {m['dim']} "
                                      "channels; it must be an even number of them")
                if not (float(_need(rot, "base", f"layers[{i}].mixer.rot")) > 0):
                    raise ConfigError(f"config.json: layers[{i}].mixer.rot.base must be > 0")
                sc = rot.get("scaling")
                if sc is not None:
                    for k in ("factor", "low", "high", "original"):
                        _need(sc, k, f"layers[{i}].mixer.rot.scaling")
                    if float(sc["high"]) == float(sc["low"]) or float(sc["factor"]) == 0:
                        raise ConfigError(f"config.json: layers[{i}].mixer.rot.scaling needs "
                                          "high != low and factor != 0")

    def run_order(self) -> list[tuple[int, int | None]]:
        """The runs of a step as ``(layer, pass number if the run starts a pass of the loop)``."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        out: list[tuple[int, int | None]] = [(i, None) for i in range(a)]
        for t in range(times):
            out += [(i, t if i == a else None) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = dict(self.extra)
        d.update(architecture="Zolapel", width=self.width, vocab=self.vocab,
                 norm={"eps": self.norm_eps}, residual_mult=self.residual_mult,
                 layers=[L.to_dict() for L in self.layers], torch_dtype=self.torch_dtype)
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
