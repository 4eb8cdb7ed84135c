"""Typed configuration of the Vilepel design, read from its own ``config.json`` keys.

A Vilepel folder names its design under ``architecture`` and describes every layer on its own:
``layers[i] = {"type": mixer kind, "mixer": its sizes and constants, "mlp": feed-forward or null,
"weights_of": j}`` where ``weights_of`` (optional) makes layer ``i`` run with the tensors of layer
``j`` and a cache or state of its own.  Beside the layers: ``width``, ``vocab``,
``embedding.scale`` and ``norm.eps``.  Every size and constant of a model comes from this object.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class VilepelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None
    weights_of: int | None = None

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"type": self.type, "mixer": _plain(self.mixer),
                             "mlp": _plain(self.mlp)}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _plain(x):
    if isinstance(x, Mapping):
        return {k: _plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_plain(v) for v in x]
    return x


@dataclass(frozen=True)
class VilepelConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[VilepelLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VilepelConfig":
        width = _positive_int(_need(d, "width", "the model"), "width")
        vocab = _positive_int(_need(d, "vocab", "the model"), "vocab")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        scale = float(_need(_need(d, "embedding", "the model"), "scale", "embedding"))
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
                if mk == "dense":
                    _positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
                    _need(mlp, "limit", f"{where}.mlp")
                elif mk == "moe":
                    ex = _need(mlp, "expert", f"{where}.mlp")
                    _positive_int(_need(ex, "ff", f"{where}.mlp.expert"), f"{where}.mlp.expert.ff")
                    _need(ex, "limit", f"{where}.mlp.expert")
                    ro = _need(mlp, "router", f"{where}.mlp")
                    n = _positive_int(_need(ro, "experts", f"{where}.mlp.router"), "experts")
                    top = _positive_int(_need(ro, "top", f"{where}.mlp.router"), "top")
                    if top > n:
                        raise ConfigError(f"config.json: {where} chooses {top} of {n} experts")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r} is not 'dense' or "
                                      "'moe'")
            wo = L.get("weights_of")
            if wo is not None:
                if isinstance(wo, bool) or not isinstance(wo, int) or not (0 <= wo < len(raw_layers)):
                    raise ConfigError(f"config.json: {where}.weights_of {wo!r} names no layer")
                if raw_layers[wo].get("weights_of") is not None:
                    raise ConfigError(f"config.json: {where}.weights_of names layer {wo}, which "
                                      "has no tensors of its own")
                if raw_layers[wo].get("type") != kind:
                    raise ConfigError(f"config.json: {where} is {kind!r} but uses the weights of "
                                      f"a {raw_layers[wo].get('type')!r} layer")
            layers.append(VilepelLayer(kind, mixer, mlp, wo))
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, embedding_scale=scale,
                  layers=tuple(layers),
                  eos_token_ids=_eos(d.get("eos_token_id"), vocab),
                  torch_dtype=str(d.get("torch_dtype", "bfloat16")),
                  extra={k: v for k, v in d.items()
                         if k not in ("width", "vocab", "norm", "embedding", "layers",
                                      "eos_token_id", "torch_dtype")})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        for i, L in enumerate(self.layers):
            m = L.mixer
            for k in ("heads", "dim", "vdim"):
                _positive_int(m[k], f"layers[{i}].mixer.{k}")
            if L.type == "latent_attention":
                _positive_int(m["kv_rank"], f"layers[{i}].mixer.kv_rank")
                _positive_int(m["rot_dim"], f"layers[{i}].mixer.rot_dim")
                dims = _positive_int(_need(m["rot"], "dims", f"layers[{i}].mixer.rot"), "rot.dims")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: layers[{i}] rotates {dims} of {m['rot_dim']} "
                                      "channels; it must be an even number of them")
                if not (float(_need(m["rot"], "base", f"layers[{i}].mixer.rot")) > 0):
                    raise ConfigError(f"config.json: layers[{i}].mixer.rot.base must be > 0")
                if m.get("mask") is not None:          # no mask: every earlier token is seen
                    _positive_int(_need(m["mask"], "size", f"layers[{i}].mixer.mask"), "mask.size")
            else:
                _positive_int(m["kv_heads"], f"layers[{i}].mixer.kv_heads")
                _positive_int(m["conv"], f"layers[{i}].mixer.conv")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: layers[{i}] has {m['heads']} heads for "
                                      f"{m['kv_heads']} kv heads")

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = dict(self.extra)
        d.update(architecture="Vilepel", width=self.width, vocab=self.vocab,
                 norm={"eps": self.norm_eps}, embedding={"scale": self.embedding_scale},
                 layers=[L.to_dict() for L in self.layers], torch_dtype=self.torch_dtype)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _eos(eos, vocab: int) -> tuple[int, ...]:
    if eos is None:
        return ()
    ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
    for e in ids:
        if not (0 <= e < vocab):
            raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary")
    return ids
