"""Tiny Vilepel configurations and model folders for the tests.  The folders' weights are drawn
at random and then shaped so that faults show: queries and key up-projections are scaled up (peaked
attention: a key that is wrongly seen or missed moves the logits), the decays are slow (a token far
back still matters), norm weights and biases are not small."""
from __future__ import annotations

import copy
import json
import os

import torch

from ginfer_b200.config.registry import resolve_architecture
from ginfer_b200.parts.model import DecoderModel
from ginfer_b200.weights.random_init import random_tensors
from ginfer_b200.weights.safetensors_io import write_safetensors


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=37, rot_dims=None, base=1000.0,
           scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
        "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
        "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims or rot_dim}}}


def delta(heads=4, kv_heads=2, dim=16, vdim=12, conv=3, decay_rank=6, gate_rank=5):
    return {"type": "channel_delta", "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
        "decay_rank": decay_rank, "gate_rank": gate_rank}}


def dense(ff=72, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, top=2, ff=40, limit=1.25):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top}}


def layer(mixer, mlp, weights_of=None):
    d = dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def config(layers, width=48, vocab=211, eps=2e-5, scale=7.0):
    return {"architecture": "Vilepel", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": layers, "torch_dtype": "float32"}


# sizes chosen so that nothing is a power of two, heads differ from kv heads, the value size
# differs from the key size, only part of the rotated channels rotates, a layer has no
# feed-forward, layers share weights, and one router chooses a single expert
MIXED = config([
    layer(latent(), dense()),
    layer(delta(), moe()),
    layer(latent(), dense(), weights_of=0),
    layer(delta(heads=2, kv_heads=2, dim=20, vdim=28, conv=2), None),
    layer(latent(heads=2, dim=24, rot_dim=16, vdim=8, kv_rank=33, window=21, rot_dims=10),
          moe(experts=3, top=1, ff=24)),
    layer(delta(), moe(), weights_of=1),
])

# other sizes: one kv head for several heads, five taps, all experts chosen, wide heads
OTHER = config([
    layer(delta(heads=3, kv_heads=1, dim=36, vdim=40, conv=5, decay_rank=3, gate_rank=8),
          moe(experts=4, top=4, ff=32, limit=0.8)),
    layer(latent(heads=5, dim=32, rot_dim=32, vdim=16, kv_rank=64, window=64), dense(ff=100)),
], width=80, vocab=173, eps=1e-6, scale=3.0)

LATENT_ONLY = config([layer(latent(window=19), None)], width=40, vocab=97)
DELTA_ONLY = config([layer(delta(), None)], width=40, vocab=97)
DENSE_FF = config([layer(latent(window=1000), dense())], width=40, vocab=97)
ROUTED_FF = config([layer(latent(window=1000), moe(experts=7, top=3))], width=40, vocab=97)


def shaped_tensors(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    arch = resolve_architecture(cfg)
    model = DecoderModel(arch.build_plan(arch.config_cls.from_dict(cfg)))
    t = random_tensors(model, seed, torch.float32)
    g = torch.Generator().manual_seed(seed + 1)

    def rnd(like, std):
        return torch.randn(like.shape, generator=g) * std
    for name in list(t):
        x = t[name]
        leaf = name.split(".", 1)[1] if "." in name else name
        if leaf in ("norm1", "norm2", "norm") or name == "final.norm":
            t[name] = rnd(x, 0.3)
        elif leaf == "mix.dkv.norm" or leaf == "mix.norm":
            t[name] = 1.0 + rnd(x, 0.3)
        elif leaf == "mix.A_log":
            t[name] = -3.0 + rnd(x, 1.0)                 # slow decays: far tokens matter
        elif leaf == "mix.dt_bias":
            t[name] = rnd(x, 1.0)
        elif leaf.endswith(".conv"):
            t[name] = rnd(x, 0.6)
        elif leaf in ("mix.q", "mix.uk", "mix.dkv"):
            t[name] = x * 9.0                            # peaked attention
        elif leaf == "mlp.router":
            t[name] = x * 20.0                           # clear choices
        elif x.dim() == 2:
            t[name] = x * 4.0
    return t


def write_folder(path: str, cfg: dict, seed: int = 0, storage=torch.float32) -> str:
    os.makedirs(path, exist_ok=True)
    out = dict(cfg, torch_dtype="bfloat16" if storage == torch.bfloat16 else "float32")
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f)
    tensors = {k: (v if not v.is_floating_point() else v.to(storage))
               for k, v in shaped_tensors(cfg, seed).items()}
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path
