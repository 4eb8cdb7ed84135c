"""Tiny Zolapel configurations and model folders for the tests.  The folders' weights are drawn at
random and then shaped so that faults show: the score scale is large (peaked attention: a key that
is wrongly seen or missed moves the logits), norm weights, biases, layer scales and the loop's
vectors are not small, and the router's choices are clear."""
from __future__ import annotations

import copy
import json
import os

import torch

from ginfer_b200.config.registry import resolve_architecture
from ginfer_b200.parts.model import DecoderModel
from ginfer_b200.weights.random_init import random_tensors
from ginfer_b200.weights.safetensors_io import write_safetensors


def attention(heads=4, kv_heads=2, dim=24, window=37, rot_dims=16, base=1000.0, scale=0.7,
              scaling="default"):
    rot = None
    if rot_dims is not None:
        rot = {"base": base, "dims": rot_dims}
        if scaling == "default":     # wavelengths of 16 rotated channels at base 1000 span 6..2,600
            scaling = {"factor": 3.0, "low": 1.0, "high": 6.0, "original": 200}
        if scaling is not None:
            rot["scaling"] = scaling
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def moe(experts=5, top=2, ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))


def config(layers, width=48, vocab=211, eps=2e-5, mult=0.6, side=6, loop=None):
    d = {"architecture": "Zolapel", "width": width, "vocab": vocab, "norm": {"eps": eps},
         "residual_mult": mult, "layers": layers, "torch_dtype": "float32"}
    if side:
        d["token_side"] = {"dim": side}
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# nothing is a power of two; several kv heads; part of a head rotates; a layer has no
# feed-forward; two and three experts chosen; the loop starts behind the first layer
MIXED = config([
    layer(attention(), moe()),
    layer(attention(heads=3, kv_heads=3, dim=20, window=21, rot_dims=12), None),
    layer(attention(heads=6, kv_heads=2, dim=16, window=50, rot_dims=16, scaling=None),
          moe(experts=7, top=3, ff=24)),
    layer(attention(heads=2, kv_heads=1, dim=40, window=18, rot_dims=40), moe(experts=3, top=1)),
], loop=(1, 3, 2))

# other sizes: a width that is no multiple of 8, a head size that no tensor-core kernel takes, a
# head size of 64 (the kernels of large models), no window on one layer, all experts chosen, no
# side input, a loop over everything
OTHER = config([
    layer(attention(heads=5, kv_heads=1, dim=12, window=64, rot_dims=8, base=50.0, scale=0.9),
          moe(experts=4, top=4, ff=32)),
    layer(attention(heads=2, kv_heads=2, dim=64, window=None, rot_dims=32, scale=0.4),
          moe(experts=9, top=2, ff=20)),
], width=52, vocab=173, eps=1e-6, mult=1.0, side=0, loop=(0, 2, 3))

# sizes that fit no vector access and no tensor-core tile: a head of 50 channels of which 6
# rotate, experts of 36, a width of 100, a side input of 7; a window of one token (a token sees
# itself only) and a window of two; the loop is the first layer alone
ODD = config([
    layer(attention(heads=3, kv_heads=1, dim=50, window=2, rot_dims=6, base=30.0, scale=0.5),
          moe(experts=5, top=3, ff=36)),
    layer(attention(heads=2, kv_heads=2, dim=18, window=1, rot_dims=18, scale=0.8), None),
    layer(attention(heads=4, kv_heads=1, dim=32, window=None, rot_dims=None, scale=0.3),
          moe(experts=2, top=1, ff=16)),
], width=100, vocab=131, eps=1e-4, mult=0.8, side=7, loop=(0, 1, 2))

ATTENTION_ONLY = config([layer(attention(window=19), None)], width=40, vocab=97, side=0)
ROUTED = config([layer(attention(window=1000), moe(experts=7, top=3))], width=40, vocab=97, side=0)
SIDE = config([layer(attention(window=1000), None), layer(attention(window=1000), None)],
              width=40, vocab=97, side=10)
LOOPED = config([layer(attention(window=1000), None)], width=40, vocab=97, side=0, loop=(0, 1, 3))
# one layer, no rotation: a score depends on the two tokens only, wherever they stand
NEEDLE = config([layer(attention(heads=2, kv_heads=1, dim=16, window=23, rot_dims=None,
                                 scale=6.0), None)], width=32, vocab=61, side=0, mult=1.0)


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
        if name == "embed":
            t[name] = x * 30.0
        elif name == "side.embed":
            t[name] = x * 50.0
        elif name == "loop.step":
            t[name] = rnd(x, 0.5)
        elif name.endswith(".b"):
            t[name] = rnd(x, 0.3)
        elif leaf in ("norm1", "norm2", "side.norm", "mix.q.norm", "mix.k.norm", "ls1", "ls2") \
                or name == "final.norm":
            t[name] = 1.0 + rnd(x, 0.3)
        elif leaf == "mlp.router":
            t[name] = x * 20.0                           # clear choices
        elif leaf == "mix.g":
            t[name] = x * 15.0                           # gates that open and close
        elif x.dim() == 2:
            t[name] = x * 5.0
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


def read_folder(path: str):
    """``(config dict, {name: float64 numpy array})`` as stored."""
    from ginfer_b200.weights.safetensors_io import open_model_tensors
    cfg = json.load(open(os.path.join(path, "config.json")))
    out = {}
    for n, (f, k) in open_model_tensors(path).items():
        v = f.get(k)
        out[n] = v.to(torch.float64).numpy() if v.is_floating_point() else v.numpy()
    return cfg, out
