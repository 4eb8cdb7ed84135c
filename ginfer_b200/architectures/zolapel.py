"""Zolapel as a plan of parts.

A decoder on a 32-bit residual stream.  A layer is ``x += m * ls1 * attention(LN1(x))``,
``x += m * ls2 * experts(LN2(x))`` and then a token side input: a slice of a second token table,
gated by the stream, projected to the width, RMS-normed and added (times ``m``).  The norms are
layer norms with weight and bias.  The attention has normed queries and keys, rotation of
neighbouring channel pairs with stretched long wavelengths, a sliding window, values that are the
keys as projected, and a sigmoid gate on every head's output.  The feed-forward routes every token
to the ``top`` experts with the largest sigmoid scores and scales what each expert reads by its
score; an expert is ``W_down relu(W_up h)^2``.  A range of layers may run several times in a row
(a loop): each pass has caches of its own and is entered through a :class:`LoopEntry`.  The head
is the embedding matrix.

Tensor names: ``embed``, ``side.embed``, ``loop.step``, ``l<i>.norm1|norm2`` (+ ``.b``),
``l<i>.ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm`` (+ ``.b``).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zolapel_config import ZolapelConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry

# Positions are exact in 32-bit floats up to here; nothing else bounds a sequence's length.
MAX_POSITIONS = 1 << 24


def _mixer(cfg: ZolapelConfig, m) -> PartSpec:
    rot = m.get("rot")
    position = PartSpec("pair_rotary", dict(
        dims=rot["dims"] if rot else 0, base=rot["base"] if rot else 1.0,
        scaling=rot.get("scaling") if rot else None, interleaved=True))
    return PartSpec("qknorm_attention", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        head_dim=m["dim"], scale=m["scale"], position=position,
        window=m["mask"]["size"] if m.get("mask") is not None else 0,
        qk_norm=True, qk_norm_eps=cfg.norm_eps, value_projection=False, head_gate=True,
        prefix="mix"))


def _feed_forward(cfg: ZolapelConfig, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"],
        num_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"], score="sigmoid",
        renormalize=False, weight_on="input", prefix="mlp"))


def zolapel_plan(cfg: ZolapelConfig) -> ModelPlan:
    def norm(name):
        return PartSpec("layernorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=name,
                                          bias_name=name + ".b"))
    n = len(cfg.layers)
    layers = []
    for i, L in enumerate(cfg.layers):
        ff = _feed_forward(cfg, L.mlp)
        after = None
        if cfg.side_dim:
            after = PartSpec("token_side", dict(
                hidden_size=cfg.width, vocab_size=cfg.vocab, dim=cfg.side_dim,
                offset=i * cfg.side_dim, total=n * cfg.side_dim, eps=cfg.norm_eps,
                table_name="/side.embed", prefix="side"))
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=_mixer(cfg, L.mixer), feed_forward=ff,
            mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
            block=PartSpec("scaled_prenorm", dict(
                residual_mult=cfg.residual_mult, mixer_scale="ls1", feed_forward_scale="ls2",
                after=after))))
    # every run has a cache of its own: a layer inside the loop keeps one per pass
    run = tuple(RunEntry(layer=i, cache=r, enter=None if t is None else (0, t))
                for r, (i, t) in enumerate(cfg.run_order()))
    stream_inputs = ()
    if cfg.loop is not None:
        stream_inputs = (PartSpec("loop_entry", dict(hidden_size=cfg.width, times=cfg.loop[2],
                                                     name="/loop.step")),)
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                         name="embed", scale=1.0)),
        layers=tuple(layers), run=run, final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied_to="embed")),
        eos_token_ids=tuple(cfg.eos_token_ids), stream_inputs=stream_inputs)


register_architecture("Zolapel", ZolapelConfig, zolapel_plan, model_types=("zolapel",))
