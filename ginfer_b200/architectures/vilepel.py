"""Vilepel as a plan of parts.

A decoder whose layers differ: each is a latent-attention mixer (one cached latent vector and one
shared rotated key part a token, sliding window) or a gated delta-rule mixer with a decay per key
channel (state of fixed size), followed by a dense or routed feed-forward with a clamped,
sigmoid-gated activation.  The norms sit on the sublayers' outputs (``x + norm(sublayer(x))``),
their weights are stored around zero, the embedding is scaled, and a layer may run with the
tensors of another layer and a cache of its own: such a layer becomes a second run of that layer
in the plan's run list.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vilepel_config import VilepelConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry

# Positions are exact in 32-bit floats up to here; nothing else bounds a sequence's length.
MAX_POSITIONS = 1 << 24


def _mixer(cfg: VilepelConfig, kind: str, m) -> PartSpec:
    if kind == "latent_attention":
        return PartSpec("latent_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], nope_dim=m["dim"], rope_dim=m["rot_dim"],
            v_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
            window=m["mask"]["size"] if m.get("mask") is not None else 0,
            rotary_dims=m["rot"]["dims"], rotary_base=m["rot"]["base"], latent_eps=cfg.norm_eps,
            prefix="mix"))
    # the inner sizes of the two low-rank projections are the tensors' own; a configuration may
    # name them (``decay_rank``, ``gate_rank``) so that random weights can be drawn
    return PartSpec("channel_delta", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        key_dim=m["dim"], v_dim=m["vdim"], conv_taps=m["conv"], out_norm_eps=cfg.norm_eps,
        decay_rank=m.get("decay_rank", -1), gate_rank=m.get("gate_rank", -1), prefix="mix"))


def _feed_forward(cfg: VilepelConfig, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("clamped_glu", dict(hidden_size=cfg.width, intermediate_size=mlp["ff"],
                                            limit=mlp["limit"], prefix="mlp"))
    return PartSpec("routed_glu", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"],
        limit=mlp["expert"]["limit"], num_experts=mlp["router"]["experts"],
        top_k=mlp["router"]["top"], prefix="mlp"))


def vilepel_plan(cfg: VilepelConfig) -> ModelPlan:
    def norm(name):
        return PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=name,
                                        weight_offset=1.0))
    layers, index_of = [], {}
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        index_of[i] = len(layers)
        ff = _feed_forward(cfg, L.mlp)
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=_mixer(cfg, L.type, L.mixer), feed_forward=ff,
            mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
            block=PartSpec("outnorm")))
    run = tuple(RunEntry(layer=index_of[i if L.weights_of is None else L.weights_of], cache=i)
                for i, L in enumerate(cfg.layers))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                         name="embed", scale=cfg.embedding_scale)),
        layers=tuple(layers), run=run, final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, name="head")),
        eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture("Vilepel", VilepelConfig, vilepel_plan, model_types=("vilepel",))
