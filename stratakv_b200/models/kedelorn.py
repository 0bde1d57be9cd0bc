"""The Kedelorn decoder as a list of parts.

Embedding ``embed``, head ``head``, last norm ``final.norm``.  Every layer ``l<i>`` is a pre-norm block over ``streams``
copies of the residual stream (``l<i>.hc1.*`` connect the mixer, ``l<i>.hc2.*`` the feed-forward; a model without
``streams`` has one stream and the plain sum).  The norms keep their weights as distances from one.  Two mixers,
chosen per layer:

* ``retention``: linear attention with a fixed decay per head (``mix.q``, ``mix.k``, ``mix.v``, ``mix.g``, ``mix.o``),
  rotary positions on queries and keys;
* ``latent_attention``: attention over one compressed vector per position and one rotated key part that all heads
  share (``mix.q``, ``mix.dkv``, ``mix.dkv.norm``, ``mix.uk``, ``mix.uv``, ``mix.sink``, ``mix.g``, ``mix.o``), rotary
  positions with stretched frequencies, a sink in the softmax, a gate per head; a layer may attend over what an
  earlier layer cached (``kv_from``) and then has no ``mix.dkv``.

The feed-forward is a mixture of experts (``mlp.e<k>.up/down``, ``mlp.router``, ``mlp.correction``) with a shared,
gated expert (``mlp.shared.up/down/sg``).  Layers may differ in every size.
"""
from __future__ import annotations

from ..config.kedelorn import ARCHITECTURE, KedelornConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, HeadSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec, RetentionSpec,
                          RotarySpec, RoutedMlpSpec, ScheduleEntry, SharedExpertSpec, StreamMixSpec, YarnSpec)

# what the design fixes
EXPERT_ACTIVATION = "relu2"
NORM_WEIGHT_OFFSET = 1.0             # the layers' norms and the last one store their weights around zero


def _rotation(rot):
    if rot is None:
        return None
    scaling = YarnSpec(rot.factor, rot.original, rot.fast, rot.slow) if rot.factor else None
    return RotarySpec(rot.dims, rot.base, scaling)


def _mixer_spec(config: KedelornConfig, layer, p: str):
    if layer.type == "retention":
        return RetentionSpec(
            hidden_size=config.width, num_heads=layer.heads, head_dim=layer.dim, v_head_dim=layer.vdim,
            decay=layer.decay, eps=config.norm_eps, rope=_rotation(layer.rot), q_weight=p + "mix.q",
            k_weight=p + "mix.k", v_weight=p + "mix.v", gate_weight=p + "mix.g", o_weight=p + "mix.o")
    return LatentAttentionSpec(
        hidden_size=config.width, num_heads=layer.heads, head_dim=layer.dim, v_head_dim=layer.vdim,
        latent_dim=layer.kv_rank, scale=layer.scale, eps=config.norm_eps, q_weight=p + "mix.q",
        down_weight=p + "mix.dkv", latent_norm=p + "mix.dkv.norm", k_up_weight=p + "mix.uk", v_up_weight=p + "mix.uv",
        o_weight=p + "mix.o", rope_dim=layer.rot_dim, rope=_rotation(layer.rot), sink=p + "mix.sink",
        gate_weight=p + "mix.g", shares_kv=layer.kv_from is not None)


def _mlp_spec(config: KedelornConfig, mlp, p: str):
    shared = None
    if mlp.shared_ff:
        shared = SharedExpertSpec(mlp.shared_ff, p + "mlp.shared.up", p + "mlp.shared.down", p + "mlp.shared.sg")
    return RoutedMlpSpec(
        hidden_size=config.width, intermediate_size=mlp.ff, experts=mlp.experts, top=mlp.top,
        activation=EXPERT_ACTIVATION, route_scale=mlp.scale, router_weight=p + "mlp.router",
        up_weights=tuple(f"{p}mlp.e{k}.up" for k in range(mlp.experts)),
        down_weights=tuple(f"{p}mlp.e{k}.down" for k in range(mlp.experts)),
        correction=p + "mlp.correction", renormalize=False, shared=shared)


def kedelorn_spec(config: KedelornConfig) -> ModelSpec:
    layers, schedule, entry_of = [], [], {}
    streams = config.streams

    def connection(prefix):
        if not streams:
            return StreamMixSpec(1)
        return StreamMixSpec(streams, prefix + ".in", prefix + ".out", prefix + ".mix")

    def norm(name):
        return NormSpec(config.width, config.norm_eps, name, weight_offset=NORM_WEIGHT_OFFSET)

    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        extras = [("mixer_streams", "stream_mix", connection(p + "hc1"))]
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn, ffn_norm = _mlp_spec(config, layer.mlp, p), norm(p + "norm2")
            extras.append(("ffn_streams", "stream_mix", connection(p + "hc2")))
        layers.append(LayerSpec(mixer_norm=norm(p + "norm1"), mixer=_mixer_spec(config, layer, p), ffn_norm=ffn_norm,
                                ffn=ffn, arrangement="multi_stream", extras=tuple(extras)))
        # a cache entry per layer that keeps something of its own; a layer that borrows a latent names the lender's
        if layer.kv_from is not None:
            schedule.append(ScheduleEntry(layer=i, cache=entry_of[layer.kv_from], writes_cache=False))
        else:
            entry_of[i] = len(entry_of)
            schedule.append(ScheduleEntry(layer=i, cache=entry_of[i]))
    return ModelSpec(
        architecture=config.architecture, hidden_size=config.width, vocab_size=config.vocab,
        embedding=EmbeddingSpec(config.vocab, config.width, "embed"), layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("final.norm"), head=HeadSpec(config.vocab, config.width, "head"))


register_architecture(ARCHITECTURE, KedelornConfig, kedelorn_spec)
