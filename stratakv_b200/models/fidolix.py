"""The Fidolix decoder as a list of parts.

Embedding ``embed`` times a constant, head ``head``, last norm ``final.norm``.  Every layer ``l<i>`` adds two branches
that read the same stream through a norm each, ``x += mixer(norm1(x)) + mlp(norm2(x))``, and then a per-layer token input
``x += rmsnorm(side.proj(gelu_tanh(side.gate x) * side.embed[token, layer's part]))``.  Two mixers, chosen per layer:

* ``attention``: grouped-query attention without a rotation; biased projections, one RMS norm with a weight over all
  query heads and one over all key heads (``mix.q.norm``, ``mix.k.norm``), capped scores, a sigmoid gate (``mix.g``) on
  every output number;
* ``parallel``: two mixers side by side whose results are added with a weight each.  ``mix.left.*``: attention whose
  biased queries and keys pass a short convolution over time (``mix.left.q.conv``, ``mix.left.k.conv``), whose values are
  the convolved keys, with rotary positions in interleaved pairs (frequencies stretched for long contexts), a sliding
  window and a sink per head (``mix.left.sink``).  ``mix.right.*``: time mixing with a matrix state per head and a decay
  per token and key channel (``mu.r/k/v/g/w``, ``r``, ``k``, ``v``, ``g``, ``w1``, ``w2``, ``w0``, ``u``, ``norm``, ``o``).

The feed-forward is a gated unit with both branches clamped (``mlp.gate/up/down``), or a mixture of gated experts
(``mlp.e<k>.gate/up/down``, ``mlp.router``) chosen by softmax scores among the best groups of experts; a layer may have
none.  Some layers in a row may run several times with the same weights; every pass has cache entries of its own and
the embedding's output is added to the stream again before every pass but the first.
"""
from __future__ import annotations

from ..config.fidolix import ARCHITECTURE, FidolixConfig
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, ConvAttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LayerSpec, MixerPairSpec,
                          ModelSpec, NormSpec, RotarySpec, RoutedMlpSpec, ScheduleEntry, TimeMixSpec, TokenSideSpec,
                          YarnSpec)

# what the design fixes
DENSE_ACTIVATION = "swiglu_clamp"
EXPERT_ACTIVATION = "silu"
ROUTER_SCORES = "softmax"
RENORMALIZE_EPS = 1e-20
ROTATION_INTERLEAVED = True


def _rotation(rot):
    if rot is None:
        return None
    scaling = YarnSpec(rot.factor, rot.original, rot.fast, rot.slow) if rot.factor else None
    return RotarySpec(rot.dims, rot.base, scaling, interleaved=ROTATION_INTERLEAVED)


def _mixer_spec(config: FidolixConfig, layer, p: str):
    a = layer.attention
    if layer.type == "attention":
        return AttentionSpec(
            hidden_size=config.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
            position=None, q_weight=p + "q", k_weight=p + "k", v_weight=p + "v", o_weight=p + "o", v_head_dim=a.vdim,
            q_bias=p + "q.b", k_bias=p + "k.b", v_bias=p + "v.b", gate_weight=p + "g", gate_per_element=True,
            softcap=a.softcap, q_norm_weight=p + "q.norm", k_norm_weight=p + "k.norm",
            projection_norm_eps=config.norm_eps)
    l, r = p + "left.", p + "right."
    left = ConvAttentionSpec(
        hidden_size=config.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
        q_weight=l + "q", k_weight=l + "k", o_weight=l + "o", taps=a.conv,
        q_conv=l + "q.conv" if a.conv else None, k_conv=l + "k.conv" if a.conv else None, q_bias=l + "q.b",
        k_bias=l + "k.b", rope=_rotation(a.rot), window=a.window, sink=l + "sink")
    right = TimeMixSpec(
        hidden_size=config.width, num_heads=layer.right.heads, head_dim=layer.right.dim, decay_rank=layer.right.rank,
        eps=config.norm_eps, mix=tuple(r + "mu." + s for s in "rkvgw"), r_weight=r + "r", k_weight=r + "k",
        v_weight=r + "v", g_weight=r + "g", w1_weight=r + "w1", w2_weight=r + "w2", w0=r + "w0", bonus=r + "u",
        norm=r + "norm", o_weight=r + "o")
    return MixerPairSpec(left, right, layer.left_scale, layer.right_scale)


def _mlp_spec(config: FidolixConfig, mlp, p: str):
    if mlp.kind == "dense":
        return GatedMlpSpec(config.width, mlp.ff, DENSE_ACTIVATION, p + "gate", p + "up", p + "down",
                            activation_param=mlp.limit)
    names = lambda part: tuple(f"{p}e{k}.{part}" for k in range(mlp.experts))
    return RoutedMlpSpec(
        hidden_size=config.width, intermediate_size=mlp.ff, experts=mlp.experts, top=mlp.top,
        activation=EXPERT_ACTIVATION, route_scale=1.0, router_weight=p + "router", up_weights=names("up"),
        down_weights=names("down"), renormalize=True, gate_weights=names("gate"), score=ROUTER_SCORES,
        groups=mlp.groups, keep_groups=mlp.keep, renormalize_eps=RENORMALIZE_EPS)


def layer_runs(config: FidolixConfig):
    """The layers in the order they run, and the indices of the runs before which the embedding's output is added."""
    order, again = list(range(config.loop_start)), set()
    for time in range(config.loop_times):
        if time > 0 and config.loop_stop > config.loop_start:
            again.add(len(order))
        order += list(range(config.loop_start, config.loop_stop))
    return order + list(range(config.loop_stop, len(config.layers))), again


def fidolix_spec(config: FidolixConfig) -> ModelSpec:
    if any(layer.right is not None and not layer.right.rank for layer in config.layers):
        raise ValueError("Fidolix: the rank of a decay's low-rank part is open; open the model through load_config, which "
                         "reads it from the checkpoint, or give mixer.right.rank")
    layers = []
    side_width = config.side_dim * len(config.layers)
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        norm = lambda name: NormSpec(config.width, config.norm_eps, p + name)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn, ffn_norm = _mlp_spec(config, layer.mlp, p + "mlp."), norm("norm2")
        extras = []
        if config.side_dim:
            extras.append(("token_input", "token_input", TokenSideSpec(
                hidden_size=config.width, vocab_size=config.vocab, dim=config.side_dim, offset=i * config.side_dim,
                table_width=side_width, eps=config.norm_eps, table="side.embed", gate_weight=p + "side.gate",
                proj_weight=p + "side.proj", norm_weight=p + "side.norm")))
        layers.append(LayerSpec(mixer_norm=norm("norm1"), mixer=_mixer_spec(config, layer, p + "mix."), ffn_norm=ffn_norm,
                                ffn=ffn, arrangement="parallel_pair", extras=tuple(extras)))
    # every run of a layer has a cache entry of its own: a layer that runs again starts from nothing
    order, again = layer_runs(config)
    schedule = tuple(ScheduleEntry(layer=i, cache=run, adds_embedding=run in again) for run, i in enumerate(order))
    return ModelSpec(
        architecture=config.architecture, hidden_size=config.width, vocab_size=config.vocab,
        embedding=EmbeddingSpec(config.vocab, config.width, "embed", scale=config.embedding_scale),
        layers=tuple(layers), schedule=schedule, final_norm=NormSpec(config.width, config.norm_eps, "final.norm"),
        head=HeadSpec(config.vocab, config.width, "head"),
        # a layer without a feed-forward has no use for a second norm; a checkpoint may carry one all the same
        ignorable=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.mlp is None))


register_architecture(ARCHITECTURE, FidolixConfig, fidolix_spec)
