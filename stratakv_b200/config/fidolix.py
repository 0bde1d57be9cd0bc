"""Typed configuration of the Fidolix decoder, read from its ``config.json``.

The file names the design under ``architecture`` and lists its layers, each with its own mixer and feed-forward::

    {"architecture": "Fidolix", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": c},
     "token_side": {"dim": n} | absent, "loop": {"start": a, "stop": b, "times": k} | absent,
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": c, "softcap": cap},
        "mlp": {"kind": "dense", "ff": F, "limit": c}
             | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k, "groups": {"count": g, "keep": m}}}
             | null},
       {"type": "parallel",
        "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "conv": taps, "scale": c,
                           "mask": {"size": w}, "rot": {"dims": n, "base": b, "scaling": {"factor": f, "original": n,
                           "fast": x, "slow": y} | absent}},
                  "right": {"heads": H, "dim": d}, "left_scale": a, "right_scale": b},
        "mlp": ...}]}

Layers ``start .. stop - 1`` run ``times`` times in a row with the same weights.  Every size and every constant that
differs between models of the design comes from there; sizes that only a tensor's shape gives (the rank of the decay's
low-rank part) are read from the checkpoint's header by the loader, or are given as ``mixer.right.rank``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError, _need, _optional
from .zepavik import _positive, _section

ARCHITECTURE = "Fidolix"
MIXERS = ("attention", "parallel")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class FidolixRotation:
    dims: int
    base: float
    factor: float = 0.0              # 0: no scaling of the frequencies
    original: int = 0
    fast: float = 0.0
    slow: float = 0.0

    @classmethod
    def from_dict(cls, raw, where: str) -> "FidolixRotation":
        dims = _positive(_need(raw, "dims", int), where + "dims")
        if dims % 2:
            raise ConfigError(f"config.json: {where}dims ({dims}) must be even: numbers are rotated in pairs")
        base = _need(raw, "base", float)
        if not base > 0.0:
            raise ConfigError(f"config.json: {where}base must be positive")
        scaling = _section(raw, "scaling", where, required=False)
        if scaling is None:
            return cls(dims, base)
        factor = _need(scaling, "factor", float)
        fast, slow = _need(scaling, "fast", float), _need(scaling, "slow", float)
        if not (factor > 0.0 and fast > 0.0 and slow > 0.0):
            raise ConfigError(f"config.json: {where}scaling.factor, scaling.fast and scaling.slow must be positive")
        return cls(dims, base, factor, _positive(_need(scaling, "original", int), where + "scaling.original"), fast, slow)

    def to_dict(self) -> dict:
        raw = {"base": self.base, "dims": self.dims}
        if self.factor:
            raw["scaling"] = {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}
        return raw


@dataclass(frozen=True)
class FidolixMlp:
    kind: str
    ff: int
    limit: float = 0.0               # dense: both branches are clamped to it
    experts: int = 0                 # moe
    top: int = 0
    groups: int = 0                  # 0: the experts form no groups
    keep: int = 0

    @classmethod
    def from_dict(cls, raw, where: str) -> "FidolixMlp":
        kind = _need(raw, "kind", str)
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}kind '{kind}' is not a feed-forward of this design ({', '.join(MLP_KINDS)})")
        if kind == "dense":
            limit = _need(raw, "limit", float)
            if not limit > 0.0:
                raise ConfigError(f"config.json: {where}limit must be positive")
            return cls(kind, _positive(_need(raw, "ff", int), where + "ff"), limit=limit)
        expert, router = _section(raw, "expert", where), _section(raw, "router", where)
        experts = _positive(_need(router, "experts", int), where + "router.experts")
        top = _positive(_need(router, "top", int), where + "router.top")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top ({top}) exceeds router.experts ({experts})")
        groups_raw = _section(router, "groups", where + "router.", required=False)
        groups = keep = 0
        if groups_raw is not None:
            groups = _positive(_need(groups_raw, "count", int), where + "router.groups.count")
            keep = _positive(_need(groups_raw, "keep", int), where + "router.groups.keep")
            if experts % groups or keep > groups or keep * (experts // groups) < top:
                raise ConfigError(f"config.json: {where}router.groups: {groups} groups must divide {experts} experts, and "
                                  f"the {keep} kept ones must hold the {top} choices")
        return cls(kind, _positive(_need(expert, "ff", int), where + "expert.ff"), experts=experts, top=top,
                   groups=groups, keep=keep)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": self.kind, "limit": self.limit}
        router = {"experts": self.experts, "top": self.top}
        if self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"expert": {"ff": self.ff}, "kind": self.kind, "router": router}


@dataclass(frozen=True)
class FidolixAttention:
    """The softmax attention of an ``attention`` layer, or the left side of a ``parallel`` one (which has ``conv``,
    ``window``, ``rot`` and no ``softcap``)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0
    conv: int = 0
    window: int = 0
    rot: Optional[FidolixRotation] = None

    @classmethod
    def from_dict(cls, raw, where: str, left: bool) -> "FidolixAttention":
        heads = _positive(_need(raw, "heads", int), where + "heads")
        kv_heads = _positive(_optional(raw, "kv_heads", int, heads), where + "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(raw, "dim", int), where + "dim")
        vdim = _positive(_optional(raw, "vdim", int, dim), where + "vdim")
        scale = _need(raw, "scale", float)
        if not left:
            softcap = _optional(raw, "softcap", float, 0.0)
            if softcap < 0.0:
                raise ConfigError(f"config.json: {where}softcap must not be negative")
            return cls(heads, kv_heads, dim, vdim, scale, softcap=softcap)
        if vdim != dim:
            raise ConfigError(f"config.json: {where}vdim ({vdim}) must equal dim ({dim}): the values are the keys")
        conv = _optional(raw, "conv", int, 0)
        if conv < 0:
            raise ConfigError(f"config.json: {where}conv must not be negative")
        mask = _section(raw, "mask", where, required=False)
        window = _positive(_need(mask, "size", int), where + "mask.size") if mask is not None else 0
        rot_raw = _section(raw, "rot", where, required=False)
        rot = FidolixRotation.from_dict(rot_raw, where + "rot.") if rot_raw is not None else None
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims ({rot.dims}) exceeds dim ({dim})")
        return cls(heads, kv_heads, dim, vdim, scale, conv=conv, window=window, rot=rot)

    def to_dict(self, left: bool) -> dict:
        raw = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if not left:
            raw["softcap"] = self.softcap
            return raw
        if self.conv:
            raw["conv"] = self.conv
        if self.window:
            raw["mask"] = {"size": self.window}
        if self.rot is not None:
            raw["rot"] = self.rot.to_dict()
        return raw


@dataclass(frozen=True)
class FidolixTimeMix:
    heads: int
    dim: int
    rank: int = 0                    # of the decay's low-rank part; 0: read from the checkpoint (``w1``'s rows)

    @classmethod
    def from_dict(cls, raw, where: str) -> "FidolixTimeMix":
        rank = _optional(raw, "rank", int, 0)
        if rank < 0:
            raise ConfigError(f"config.json: {where}rank must not be negative")
        return cls(_positive(_need(raw, "heads", int), where + "heads"), _positive(_need(raw, "dim", int), where + "dim"), rank)

    def to_dict(self) -> dict:
        raw = {"dim": self.dim, "heads": self.heads}
        if self.rank:
            raw["rank"] = self.rank
        return raw


@dataclass(frozen=True)
class FidolixLayer:
    type: str
    mlp: Optional[FidolixMlp]
    attention: FidolixAttention                      # the mixer of an attention layer, the left side of a parallel one
    right: Optional[FidolixTimeMix] = None
    left_scale: float = 1.0
    right_scale: float = 1.0

    @classmethod
    def from_dict(cls, raw, index: int) -> "FidolixLayer":
        where = f"layers[{index}]."
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: layers[{index}] must be an object")
        kind = _need(raw, "type", str)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design ({', '.join(MIXERS)})")
        mixer = _section(raw, "mixer", where)
        mlp_raw = _section(raw, "mlp", where, required=False)
        mlp = FidolixMlp.from_dict(mlp_raw, where + "mlp.") if mlp_raw is not None else None
        if kind == "attention":
            return cls(kind, mlp, FidolixAttention.from_dict(mixer, where + "mixer.", left=False))
        left = FidolixAttention.from_dict(_section(mixer, "left", where + "mixer."), where + "mixer.left.", left=True)
        right = FidolixTimeMix.from_dict(_section(mixer, "right", where + "mixer."), where + "mixer.right.")
        return cls(kind, mlp, left, right, _optional(mixer, "left_scale", float, 1.0),
                   _optional(mixer, "right_scale", float, 1.0))

    def to_dict(self) -> dict:
        if self.type == "attention":
            mixer = self.attention.to_dict(left=False)
        else:
            mixer = {"left": self.attention.to_dict(left=True), "left_scale": self.left_scale,
                     "right": self.right.to_dict(), "right_scale": self.right_scale}
        return {"type": self.type, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclass(frozen=True)
class FidolixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    side_dim: int                      # 0: no per-layer token input
    loop_start: int
    loop_stop: int
    loop_times: int                    # 1: every layer runs once
    layers: Tuple[FidolixLayer, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FidolixConfig":
        vocab = _positive(_need(raw, "vocab", int), "vocab")
        width = _positive(_need(raw, "width", int), "width")
        norm = _section(raw, "norm", "")
        embedding = _section(raw, "embedding", "", required=False)
        scale = _optional(embedding, "scale", float, 1.0) if embedding is not None else 1.0
        side = _section(raw, "token_side", "", required=False)
        side_dim = _optional(side, "dim", int, 0) if side is not None else 0
        if side_dim < 0:
            raise ConfigError("config.json: token_side.dim must not be negative")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(FidolixLayer.from_dict(layer, i) for i, layer in enumerate(layers))
        loop = _section(raw, "loop", "", required=False)
        start, stop, times = 0, 0, 1
        if loop is not None:
            start, stop = _need(loop, "start", int), _need(loop, "stop", int)
            times = _positive(_need(loop, "times", int), "loop.times")
            if not 0 <= start <= stop <= len(parsed):
                raise ConfigError(f"config.json: loop.start ({start}) and loop.stop ({stop}) must bound layers of the "
                                  f"{len(parsed)} there are")
        return cls(vocab, width, _need(norm, "eps", float), scale, side_dim, start, stop, times, parsed)

    def needs_tensor_shapes(self) -> bool:
        """True if a size is still open that only the checkpoint's tensors give."""
        return any(layer.right is not None and not layer.right.rank for layer in self.layers)

    def with_tensor_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "FidolixConfig":
        """The configuration with the sizes that ``config.json`` leaves to the tensors' shapes filled in."""
        import dataclasses
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.right is not None and not layer.right.rank:
                name = f"l{i}.mix.right.w1"
                shape = shapes.get(name)
                if shape is None or len(shape) != 2 or shape[0] <= 0:
                    raise ConfigError(f"the checkpoint has no matrix '{name}' to read the decay's rank from")
                layer = dataclasses.replace(layer, right=dataclasses.replace(layer.right, rank=int(shape[0])))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.side_dim:
            raw["token_side"] = {"dim": self.side_dim}
        if self.loop_times != 1 or self.loop_stop > self.loop_start:
            raw["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return raw
