"""Typed configuration of the Kedelorn decoder, read from its ``config.json``.

The file names the design under ``architecture`` and lists its layers, each with its own mixer and sizes::

    {"architecture": "Kedelorn", "vocab": V, "width": W, "norm": {"eps": e}, "streams": s | absent,
     "layers": [
       {"type": "retention",
        "mixer": {"heads": H, "dim": d, "vdim": dv, "decay": [per head], "rot": {"dims": n, "base": b, "scaling": ...}},
        "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k, "scale": c},
                "shared": {"ff": Fs} | absent} | null},
       {"type": "latent_attention",
        "mixer": {"heads": H, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": r, "scale": c, "kv_from": j | absent,
                  "rot": {"dims": dr, "base": b, "scaling": {"factor": f, "original": n, "fast": x, "slow": y} | absent}},
        "mlp": ...}]}

``streams`` absent: one residual stream and the plain residual sum.  Every size and every constant that differs
between models of the design comes from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError, _need, _optional
from .zepavik import _positive, _section

ARCHITECTURE = "Kedelorn"
MIXERS = ("retention", "latent_attention")
MLP_KINDS = ("moe",)


@dataclass(frozen=True)
class KedelornRotation:
    dims: int
    base: float
    factor: float = 0.0              # 0: no scaling of the frequencies
    original: int = 0
    fast: float = 0.0
    slow: float = 0.0

    @classmethod
    def from_dict(cls, raw, where: str) -> "KedelornRotation":
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
        if not factor > 0.0:
            raise ConfigError(f"config.json: {where}scaling.factor must be positive")
        fast, slow = _need(scaling, "fast", float), _need(scaling, "slow", float)
        if not (fast > 0.0 and slow > 0.0):
            raise ConfigError(f"config.json: {where}scaling.fast and scaling.slow must be positive")
        return cls(dims, base, factor, _positive(_need(scaling, "original", int), where + "scaling.original"), fast, slow)

    def to_dict(self) -> dict:
        raw = {"base": self.base, "dims": self.dims}
        if self.factor:
            raw["scaling"] = {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}
        return raw


@dataclass(frozen=True)
class KedelornMlp:
    ff: int
    experts: int
    top: int
    scale: float
    shared_ff: int = 0               # 0: no shared expert
    kind: str = "moe"

    @classmethod
    def from_dict(cls, raw, where: str) -> "KedelornMlp":
        kind = _optional(raw, "kind", str, "moe")
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}kind '{kind}' is not a feed-forward of this design")
        expert, router = _section(raw, "expert", where), _section(raw, "router", where)
        experts = _positive(_need(router, "experts", int), where + "router.experts")
        top = _positive(_need(router, "top", int), where + "router.top")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top ({top}) exceeds router.experts ({experts})")
        shared = _section(raw, "shared", where, required=False)
        return cls(_positive(_need(expert, "ff", int), where + "expert.ff"), experts, top, _need(router, "scale", float),
                   _positive(_need(shared, "ff", int), where + "shared.ff") if shared is not None else 0, kind)

    def to_dict(self) -> dict:
        raw = {"expert": {"ff": self.ff}, "kind": self.kind,
               "router": {"experts": self.experts, "scale": self.scale, "top": self.top}}
        if self.shared_ff:
            raw["shared"] = {"ff": self.shared_ff}
        return raw


@dataclass(frozen=True)
class KedelornLayer:
    """One layer.  Retention uses heads, dim, vdim, decay and rot; latent attention heads, dim, rot_dim, vdim, kv_rank,
    scale, rot and kv_from (None: a latent of its own)."""
    type: str
    mlp: Optional[KedelornMlp]
    heads: int
    dim: int
    vdim: int
    rot: Optional[KedelornRotation]
    decay: Tuple[float, ...] = ()
    rot_dim: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, raw, index: int) -> "KedelornLayer":
        where = f"layers[{index}]."
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: layers[{index}] must be an object")
        kind = _need(raw, "type", str)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design ({', '.join(MIXERS)})")
        mixer = _section(raw, "mixer", where)
        mlp_raw = _section(raw, "mlp", where, required=False)
        mlp = KedelornMlp.from_dict(mlp_raw, where + "mlp.") if mlp_raw is not None else None
        heads = _positive(_need(mixer, "heads", int), where + "mixer.heads")
        dim = _positive(_need(mixer, "dim", int), where + "mixer.dim")
        vdim = _positive(_optional(mixer, "vdim", int, dim), where + "mixer.vdim")
        rot_raw = _section(mixer, "rot", where + "mixer.", required=False)
        rot = KedelornRotation.from_dict(rot_raw, where + "mixer.rot.") if rot_raw is not None else None
        if kind == "retention":
            decay = mixer.get("decay")
            if (not isinstance(decay, list) or len(decay) != heads
                    or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 <= d <= 1.0 for d in decay)):
                raise ConfigError(f"config.json: {where}mixer.decay must list one number from 0 to 1 per head")
            if rot is not None and rot.dims > dim:
                raise ConfigError(f"config.json: {where}mixer.rot.dims ({rot.dims}) exceeds mixer.dim ({dim})")
            return cls(kind, mlp, heads, dim, vdim, rot, decay=tuple(float(d) for d in decay))
        rot_dim = _optional(mixer, "rot_dim", int, 0)
        if rot_dim < 0 or (rot_dim > 0) != (rot is not None) or (rot is not None and rot.dims > rot_dim):
            raise ConfigError(f"config.json: {where}mixer.rot_dim and mixer.rot go together, rot.dims within rot_dim")
        kv_from = mixer.get("kv_from")
        if kv_from is not None:
            kv_from = _need(mixer, "kv_from", int)
            if not 0 <= kv_from < index:
                raise ConfigError(f"config.json: {where}mixer.kv_from ({kv_from}) must name an earlier layer")
        return cls(kind, mlp, heads, dim, vdim, rot, rot_dim=rot_dim,
                   kv_rank=_positive(_need(mixer, "kv_rank", int), where + "mixer.kv_rank"),
                   scale=_need(mixer, "scale", float), kv_from=kv_from)

    def to_dict(self) -> dict:
        mixer = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.rot is not None:
            mixer["rot"] = self.rot.to_dict()
        if self.type == "retention":
            mixer["decay"] = list(self.decay)
        else:
            mixer.update(kv_rank=self.kv_rank, scale=self.scale)
            if self.rot_dim:
                mixer["rot_dim"] = self.rot_dim
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": dict(sorted(mixer.items())),
                "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclass(frozen=True)
class KedelornConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int                       # 0: one stream and the plain residual sum
    layers: Tuple[KedelornLayer, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KedelornConfig":
        vocab = _positive(_need(raw, "vocab", int), "vocab")
        width = _positive(_need(raw, "width", int), "width")
        norm = _section(raw, "norm", "")
        streams = raw.get("streams")
        streams = 0 if streams is None else _positive(_need(raw, "streams", int), "streams")
        if streams > 8:
            raise ConfigError(f"config.json: streams ({streams}) is not supported (at most 8)")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(KedelornLayer.from_dict(layer, i) for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            if layer.kv_from is None:
                continue
            source = parsed[layer.kv_from]
            if source.type != "latent_attention" or source.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {layer.kv_from}, "
                                  "which has no latent of its own")
            if (source.kv_rank, source.rot_dim, source.rot) != (layer.kv_rank, layer.rot_dim, layer.rot):
                raise ConfigError(f"config.json: layers[{i}] uses the latent of layer {layer.kv_from} "
                                  "but differs from it in kv_rank, rot_dim or rot")
        return cls(vocab, width, _need(norm, "eps", float), streams, parsed)

    def to_dict(self) -> dict:
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.streams:
            raw["streams"] = self.streams
        return raw
