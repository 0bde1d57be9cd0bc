"""Small Fidolix configurations for the tests, and folders with random weights for them.

The weights are drawn so that a fault shows.  Queries and keys are large (peaked attention: a key that is lost, shifted
by one, seen through a window that is one token off or taken from another page moves the logits by far more than
rounding does), the sinks are a few units apart, the gates far from one half, the norms' weights between 0.4 and 1.6,
the decays of the time mixing between "forgets in a few tokens" and "keeps for hundreds", the routers' logits a few
units apart.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def rotation(dims, base, scaling=None):
    raw = {"dims": dims, "base": base}
    if scaling is not None:
        raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return raw


def attention(heads, kv_heads, dim, vdim, scale, softcap, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        mixer["softcap"] = softcap
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right, scales, mlp):
    heads, kv_heads, dim, conv, window, rot, scale = left
    side = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if conv:
        side["conv"] = conv
    if window:
        side["mask"] = {"size": window}
    if rot is not None:
        side["rot"] = rot
    other = {"heads": right[0], "dim": right[1], "rank": right[2]}
    return {"type": "parallel", "mixer": {"left": side, "right": other, "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": mlp}


def config(vocab, width, layers, eps=1e-5, scale=None, side=None, loop=None):
    raw = {"architecture": "Fidolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        raw["embedding"] = {"scale": scale}
    if side is not None:
        raw["token_side"] = {"dim": side}
    if loop is not None:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


STRETCHED = rotation(8, 100.0, (4.0, 16, 4.0, 1.0))
# FA: values wider and narrower than keys; a window of 7 (shorter than a page of 16) and one of 33 (two pages and one);
#     three and two taps; a rotation over half a head with stretched frequencies and one over a whole head without;
#     six experts in three groups of which one is kept (both choices come from it); a layer without a feed-forward; layers 1 and 2 run twice.
FA = config(101, 64, [
    attention(4, 2, 16, 24, 0.25, 20.0, dense(40, 1.0)),
    parallel((4, 2, 16, 3, 7, STRETCHED, 0.3), (2, 16, 5), (0.7, 1.3), moe(24, 6, 2, (3, 1))),
    attention(2, 1, 24, 8, 0.2, None, None),
    parallel((2, 1, 24, 2, 33, rotation(24, 10000.0), 0.25), (4, 8, 3), (1.2, 0.6), dense(36, 2.0))],
    scale=2.5, side=8, loop=(1, 3, 2))
# FB: no token input, no embedding scale, sizes that are multiples of nothing much; a parallel layer first; a window
#     of 4 under five taps; three query heads a key head; eight experts in four groups of which two, three chosen;
#     one layer alone runs three times; every query head with a key head of its own in the attention layer.
FB = config(211, 72, [
    parallel((6, 2, 12, 5, 4, rotation(4, 50.0), 0.35), (3, 20, 9), (1.0, 1.0), moe(20, 8, 3, (4, 2))),
    attention(3, 3, 20, 20, 0.22, 8.0, moe(28, 5, 1)),
    parallel((3, 3, 8, 1, 70, rotation(8, 1000.0, (2.0, 32, 8.0, 2.0)), 0.4), (1, 40, 4), (0.5, 2.0), None)],
    eps=1e-6, loop=(1, 2, 3))
# FC: the head sizes at which bfloat16 prompts run on the tensor cores: 64 in the attention layer and in the left side
#     of one parallel layer, 128 in the other's; windows of 100 and of 64 (a page); four taps; sixteen experts of which
#     one, without groups; heads of 64 and of 32 in the time mixing; the first layer runs twice.
FC = config(300, 128, [
    attention(2, 1, 64, 64, 0.125, 30.0, moe(40, 16, 1)),
    parallel((2, 1, 64, 4, 100, rotation(32, 10000.0, (4.0, 64, 16.0, 1.0)), 0.125), (2, 64, 16), (0.8, 1.1), dense(136, 1.5)),
    parallel((1, 1, 128, 2, 64, rotation(128, 500000.0), 0.09), (4, 32, 8), (1.0, 0.9), moe(48, 4, 2, (2, 1)))],
    scale=3.0, side=4, loop=(0, 1, 2))
# FD: a left side without a convolution, without a window and without a rotation; one group of experts; a time mixing
#     head of 40 numbers; three query heads a key head everywhere; no loop.
FD = config(160, 96, [
    parallel((3, 1, 32, 0, 0, None, 0.18), (2, 40, 6), (0.9, 1.0), moe(32, 4, 2, (1, 1))),
    attention(6, 2, 16, 16, 0.25, 15.0, dense(100, 0.75))], side=12, scale=0.5)
FIDOLIX = {"FA": FA, "FB": FB, "FC": FC, "FD": FD}


def make_folder(folder, raw_config, seed, dtype=torch.float32):
    """A model folder with random weights stored in ``dtype``."""
    from stratakv_b200.config import FidolixConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.models.fidolix import fidolix_spec
    from stratakv_b200.weights.random_init import random_tensors
    from stratakv_b200.weights.safetensors_io import write_safetensors
    typed = FidolixConfig.from_dict(raw_config)
    tensors = random_tensors(expected_tensors(fidolix_spec(typed)), seed, std=0.05, dtype=torch.float32)
    sharpen = (2304.0 / typed.width) ** 0.25
    for name in tensors:
        if name.endswith((".left.q", ".left.k")):
            tensors[name] = tensors[name] * 2.0 * sharpen
        elif name.endswith((".q.b", ".k.b", ".v.b")):
            tensors[name] = tensors[name] * 4.0
        elif name.endswith((".q.norm", ".k.norm")):
            tensors[name] = 1.0 + (tensors[name] - 1.0) * 6.0 + (0.8 if name.endswith(".q.norm") else 0.0)
        elif name.endswith(".left.sink"):
            tensors[name] = 2.0 + tensors[name] * 60.0           # sinks of a few units, as large as the largest scores
        elif name.endswith(".mix.g"):
            tensors[name] = tensors[name] * 5.0
        elif name.endswith((".norm1", ".norm2", ".side.norm", ".right.norm")) or name == "final.norm":
            tensors[name] = 1.0 + (tensors[name] - 1.0) * 6.0    # from 0.4 to 1.6
        elif name.endswith(".mlp.router"):
            tensors[name] = tensors[name] * 8.0
        elif name.endswith((".right.w1", ".right.w2")):
            tensors[name] = tensors[name] * (6.0 if name.endswith("w1") else 24.0)   # the decays move with the token
        elif ".mlp.e" in name and name.endswith((".down", ".up")):
            tensors[name] = tensors[name] * 3.0                  # experts that differ, so that a wrong choice shows
        elif name.endswith(".right.u"):
            tensors[name] = tensors[name] * 6.0                  # the current token counts as much as all before it
        elif name.endswith(".side.gate") or name == "side.embed":
            tensors[name] = tensors[name] * 4.0
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    write_safetensors(folder / "model.safetensors", {n: t.to(dtype) for n, t in tensors.items()})
    return folder
