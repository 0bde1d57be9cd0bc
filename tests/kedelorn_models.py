"""Small Kedelorn configurations for the tests, and folders with random weights for them.

The weights are drawn so that a fault shows.  Queries and the keys' up-projection are large (peaked attention: a key
that is lost, shifted by one or taken from another page moves the logits by far more than rounding does), the sinks
are a few units apart, the gates far from one half, the decays of the retention layers between "forgets in a few
tokens" and "never forgets", the streams' mixing matrices far from the identity, the router's corrections as large
as the differences between its scores.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def moe(ff, experts, top, scale, shared=0):
    raw = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        raw["shared"] = {"ff": shared}
    return raw


def rotation(dims, base, scaling=None):
    raw = {"dims": dims, "base": base}
    if scaling is not None:
        raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return raw


def retention(heads, dim, vdim, decay, rot, mlp):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": rot},
            "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, rot, mlp, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def config(vocab, width, layers, streams=None, eps=1e-5):
    raw = {"architecture": "Kedelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    return raw


# stretched frequencies whose ramp runs over the middle pairs of eight (pairs 0 and 1 stay or blend, 2 and 3 are slowed)
STRETCHED = rotation(8, 10000.0, (8.0, 64, 4.0, 1.0))
# KA: three streams; retention first (three heads, values wider than keys, a rotation over half a head, one decay
#     of exactly one and one that forgets within a few tokens), a latent layer whose latent is wider than a head, a
#     layer without a feed-forward, and a last layer with other heads and sizes on the latent of layer 1 across one
#     other; five experts of which two, one shared expert; then one of three experts without a shared one.
KA = config(101, 64, [retention(3, 16, 24, (1.0, 0.5, 0.96875), rotation(8, 100.0), moe(40, 5, 2, 1.5, shared=24)),
                      latent(3, 16, 8, 8, 40, 0.3, STRETCHED, moe(32, 3, 1, 1.0)),
                      retention(2, 8, 8, (0.9, 0.0), rotation(8, 50.0), None),
                      latent(2, 24, 8, 16, 40, 0.25, STRETCHED, moe(40, 5, 2, 1.5, shared=24), kv_from=1)], streams=3)
# KB: no streams at all (the plain residual sum); sizes that are multiples of nothing much; a rotation without
#     stretched frequencies on the latent layers; seven experts of which three, all of four, and a shared expert wider
#     than the routed ones; a latent layer first, which lends to the last.
PLAIN_TWELVE = rotation(12, 3000.0)
KB = config(211, 72, [latent(5, 20, 12, 12, 24, 0.22, PLAIN_TWELVE, moe(52, 7, 3, 0.75, shared=60)),
                      retention(5, 20, 12, (0.75, 0.875, 0.9375, 0.984375, 0.998046875), rotation(20, 1e6), moe(36, 4, 4, 2.0)),
                      latent(1, 40, 12, 40, 24, 0.15, PLAIN_TWELVE, None, kv_from=0),
                      latent(2, 28, 12, 20, 24, 0.2, PLAIN_TWELVE, moe(52, 7, 3, 0.75, shared=60), kv_from=0)], eps=1e-6)
# KC: one stream WITH its connection tensors; heads of 128 keys in the retention layers (their kernels then reserve
#     more shared memory than a block has by default) and of 64 and 32 in the latent ones, a latent of 64 and a
#     rotated part as wide as the unrotated one; sixteen experts of which one.
KC = config(300, 128, [retention(2, 128, 64, (0.99, 0.999), rotation(128, 10000.0), moe(64, 16, 1, 2.5, shared=72)),
                       latent(4, 32, 32, 64, 64, 0.125, rotation(32, 20000.0, (4.0, 256, 32.0, 1.0)), moe(136, 2, 2, 1.0)),
                       latent(2, 64, 32, 32, 64, 0.1, rotation(32, 20000.0, (4.0, 256, 32.0, 1.0)), None, kv_from=1),
                       retention(4, 32, 160, (0.5, 0.9, 0.99, 1.0), rotation(16, 500.0), moe(64, 16, 1, 2.5, shared=72))],
            streams=1)
# KD: two streams; both latent layers have heads whose unrotated and rotated parts together are as wide as their values,
#     64 numbers, the size at which prompts in bfloat16 make every head's keys and attend on the tensor cores; the
#     second one borrows the first one's cache across a retention layer, with other heads; twelve experts of which two.
ROTATED_SIXTEEN = rotation(16, 20000.0, (4.0, 128, 16.0, 1.0))
KD = config(160, 64, [latent(2, 48, 16, 64, 32, 0.12, ROTATED_SIXTEEN, moe(24, 12, 2, 2.0, shared=32)),
                      retention(2, 16, 16, (0.984375, 0.998046875), rotation(16, 1e6), moe(24, 12, 2, 2.0, shared=32)),
                      latent(3, 48, 16, 64, 32, 0.1, ROTATED_SIXTEEN, moe(24, 12, 2, 2.0, shared=32), kv_from=0)], streams=2)
KEDELORN = {"KA": KA, "KB": KB, "KC": KC, "KD": KD}


def make_folder(folder, raw_config, seed, dtype=torch.float32):
    """A model folder with random weights stored in ``dtype``."""
    from stratakv_b200.config import KedelornConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.models.kedelorn import kedelorn_spec
    from stratakv_b200.weights.random_init import random_tensors
    from stratakv_b200.weights.safetensors_io import write_safetensors
    typed = KedelornConfig.from_dict(raw_config)
    tensors = random_tensors(expected_tensors(kedelorn_spec(typed)), seed, std=0.05, dtype=torch.float32)
    sharpen = (2304.0 / typed.width) ** 0.5
    for name in tensors:
        layer = int(name[1:name.index(".")]) if name.startswith("l") and name[1].isdigit() else None
        kind = typed.layers[layer].type if layer is not None else None
        if kind == "latent_attention" and name.endswith((".mix.q", ".mix.uk")):
            tensors[name] = tensors[name] * (sharpen if name.endswith(".mix.q") else sharpen ** 0.5)
        elif name.endswith(".mix.dkv"):
            # the rotated key part is not normed: make it as large as the normed latent's numbers
            tensors[name] = tensors[name] * 6.0
        elif name.endswith(".mix.dkv.norm"):
            tensors[name] = 1.0 + (tensors[name] - 1.0) * 8.0
        elif name.endswith(".mix.sink"):
            tensors[name] = 3.0 + tensors[name] * 80.0            # sinks of a few units, as large as the largest scores
        elif name.endswith(".mix.g"):
            tensors[name] = tensors[name] * 5.0
        elif name.endswith((".norm1", ".norm2")) or name == "final.norm":
            tensors[name] = tensors[name] * 6.0                   # 1 + w from 0.4 to 1.6
        elif name.endswith(".mlp.router"):
            tensors[name] = tensors[name] * 6.0
        elif name.endswith(".mlp.correction"):
            tensors[name] = tensors[name] * 6.0
        elif name.endswith(".mlp.shared.sg"):
            tensors[name] = tensors[name] * 6.0
        elif name.endswith((".in", ".out")) and ".hc" in name:
            tensors[name] = 1.0 + (tensors[name] - 1.0) * 6.0
        elif name.endswith(".mix") and ".hc" in name:
            s = tensors[name].shape[0]
            tensors[name] = torch.eye(s) * 0.8 + (tensors[name] - torch.eye(s)) * 10.0 + 0.1
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    write_safetensors(folder / "model.safetensors", {n: t.to(dtype) for n, t in tensors.items()})
    return folder
