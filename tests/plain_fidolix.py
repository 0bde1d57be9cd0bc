"""A plain, slow restatement of the Fidolix decoder: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the library; the GPU tests compare the engine with it.

Notation: a sequence of T tokens at positions 0..T-1, width W.  ``P`` maps tensor names to float64 tensors,
``cfg`` is the dictionary of a ``config.json`` of this design, ``p`` a tensor prefix (``"l3.mix."``), ``m`` a mixer's
section of the configuration.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def linear(h, P, name, bias=False):
    y = h @ P[name].T
    return y + P[name + ".b"] if bias else y


# ---- the attention mixer ------------------------------------------------------------------------------------------

def capped(scores, cap):
    return cap * torch.tanh(scores / cap) if cap else scores


def attention_mixer(h, P, p, m, eps):
    """Grouped-query attention without positions: biased projections, one RMS norm over all of q and one over all
    of k, capped scores, causal softmax, a sigmoid gate on every output number."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = norm(linear(h, P, p + "q", True), P[p + "q.norm"], eps).view(T, H, d)
    k = norm(linear(h, P, p + "k", True), P[p + "k.norm"], eps).view(T, G, d)
    v = linear(h, P, p + "v", True).view(T, G, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(H):
        g = head // (H // G)
        scores = capped((q[:, head] @ k[:, g].T) * m["scale"], m.get("softcap", 0.0))
        scores = scores.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, g]
    gate = sigmoid(linear(h, P, p + "g"))
    return (out.reshape(T, H * dv) * gate) @ P[p + "o"].T


# ---- the left half of the parallel mixer ------------------------------------------------------------------------

def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def rotary_frequencies(rot):
    """The dims/2 frequencies of a rotation and the factor on its cosines and sines."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(scaling["fast"])), 0)
    hi = min(math.ceil(pair_of(scaling["slow"])), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot):
    """x [T, heads, n]: of the first rot.dims numbers of a head, number 2i is paired with number 2i + 1."""
    dims = rot["dims"]
    f, magnitude = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_with_sink(scores, sink):
    """Rows of scores (-inf where unseen); the denominator also holds exp(sink)."""
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, torch.as_tensor(sink, dtype=F64))
    e = torch.exp(scores - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))


def windowed_mixer(h, P, p, m, positions=None):
    """Queries and keys through a short convolution over time, the values are the convolved keys before they are
    rotated; rotary positions; a sliding window; a sink in the softmax."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(T) if positions is None else positions
    q, k = linear(h, P, p + "q", True), linear(h, P, p + "k", True)
    if m.get("conv"):
        q, k = short_convolution(q, P[p + "q.conv"]), short_convolution(k, P[p + "k.conv"])
    q, k = q.view(T, H, d), k.view(T, G, d)
    v = k.clone()
    if m.get("rot"):
        q, k = rotate_interleaved(q, positions, m["rot"]), rotate_interleaved(k, positions, m["rot"])
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    window = (m.get("mask") or {}).get("size", 0)
    if window:
        seen = seen & (distance < window)
    out = torch.zeros(T, H, d, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        scores = ((q[:, head] @ k[:, g].T) * m["scale"]).masked_fill(~seen, -math.inf)
        out[:, head] = softmax_with_sink(scores, P[p + "sink"][head]) @ v[:, g]
    return out.reshape(T, H * d) @ P[p + "o"].T


# ---- the right half of the parallel mixer -----------------------------------------------------------------------

def shifted_mixes(h, P, p):
    """For each of r, k, v, g, w: h + (previous h - h) * mu, with zeros before the first token."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return {s: h + (before - h) * P[p + "mu." + s] for s in "rkvgw"}


def decays(mix_w, P, p):
    return torch.exp(-torch.exp(torch.tanh(mix_w @ P[p + "w1"].T) @ P[p + "w2"].T + P[p + "w0"]))


def time_mixing(h, P, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    mix = shifted_mixes(h, P, p)
    r = (mix["r"] @ P[p + "r"].T).view(T, H, d)
    k = (mix["k"] @ P[p + "k"].T).view(T, H, d)
    v = (mix["v"] @ P[p + "v"].T).view(T, H, d)
    gate = silu(mix["g"] @ P[p + "g"].T)
    w = decays(mix["w"], P, p).view(T, H, d)
    u = P[p + "u"].view(H, d)
    S = torch.zeros(H, d, d, dtype=F64)                  # [head, key channel, value channel]
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    o = unit_rms(o, eps).reshape(T, H * d) * P[p + "norm"] * gate
    return o @ P[p + "o"].T


def parallel_mixer(h, P, p, m, eps):
    left = windowed_mixer(h, P, p + "left.", m["left"])
    right = time_mixing(h, P, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---- feed-forwards ------------------------------------------------------------------------------------------------

def dense_ff(h, P, p, mlp):
    limit = mlp["limit"]
    g = torch.clamp(h @ P[p + "gate"].T, max=limit)
    u = torch.clamp(h @ P[p + "up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ P[p + "down"].T


# Where the engine computes in bfloat16 its router sees a rounded input, and where two experts (or two groups) score
# nearly alike it may choose the other one: that is no fault.  ``proposed`` ([T, top] expert indices, -1 where unknown)
# is the engine's choice; it is followed where its experts score at least CLOSE_CALL of what the plain choice's do,
# and counted in FAR_CALLS otherwise (DECISIONS counts all choices that were compared).  The test models' routers are
# sharp and their later runs see a stream that rounding has moved by a few hundredths, hence the wide call; float32
# runs follow nobody and hold every choice.
CLOSE_CALL = 0.6
FAR_CALLS, DECISIONS = [], [0]


def route(h, P, p, router, proposed=None):
    """Per token: the chosen experts and their weights."""
    E, top = router["experts"], router["top"]
    s = torch.softmax(h @ P[p + "router"].T, dim=-1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        size = E // groups["count"]
        best = s.view(-1, groups["count"], size).max(dim=-1).values
        kept = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros(s.shape[0], groups["count"], dtype=torch.bool).scatter_(1, kept, True)
        allowed = allowed.repeat_interleave(size, dim=1)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    if proposed is not None:
        for t in range(s.shape[0]):
            theirs = proposed[t]
            if int(theirs.min()) < 0 or set(theirs.tolist()) == set(chosen[t].tolist()):
                continue
            DECISIONS[0] += 1
            if float(s[t, theirs].sum()) >= CLOSE_CALL * float(s[t, chosen[t]].sum()):
                chosen[t] = theirs
            else:
                FAR_CALLS.append((p, t))
        DECISIONS[0] += s.shape[0]
    weights = s.gather(1, chosen)
    return chosen, weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)


def expert(h, P, p):
    return (silu(h @ P[p + "gate"].T) * (h @ P[p + "up"].T)) @ P[p + "down"].T


def moe(h, P, p, mlp, proposed=None):
    chosen, weights = route(h, P, p, mlp["router"], proposed)
    y = torch.zeros(h.shape[0], P[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            y[t] += w * expert(h[t:t + 1], P, f"{p}e{e}.")[0]
    return y


def feed_forward(h, P, p, mlp, proposed=None):
    return dense_ff(h, P, p, mlp) if mlp["kind"] == "dense" else moe(h, P, p, mlp, proposed)


# ---- the model ------------------------------------------------------------------------------------------------------

def token_side(x, tokens, P, i, dim, eps):
    p = f"l{i}.side."
    e = P["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ P[p + "gate"].T) * e) @ P[p + "proj"].T
    return x + unit_rms(y, eps) * P[p + "norm"]


def layer(x, tokens, cfg, P, i, proposed=None):
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = norm(x, P[p + "norm1"], eps)
    if spec["type"] == "attention":
        branch = attention_mixer(h, P, p + "mix.", spec["mixer"], eps)
    else:
        branch = parallel_mixer(h, P, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp"):
        branch = branch + feed_forward(norm(x, P[p + "norm2"], eps), P, p + "mlp.", spec["mlp"], proposed)
    x = x + branch
    side = (cfg.get("token_side") or {}).get("dim", 0)
    return token_side(x, tokens, P, i, side, eps) if side else x


def layer_runs(cfg):
    """The layers in the order they run, and the runs before which the embedding's output is added again."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order, again = list(range(loop["start"])), set()
    for time in range(loop["times"]):
        if time > 0 and loop["stop"] > loop["start"]:
            again.add(len(order))
        order += list(range(loop["start"], loop["stop"]))
    return order + list(range(loop["stop"], n)), again


def forward(cfg, P, tokens, layer_outputs=None, proposed=None):
    """Logits [T, vocab] of one sequence; ``layer_outputs`` (a list) gets the stream after every run of a layer;
    ``proposed``: run index -> the experts another implementation chose there (see ``route``)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    first = P["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x = first
    order, again = layer_runs(cfg)
    for run, i in enumerate(order):
        if run in again:
            x = x + first
        x = layer(x, tokens, cfg, P, i, proposed.get(run) if proposed else None)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return norm(x, P["final.norm"], cfg["norm"]["eps"]) @ P["head"].T


def load_folder(folder):
    """``(cfg, P)`` of a model folder; floating tensors widened to float64."""
    import numpy as np
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    size = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + size])
    data = raw[8 + size:]
    P = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        chunk = np.frombuffer(data[lo:hi], dtype=np.uint8)
        if info["dtype"] == "BF16":
            bits = chunk.view(np.uint16).astype(np.uint32) << 16
            value = torch.from_numpy(bits.view(np.float32).copy())
        elif info["dtype"] == "F32":
            value = torch.from_numpy(chunk.view(np.float32).copy())
        elif info["dtype"] == "F16":
            value = torch.from_numpy(chunk.view(np.float16).astype(np.float32))
        elif info["dtype"] == "I32":
            P[name] = torch.from_numpy(chunk.view(np.int32).copy()).view(info["shape"])
            continue
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        P[name] = value.view(info["shape"]).to(F64)
    return cfg, P


def logits_of(cfg, P, tokens, proposed=None):
    return forward(cfg, P, tokens, proposed=proposed).to(torch.float32).numpy()
