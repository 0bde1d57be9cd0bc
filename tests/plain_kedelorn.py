"""A plain, slow restatement of the Kedelorn decoder: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the library; the GPU tests compare the engine with it.

Notation: a sequence of T tokens at positions 0..T-1, width W.  ``P`` maps tensor names to float64 tensors,
``cfg`` is the dictionary of a ``config.json`` of this design, ``p`` a layer's prefix (``"l3."``), ``m`` a layer's
``mixer`` section.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, weight, eps):
    """The layers' norm and the model's last one: the weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def norm_plain(x, weight, eps):
    return unit_rms(x, eps) * weight


def rotary_frequencies(rot):
    """The dims/2 frequencies of a rotation and the factor on its cosines and sines.  Without ``scaling`` these are
    base^(-2i/dims) and 1; with it (YaRN) slow pairs are divided by ``factor``, fast ones stay, pairs between blend."""
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


def rotate(x, positions, rot):
    """x [T, ..., n]: the first rot.dims numbers of the last axis are rotated, number i with number i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    f, magnitude = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
    cos, sin = (torch.cos(angle) * magnitude).view(shape), (torch.sin(angle) * magnitude).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def retention_mixer(h, P, p, m, eps, positions=None):
    """Linear attention with a fixed decay per head, no softmax: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = rotate((h @ P[p + "mix.q"].T).view(T, H, d), positions, m["rot"])
    k = rotate((h @ P[p + "mix.k"].T).view(T, H, d), positions, m["rot"]) * d ** -0.5
    v = (h @ P[p + "mix.v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    out = unit_rms(out, eps).reshape(T, H * dv)
    gate = h @ P[p + "mix.g"].T
    return (out * gate * torch.sigmoid(gate)) @ P[p + "mix.o"].T


def latent_kept(h, P, p, m, eps, positions=None):
    """What a latent-attention layer keeps per position: the normed latent and the one rotated key part."""
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    down = h @ P[p + "mix.dkv"].T
    r = m["kv_rank"]
    c = norm_plain(down[:, :r], P[p + "mix.dkv.norm"], eps)
    k_rot = rotate(down[:, r:], positions, m["rot"])
    return c, k_rot


def softmax_with_sink(scores, sink):
    """scores [H, T, T] (causal), sink [H]: exp(sink) counts once in every row's denominator and brings nothing."""
    T = scores.shape[-1]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    scores = scores.masked_fill(hidden, -math.inf)
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def latent_attention_mixer(h, P, p, m, eps, kept):
    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, k_rot = kept
    q = (h @ P[p + "mix.q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], torch.arange(T), m["rot"])
    k_plain = (c @ P[p + "mix.uk"].T).view(T, H, d)
    v = (c @ P[p + "mix.uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    weights = softmax_with_sink(scores, P[p + "mix.sink"])
    out = torch.einsum("hij,jhd->ihd", weights, v)
    out = out * torch.sigmoid(h @ P[p + "mix.g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ P[p + "mix.o"].T


def expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


# Choice scores nearer than this are a close call for an implementation in bfloat16: the router reads a normed stream
# that carries the rounding of every layer before it (a few hundredths of its spread in the test models), through
# rows of the router's matrix whose length is two to three, and the sigmoid's slope is at most a quarter.
CLOSE_CALL = 0.08
# (layer prefix, token, distance from a tie) of the proposals since the last forward that differed from the choice
# here by more than a close call; they are followed all the same, and the caller decides how many it accepts
FAR_CALLS = []
DECISIONS = [0]          # how many tokens' choices were compared with a proposal since the last forward


def route(h, P, p, mlp, proposed=None):
    """Which experts each token uses, and with which weights: [T, top] indices and [T, top] weights.

    ``proposed`` ([T, top] indices, -1 where nothing is proposed) is another implementation's choice, which is followed:
    where two choice scores are nearer than the other implementation's rounding, either choice is right, and everything
    after it has to be compared along the same path.  A proposal that differs by more than CLOSE_CALL (its weakest
    expert that far below the last chosen one's score, or an expert it leaves out that far above) is noted in
    FAR_CALLS: a router that works has few of them, one that leaves out the correction or the sigmoid has many."""
    router = mlp["router"]
    s = torch.sigmoid(h @ P[p + "mlp.router"].T)
    choice = s + P[p + "mlp.correction"]
    best = torch.topk(choice, router["top"], dim=-1)
    chosen = best.indices.clone()
    if proposed is not None:
        for t in range(h.shape[0]):
            theirs = [int(e) for e in proposed[t]]
            if min(theirs) < 0 or len(set(theirs)) != len(theirs) or max(theirs) >= s.shape[1]:
                continue
            DECISIONS[0] += 1
            if set(theirs) == set(best.indices[t].tolist()):
                continue
            edge = float(best.values[t, -1])
            # how far from a tie the proposal is: its weakest expert below the edge, the strongest one it leaves out above
            below = edge - min(float(choice[t, e]) for e in theirs)
            above = max(float(choice[t, e]) for e in range(s.shape[1]) if e not in theirs) - edge
            if max(below, above) > CLOSE_CALL:
                FAR_CALLS.append((p, t, round(max(below, above), 4)))
            chosen[t] = torch.tensor(theirs)
    return chosen, torch.gather(s, 1, chosen) * router["scale"]


def moe(h, P, p, mlp, proposed=None):
    chosen, weights = route(h, P, p, mlp, proposed)
    out = torch.zeros(h.shape[0], P[p + "mlp.e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += w * expert(h[t], P[p + f"mlp.e{e}.up"], P[p + f"mlp.e{e}.down"])
    if mlp.get("shared"):
        share = torch.sigmoid(h @ P[p + "mlp.shared.sg"].T)
        out = out + share * expert(h, P[p + "mlp.shared.up"], P[p + "mlp.shared.down"])
    return out


def hyper_sublayer(streams, P, prefix, sublayer):
    """streams [s, T, W].  The sublayer reads a mix of the streams; every new stream is a mix of the old ones plus
    its share of the sublayer's result."""
    u = torch.einsum("s,stw->tw", P[prefix + ".in"], streams)
    y = sublayer(u)
    return torch.einsum("sr,stw->rtw", P[prefix + ".mix"], streams) + P[prefix + ".out"][:, None, None] * y[None]


def forward(cfg, P, tokens, layer_outputs=None, proposed=None):
    """Logits [T, vocab] for one sequence of token ids; ``layer_outputs`` (a list) receives the sum of the streams
    after every layer.  ``proposed`` maps a layer's index to the experts another implementation chose there
    ([T, top]; see ``route``)."""
    eps = cfg["norm"]["eps"]
    FAR_CALLS.clear()
    DECISIONS[0] = 0
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = P["embed"][tokens]
    n_streams = cfg.get("streams", 0)
    streams = x[None].repeat(max(n_streams, 1), 1, 1)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]

        def mixer(u):
            h = norm_around_zero(u, P[p + "norm1"], eps)
            if layer["type"] == "retention":
                return retention_mixer(h, P, p, m, eps)
            if m.get("kv_from") is None:
                kept[i] = latent_kept(h, P, p, m, eps)
            return latent_attention_mixer(h, P, p, m, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])

        def feed_forward(u):
            return moe(norm_around_zero(u, P[p + "norm2"], eps), P, p, layer["mlp"],
                       proposed.get(i) if proposed else None)

        if n_streams:
            streams = hyper_sublayer(streams, P, p + "hc1", mixer)
            if layer.get("mlp"):
                streams = hyper_sublayer(streams, P, p + "hc2", feed_forward)
        else:
            streams = streams + mixer(streams[0])[None]
            if layer.get("mlp"):
                streams = streams + feed_forward(streams[0])[None]
        if layer_outputs is not None:
            layer_outputs.append(streams.sum(dim=0))
    x = streams.sum(dim=0)
    return norm_around_zero(x, P["final.norm"], eps) @ P["head"].T


def load_folder(folder):
    """(config dictionary, tensors as float64) of a model folder; reads the safetensors container itself."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (size,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + size])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    P = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        flat = torch.frombuffer(bytearray(raw[8 + size + begin:8 + size + end]), dtype=kinds[info["dtype"]])
        P[name] = flat.reshape(info["shape"]).to(F64)
    return cfg, P


def logits_of(cfg, P, tokens, proposed=None):
    return forward(cfg, P, tokens, proposed=proposed)
