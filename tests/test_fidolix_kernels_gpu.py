"""The mechanisms of the Fidolix decoder one at a time, each kernel against the plain implementation's function
(tests/plain_fidolix.py): the norm over a whole projection; the short convolution with rotation over portions, unequal
batches, scrambled pages, used slots and one-token steps that run twice; attention with a window and a sink where one
key is made to dominate just inside and just outside the window, at page borders, far back, at the first position and
at the query itself, in prompts and in one-token steps, on the general kernel (also with the keys cut into parts) and on
the tensor-core prompt kernel; the time mixing over portions, batches, used slots and steps that run twice, and a token
hundreds back that a slow head keeps and a fast head has lost; the router (softmax scores, groups, equal scores) and the
gated experts."""
import math

import pytest
import torch

import plain_fidolix as plain

pytestmark = pytest.mark.gpu

F64 = torch.float64
DTYPES = [torch.float32, torch.bfloat16]


def kernels(dtype, head_dim=64):
    from stratakv_b200 import ops
    return ops.kernels_for(dtype, head_dim, verbose=False)


def i32(values):
    return torch.as_tensor(values, dtype=torch.int32).cuda()


def close(got, want, dtype, what="", loose=1.0):
    got, want = got.detach().double().cpu(), want.double()
    allowed = (2e-5 if dtype == torch.float32 else 1.2e-2) * loose * max(1.0, float(want.abs().max()))
    worst = float((got - want).abs().max())
    assert worst <= allowed, f"{what}: off by {worst:.3e} (allowed {allowed:.3e})"


def table_of(rot, positions):
    """[positions, dims / 2, 2] float32 of (cos, sin) from the plain implementation's frequencies."""
    f, magnitude = plain.rotary_frequencies(rot)
    angle = torch.arange(positions, dtype=F64)[:, None] * f[None, :]
    return torch.stack([torch.cos(angle) * magnitude, torch.sin(angle) * magnitude], dim=-1).float().cuda()


def scrambled_table(n_seqs, blocks_each, generator):
    """Every sequence's pages in a random order among all pages (page 0 is left to nobody)."""
    order = (torch.randperm(n_seqs * blocks_each, generator=generator) + 1).view(n_seqs, blocks_each)
    return order.to(torch.int32)


def batch_meta(live, at, counts, slots):
    positions = [p for i in live for p in range(at[i], at[i] + counts[i])]
    token_seq = [s for s, i in enumerate(live) for _ in range(counts[i])]
    cu_q = [0]
    for i in live:
        cu_q.append(cu_q[-1] + counts[i])
    return (i32(positions), i32(token_seq), i32(cu_q), i32([slots[i] for i in live])), cu_q


# ---- the norm over a whole projection ---------------------------------------------------------------------------
def test_projection_norm_over_all_heads_at_once():
    ops = kernels(torch.float32)
    g = torch.Generator().manual_seed(1)
    rows = torch.randn(9, 200, generator=g)
    bias_a, weight_a = torch.randn(72, generator=g), torch.rand(72, generator=g) + 0.5
    weight_b = torch.rand(40, generator=g) + 0.5
    want = rows.double().clone()
    want[:, 8:80] = plain.norm(rows[:, 8:80].double() + bias_a.double(), weight_a.double(), 1e-5)
    want[:, 120:160] = plain.norm(rows[:, 120:160].double(), weight_b.double(), 1e-5)
    got = rows.cuda()
    ops.projection_norm(got, 1e-5, [(8, 72, bias_a.cuda(), weight_a.cuda()), (120, 40, None, weight_b.cuda())])
    close(got, want, torch.float32, "two segments")
    # not one norm per head: the heads of a row share one root mean square
    per_head = plain.norm((rows[:, 8:80].double() + bias_a.double()).view(9, 3, 24), torch.ones(24, dtype=F64), 1e-5)
    assert float((per_head.reshape(9, 72) * weight_a.double() - want[:, 8:80]).abs().max()) > 0.05


# ---- the short convolution, the rotation and the cache write --------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 2, 16, 3, 8, True), (2, 1, 24, 2, 24, True), (3, 3, 8, 5, 4, False),
                                   (1, 1, 80, 4, 80, True), (2, 2, 12, 1, 0, True), (2, 1, 20, 0, 20, True)])
def test_short_convolution_rotation_and_cache_over_portions(dtype, shape):
    heads, kv_heads, dim, taps, rotated, interleaved = shape
    g = torch.Generator().manual_seed(heads * 100 + dim + taps)
    ops = kernels(dtype)
    block_size, channels = 16, (heads + kv_heads) * dim
    rot = {"dims": rotated, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    lengths = [70, 1, 37, 5]
    width = channels + 8                                    # (a row may be wider than its parts)
    rows = [torch.randn(n, width, generator=g) for n in lengths]
    bias = torch.randn(channels, generator=g)
    conv_w = torch.randn(channels, max(taps, 1), generator=g)
    want_q, want_k, want_v = [], [], []
    for r in rows:
        u = r[:, :channels].double() + bias.double()
        y = plain.short_convolution(u, conv_w.double()) if taps else u
        y = y.view(-1, heads + kv_heads, dim)
        if rotated and interleaved:
            turned = plain.rotate_interleaved(y, torch.arange(y.shape[0]), rot)
        elif rotated:                                       # the other layout: number i with number i + rotated / 2
            f, magnitude = plain.rotary_frequencies(rot)
            angle = torch.arange(y.shape[0], dtype=F64)[:, None] * f[None, :]
            c, s = (torch.cos(angle) * magnitude)[:, None], (torch.sin(angle) * magnitude)[:, None]
            a, b = y[..., :rotated // 2], y[..., rotated // 2:rotated]
            turned = torch.cat([a * c - b * s, b * c + a * s, y[..., rotated:]], dim=-1)
        else:
            turned = y
        want_q.append(turned[:, :heads].reshape(-1, heads * dim))
        want_k.append(turned[:, heads:])
        want_v.append(y[:, heads:])
    table = table_of(rot, 128) if rotated else None
    blocks_each = 5
    block_table = scrambled_table(len(lengths), blocks_each, g).cuda()
    k_cache = torch.zeros(len(lengths) * blocks_each + 1, kv_heads, block_size, dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    slots = [5, 0, 3, 2]
    state = torch.full((7, 3 + max(taps, 1) * channels), 1e30, device="cuda")      # what an earlier user left behind
    at, got = [0] * len(lengths), [[] for _ in lengths]

    def step(counts, twice=False):
        live = [i for i, c in enumerate(counts) if c]
        fused = torch.cat([rows[i][at[i]:at[i] + counts[i]] for i in live]).cuda()
        meta, cu_q = batch_meta(live, at, counts, slots)
        q_out = torch.empty(fused.shape[0], heads * dim, dtype=dtype, device="cuda")
        tables = block_table[[i for i in live]].contiguous()
        for _ in range(2 if twice else 1):
            ops.short_conv_rotary(fused, bias.cuda(), conv_w.cuda() if taps else None, taps, table, rotated, interleaved,
                                  tables, q_out, k_cache, v_cache, heads, kv_heads, dim, block_size, True, meta, state, 3)
            ops.short_conv_remember(fused, bias.cuda(), channels, taps, len(live), meta, state, 3)
        for s, i in enumerate(live):
            got[i].append(q_out[cu_q[s]:cu_q[s + 1]].clone())
            at[i] += counts[i]

    step([15, 1, 2, 1])                                     # ends just before a page's border; a first token alone
    step([1, 0, 1, 1], twice=True)                          # one token each; the step runs twice as under a graph
    step([2, 0, 1, 2])                                      # portions shorter than the convolution reaches
    step([52, 0, 33, 1])
    for i, n in enumerate(lengths):
        close(torch.cat(got[i]), want_q[i], dtype, f"queries of sequence {i}", loose=4.0)
        for p in range(n):
            block = int(block_table[i, p // block_size])
            close(k_cache[block, :, p % block_size], want_k[i][p], dtype, f"key {p} of sequence {i}", loose=4.0)
            close(v_cache[block, :, p % block_size], want_v[i][p], dtype, f"value {p} of sequence {i}", loose=4.0)
    assert bool((state[:, :3] == state.new_tensor(1e30)).all())      # what lies before the mixer's own state is left alone


# ---- attention with a window and a sink ---------------------------------------------------------------------------
def plain_windowed(q, k, v, scale, window, sink):
    """[T, H, d] queries over [T, G, d] keys and values of one sequence: the plain left side behind its projections."""
    T, H, d = q.shape
    G = k.shape[1]
    distance = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    seen = (distance >= 0) & ((distance < window) if window else True)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for head in range(H):
        scores = ((q[:, head] @ k[:, head // (H // G)].T) * scale).masked_fill(~seen, -math.inf)
        out[:, head] = plain.softmax_with_sink(scores, sink[head]) @ v[:, head // (H // G)]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 2, 16, 7, 16), (2, 1, 80, 90, 64), (2, 1, 64, 100, 64), (1, 1, 128, 64, 64),
                                   (3, 1, 24, 0, 16)])
def test_a_key_that_dominates_at_the_edges_of_the_window(dtype, shape):
    """One key and the queries that meet it are scaled so that its score stands out among hundreds: the query that is
    window - 1 tokens behind it still returns its value, the next one does not; the same far back without a window, at
    a page's last and first row, at position 0 and at the query itself; whole prompts, a portion after a prefix, and
    one token at a time with the keys cut into parts."""
    heads, kv_heads, dim, window, block_size = shape
    g = torch.Generator().manual_seed(dim + window)
    ops = kernels(dtype, dim if dim in (64, 128) else 64)
    T = 330
    q = torch.randn(T, heads, dim, generator=g).double() * 0.3
    k = torch.randn(T, kv_heads, dim, generator=g).double() * 0.3
    v = torch.randn(T, kv_heads, dim, generator=g).double()
    sink = torch.tensor([1.5, -2.0, 0.5, 3.0][:heads], dtype=F64)
    reach = window if window else T
    marked = [0, block_size - 1, block_size, 200, T - 1]
    direction = torch.zeros(dim, dtype=F64)
    direction[0] = 1.0
    for j in marked:
        k[j] = direction * 6.0
        v[j, :, 0] = 50.0 + j                               # a value nobody else has
        for i in {j, min(T - 1, j + reach - 1), min(T - 1, j + reach)}:
            q[i] = direction * 6.0
    round_trip = (lambda x: x.to(dtype).double())           # what the cache and the query rows hold
    q, k, v = round_trip(q), round_trip(k), round_trip(v)
    scale = 0.5
    want = plain_windowed(q, k, v, scale, window, sink).reshape(T, heads * dim)
    # the marked key's value comes back just inside the window and not just outside it
    if window:
        j = 200
        assert abs(float(want[j + window - 1, 0]) - (50.0 + j)) < 1.0 and abs(float(want[j + window, 0])) < 25.0
    blocks = -(-T // block_size)
    table = scrambled_table(1, blocks, g).cuda()
    k_cache = torch.zeros(blocks + 1, kv_heads, block_size, dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    for p in range(T):
        block = int(table[0, p // block_size])
        k_cache[block, :, p % block_size] = k[p].to(dtype).cuda()
        v_cache[block, :, p % block_size] = v[p].to(dtype).cuda()
    q_rows = q.reshape(T, heads * dim).to(dtype).cuda()
    sink_f = sink.float().cuda()

    def general(first, count, splits=1):
        out = torch.empty(count, heads * dim + 8, dtype=dtype, device="cuda")
        positions, seqs = i32(range(first, first + count)), i32([0] * count)
        scratch_o = torch.empty(count * heads * splits * dim, device="cuda") if splits > 1 else None
        scratch_ml = torch.empty(count * heads * splits * 2, device="cuda") if splits > 1 else None
        ops.attention_general(q_rows[first:first + count].contiguous(), k_cache, v_cache, table, positions, seqs, out,
                              heads, kv_heads, dim, dim, block_size, scale, window, sink=sink_f, splits=splits,
                              scratch_o=scratch_o, scratch_ml=scratch_ml)
        return out[:, :heads * dim]

    close(general(0, T), want, dtype, "a whole prompt")
    close(general(150, T - 150), want[150:], dtype, "a portion after a prefix")
    for p in sorted({0, 1, block_size - 1, block_size, 200, 200 + reach - 1, min(T - 1, 200 + reach), T - 1}):
        if p < T:
            for splits in (1, 2, 5):
                close(general(p, 1, splits), want[p:p + 1], dtype, f"position {p} alone, keys in {splits} parts")
    if dtype == torch.bfloat16 and dim in (64, 128):
        # one token a sequence on the split kernel of the head size's own library, the sink in its merge
        for p in sorted({0, 1, block_size - 1, block_size, 200, 200 + reach - 1, min(T - 1, 200 + reach), T - 1}):
            for splits in (1, 2, 5):
                out = torch.empty(1, heads * dim, dtype=dtype, device="cuda")
                scratch_o = torch.empty(heads * splits * dim, device="cuda") if splits > 1 else None
                scratch_ml = torch.empty(heads * splits * 2, device="cuda") if splits > 1 else None
                ops.attention_decode(q_rows[p:p + 1].contiguous(), k_cache, v_cache, table, i32([p + 1]), out, heads,
                                     kv_heads, dim, block_size, scale, window, splits, scratch_o, scratch_ml, sink=sink_f)
                close(out, want[p:p + 1], dtype, f"the split kernel at position {p}, {splits} pieces", loose=2.0)
    if dtype == torch.bfloat16 and dim in (64, 128) and ops.has_attention_prefill_tc():
        for first in (0, 150):
            count = T - first
            out = torch.empty(count, heads * dim, dtype=dtype, device="cuda")
            ops.attention_prefill_tc(q_rows[first:].contiguous(), k_cache, v_cache, table, i32([0, count]), i32([T]), out,
                                     count, heads, kv_heads, dim, block_size, scale, window, sink=sink_f)
            close(out, want[first:], dtype, f"the tensor-core prompt kernel from {first}", loose=2.0)


# ---- time mixing ------------------------------------------------------------------------------------------------------
def plain_time_mix(h, P, heads, dim, eps):
    return plain.time_mixing(h, P, "x.", {"heads": heads, "dim": dim}, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 16, 5, 64), (4, 8, 3, 40), (1, 40, 4, 72), (2, 64, 16, 128), (3, 96, 8, 64)])
def test_time_mixing_over_portions_batches_and_used_slots(dtype, shape):
    """The kernels between the projections (the mixes, the decay, the recurrence, the finish) with identity-like
    projections, so that what they get and give is known exactly."""
    heads, dim, rank, hidden = shape
    inner = heads * dim
    g = torch.Generator().manual_seed(inner + rank)
    ops = kernels(dtype)
    eps, out_scale = 1e-5, 1.1
    lengths = [90, 1, 37, 20]
    hs = [(torch.randn(n, hidden, generator=g) * 0.7).to(dtype) for n in lengths]
    mu = torch.rand(5, hidden, generator=g)
    mats = {s: (torch.randn(inner, hidden, generator=g) * hidden ** -0.5).to(dtype) for s in "rkvg"}
    w1 = (torch.randn(rank, hidden, generator=g) * 0.3).to(dtype)
    w2 = (torch.randn(inner, rank, generator=g)).to(dtype)
    w0 = torch.randn(inner, generator=g) * 1.5 - 2.0
    bonus, norm_w = torch.rand(heads, dim, generator=g), torch.rand(inner, generator=g) + 0.5
    P = {"x." + s: mats[s].double() for s in "rkvg"}
    P.update({"x.mu." + s: mu[i].double() for i, s in enumerate("rkvgw")})
    P.update({"x.w1": w1.double(), "x.w2": w2.double(), "x.w0": w0.double(), "x.u": bonus.double(),
              "x.norm": norm_w.double(), "x.o": torch.eye(inner, dtype=F64)})
    want = [plain_time_mix(h.double(), P, heads, dim, eps) * out_scale for h in hs]
    slots = [5, 0, 3, 2]
    floats = ops.time_mix_state_floats(hidden, heads, dim)
    state = torch.full((7, 2 + floats), 1e30, device="cuda")          # what an earlier user left behind
    at, got = [0] * len(lengths), [[] for _ in lengths]

    def step(counts, twice=False):
        live = [i for i, c in enumerate(counts) if c]
        h = torch.cat([hs[i][at[i]:at[i] + counts[i]] for i in live]).cuda()
        n = h.shape[0]
        meta, cu_q = batch_meta(live, at, counts, slots)
        out = torch.empty(n, inner + 8, dtype=dtype, device="cuda")
        for _ in range(2 if twice else 1):
            mixes = torch.empty(5, n, hidden, dtype=dtype, device="cuda")
            ops.token_shift_mix(h, mu.cuda(), mixes, heads, dim, meta, state, 2)
            rows = torch.empty(6, n, inner, device="cuda")
            for index, s in enumerate("rkvg"):                  # the library's projection is tested elsewhere
                rows[index] = (mixes[index].double() @ mats[s].double().cuda().T).float()
            lora = (mixes[4].double() @ w1.double().cuda().T).float().contiguous()
            ops.time_mix_decay(lora, rank, w2.t().contiguous().cuda(), w0.cuda(), rows[4])
            ops.time_mix_scan(rows[0], rows[1], rows[2], rows[4], bonus.reshape(-1).cuda(), rows[5], h, len(live), heads,
                              dim, meta, state, 2)
            ops.time_mix_finish(rows[5], rows[3], norm_w.cuda(), eps, out_scale, out, heads, dim)
        assert float(out[:, inner:].float().abs().max()) == 0.0
        for s, i in enumerate(live):
            got[i].append(out[cu_q[s]:cu_q[s + 1], :inner].clone())
            at[i] += counts[i]

    step([15, 1, 2, 1])
    step([1, 0, 1, 1], twice=True)                          # one token each; the step runs twice as under a graph
    step([2, 0, 1, 2])                                      # an even and an odd count: both halves of the state
    step([72, 0, 33, 16])
    for i in range(len(lengths)):
        close(torch.cat(got[i]), want[i], dtype, f"sequence {i}", loose=4.0)
    assert bool((state[:, :2] == state.new_tensor(1e30)).all())


def test_a_token_far_back_that_a_slow_head_keeps():
    """Two heads, decays 0.999 and 0.5 in every channel: 300 tokens after a marked token the first head's output still
    points at its value and the second head's does not."""
    ops = kernels(torch.float32)
    heads, dim, T = 2, 16, 320
    inner = heads * dim
    g = torch.Generator().manual_seed(3)
    r = torch.randn(T, inner, generator=g) * 0.05
    k = torch.randn(T, inner, generator=g) * 0.05
    v = torch.randn(T, inner, generator=g) * 0.05
    k[10], v[10] = 0.0, 0.0
    k[10, 0], k[10, dim] = 4.0, 4.0                         # both heads' first key channel
    v[10, 3], v[10, dim + 3] = 9.0, 9.0
    r[T - 1, 0], r[T - 1, dim] = 2.0, 2.0
    decay = torch.cat([torch.full((T, dim), 0.999), torch.full((T, dim), 0.5)], dim=1)
    out = torch.empty(T, inner, device="cuda")
    state = torch.zeros(2, ops.time_mix_state_floats(8, heads, dim), device="cuda")
    meta = (i32(range(T)), i32([0] * T), i32([0, T]), i32([1]))
    h = torch.zeros(T, 8, device="cuda")
    ops.time_mix_scan(r.cuda(), k.cuda(), v.cuda(), decay.cuda(), torch.zeros(inner, device="cuda"), out, h, 1, heads, dim,
                      meta, state)
    last = out[T - 1].cpu()
    assert abs(float(last[3]) - 2.0 * 4.0 * 9.0 * 0.999 ** (T - 2 - 10)) < 0.5 and abs(float(last[dim + 3])) < 0.05


# ---- the router and the experts ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(6, 2, 3, 1), (8, 3, 4, 2), (16, 2, 2, 1), (5, 1, 0, 0), (4, 4, 1, 1), (12, 4, 3, 2)])
def test_router_with_softmax_scores_and_groups(dtype, shape):
    experts, top, groups, keep = shape
    g = torch.Generator().manual_seed(experts * 10 + top)
    ops = kernels(dtype)
    n, hidden = 50, 64
    h = torch.randn(n, hidden, generator=g).to(dtype)
    router_w = (torch.randn(experts, hidden, generator=g) * 0.4).to(dtype)
    cfg = {"experts": experts, "top": top}
    if groups:
        cfg["groups"] = {"count": groups, "keep": keep}
    want_chosen, want_weights = plain.route(h.double(), {"x.router": router_w.double()}, "x.", cfg)
    chosen = torch.empty(n, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(n, top, device="cuda")
    ops.route_tokens(h.cuda(), router_w.cuda(), None, top, 1.0, True, chosen, weights, softmax=True, groups=groups, keep=keep,
                     renorm_eps=1e-20)
    assert chosen.cpu().tolist() == want_chosen.tolist()
    close(weights, want_weights, dtype, "weights", loose=0.1)
    assert float((weights.sum(dim=-1) - 1.0).abs().max()) < 1e-5


def test_router_with_equal_scores_takes_the_lower_index_and_group():
    ops = kernels(torch.float32)
    h = torch.zeros(3, 16, device="cuda")
    router_w = torch.randn(8, 16).cuda()
    chosen = torch.empty(3, 2, dtype=torch.int32, device="cuda")
    weights = torch.empty(3, 2, device="cuda")
    ops.route_tokens(h, router_w, None, 2, 1.0, True, chosen, weights, softmax=True, groups=4, keep=1, renorm_eps=1e-20)
    assert chosen.cpu().tolist() == [[0, 1]] * 3
    close(weights, torch.full((3, 2), 0.5), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_experts(dtype):
    from stratakv_b200.parts.ffn import pack_gate_up
    ops = kernels(dtype)
    g = torch.Generator().manual_seed(9)
    experts, hidden, ff, n, top = 5, 64, 24, 40, 2
    h = torch.randn(n, hidden, generator=g).to(dtype)
    gate = (torch.randn(experts, ff, hidden, generator=g) * 0.2).to(dtype)
    up = (torch.randn(experts, ff, hidden, generator=g) * 0.2).to(dtype)
    chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    chosen[:, 0][chosen[:, 0] == 3] = 4                     # expert 3 gets nobody ... almost
    chosen[:, 1][chosen[:, 1] == 3] = 4
    offsets = torch.empty(experts + 1, dtype=torch.int32, device="cuda")
    order = torch.empty(n * top, dtype=torch.int32, device="cuda")
    place = torch.empty(n, top, dtype=torch.int32, device="cuda")
    ops.sort_by_expert(chosen.cuda(), experts, offsets, order, place)
    packed = torch.stack([pack_gate_up(gate[e].cuda(), up[e].cuda()) for e in range(experts)]).contiguous()
    hidden_rows = torch.empty(n * top, ff, dtype=dtype, device="cuda")
    ops.expert_linear(h.cuda(), packed, offsets, hidden_rows, rows=order, activation="silu", gated=True)
    for t in range(n):
        for choice in range(top):
            e = int(chosen[t, choice])
            want = plain.silu(h[t].double() @ gate[e].double().T) * (h[t].double() @ up[e].double().T)
            close(hidden_rows[int(place[t, choice])], want, dtype, f"token {t} expert {e}")
