"""The mechanisms of the Kedelorn decoder one at a time, each kernel against the plain implementation's function
(tests/plain_kedelorn.py): retention over portions, unequal batches, chunk borders, used slots and a one-token step
that runs twice; the finish of the latent layer's projection (rotated query parts with stretched frequencies, the
normed latent and the shared rotated key part into scrambled pages); attention over the cached rows with a sink and a
gate per head, with one key made to dominate far back, at page borders, at the first position and at the query
itself; the router (a correction that chooses and does not weigh, equal scores, the shared expert's gate), the sort by
expert, the experts' projections and their weighted sum; and the pass over several residual streams."""
import math

import pytest
import torch

import plain_kedelorn as plain

pytestmark = pytest.mark.gpu

F64 = torch.float64
DTYPES = [torch.float32, torch.bfloat16]


def kernels(dtype, head_dim=16):
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


def selecting(width, start, count):
    """A [count, width] matrix that picks columns start .. start + count of a row."""
    m = torch.zeros(count, width, dtype=F64)
    m[torch.arange(count), start + torch.arange(count)] = 1.0
    return m


# ---- retention --------------------------------------------------------------------------------------------------
def plain_retention(rows, heads, dim, vdim, decay, rot, eps):
    """The plain mixer on rows that already are [q | k | v | gate]: its projections pick the columns, Wo is one."""
    width = rows.shape[1]
    P = {"l0.mix.q": selecting(width, 0, heads * dim), "l0.mix.k": selecting(width, heads * dim, heads * dim),
         "l0.mix.v": selecting(width, 2 * heads * dim, heads * vdim),
         "l0.mix.g": selecting(width, 2 * heads * dim + heads * vdim, heads * vdim),
         "l0.mix.o": torch.eye(heads * vdim, dtype=F64)}
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": rot}
    return plain.retention_mixer(rows.double(), P, "l0.", m, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 16, 24, 8, (1.0, 0.5, 0.96875)), (2, 128, 64, 128, (0.99, 0.0)),
                                   (4, 32, 160, 16, (0.5, 0.9, 0.999, 1.0)), (1, 6, 2, 2, (0.75,))])
def test_retention_over_portions_batches_and_used_slots(dtype, shape):
    heads, dim, vdim, rotated, decay = shape
    g = torch.Generator().manual_seed(heads * 100 + dim)
    ops = kernels(dtype)
    eps, rot = 1e-5, {"dims": rotated, "base": 100.0}
    lengths = [150, 1, 37, 66]                              # sequences of a batch; 32 tokens are one chunk of a prompt
    width = 2 * heads * (dim + vdim) + 8                    # (a row may be wider than its parts)
    rows = [torch.randn(n, width, generator=g) for n in lengths]
    want = [plain_retention(r, heads, dim, vdim, decay, rot, eps) for r in rows]
    table = table_of(rot, 256)
    slots = [5, 0, 3, 2]
    state = torch.full((7, 2 * heads * dim * vdim + 4), 1e30, device="cuda")      # what an earlier user left behind
    decay_t = torch.tensor(decay, dtype=torch.float32).cuda()
    at = [0] * len(lengths)
    got = [[] for _ in lengths]

    def step(counts, twice=False):
        live = [i for i, c in enumerate(counts) if c]
        fused = torch.cat([rows[i][at[i]:at[i] + counts[i]] for i in live]).cuda()
        positions = [p for i in live for p in range(at[i], at[i] + counts[i])]
        token_seq = [s for s, i in enumerate(live) for _ in range(counts[i])]
        cu_q = [0]
        for i in live:
            cu_q.append(cu_q[-1] + counts[i])
        longest = max(counts)
        need = ops.retention_scratch(len(live), longest, heads, dim, vdim)
        scratch = torch.empty(max(need, 1), device="cuda")
        out = torch.empty(fused.shape[0], heads * vdim + 8, dtype=dtype, device="cuda")
        meta = (i32(positions), i32(token_seq), i32(cu_q), i32([slots[i] for i in live]))
        for _ in range(2 if twice else 1):
            ops.retention(fused.clone(), table, rotated, decay_t, eps, out, state, meta, heads, dim, vdim, longest, scratch)
        assert float(out[:, heads * vdim:].float().abs().max()) == 0.0
        for s, i in enumerate(live):
            got[i].append(out[cu_q[s]:cu_q[s + 1], :heads * vdim].clone())
            at[i] += counts[i]

    step([31, 1, 2, 33])                                    # ends just before, and just after, a chunk's border
    step([1, 0, 1, 1], twice=True)                          # one token each; the step runs twice as under a graph
    step([66, 0, 34, 32])                                   # portions that start inside a chunk of the sequence
    step([2, 0, 0, 0])
    for _ in range(50):
        step([1, 0, 0, 0], twice=True)
    assert at == lengths
    for i, n in enumerate(lengths):
        close(torch.cat(got[i]), want[i], dtype, f"sequence {i} of {n} tokens", loose=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_retention_remembers_one_far_token(dtype):
    """A head that never forgets (decay 1) gives a token 300 positions back its full weight; a head with decay 0.5
    has forgotten it; a head with decay 0 sees only the newest token.  The far token's key meets the queries with
    weight 8, those between with 0.02, the newest with 1."""
    ops = kernels(dtype)
    g = torch.Generator().manual_seed(9)
    heads, dim, vdim, n, eps = 3, 8, 4, 301, 1e-6
    decay = (1.0, 0.5, 0.0)
    far, new = torch.tensor([1.0, -1.0, 2.0, 0.5]), torch.tensor([0.0, 0.0, 0.0, 3.0])
    rows = torch.zeros(n, 2 * heads * (dim + vdim))
    k0, v0, g0 = heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim
    rows[:, g0:] = 1.0
    rows[:, v0:g0] = torch.randn(n, heads * vdim, generator=g)
    for head in range(heads):
        rows[:, head * dim + 2] = 1.0                                      # every query: a unit vector (not a rotated one)
        rows[:, k0 + head * dim + 2] = 0.02
        rows[:, k0 + head * dim + 3] = 1.0                                 # (most of a key is across the queries)
        rows[0, k0 + head * dim + 2] = 8.0
        rows[0, v0 + head * vdim:v0 + (head + 1) * vdim] = far
        rows[n - 1, k0 + head * dim + 2] = 1.0
        rows[n - 1, v0 + head * vdim:v0 + (head + 1) * vdim] = new
    rot = {"dims": 2, "base": 10.0}
    want = plain_retention(rows, heads, dim, vdim, decay, rot, eps)
    rot_table = table_of(rot, n)
    state = torch.zeros(1, 2 * heads * dim * vdim, device="cuda")
    decay_t = torch.tensor(decay).cuda()
    outs = []
    for first, count in ((0, 200), (200, 100), (300, 1)):
        meta = (i32(range(first, first + count)), i32([0] * count), i32([0, count]), i32([0]))
        need = ops.retention_scratch(1, count, heads, dim, vdim)
        out = torch.empty(count, heads * vdim, dtype=dtype, device="cuda")
        ops.retention(rows[first:first + count].cuda(), rot_table, 2, decay_t, eps, out, state, meta, heads, dim,
                      vdim, count, torch.empty(max(need, 1), device="cuda"))
        outs.append(out)
    got = torch.cat(outs)
    close(got, want, dtype, "all positions", loose=4.0)
    last = got[-1].float().cpu().view(heads, vdim)
    cosine = lambda a, b: float((a * b).sum() / (a.norm() * b.norm()))
    assert cosine(last[0], far) > 0.97, "the head that never forgets has lost the far token"
    assert cosine(last[1], new) > 0.97 and cosine(last[2], new) > 0.9999, "a head that forgets has kept the far token"


# ---- latent attention ---------------------------------------------------------------------------------------------
STRETCHED = {"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 16, 8, 40, STRETCHED), (2, 20, 12, 24, {"dims": 12, "base": 3000.0}),
                                   (1, 8, 16, 8, {"dims": 10, "base": 50.0})])
def test_finish_of_the_latent_projection(dtype, shape):
    """Rotated query parts behind the place of each head's folded query, the unrotated ones apart; the latent divided by
    its root mean square, times its weight, and the rotated shared key part behind it, into scrambled pages."""
    heads, dim, rope_dim, rank, rot = shape
    g = torch.Generator().manual_seed(rank)
    ops = kernels(dtype)
    block, eps, key_dim = 16, 1e-4, rank + rope_dim
    positions = [0, 1, 15, 16, 17, 63, 64, 100, 3, 31, 32]
    token_seq = [0] * 8 + [1] * 3
    n = len(positions)
    q_width = heads * (dim + rope_dim)
    rows = torch.randn(n, q_width + key_dim + heads + 5, generator=g) * 2
    gamma = torch.randn(rank, generator=g)
    table = scrambled_table(2, 7, g)
    cache = torch.zeros(15, 1, block, key_dim, dtype=dtype, device="cuda")
    q_plain = torch.empty(n, heads * dim, dtype=dtype, device="cuda")
    q_folded = torch.zeros(n, heads * key_dim, dtype=dtype, device="cuda")
    ops.latent_finish(rows.cuda(), q_plain, q_folded, cache, i32(positions), i32(token_seq), table.cuda(), heads, dim,
                      rope_dim, rank, block, rotation=table_of(rot, 128), rotated=rot["dims"], latent_offset=q_width,
                      latent_gamma=gamma.float().cuda(), eps=eps)
    where = torch.tensor(positions)
    q = rows[:, :q_width].double().view(n, heads, dim + rope_dim)
    close(q_plain.view(n, heads, dim), q[:, :, :dim], dtype, "unrotated query parts")
    close(q_folded.view(n, heads, key_dim)[:, :, rank:], plain.rotate(q[:, :, dim:], where, rot), dtype, "rotated query parts")
    assert float(q_folded.view(n, heads, key_dim)[:, :, :rank].float().abs().max()) == 0.0       # left to the folding
    down = rows[:, q_width:q_width + key_dim].double()
    latent = plain.norm_plain(down[:, :rank], gamma.double(), eps)
    key_part = plain.rotate(down[:, rank:], where, rot)
    for t in range(n):
        page = int(table[token_seq[t], positions[t] // block])
        row = cache[page, 0, positions[t] % block]
        close(row[:rank], latent[t], dtype, f"latent of token {t}")
        close(row[rank:], key_part[t], dtype, f"key part of token {t}")
    # whole query heads [unrotated | rotated] in one place, for steps that make every head's keys
    q_whole = torch.empty(n, q_width, dtype=dtype, device="cuda")
    ops.latent_finish(rows.cuda(), None, None, cache, i32(positions), i32(token_seq), table.cuda(), heads, dim, rope_dim,
                      rank, block, rotation=table_of(rot, 128), rotated=rot["dims"], write_cache=False, q_whole=q_whole)
    whole = torch.cat([q[:, :, :dim], plain.rotate(q[:, :, dim:], where, rot)], dim=-1)
    close(q_whole.view(n, heads, dim + rope_dim), whole, dtype, "whole query heads")
    # a layer that attends over another's cache writes nothing
    before = cache.clone()
    ops.latent_finish(rows.cuda(), q_plain, q_folded, cache, i32([p + 1 for p in positions]), i32(token_seq), table.cuda(),
                      heads, dim, rope_dim, rank, block, rotation=table_of(rot, 128), rotated=rot["dims"], write_cache=False)
    assert torch.equal(cache, before)


def plain_sink_attention(q, rows, rank, scale, sink, gate):
    """q [T, H, key_dim] against the cached rows [T, key_dim] of one sequence (keys: the whole row; values: its first
    ``rank`` numbers); a sink per head in the denominator; every head's output times the sigmoid of its gate."""
    scores = torch.einsum("ihd,jd->hij", q, rows) * scale
    weights = plain.softmax_with_sink(scores, sink)
    return torch.einsum("hij,jd->ihd", weights, rows[:, :rank]) * torch.sigmoid(gate)[:, :, None]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 40, 8, 16), (2, 24, 12, 16), (4, 64, 32, 64), (1, 288, 32, 16)])
def test_attention_with_a_sink_and_a_gate_finds_the_one_key(dtype, shape):
    """All heads over one cached row per position, keys wider than values.  In the marked queries one key is made to
    dominate: far back, the last of a page, the first of the next, position 0 and the query's own; the sink is as
    large as the largest other scores, so leaving it out, scaling it or giving it a value shows."""
    heads, rank, rope_dim, block = shape
    g = torch.Generator().manual_seed(rank + heads)
    ops = kernels(dtype)
    key_dim, T, scale = rank + rope_dim, 4 * block + 5, 0.3
    rows = torch.randn(T, key_dim, generator=g)
    q = torch.randn(T, heads, key_dim, generator=g)
    marked = {T - 1: 2, T - 2: block - 1, T - 3: block, T - 4: 0, T - 5: T - 5, 3 * block: 2 * block + 1}
    for query, key in marked.items():
        q[query] = rows[key][None, :] * (9.0 / scale / float(rows[key] @ rows[key])) + 0.1 * q[query]
    sink = torch.tensor([3.0, -2.0, 6.0, 0.5])[:heads].double()
    gate = torch.randn(T, heads, generator=g) * 2
    if dtype == torch.bfloat16:                                   # both sides start from the same rounded numbers
        rows, q = rows.bfloat16().float(), q.bfloat16().float()
    want = plain_sink_attention(q.double(), rows.double(), rank, scale, sink, gate.double())
    table = scrambled_table(1, 5, g)
    cache = torch.zeros(6, 1, block, key_dim, dtype=dtype, device="cuda")
    for p in range(T):
        cache[int(table[0, p // block]), 0, p % block] = rows[p].to(dtype)
    gate_rows = torch.zeros(T, heads + 3)
    gate_rows[:, 2:2 + heads] = gate
    gate_rows = gate_rows.cuda()
    for first, count in ((0, T), (0, 3 * block - 1), (3 * block - 1, 1), (3 * block, 1), (T - 5, 5)):
        out = torch.empty(count, heads * rank + 8, dtype=dtype, device="cuda")
        ops.attention_general(q[first:first + count].reshape(count, -1).to(dtype).cuda(), cache, cache, table.cuda(),
                              i32(range(first, first + count)), i32([0] * count), out, heads, 1, key_dim, rank, block, scale,
                              gate=gate_rows[first:first + count, 2:], gate_stride=heads + 3, sink=sink.float().cuda(),
                              value_stride=key_dim)
        close(out[:, :heads * rank].view(count, heads, rank), want[first:first + count], dtype, f"tokens {first}..{first + count}")
    # one token a sequence with the keys cut into parts that run side by side: parts without keys, of one run, of many
    for splits in (2, 3, 7, 64):
        for first in (0, 1, 31, 32, 3 * block - 1, 3 * block, T - 1):
            out = torch.empty(1, heads * rank + 8, dtype=dtype, device="cuda")
            scratch_o = torch.full((heads * splits * rank,), float("nan"), device="cuda")
            scratch_ml = torch.full((heads * splits * 2,), float("nan"), device="cuda")
            ops.attention_general(q[first:first + 1].reshape(1, -1).to(dtype).cuda(), cache, cache, table.cuda(),
                                  i32([first]), i32([0]), out, heads, 1, key_dim, rank, block, scale,
                                  gate=gate_rows[first:first + 1, 2:], gate_stride=heads + 3, sink=sink.float().cuda(),
                                  value_stride=key_dim, splits=splits, scratch_o=scratch_o, scratch_ml=scratch_ml)
            close(out[:, :heads * rank].view(1, heads, rank), want[first:first + 1], dtype, f"token {first} in {splits} parts")
            assert float(out[:, heads * rank:].float().abs().max()) == 0.0
    for query, key in marked.items():                             # the marked queries do return the marked key's values
        head_out = want[query, 0] / torch.sigmoid(gate[query, 0].double())
        assert float((head_out - rows[key, :rank].double()).abs().max()) < 0.35 * float(rows[key, :rank].abs().max()), (query, key)


# ---- routed feed-forward --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(5, 2, 1.5, 64), (7, 3, 0.75, 72), (4, 4, 2.0, 40), (16, 1, 2.5, 128), (3, 1, 1.0, 24)])
def test_router_chooses_by_corrected_scores_and_weighs_by_plain_ones(dtype, shape):
    experts, top, scale, hidden = shape
    g = torch.Generator().manual_seed(experts * 10 + top)
    ops = kernels(dtype)
    n = 90
    h = torch.randn(n, hidden, generator=g)
    router = torch.randn(experts, hidden, generator=g) * 0.3
    correction = torch.randn(experts, generator=g) * 0.5             # as large as the differences between the scores
    shared_gate = torch.randn(hidden, generator=g) * 0.3
    h[0] = 0.0                                                        # all scores one half: the correction alone chooses
    if dtype == torch.bfloat16:
        h, router, shared_gate = h.bfloat16().float(), router.bfloat16().float(), shared_gate.bfloat16().float()
    P = {"l0.mlp.router": router.double(), "l0.mlp.correction": correction.double()}
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}}
    want_chosen, want_weights = plain.route(h.double(), P, "l0.", mlp)
    chosen = torch.empty(n, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(n, top, device="cuda")
    share = torch.empty(n, device="cuda")
    ops.route_tokens(h.to(dtype).cuda(), router.to(dtype).cuda(), correction.float().cuda(), top, scale, False, chosen,
                     weights, shared_gate_weight=shared_gate.to(dtype).cuda(), shared_gate_out=share)
    got_chosen, got_weights = chosen.cpu().long(), weights.cpu().double()
    scores = torch.sigmoid(h.double() @ router.double().T) + correction.double()
    for t in range(n):
        ours, theirs = sorted(got_chosen[t].tolist()), sorted(want_chosen[t].tolist())
        if ours != theirs:                                            # only where the choice is a tie to float rounding
            edge = torch.sort(scores[t], descending=True).values
            assert abs(float(edge[top - 1] - edge[top])) < 1e-5, f"token {t}: {ours} for {theirs}"
            continue
        by_expert = dict(zip(want_chosen[t].tolist(), want_weights[t].tolist()))
        for e, w in zip(got_chosen[t].tolist(), got_weights[t].tolist()):
            assert abs(w - by_expert[e]) < 2e-5 * scale, f"token {t}, expert {e}"
    assert sorted(got_chosen[0].tolist()) == sorted(torch.topk(correction, top).indices.tolist())
    assert torch.allclose(got_weights[0], torch.full((top,), 0.5 * scale, dtype=F64))
    close(share, torch.sigmoid(h.double() @ shared_gate.double()), torch.float32, "the shared expert's gate", loose=2.0)
    # equal choice scores: the lower index
    ops.route_tokens(torch.zeros(2, hidden, dtype=dtype, device="cuda"), router.to(dtype).cuda(), None, top, scale, False,
                     chosen[:2], weights[:2])
    assert sorted(chosen[0].tolist()) == list(range(top))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(5, 2, 64, 40, 24), (7, 3, 72, 56, 0), (16, 1, 128, 64, 72), (2, 2, 40, 136, 8)])
def test_experts_over_sorted_pairs_and_their_weighted_sum(dtype, shape):
    """Tokens sorted by expert (some experts get none, one gets most), both projections with the squared relu between,
    and the sum weighted by the router, plus the gated shared expert, added to the stream."""
    experts, top, hidden, ff, shared_ff = shape
    g = torch.Generator().manual_seed(experts + ff)
    ops = kernels(dtype)
    n = 75
    rnd = lambda *size: (torch.randn(*size, generator=g) * 0.3).to(dtype).float()
    h, up, down = rnd(n, hidden) * 3, rnd(experts, ff, hidden), rnd(experts, hidden, ff)
    favourite = experts - 1
    chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)])
    for t in range(0, n, 2):                                        # every second token takes the last expert
        if favourite not in chosen[t].tolist():
            chosen[t, 0] = favourite
    if experts > 3:
        chosen[chosen == 1] = favourite if top == 1 else 1          # (top 1: expert 1 gets nobody)
    weights = torch.rand(n, top, generator=g) + 0.2
    share = torch.rand(n, generator=g)
    x0 = torch.randn(n, hidden, generator=g)
    want = x0.double().clone()
    for t in range(n):
        for e, w in zip(chosen[t].tolist(), weights[t].tolist()):
            want[t] += w * plain.expert(h[t:t + 1].double(), up[e].double(), down[e].double())[0]
    if shared_ff:
        s_up, s_down = rnd(shared_ff, hidden), rnd(hidden, shared_ff)
        want += share.double()[:, None] * plain.expert(h.double(), s_up.double(), s_down.double())
    chosen_d = chosen.to(torch.int32).cuda()
    offsets = torch.empty(experts + 1, dtype=torch.int32, device="cuda")
    order = torch.empty(n * top, dtype=torch.int32, device="cuda")
    place = torch.empty(n, top, dtype=torch.int32, device="cuda")
    ops.sort_by_expert(chosen_d, experts, offsets, order, place)
    counts = torch.bincount(chosen.flatten(), minlength=experts)
    assert offsets.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    flat_expert = chosen.flatten()
    for pair in range(n * top):
        at = int(place.flatten()[pair])
        assert int(offsets[flat_expert[pair]]) <= at < int(offsets[flat_expert[pair] + 1]) and int(order[at]) == pair // top
    hidden_rows = torch.empty(n * top, ff, dtype=dtype, device="cuda")
    ops.expert_linear(h.to(dtype).cuda(), up.to(dtype).cuda(), offsets, hidden_rows, rows=order, activation="relu2")
    if ops.expert_rows_sorted_first(hidden):                      # the other way: rows brought into sorted order first
        gathered = torch.empty(n * top, hidden, dtype=dtype, device="cuda")
        ops.gather_rows(h.to(dtype).cuda(), order, gathered)
        assert torch.equal(gathered.cpu(), h.to(dtype)[order.cpu().long()])
        other = torch.full_like(hidden_rows, 5.0)
        ops.expert_linear(gathered, up.to(dtype).cuda(), offsets, other, activation="relu2")
        close(other, hidden_rows.double().cpu(), dtype, "hidden rows from sorted rows", loose=2.0)
        hidden_rows = other
    results = torch.empty(n * top, hidden, device="cuda")
    ops.expert_linear(hidden_rows, down.to(dtype).cuda(), offsets, results)
    shared_out = None
    if shared_ff:
        z = torch.relu(h.double() @ s_up.double().T) ** 2
        shared_out = (z.to(dtype).double() @ s_down.double().T).float().cuda()
    x = x0.clone().cuda()
    ops.combine_experts(results, place, weights.cuda(), shared_out, share.cuda() if shared_ff else None, x)
    close(x, want, dtype, "the stream after the feed-forward", loose=3.0)
    stored = torch.full_like(x, 7.0)
    ops.combine_experts(results, place, weights.cuda(), shared_out, share.cuda() if shared_ff else None, stored, add=False)
    close(stored, want - x0.double(), dtype, "the feed-forward's result stored", loose=3.0)


# ---- several residual streams ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count,hidden", [(3, 64), (1, 128), (2, 72), (4, 40), (8, 24)])
def test_streams_are_read_mixed_and_summed(dtype, count, hidden):
    g = torch.Generator().manual_seed(count)
    ops = kernels(dtype)
    n, eps = 37, 1e-5
    P = {"c.in": torch.randn(count, generator=g).double() + 1, "c.out": torch.randn(count, generator=g).double() + 1,
         "c.mix": torch.eye(count, dtype=F64) + torch.randn(count, count, generator=g).double()}
    weight = torch.randn(hidden, generator=g).double() * 0.5
    f32 = lambda t: t.float().cuda().contiguous()
    # before the first layer every stream is the embedding's output: the kernel reads that one copy
    source = torch.randn(n, hidden, generator=g)
    normed = torch.empty(n, hidden, dtype=dtype, device="cuda")
    streams = torch.full((count, n, hidden), 9.0, device="cuda")
    ops.stream_mix(streams, count, source=f32(source), read=f32(P["c.in"]), gamma=f32(1 + weight), eps=eps, normed_out=normed)
    old = source.double()[None].repeat(count, 1, 1)
    u = torch.einsum("s,stw->tw", P["c.in"], old)
    close(normed, plain.norm_around_zero(u, weight, eps), dtype, "what the first sublayer reads")
    # the sublayer's result: every stream from all the old ones (mix is [from, to]); then the next reading and the sum
    branch = torch.randn(n, hidden, generator=g)
    want = plain.hyper_sublayer(old, P, "c", lambda _: branch.double())
    total = torch.empty(n, hidden, device="cuda")
    ops.stream_mix(streams, count, source=f32(source), branch=f32(branch), mix=f32(P["c.mix"]).view(-1), write=f32(P["c.out"]),
                   read=f32(P["c.in"]), gamma=f32(1 + weight), eps=eps, normed_out=normed, sum_out=total)
    close(streams, want, torch.float32, "the streams after the first sublayer", loose=4.0)
    close(total, want.sum(dim=0), torch.float32, "their sum", loose=8.0)
    close(normed, plain.norm_around_zero(torch.einsum("s,stw->tw", P["c.in"], want), weight, eps), dtype, "the next reading")
    again = plain.hyper_sublayer(want, P, "c", lambda _: -branch.double())
    ops.stream_mix(streams, count, branch=f32(-branch), mix=f32(P["c.mix"]).view(-1), write=f32(P["c.out"]))
    close(streams, again, torch.float32, "the streams after a second sublayer", loose=8.0)
