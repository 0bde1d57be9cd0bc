"""The Fidolix decoder on the CPU: its configuration and refusals, tensor names, the order of runs and their cache
entries, hand-worked numbers for the mechanisms of the plain implementation (tests/plain_fidolix.py), that a fault in
any mechanism moves the plain logits by far more than rounding, and the engine's bookkeeping (portions, batches, slots,
pages and states used again, steps that run twice) with torch stand-ins for the kernels (tests/ops_double.py)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_fidolix as plain
from fidolix_models import FIDOLIX, make_folder
from helpers import random_tokens
from ops_double import double_loader
from stratakv_b200 import Engine, EngineConfig, StepEntry
from stratakv_b200.config import ConfigError, FidolixConfig, load_config
from stratakv_b200.engine.model import cache_requests, expected_tensors
from stratakv_b200.models.fidolix import fidolix_spec, layer_runs
from stratakv_b200.weights.loader import load_checkpoint

F64 = torch.float64


def test_configuration_round_trip_and_refusals():
    for raw in FIDOLIX.values():
        typed = FidolixConfig.from_dict(raw)
        assert FidolixConfig.from_dict(typed.to_dict()) == typed
    fa = FidolixConfig.from_dict(FIDOLIX["FA"])
    assert (fa.vocab, fa.width, fa.side_dim, fa.embedding_scale, fa.loop_start, fa.loop_stop, fa.loop_times) == \
        (101, 64, 8, 2.5, 1, 3, 2)
    assert fa.layers[1].attention.window == 7 and fa.layers[1].attention.conv == 3 and fa.layers[1].right.rank == 5
    assert fa.layers[2].mlp is None and fa.layers[2].attention.softcap == 0.0
    assert FidolixConfig.from_dict(FIDOLIX["FB"]).embedding_scale == 1.0

    def broken(change):
        raw = copy.deepcopy(FIDOLIX["FA"])
        change(raw)
        with pytest.raises(ConfigError):
            FidolixConfig.from_dict(raw)

    broken(lambda r: r["layers"][0].update(type="retention"))
    broken(lambda r: r["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda r: r["layers"][1]["mixer"]["left"].update(vdim=8))
    broken(lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=18))
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(top=7))
    broken(lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4))
    broken(lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=0))
    broken(lambda r: r["layers"][0]["mlp"].update(kind="relu"))
    broken(lambda r: r["loop"].update(stop=5))
    broken(lambda r: r["loop"].update(times=0))
    broken(lambda r: r.pop("norm"))


def test_the_decay_rank_is_read_from_the_checkpoint(tmp_path):
    folder = make_folder(tmp_path / "m", FIDOLIX["FA"], seed=1)
    raw = copy.deepcopy(FIDOLIX["FA"])
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["rank"]
    import json
    (folder / "config.json").write_text(json.dumps(raw))
    with pytest.raises(ValueError):
        fidolix_spec(FidolixConfig.from_dict(raw))
    _, typed = load_config(folder)
    assert typed.layers[1].right.rank == 5 and typed.layers[3].right.rank == 3


def test_tensor_names_runs_and_cache_entries():
    typed = FidolixConfig.from_dict(FIDOLIX["FA"])
    spec = fidolix_spec(typed)
    shapes = {name: tuple(request.shape) for name, request in expected_tensors(spec).items()}
    assert shapes["embed"] == (101, 64) and shapes["head"] == (101, 64) and shapes["side.embed"] == (101, 32)
    assert shapes["l0.mix.q"] == (64, 64) and shapes["l0.mix.k.b"] == (32,) and shapes["l0.mix.v"] == (48, 64)
    assert shapes["l0.mix.q.norm"] == (64,) and shapes["l0.mix.k.norm"] == (32,) and shapes["l0.mix.g"] == (96, 64)
    assert shapes["l0.mix.o"] == (64, 96) and shapes["l0.mlp.gate"] == (40, 64) and shapes["l0.side.proj"] == (64, 8)
    assert shapes["l1.mix.left.q.conv"] == (64, 3) and shapes["l1.mix.left.k.conv"] == (32, 3)
    assert shapes["l1.mix.left.sink"] == (4,) and shapes["l1.mix.left.o"] == (64, 64) and "l1.mix.left.v" not in shapes
    assert shapes["l1.mix.right.mu.w"] == (64,) and shapes["l1.mix.right.w1"] == (5, 64)
    assert shapes["l1.mix.right.w2"] == (32, 5) and shapes["l1.mix.right.u"] == (2, 16) and shapes["l1.mix.right.r"] == (32, 64)
    assert shapes["l1.mlp.router"] == (6, 64) and shapes["l1.mlp.e5.gate"] == (24, 64) and "l1.mlp.e6.up" not in shapes
    assert "l2.norm2" not in shapes and "l2.mlp.gate" not in shapes
    # layers 1 and 2 run twice; every run has a cache entry of its own; the embedding comes back before the second pass
    order, again = layer_runs(typed)
    assert order == [0, 1, 2, 1, 2, 3] and again == {3}
    assert [(e.layer, e.cache, e.adds_embedding) for e in spec.schedule] == \
        [(0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False), (3, 5, False)]
    requests = cache_requests(spec)
    assert [r.kind for r in requests] == ["kv", "kv_window", "kv", "kv_window", "kv", "kv_window"]
    assert requests[0].v_head_dim == 24 and requests[1].window == 7 and requests[5].window == 33
    # the convolution's last inputs, then the time mixing's matrices and last input, twice each
    assert requests[1].state_bytes == 4 * (3 * (64 + 32) + 2 * 2 * 16 * 16 + 2 * 64)
    assert requests[5].state_bytes == 4 * (2 * (48 + 24) + 2 * 4 * 8 * 8 + 2 * 64)
    single = layer_runs(FidolixConfig.from_dict(FIDOLIX["FB"]))
    assert single == ([0, 1, 1, 1, 2], {2, 3})
    assert layer_runs(FidolixConfig.from_dict(FIDOLIX["FD"])) == ([0, 1], set())


# ---- hand-worked numbers for the plain implementation ---------------------------------------------------------------

def test_interleaved_rotation_by_hand():
    rot = {"dims": 4, "base": 100.0}
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64).repeat(2, 1, 1)
    out = plain.rotate_interleaved(x, torch.tensor([0, 3]), rot)
    assert torch.equal(out[0], x[0])                       # position 0 turns nothing
    a0, a1 = 3.0 * 1.0, 3.0 * 100.0 ** (-0.5)
    want = [math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + math.sin(a0),
            3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1), 5.0, 6.0]
    np.testing.assert_allclose(out[1, 0].numpy(), want, rtol=1e-12)


def test_stretched_frequencies_by_hand():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    f, magnitude = plain.rotary_frequencies(rot)
    pair = lambda turns: 8 * math.log(16 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(pair(4.0)), 0), min(math.ceil(pair(1.0)), 7)
    assert (lo, hi) == (0, 1)
    plain_f = [100.0 ** (-2 * i / 8) for i in range(4)]
    np.testing.assert_allclose(f.numpy(), [plain_f[0], plain_f[1] / 4, plain_f[2] / 4, plain_f[3] / 4], rtol=1e-12)
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_short_convolution_by_hand():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=F64)
    w = torch.tensor([[0.5, 0.25, 1.0], [0.0, 1.0, -1.0]], dtype=F64)        # the last tap weighs the current token
    y = plain.short_convolution(u, w)
    np.testing.assert_allclose(y[:, 0].numpy(), [1.0, 2.25, 4.0, 5.75])
    np.testing.assert_allclose(y[:, 1].numpy(), [-10.0, -10.0, -10.0, -10.0])


def test_softmax_with_a_sink_by_hand():
    scores = torch.tensor([[0.0, math.log(2.0), -math.inf]], dtype=F64)
    weights = plain.softmax_with_sink(scores, torch.tensor(math.log(5.0), dtype=F64))
    np.testing.assert_allclose(weights.numpy(), [[1 / 8, 2 / 8, 0.0]], rtol=1e-12)
    far = plain.softmax_with_sink(torch.tensor([[1.0]], dtype=F64), torch.tensor(800.0, dtype=F64))
    assert float(far[0, 0]) == pytest.approx(0.0, abs=1e-300)


def test_window_edges_of_the_left_side():
    """With one key made to stand out, the query that is window - 1 behind it sees it and the next one does not."""
    torch.manual_seed(0)
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "scale": 1.0, "mask": {"size": 3}}
    P = {"q": torch.zeros(4, 4, dtype=F64), "q.b": torch.tensor([1.0, 0, 0, 0], dtype=F64), "k": torch.eye(4, dtype=F64),
         "k.b": torch.zeros(4, dtype=F64), "sink": torch.tensor([-50.0], dtype=F64), "o": torch.eye(4, dtype=F64)}
    h = torch.zeros(6, 4, dtype=F64)
    h[1] = torch.tensor([30.0, 7.0, 0, 0])                 # the key (and value) at position 1 stands out
    out = plain.windowed_mixer(h, {"x." + k: v for k, v in P.items()}, "x.", m)
    assert out[1, 1] == pytest.approx(7.0) and out[2, 1] == pytest.approx(7.0) and out[3, 1] == pytest.approx(7.0)
    assert abs(float(out[4, 1])) < 1e-9 and abs(float(out[5, 1])) < 1e-9


def test_time_mixing_as_an_explicit_sum():
    """o_t = sum over s < t of (r_t . (prod of the decays between) k_s) v_s + (r_t . u k_t) v_t, before the norm."""
    torch.manual_seed(1)
    T, W, H, d = 6, 8, 2, 4
    P = {"x." + n: torch.randn(H * d, W, dtype=F64) * 0.5 for n in ("r", "k", "v", "g")}
    P.update({"x.mu." + s: torch.rand(W, dtype=F64) for s in "rkvgw"})
    P.update({"x.w1": torch.randn(3, W, dtype=F64), "x.w2": torch.randn(H * d, 3, dtype=F64), "x.w0": torch.randn(H * d, dtype=F64) - 1,
              "x.u": torch.rand(H, d, dtype=F64), "x.norm": torch.ones(H * d, dtype=F64), "x.o": torch.eye(H * d, dtype=F64)})
    h = torch.randn(T, W, dtype=F64)
    out = plain.time_mixing(h, P, "x.", {"heads": H, "dim": d}, 1e-5)
    mix = plain.shifted_mixes(h, P, "x.")
    np.testing.assert_allclose(mix["r"][0].numpy(), (h[0] * (1 - P["x.mu.r"])).numpy(), rtol=1e-12)  # zeros before the first
    r, k, v = (mix[s] @ P["x." + s].T for s in "rkv")
    w = plain.decays(mix["w"], P, "x.")
    gate = plain.silu(mix["g"] @ P["x.g"].T)
    for t in (0, 3, 5):
        for head in range(H):
            cols = slice(head * d, (head + 1) * d)
            o = (r[t, cols] * P["x.u"][head] * k[t, cols]).sum() * v[t, cols]
            for s in range(t):
                between = torch.ones(d, dtype=F64)
                for j in range(s + 1, t):
                    between = between * w[j, cols]
                o = o + (r[t, cols] * between * k[s, cols]).sum() * v[s, cols]
            want = o / torch.sqrt((o * o).mean() + 1e-5) * gate[t, cols]
            np.testing.assert_allclose(out[t, cols].numpy(), want.numpy(), rtol=1e-9, atol=1e-12)


def test_routing_among_the_best_groups_by_hand():
    logits = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.02, 0.20, 0.18]], dtype=F64))
    P = {"x.router": torch.eye(6, dtype=F64)}
    router = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}
    chosen, weights = plain.route(logits, P, "x.", router)
    # the groups score 0.30, 0.25, 0.20: the third is out although its experts beat expert 0 and 3
    assert chosen.tolist() == [[1, 2]]
    np.testing.assert_allclose(weights.numpy(), [[0.30 / 0.55, 0.25 / 0.55]], rtol=1e-12)
    one_group = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    chosen, weights = plain.route(logits, P, "x.", one_group)
    assert chosen.tolist() == [[1, 0]]                     # both from the best group, although expert 0 scores little
    np.testing.assert_allclose(weights.numpy(), [[0.30 / 0.35, 0.05 / 0.35]], rtol=1e-12)
    chosen, _ = plain.route(logits, P, "x.", {"experts": 6, "top": 3})
    assert chosen.tolist() == [[1, 2, 4]]


def test_dense_feed_forward_by_hand():
    P = {"x.gate": torch.tensor([[1.0], [1.0]], dtype=F64), "x.up": torch.tensor([[1.0], [-1.0]], dtype=F64),
         "x.down": torch.eye(2, dtype=F64)}
    y = plain.dense_ff(torch.tensor([[3.0]], dtype=F64), P, "x.", {"limit": 2.0})
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    np.testing.assert_allclose(y.numpy(), [[g * 3.0, g * -1.0]], rtol=1e-12)       # the gate is cut at 2, up at +-2


FAULTS = {
    "the embedding's scale": lambda cfg, P: cfg["embedding"].update(scale=1.0),
    "the embedding added before a later pass": lambda cfg, P: cfg["loop"].update(times=1),
    "the second norm": lambda cfg, P: P.update({"l0.norm2": P["l0.norm1"]}),
    "the query norm's weight": lambda cfg, P: P.update({"l0.mix.q.norm": torch.ones_like(P["l0.mix.q.norm"])}),
    "a key bias": lambda cfg, P: P.update({"l0.mix.k.b": torch.zeros_like(P["l0.mix.k.b"])}),
    "the cap": lambda cfg, P: cfg["layers"][0]["mixer"].update(softcap=2.0),
    "the gate": lambda cfg, P: P.update({"l0.mix.g": torch.zeros_like(P["l0.mix.g"])}),
    "the window, one token off": lambda cfg, P: cfg["layers"][1]["mixer"]["left"]["mask"].update(size=6),
    "the sink": lambda cfg, P: P.update({"l1.mix.left.sink": P["l1.mix.left.sink"] - 30.0}),
    "the convolution's oldest tap": lambda cfg, P: P["l1.mix.left.k.conv"].__setitem__((slice(None), 0), 0.0),
    "the rotation's stretch": lambda cfg, P: cfg["layers"][1]["mixer"]["left"]["rot"].pop("scaling"),
    "the bonus": lambda cfg, P: P.update({"l1.mix.right.u": torch.zeros_like(P["l1.mix.right.u"])}),
    "the decay's low-rank part": lambda cfg, P: P.update({"l1.mix.right.w2": torch.zeros_like(P["l1.mix.right.w2"])}),
    "the token shift": lambda cfg, P: P.update({"l1.mix.right.mu.k": torch.zeros_like(P["l1.mix.right.mu.k"])}),
    "the sides' weights": lambda cfg, P: cfg["layers"][1]["mixer"].update(left_scale=1.0, right_scale=1.0),
    "the groups": lambda cfg, P: cfg["layers"][1]["mlp"]["router"].pop("groups"),
    "the clamp": lambda cfg, P: cfg["layers"][0]["mlp"].update(limit=0.25),
    "the token input": lambda cfg, P: cfg.pop("token_side"),
}


@pytest.mark.parametrize("fault", list(FAULTS))
def test_a_fault_moves_the_plain_logits_far_more_than_rounding(tmp_path, fault):
    folder = make_folder(tmp_path / "FA", FIDOLIX["FA"], seed=2)
    cfg, P = plain.load_folder(folder)
    tokens = random_tokens(101, 48, seed=5)
    ref = plain.logits_of(cfg, P, tokens)
    cfg, P = copy.deepcopy(cfg), {k: v.clone() for k, v in P.items()}
    FAULTS[fault](cfg, P)
    moved = plain.logits_of(cfg, P, tokens)
    per_position = np.sqrt(((moved - ref) ** 2).mean(axis=-1)) / ref.std()
    assert per_position.max() > 0.16, f"{fault}: the logits move by {per_position.max():.3f} of their spread only"


# ---- the engine's bookkeeping, with stand-ins for the kernels ---------------------------------------------------------

def cpu_engine(folder, max_tokens=512, block_size=16, max_batch=0):
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    return Engine(spec, tensors, EngineConfig(max_tokens=max_tokens, dtype="float32", device="cpu", block_size=block_size,
                                              max_batch=max_batch), kernel_loader=double_loader())


@pytest.mark.parametrize("name", ["FA", "FB", "FD"])
def test_bookkeeping_portions_batches_and_slots_used_again(tmp_path, name):
    folder = make_folder(tmp_path / name, FIDOLIX[name], seed=3)
    cfg, P = plain.load_folder(folder)
    engine = cpu_engine(folder, max_tokens=16 * 14, max_batch=3)
    vocab = FIDOLIX[name]["vocab"]
    for turn in range(2):                     # the second turn takes the slots, pages and states of the first
        prompts = [random_tokens(vocab, n, seed=10 * turn + n) for n in (5, 40, 18)]
        refs = [plain.logits_of(cfg, P, p) for p in prompts]
        slots = [engine.open_sequence() for _ in prompts]
        cut = [1, 20, 17]
        got = engine.step([StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)])
        np.testing.assert_allclose(got.numpy(), np.concatenate([r[:c] for r, c in zip(refs, cut)]), rtol=2e-4, atol=5e-5)
        got = engine.step([StepEntry(slots[0], prompts[0][1:], [3]), StepEntry(slots[1], prompts[1][20:22], [0, 1]),
                           StepEntry(slots[2], prompts[2][17:], [0])])
        np.testing.assert_allclose(got.numpy(), np.stack([refs[0][4], refs[1][20], refs[1][21], refs[2][17]]), rtol=2e-4, atol=5e-5)
        engine.close_sequence(slots[0]); engine.close_sequence(slots[2])
        for position in range(22, 40):
            got = engine.step([StepEntry(slots[1], [prompts[1][position]], [0])])
            np.testing.assert_allclose(got.numpy()[0], refs[1][position], rtol=2e-4, atol=5e-5)
        engine.close_sequence(slots[1])
        assert engine.cache.all_free()


def test_a_step_that_runs_twice_leaves_the_states_as_one_run_does(tmp_path):
    """A decode graph's warm-up and its first replay run the same one-token step twice: no state a step reads (the
    convolution's last inputs, the time mixing's matrices and last input) is one that it writes."""
    name = "FA"
    folder = make_folder(tmp_path / name, FIDOLIX[name], seed=4)
    cfg, P = plain.load_folder(folder)
    engine = cpu_engine(folder)
    tokens = random_tokens(FIDOLIX[name]["vocab"], 14, seed=1)
    ref = plain.logits_of(cfg, P, tokens)
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:6], [])])
    rows = torch.tensor([0], dtype=torch.int32)
    for position in range(6, 14):
        step, _, _ = engine.prepare([StepEntry(slot, [tokens[position]], [0])])
        first = engine.model.forward(step, rows, 1).clone()
        second = engine.model.forward(step, rows, 1).clone()
        engine.cache.advance(slot, position + 1)
        np.testing.assert_allclose(first.numpy()[0], ref[position], rtol=2e-4, atol=5e-5)
        np.testing.assert_allclose(second.numpy(), first.numpy(), rtol=0, atol=0)
    engine.close_sequence(slot)


def test_window_pages_come_back_while_a_sequence_runs(tmp_path):
    """The left side keeps a window: a long sequence gives pages back as it goes, and what it computes stays right."""
    folder = make_folder(tmp_path / "FA", FIDOLIX["FA"], seed=6)
    cfg, P = plain.load_folder(folder)
    engine = cpu_engine(folder, max_tokens=16 * 12, block_size=16)
    tokens = random_tokens(101, 90, seed=8)
    ref = plain.logits_of(cfg, P, tokens)
    slot = engine.open_sequence()
    got = engine.step([StepEntry(slot, tokens[:50], [49])])
    np.testing.assert_allclose(got.numpy()[0], ref[49], rtol=2e-4, atol=5e-5)
    windowed = [g for g in engine.cache.groups if g.kind.windowed]
    assert windowed and all(g.blocks.free_count > g.blocks.total - 4 * len(g.entries) for g in windowed)
    for position in range(50, 90):
        got = engine.step([StepEntry(slot, [tokens[position]], [0])])
        np.testing.assert_allclose(got.numpy()[0], ref[position], rtol=2e-4, atol=5e-5)
    engine.close_sequence(slot)
    assert engine.cache.all_free()
