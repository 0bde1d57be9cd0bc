"""The Kedelorn decoder off the GPU: its configuration and description as parts, the engine's bookkeeping for it (a
retention state per slot, a latent cache with a rotated key part, a lent latent, several residual streams, routed
experts) with the torch stand-in for the kernels, and that the plain implementation the GPU tests compare with is
right on numbers worked out by hand and can tell a fault from rounding."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import plain_kedelorn as plain
from helpers import random_tokens
from kedelorn_models import KEDELORN, make_folder
from ops_double import double_loader
from stratakv_b200 import EngineConfig, StepEntry
from stratakv_b200.config import ConfigError, KedelornConfig, load_config
from stratakv_b200.engine.engine import Engine
from stratakv_b200.engine.model import cache_requests, expected_tensors
from stratakv_b200.weights import load_checkpoint

F64 = torch.float64


def test_config_round_trip_and_what_it_refuses(tmp_path):
    for raw in KEDELORN.values():
        assert KedelornConfig.from_dict(raw).to_dict() == raw
    (tmp_path / "config.json").write_text(json.dumps(KEDELORN["KA"]))
    arch, typed = load_config(tmp_path)
    assert arch.name == "Kedelorn" and typed.streams == 3
    assert [layer.type for layer in typed.layers] == ["retention", "latent_attention", "retention", "latent_attention"]
    assert typed.layers[3].kv_from == 1 and typed.layers[1].kv_from is None and typed.layers[2].mlp is None
    assert typed.layers[0].decay == (1.0, 0.5, 0.96875) and typed.layers[0].rot.dims == 8 and typed.layers[0].rot.factor == 0.0
    assert typed.layers[1].rot.factor == 8.0 and typed.layers[1].rot.original == 64 and typed.layers[1].mlp.shared_ff == 0
    assert KedelornConfig.from_dict(KEDELORN["KB"]).streams == 0 and KedelornConfig.from_dict(KEDELORN["KC"]).streams == 1
    for path, value, message in ((("layers", 0, "type"), "attention", "not a mixer"),
                                 (("layers", 0, "mixer", "decay"), [0.5, 0.5], "one number from 0 to 1 per head"),
                                 (("layers", 0, "mixer", "decay"), [0.5, 0.5, 1.5], "one number from 0 to 1 per head"),
                                 (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
                                 (("layers", 0, "mixer", "rot", "dims"), 18, "exceeds"),
                                 (("layers", 0, "mlp", "kind"), "dense", "not a feed-forward"),
                                 (("layers", 0, "mlp", "router", "top"), 6, "exceeds"),
                                 (("layers", 3, "mixer", "kv_from"), 2, "no latent of its own"),
                                 (("layers", 3, "mixer", "kv_from"), 3, "earlier layer"),
                                 (("layers", 3, "mixer", "kv_rank"), 48, "differs"),
                                 (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0, "positive"),
                                 (("streams",), 9, "not supported"),
                                 (("vocab",), None, "missing"), (("norm",), None, "missing")):
        raw = copy.deepcopy(KEDELORN["KA"])
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=message):
            KedelornConfig.from_dict(raw)


def test_description_names_the_checkpoint_tensors_and_the_cache():
    from stratakv_b200.models.kedelorn import kedelorn_spec
    spec = kedelorn_spec(KedelornConfig.from_dict(KEDELORN["KA"]))
    shapes = {name: tuple(request.shape) for name, request in expected_tensors(spec).items()}
    assert shapes["embed"] == (101, 64) and shapes["head"] == (101, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (48, 64) and shapes["l0.mix.k"] == (48, 64) and shapes["l0.mix.v"] == (72, 64)
    assert shapes["l0.mix.g"] == (72, 64) and shapes["l0.mix.o"] == (64, 72)
    assert shapes["l0.hc1.in"] == (3,) and shapes["l0.hc1.out"] == (3,) and shapes["l0.hc2.mix"] == (3, 3)
    assert shapes["l0.mlp.router"] == (5, 64) and shapes["l0.mlp.correction"] == (5,) and shapes["l0.mlp.e4.up"] == (40, 64)
    assert shapes["l0.mlp.e0.down"] == (64, 40) and shapes["l0.mlp.shared.up"] == (24, 64) and shapes["l0.mlp.shared.sg"] == (1, 64)
    assert "l0.mlp.e5.up" not in shapes and "l1.mlp.shared.up" not in shapes and "l1.mlp.e3.up" not in shapes
    assert shapes["l1.mix.q"] == (3 * 24, 64) and shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.dkv.norm"] == (40,)
    assert shapes["l1.mix.uk"] == (48, 40) and shapes["l1.mix.uv"] == (24, 40) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l1.mix.g"] == (3, 64) and shapes["l1.mix.o"] == (64, 24)
    assert "l2.norm2" not in shapes and "l2.hc2.in" not in shapes and "l2.mlp.router" not in shapes
    assert "l3.mix.dkv" not in shapes and "l3.mix.dkv.norm" not in shapes and shapes["l3.mix.q"] == (2 * 32, 64)
    assert shapes["l3.mix.uk"] == (48, 40) and shapes["l3.mix.uv"] == (32, 40)
    requests = cache_requests(spec)
    assert [r.kind for r in requests] == ["none", "latent", "none"]
    assert requests[0].state_bytes == 4 * 2 * 3 * 16 * 24 and requests[1].head_dim == 48 and requests[2].state_bytes == 4 * 2 * 2 * 8 * 8
    assert [(e.cache, e.writes_cache) for e in spec.schedule] == [(0, True), (1, True), (2, True), (1, False)]
    plain_sum = kedelorn_spec(KedelornConfig.from_dict(KEDELORN["KB"]))
    assert not any(".hc" in name for name in expected_tensors(plain_sum))
    one_stream = {n: tuple(r.shape) for n, r in expected_tensors(kedelorn_spec(KedelornConfig.from_dict(KEDELORN["KC"]))).items()}
    assert one_stream["l0.hc1.in"] == (1,) and one_stream["l0.hc1.mix"] == (1, 1)


def cpu_engine(folder, max_tokens=512, block_size=16, max_batch=0):
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    return Engine(spec, tensors, EngineConfig(max_tokens=max_tokens, dtype="float32", device="cpu", block_size=block_size,
                                              max_batch=max_batch), kernel_loader=double_loader())


@pytest.mark.parametrize("name", ["KA", "KB"])
def test_bookkeeping_portions_batches_and_slots_used_again(tmp_path, name):
    folder = make_folder(tmp_path / name, KEDELORN[name], seed=3)
    cfg, P = plain.load_folder(folder)
    engine = cpu_engine(folder, max_tokens=16 * 14, max_batch=3)
    vocab = KEDELORN[name]["vocab"]
    for turn in range(2):                     # the second turn takes the slots, pages and states of the first
        prompts = [random_tokens(vocab, n, seed=10 * turn + n) for n in (5, 40, 18)]
        refs = [plain.logits_of(cfg, P, p).numpy() for p in prompts]
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


def test_a_step_that_runs_twice_leaves_the_retention_state_as_one_run_does(tmp_path):
    """A decode graph's warm-up and its first replay run the same one-token step twice: the state a step reads is
    not the state it writes."""
    name = "KA"
    folder = make_folder(tmp_path / name, KEDELORN[name], seed=4)
    cfg, P = plain.load_folder(folder)
    engine = cpu_engine(folder)
    tokens = random_tokens(KEDELORN[name]["vocab"], 12, seed=1)
    ref = plain.logits_of(cfg, P, tokens).numpy()
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:6], [])])
    for position in range(6, 12):
        step, rows, n = engine.prepare([StepEntry(slot, [tokens[position]], [0])])
        engine.model.forward(step, rows, n)                                  # once for nothing
        got = engine.model.forward(step, rows, n).clone()
        engine.cache.advance(slot, position + 1)
        np.testing.assert_allclose(got.numpy()[0], ref[position], rtol=2e-4, atol=5e-5)


def test_the_plain_implementation_tells_faults_from_rounding(tmp_path):
    """Each fault that the GPU tests are there to catch moves the plain logits by far more than they allow."""
    name = "KA"
    folder = make_folder(tmp_path / name, KEDELORN[name], seed=5)
    cfg, P = plain.load_folder(folder)
    tokens = random_tokens(KEDELORN[name]["vocab"], 90, seed=2)
    right = plain.logits_of(cfg, P, tokens).numpy()
    allowed = 0.08 * right.std()             # what tests/test_kedelorn_gpu.py allows a position in bfloat16

    def moved(change):
        other_cfg, other_P = copy.deepcopy(cfg), dict(P)
        change(other_cfg, other_P)
        difference = plain.logits_of(other_cfg, other_P, tokens).numpy() - right
        return np.sqrt((difference ** 2).mean(axis=-1)).max()

    def no_sink(c, w): w["l1.mix.sink"] = torch.full_like(w["l1.mix.sink"], -50.0)
    def sink_scaled_like_a_score(c, w): w["l1.mix.sink"] = w["l1.mix.sink"] * 0.3; w["l3.mix.sink"] = w["l3.mix.sink"] * 0.25
    def no_gate(c, w): w["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])
    def no_rotated_part(c, w): w["l1.mix.dkv"] = torch.cat([w["l1.mix.dkv"][:40], torch.zeros(8, 64, dtype=F64)])
    def plain_frequencies(c, w): c["layers"][1]["mixer"]["rot"].pop("scaling"); c["layers"][3]["mixer"]["rot"].pop("scaling")
    def scaled_by_the_stretch(c, w): c["layers"][1]["mixer"]["scale"] *= (0.1 * math.log(8.0) + 1.0) ** 2
    def no_latent_norm_weight(c, w): w["l1.mix.dkv.norm"] = torch.ones_like(w["l1.mix.dkv.norm"])
    def a_latent_of_its_own(c, w): w["l3.mix.uk"] = torch.roll(w["l3.mix.uk"], 1, dims=1)
    def other_decay(c, w): c["layers"][0]["mixer"]["decay"][2] = 0.9
    def whole_head_rotated(c, w): c["layers"][0]["mixer"]["rot"]["dims"] = 16
    def no_retention_gate(c, w): w["l0.mix.g"] = torch.zeros_like(w["l0.mix.g"])
    def correction_in_the_weights(c, w): w["l0.mlp.router"] = w["l0.mlp.router"] * 1.5
    def no_correction(c, w): w["l0.mlp.correction"] = torch.zeros_like(w["l0.mlp.correction"])
    def other_route_scale(c, w): c["layers"][0]["mlp"]["router"]["scale"] = 1.0
    def no_shared_gate(c, w): w["l0.mlp.shared.sg"] = torch.zeros_like(w["l0.mlp.shared.sg"])
    def mix_transposed(c, w): w["l1.hc1.mix"] = w["l1.hc1.mix"].T.contiguous()
    def streams_not_mixed(c, w): w["l0.hc2.mix"] = torch.eye(3, dtype=F64)
    def norm_weight_not_offset(c, w): w["l2.norm1"] = w["l2.norm1"] - 1.0
    for change in (no_sink, sink_scaled_like_a_score, no_gate, no_rotated_part, plain_frequencies, scaled_by_the_stretch,
                   no_latent_norm_weight, a_latent_of_its_own, other_decay, whole_head_rotated, no_retention_gate,
                   correction_in_the_weights, no_correction, other_route_scale, no_shared_gate, mix_transposed,
                   streams_not_mixed, norm_weight_not_offset):
        assert moved(change) > 2 * allowed, f"{change.__name__}: {moved(change) / right.std():.3f} of the spread"


def test_rotation_by_hand():
    t = lambda values: torch.tensor(values, dtype=F64)
    rot = {"dims": 4, "base": 100.0}
    f, magnitude = plain.rotary_frequencies(rot)
    assert torch.allclose(f, t([1.0, 0.1])) and magnitude == 1.0
    x = t([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]])
    out = plain.rotate(x, torch.tensor([3]), rot)[0]
    c0, s0, c1, s1 = math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)
    assert torch.allclose(out, t([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1, 5.0, 6.0]))
    assert torch.allclose(plain.rotate(x, torch.tensor([0]), rot), x)
    # stretched: with base 10000, 8 numbers and an original length of 64, one turn within 64 positions falls between
    # pairs 1 and 2 and four turns before pair 1, so lo = 0, hi = 2 and the ramp is 0, 1/2, 1, 1
    stretched = {"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}}
    f, magnitude = plain.rotary_frequencies(stretched)
    base = t([1.0, 0.1, 0.01, 0.001])
    assert torch.allclose(f, base * t([1.0, 0.5 + 0.5 / 8, 1 / 8, 1 / 8]))
    assert magnitude == pytest.approx(0.1 * math.log(8.0) + 1.0)
    turned = plain.rotate(t([[1.0, 0, 0, 0, 0, 0, 0, 0]]), torch.tensor([2]), stretched)[0]
    assert turned[0] == pytest.approx(magnitude * math.cos(2.0)) and turned[4] == pytest.approx(magnitude * math.sin(2.0))


def test_softmax_with_a_sink_by_hand():
    scores = torch.zeros(2, 3, 3, dtype=F64)
    sink = torch.tensor([math.log(2.0), -1e9], dtype=F64)
    weights = plain.softmax_with_sink(scores, sink)
    expected_0 = torch.tensor([[1 / 3, 0, 0], [1 / 4, 1 / 4, 0], [1 / 5, 1 / 5, 1 / 5]], dtype=F64)
    expected_1 = torch.tensor([[1.0, 0, 0], [1 / 2, 1 / 2, 0], [1 / 3, 1 / 3, 1 / 3]], dtype=F64)
    assert torch.allclose(weights[0], expected_0) and torch.allclose(weights[1], expected_1)
    huge = plain.softmax_with_sink(torch.full((1, 2, 2), -5.0, dtype=F64), torch.tensor([800.0], dtype=F64))
    assert torch.isfinite(huge).all() and float(huge.abs().max()) < 1e-300


def test_retention_is_a_decaying_sum():
    """o_t = sum over j <= t of decay^(t-j) (q_t . k_j) v_j, heads apart, before the norm and the gate."""
    g = torch.Generator().manual_seed(0)
    T, W, H, d, dv = 7, 10, 2, 4, 3
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 1.0], "rot": {"dims": 2, "base": 10.0}}
    P = {"l0.mix." + n: torch.randn(s, generator=g, dtype=F64) for n, s in
         (("q", (H * d, W)), ("k", (H * d, W)), ("v", (H * dv, W)), ("g", (H * dv, W)), ("o", (W, H * dv)))}
    P["l0.mix.o"] = torch.eye(W, H * dv, dtype=F64)
    h = torch.randn(T, W, generator=g, dtype=F64)
    got = plain.retention_mixer(h, P, "l0.", m, 0.0)[:, :H * dv].view(T, H, dv)
    positions = torch.arange(T)
    q = plain.rotate((h @ P["l0.mix.q"].T).view(T, H, d), positions, m["rot"])
    k = plain.rotate((h @ P["l0.mix.k"].T).view(T, H, d), positions, m["rot"]) / 2.0
    v = (h @ P["l0.mix.v"].T).view(T, H, dv)
    gate = (h @ P["l0.mix.g"].T).view(T, H, dv)
    for t in range(T):
        for head, a in enumerate(m["decay"]):
            o = sum(a ** (t - j) * float(q[t, head] @ k[j, head]) * v[j, head] for j in range(t + 1))
            o = o / torch.sqrt((o * o).mean())
            assert torch.allclose(got[t, head], o * gate[t, head] * torch.sigmoid(gate[t, head]))


def test_routing_and_streams_by_hand():
    t = lambda values: torch.tensor(values, dtype=F64)
    P = {"l0.mlp.router": t([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]]), "l0.mlp.correction": t([0.0, 0.0, 10.0])}
    mlp = {"router": {"experts": 3, "top": 2, "scale": 3.0}}
    chosen, weights = plain.route(t([[2.0, 1.0]]), P, "l0.", mlp)
    # scores sigmoid(2), sigmoid(1), sigmoid(-2): the correction puts the weakest first, its weight stays its score
    assert chosen.tolist() == [[2, 0]]
    assert torch.allclose(weights, 3.0 * torch.sigmoid(t([[-2.0, 2.0]])))
    assert torch.allclose(plain.expert(t([[1.0, -1.0]]), t([[2.0, 0.0], [0.0, 3.0]]), t([[1.0, 1.0]])), t([[4.0]]))
    streams = t([[[1.0]], [[10.0]]])
    Q = {"c.in": t([1.0, 2.0]), "c.out": t([0.5, -1.0]), "c.mix": t([[1.0, 2.0], [3.0, 4.0]])}
    new = plain.hyper_sublayer(streams, Q, "c", lambda u: u * 2.0)      # u = 21, result 42
    assert torch.allclose(new, t([[[1 * 1.0 + 3 * 10.0 + 0.5 * 42]], [[2 * 1.0 + 4 * 10.0 - 42.0]]]))
    assert torch.allclose(plain.norm_around_zero(t([[3.0, 4.0]]), t([0.0, 1.0]), 0.0), t([[3.0, 8.0]]) / math.sqrt(12.5))
