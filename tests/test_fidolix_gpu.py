"""The Fidolix decoder in the engine against the plain implementation (tests/plain_fidolix.py): whole prompts,
prompts then tokens one by one (the first tokens of a sequence, decoding past every window), prompts in portions down
to two tokens, batches of unequal requests with early finishers and slots, pages and states used again, long decoding,
the stream after every run of a layer, greedy generation through Engine.generate, the command line and the trace
runner; in float32 and in bfloat16, on configurations that differ in every size."""
import numpy as np
import pytest
import torch

import plain_fidolix
from fidolix_models import FIDOLIX, make_folder
from helpers import random_tokens, run_trace, stored_dtype

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# float32: a position's logits differ from the plain ones by at most this fraction of the logits' spread, in the root
# mean square over the vocabulary (the order of the sums), and a single logit by four times that.  This is the sharp
# test of every mechanism, position by position; both builds run the same kernels apart from the projections.
# bfloat16: the test models' attention is peaked and their time mixing remembers long, so the rounding of a
# projection's inputs moves most positions by a few hundredths of the spread and a few by more; a lost sink, gate,
# state, tap, window edge or group moves positions by 0.16 or more (tests/test_fidolix.py shows that on the plain
# implementation).  So: ROW_NOISE for all but ROWS_OVER of a request's positions (one, in a short request), ROW_LIMIT
# for every position (a router that chooses one expert of sixteen sharpened ones moves a position that far when it
# makes a call that is not close enough to be followed), MEAN_NOISE for their root mean square; and the routers' choices may differ from the plain ones by
# more than a close call in FAR_CALLS of the decisions (plus one).
ROW_NOISE = {"bfloat16": 0.08, "float32": 1.5e-4}
ROWS_OVER, ROW_LIMIT, MEAN_NOISE, FAR_CALLS = 0.04, 0.45, 0.05, 0.02


class Folders:
    def __init__(self, root):
        self.root, self.made, self.logits, self.loaded = root, {}, {}, {}

    def __getitem__(self, key):
        name, dtype = key
        if key not in self.made:
            self.made[key] = make_folder(self.root / f"{name}_{dtype}", FIDOLIX[name], seed=5 + list(FIDOLIX).index(name),
                                         dtype=stored_dtype(dtype))
        return self.made[key]

    def weights(self, name, dtype):
        if (name, dtype) not in self.loaded:
            self.loaded[name, dtype] = plain_fidolix.load_folder(self[name, dtype])
        return self.loaded[name, dtype]

    def plain(self, name, dtype, tokens, proposed=None):
        key = (name, dtype, tuple(tokens))
        if proposed is not None or key not in self.logits:
            config, weights = self.weights(name, dtype)
            logits = plain_fidolix.logits_of(config, weights, list(tokens), proposed)
            if proposed is not None:
                return logits
            self.logits[key] = logits
        return self.logits[key]


class Choices:
    """The experts the engine's routers chose, per slot, run of a layer and position.  In bfloat16 the router's input is
    a rounded number, and where two scores are nearer than that rounding the engine may choose the other expert; the
    plain implementation then follows it (``plain_fidolix.route``), for that is no fault.  A choice that is not a close
    call is not followed and shows as a difference.  A step that is watched does not run as a graph."""

    def __init__(self, engine):
        self.seen = {}
        engine.model.choice_probe = self

    def __call__(self, run_index, step, chosen):
        rows, at = chosen.cpu().tolist(), 0
        for slot, count, before in zip(step.slots, step.q_lens, step.ctx_before):
            layer = self.seen.setdefault(slot, {}).setdefault(run_index, {})
            for j in range(count):
                layer[before + j] = rows[at + j]
            at += count

    def take(self, slot, length):
        proposed = {}
        for run, by_position in self.seen.pop(slot, {}).items():
            table = torch.full((length, len(next(iter(by_position.values())))), -1, dtype=torch.long)
            for position, experts in by_position.items():
                table[position] = torch.tensor(experts)
            proposed[run] = table
        return proposed


class Session:
    """An engine with what a test needs to compare a finished request with the plain implementation."""

    def __init__(self, folders, name, dtype, watch=None, **more):
        self.folders, self.name, self.dtype = folders, name, dtype
        self.engine = engine_for(folders[name, dtype], dtype, **more)
        watch = dtype == "bfloat16" if watch is None else watch
        self.choices = Choices(self.engine) if watch else None

    def reference(self, slot, tokens):
        """The plain logits of ``tokens``, a request that ran in ``slot`` (call it once, after the request's last step)."""
        proposed = self.choices.take(slot, len(tokens)) if self.choices is not None else None
        return self.folders.plain(self.name, self.dtype, tokens, proposed)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return Folders(tmp_path_factory.mktemp("fidolix"))


def engine_for(folder, dtype, max_tokens=2048, block_size=64, **more):
    from stratakv_b200 import Engine, EngineConfig
    return Engine.from_folder(folder, EngineConfig(max_tokens=max_tokens, dtype=dtype, block_size=block_size, **more),
                              verbose=False)


def check(got, ref, dtype, what=""):
    got = got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert got.shape == ref.shape, what
    spread = float(np.asarray(ref, dtype=np.float64).std())
    difference = got.astype(np.float64) - ref
    per_position = np.sqrt((difference ** 2).mean(axis=-1)) / spread
    worst = int(per_position.argmax())
    if dtype == "float32":
        assert per_position[worst] <= ROW_NOISE[dtype], f"{what}: row {worst} is off by {per_position[worst]:.2e} of the spread"
        assert np.abs(difference).max() <= 4 * ROW_NOISE[dtype] * spread, f"{what}: a logit is off by {np.abs(difference).max() / spread:.2e} of the spread"
        return
    far = plain_fidolix.FAR_CALLS
    assert len(far) <= 1 + FAR_CALLS * plain_fidolix.DECISIONS[0], \
        f"{what}: {len(far)} of {plain_fidolix.DECISIONS[0]} choices of experts differ by more than a close call: {far[:8]}"
    over = per_position > ROW_NOISE[dtype]
    told = f"{what}: {int(over.sum())} of {len(per_position)} rows are off by more than {ROW_NOISE[dtype]} of the spread " \
           f"(rows {np.nonzero(over)[0][:8].tolist()}), the worst, row {worst}, by {per_position[worst]:.2e}; " \
           f"root mean square {np.sqrt((per_position ** 2).mean()):.2e}"
    assert over.sum() <= max(1, ROWS_OVER * len(per_position)), told
    assert per_position.max() <= ROW_LIMIT, told
    assert per_position.size < 8 or np.sqrt((per_position ** 2).mean()) <= MEAN_NOISE, told


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FIDOLIX))
def test_whole_prompts(folders, dtype, name):
    from stratakv_b200 import StepEntry
    session = Session(folders, name, dtype)
    engine = session.engine
    for length in (1, 2, 3, 33, 64, 65, 150, 300):
        tokens = random_tokens(FIDOLIX[name]["vocab"], length, seed=length)
        slot = engine.open_sequence()
        got = engine.step([StepEntry(slot, tokens, list(range(length)))]).clone()
        check(got, session.reference(slot, tokens), dtype, f"{name} whole length {length}")
        engine.close_sequence(slot)
    engine.check_flags()
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["FA", "FC"])
def test_the_stream_after_every_run_of_a_layer(folders, dtype, name):
    """Run by run (a layer that runs twice counts twice): the float32 residual stream against the plain one."""
    from stratakv_b200 import StepEntry
    session = Session(folders, name, dtype)
    engine = session.engine
    tokens = random_tokens(FIDOLIX[name]["vocab"], 70, seed=12)
    seen = []
    engine.model.layer_probe = lambda index, x: seen.append(x.detach().cpu().double().clone())
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens, [])])
    engine.model.layer_probe = None
    config, weights = folders.weights(name, dtype)
    streams = []
    proposed = session.choices.take(slot, len(tokens)) if session.choices is not None else None
    plain_fidolix.forward(config, weights, tokens, layer_outputs=streams, proposed=proposed)
    order, _ = plain_fidolix.layer_runs(config)
    assert len(seen) == len(order) == len(streams)
    for index, (got, ref) in enumerate(zip(seen, streams)):
        allowed = (3e-5 if dtype == "float32" else 0.06) * float(ref.std())
        worst = float(torch.sqrt(((got - ref) ** 2).mean(dim=-1)).max())
        assert worst <= allowed, f"after run {index} (layer {order[index]}): {worst / float(ref.std()):.2e} of the spread"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FIDOLIX))
def test_prompt_then_tokens_one_by_one(folders, dtype, name):
    """The first tokens of a sequence decoded alone (prompts of 1 and 2: the convolution and the token shift start
    from nothing), and decoding that starts inside a page, runs over page borders, past every window and through the
    graphs of a step."""
    from stratakv_b200 import StepEntry
    session = Session(folders, name, dtype)
    engine = session.engine
    for prompt, total in ((1, 40), (2, 10), (50, 140), (120, 330)):
        tokens = random_tokens(FIDOLIX[name]["vocab"], total, seed=total)
        slot = engine.open_sequence()
        got = [engine.step([StepEntry(slot, tokens[:prompt], list(range(prompt)))]).clone()]
        for p in range(prompt, total):
            got.append(engine.step([StepEntry(slot, [tokens[p]], [0])]).clone())
        check(torch.cat(got), session.reference(slot, tokens), dtype, f"{name} a prompt of {prompt}, then one by one")
        engine.close_sequence(slot)
    engine.check_flags()


@pytest.mark.parametrize("name", ["FA", "FC"])
def test_decoding_through_the_graphs(folders, name):
    """bfloat16 steps of one token that nobody watches run as CUDA graphs (a watched router's step does not): a graph's
    warm-up and first replay run a step twice, which the states must survive."""
    from stratakv_b200 import StepEntry
    dtype = "bfloat16"
    session = Session(folders, name, dtype, watch=False)
    engine = session.engine
    tokens = random_tokens(FIDOLIX[name]["vocab"], 150, seed=3)
    ref = folders.plain(name, dtype, tokens)
    slot = engine.open_sequence()
    got = [engine.step([StepEntry(slot, tokens[:20], [19])]).clone()]
    for p in range(20, 150):
        got.append(engine.step([StepEntry(slot, [tokens[p]], [0])]).clone())
    assert engine.graph_launches > 0
    difference = torch.cat(got).float().cpu().numpy().astype(np.float64) - ref[19:]
    per_position = np.sqrt((difference ** 2).mean(axis=-1)) / ref.std()
    # no router is followed here, so a close call may move a position; most positions say whether the states held
    assert np.median(per_position) <= 0.04 and (per_position > ROW_NOISE[dtype]).mean() <= 0.1, \
        f"{name}: median {np.median(per_position):.3f}, {(per_position > ROW_NOISE[dtype]).sum()} rows over"
    engine.close_sequence(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FIDOLIX))
def test_prompts_in_portions(folders, dtype, name):
    """Portions of one and two tokens (shorter than the convolution reaches), ones that end at and after a page's
    border, ones shorter and longer than the windows."""
    from stratakv_b200 import StepEntry
    session = Session(folders, name, dtype)
    engine = session.engine
    for portions in ((70, 65, 40), (2, 2, 2, 2, 2), (63, 2, 1, 64, 33), (130, 2, 100), (1, 1, 3, 1, 2, 5)):
        tokens = random_tokens(FIDOLIX[name]["vocab"], sum(portions), seed=sum(portions))
        slot, at, got = engine.open_sequence(), 0, []
        for count in portions:
            got.append(engine.step([StepEntry(slot, tokens[at:at + count], list(range(count)))]).clone())
            at += count
        check(torch.cat(got), session.reference(slot, tokens), dtype, f"{name} in portions of {portions}")
        engine.close_sequence(slot)
    engine.check_flags()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FIDOLIX))
def test_unequal_batches_with_early_finishers_and_reuse(folders, dtype, name):
    """Two batches one after the other in one engine whose cache just holds one of them: the second takes the
    slots, pages and states that the first gave back."""
    from stratakv_b200 import StepEntry
    vocab = FIDOLIX[name]["vocab"]
    session = Session(folders, name, dtype, max_tokens=64 * 12, max_batch=4)
    engine = session.engine
    for batch, shapes in enumerate((((1, 5), (70, 12), (200, 30), (129, 31)), ((3, 33), (190, 3), (64, 40), (2, 1)))):
        requests = [random_tokens(vocab, prompt + more, seed=100 * batch + i) for i, (prompt, more) in enumerate(shapes)]
        slots = [engine.open_sequence() for _ in requests]
        first = engine.step([StepEntry(slot, tokens[:prompt], [prompt - 1])
                             for slot, tokens, (prompt, _) in zip(slots, requests, shapes)]).clone()
        got = [[first[row:row + 1]] for row in range(len(requests))]

        def finish(i):
            # the positions from the prompt's last on, against the plain run of the whole request
            ref = session.reference(slots[i], requests[i])
            check(torch.cat(got[i]), ref[shapes[i][0] - 1:], dtype, f"{name} batch {batch} request {i}")
            engine.close_sequence(slots[i])

        for step in range(max(more for _, more in shapes)):
            live = [i for i, (_, more) in enumerate(shapes) if step < more]
            rows = engine.step([StepEntry(slots[i], [requests[i][shapes[i][0] + step]], [0]) for i in live]).clone()
            for row, i in enumerate(live):
                got[i].append(rows[row:row + 1])
            for i in live:
                if step + 1 == shapes[i][1]:
                    finish(i)
        engine.check_flags()
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_of_sixteen_and_long_decoding(folders, dtype):
    """Small pages and 400 tokens one by one: the time mixing's state is carried for hundreds of steps, the windows
    pass over many pages (which come back as they go) and the attention layers read across twenty-odd."""
    from stratakv_b200 import StepEntry
    name = "FA"
    session = Session(folders, name, dtype, max_tokens=16 * 30, block_size=16, max_batch=1)
    engine = session.engine
    tokens = random_tokens(FIDOLIX[name]["vocab"], 430, seed=77)
    slot = engine.open_sequence()
    got = [engine.step([StepEntry(slot, tokens[:30], [29])]).clone()]
    for p in range(30, 430):
        got.append(engine.step([StepEntry(slot, [tokens[p]], [0])]).clone())
    check(torch.cat(got), session.reference(slot, tokens)[29:], dtype, "a prompt of 30, then 400 one by one")
    engine.close_sequence(slot)
    assert engine.cache.all_free()


@pytest.mark.parametrize("name", ["FA", "FB"])
def test_greedy_generation_through_the_engine(folders, name):
    """Engine.generate (the scheduler, the graph steps that run ahead of the host, the sampler): every token it
    chooses is the plain implementation's best or within rounding of it."""
    dtype = "float32"
    engine = engine_for(folders[name, dtype], dtype, max_tokens=1024)
    vocab = FIDOLIX[name]["vocab"]
    prompts = [random_tokens(vocab, n, seed=900 + n) for n in (1, 9, 70)]
    output = engine.generate(prompts, 24, ignore_eos=True)
    config, weights = folders.weights(name, dtype)
    for prompt, sequence in zip(prompts, output.sequences):
        assert len(sequence) == len(prompt) + 24 and sequence[:len(prompt)] == prompt
        logits = plain_fidolix.logits_of(config, weights, sequence)
        for at in range(len(prompt), len(sequence)):
            row = logits[at - 1]
            assert row[sequence[at]] >= row.max() - 1e-4 * max(1.0, abs(row.max())), f"{name}: token {at} is not the best"
    assert engine.cache.all_free()


def test_generation_in_bfloat16_repeats_itself(folders):
    """Generation through graphs and through eager steps chooses the same tokens (every state included)."""
    name, dtype = "FA", "bfloat16"
    prompts = [random_tokens(FIDOLIX[name]["vocab"], n, seed=40 + n) for n in (5, 31)]
    outputs = []
    for graphs in (True, False):
        engine = engine_for(folders[name, dtype], dtype, max_tokens=512, use_cuda_graphs=graphs)
        outputs.append(engine.generate(prompts, 20, ignore_eos=True).sequences)
    assert outputs[0] == outputs[1]


def test_command_line_generates_from_a_fidolix_folder(folders):
    """bin/stratakv_cli opens the folder through the registry like every other entry point; greedy, float32."""
    import subprocess
    import sys
    from helpers import ROOT
    name = "FD"
    folder = folders[name, "float32"]
    prompt = random_tokens(FIDOLIX[name]["vocab"], 12, seed=8)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "stratakv_cli"), "--dtype", "float32", "--temp", "0",
                           "--ignore-eos", str(folder), "10", *[str(t) for t in prompt]],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    sequence = [int(word) for word in done.stdout.split()]
    assert len(sequence) == 22 and sequence[:12] == prompt
    config, weights = folders.weights(name, "float32")
    logits = plain_fidolix.logits_of(config, weights, sequence)
    for at in range(12, 22):
        row = logits[at - 1]
        assert row[sequence[at]] >= row.max() - 1e-4 * max(1.0, abs(row.max()))


def test_trace_runner_chooses_the_model_by_its_config(folders, tmp_path):
    name, dtype = "FB", "float32"
    folder = folders[name, dtype]
    vocab = FIDOLIX[name]["vocab"]
    a, b = random_tokens(vocab, 75, seed=1), random_tokens(vocab, 20, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:18], "want": [17]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:71], "want": [0]}, {"id": "b", "tokens": b[18:19], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[71:72], "want": [0]}, {"id": "b", "tokens": b[19:20], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[72:75], "want": [2]}], "end": ["a"]}]
    logits = run_trace(folder, dtype, steps, tmp_path / "out", max_tokens=256, vocab=vocab)
    ref_a, ref_b = folders.plain(name, dtype, a), folders.plain(name, dtype, b)
    check(logits[0], np.stack([ref_a[0], ref_a[69], ref_b[17]]), dtype, "step 0")
    check(logits[1], ref_a[70:71], dtype, "step 1")
    check(logits[2], np.stack([ref_a[71], ref_b[19]]), dtype, "step 2")
    check(logits[3], ref_a[74:75], dtype, "step 3")
