"""Nunivik on the GPU against the plain implementation (``tests/plain/nunivik_plain.py``): every mixer alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests against each alone,
pages and state slots that are freed and taken again, keys at window and page borders, the first tokens, long decoding,
sizes that differ in every respect between the configurations, and greedy generation through ``Engine.generate``.

The configurations and weights are made here.  Weights are drawn so that a fault shows: query and key norm weights
around 2 make the attention peaked, and where a test is about one key a marker token, whose key points where the last
query points, makes that key's score stand out.  float32 runs are held to 3e-4 of the largest logit, which no wrong key, window edge or lost state
survives; bfloat16 runs to 5e-2 of a row's root-mean-square logit.
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import nunivik_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOLERANCE = {"float32": 3e-4, "bfloat16": 5e-2}


# ------------------------------------------------------------------------------------------ configurations
def attention(heads, kv_heads, dim, vdim, window=None, rot=None, factor=None, softcap=None, v_mix=False, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot, "base": 10000.0, "scaling": {"factor": factor or 1.0}}
    if softcap:
        m["softcap"] = softcap
    return m


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def document(width, vocab, layers, scale=3.0, eps=1e-5):
    return {"architecture": "Nunivik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}


DELTA_A = {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 20, "conv": 3}
MAMBA_A = {"heads": 6, "vdim": 16, "state": 24, "groups": 2, "norm_groups": 3, "conv": 4}
DELTA_B = {"heads": 2, "kv_heads": 2, "dim": 36, "vdim": 12, "conv": 5}
MAMBA_B = {"heads": 4, "vdim": 8, "state": 40, "groups": 4, "norm_groups": 1, "conv": 2}

CONFIGS = {
    # a state layer first; keys and values of one size (pages of [2, heads, page, d]); a window smaller than a page; rotation of
    # half a head without stretching; three layers that mix values; a last attention without window, cap or rotation
    "A": document(96, 211, [
        layer("delta", DELTA_A, ff=136),
        layer("attention", attention(6, 3, 32, 32, window=24, rot=16, softcap=30.0, v_mix=True, scale=0.2), ff=120),
        layer("mamba2", MAMBA_A),
        layer("attention", attention(6, 3, 32, 32, window=9, rot=32, factor=2.0, v_mix=True)),
        layer("attention", attention(3, 3, 16, 32, v_mix=True), ff=88),
        layer("attention", attention(4, 1, 16, 40)),
    ]),
    # keys and values of two sizes; one query head per key head; a window of several pages; sizes that are no multiple of
    # 4, 8 or 32; a state-space layer with a group per head and a feed-forward; a single layer that mixes values
    "B": document(64, 130, [
        layer("attention", attention(2, 2, 48, 24, window=70, rot=48, factor=2.5, softcap=15.0)),
        layer("mamba2", MAMBA_B, ff=72),
        layer("delta", DELTA_B),
        layer("attention", attention(4, 2, 24, 10, window=33, rot=8, v_mix=True), ff=40),
    ], scale=1.5, eps=1e-6),
    # heads of 64 for keys and values alike: in bfloat16 the tensor-core kernels read the cache (with the cap and the window as arguments)
    "C": document(128, 300, [
        layer("attention", attention(4, 2, 64, 64, window=100, rot=32, factor=1.0, softcap=25.0, v_mix=True), ff=264),
        layer("delta", {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "conv": 4}),
        layer("attention", attention(4, 2, 64, 64, rot=64, softcap=12.0, v_mix=True), ff=136),
    ], scale=2.0),
}
ALONE = {
    "attention": document(48, 97, [layer("attention", attention(4, 2, 24, 12, window=21, rot=12, factor=3.0, softcap=20.0))], scale=0.4),
    "attention_full": document(48, 97, [layer("attention", attention(2, 1, 40, 40, rot=40))]),
    "delta": document(48, 97, [layer("delta", {"heads": 4, "kv_heads": 2, "dim": 72, "vdim": 18, "conv": 4})]),
    "delta_wide": document(40, 61, [layer("delta", {"heads": 1, "kv_heads": 1, "dim": 136, "vdim": 8, "conv": 2})]),
    "mamba2": document(48, 97, [layer("mamba2", {"heads": 3, "vdim": 24, "state": 16, "groups": 1, "norm_groups": 2, "conv": 3})]),
    "feed_forward": document(48, 97, [layer("mamba2", {"heads": 2, "vdim": 8, "state": 8, "groups": 2, "norm_groups": 1, "conv": 1}, ff=100)]),
}


def make_weights(doc: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors under the design's names: matrices N(0, 1/in), norm weights near 1 (query/key norms near 2),
    decays and step sizes spread over their useful range."""
    from hyperion_b200.models import DecoderModel, get_architecture

    entry = get_architecture("Nunivik")
    model = DecoderModel(entry.build_spec(entry.read_config(doc)), torch.float32, torch.device("meta"))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, wanted in model.expected_tensors().items():
        shape = tuple(wanted.shape)
        leaf = name.split(".", 1)[-1]
        if leaf.endswith("q.norm") or leaf.endswith("k.norm"):
            t = 2.0 + 0.2 * torch.randn(shape, generator=g)
        elif "norm" in leaf:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf.endswith("vmix"):
            t = torch.tensor(0.3 + 0.4 * torch.rand((), generator=g).item())
        elif leaf.endswith("A_log"):
            t = -1.0 + 1.5 * torch.randn(shape, generator=g)
        elif leaf.endswith("dt_bias") or leaf.endswith("conv.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf.endswith(".D"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf.endswith("conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def align_keys_with_queries(doc: dict, weights: dict[str, torch.Tensor], norm: float = 1.6) -> None:
    """Make one score stand out: every key head gets the matrix of its first query head and both norms one weight, so a
    key made from the same token as the query meets it with cosine 1 (before rotation) where other keys' cosines are
    about 1 / sqrt(dim)."""
    for index, entry in enumerate(doc["layers"]):
        if entry["type"] != "attention":
            continue
        m, p = entry["mixer"], f"l{index}.mix."
        rep, d = m["heads"] // m["kv_heads"], m["dim"]
        q = weights[p + "q"].view(m["heads"], d, -1)
        weights[p + "k"] = q[::rep].reshape(m["kv_heads"] * d, -1).clone()
        weights[p + "q.norm"] = torch.full((d,), norm, dtype=torch.bfloat16)
        weights[p + "k.norm"] = torch.full((d,), norm, dtype=torch.bfloat16)
    # the last token of the vocabulary is the marker, the one before it the query: the marker's embedding is mostly the
    # query's, so its key points where the query points, and partly its own, so its value is another
    own = torch.randn(weights["embed"].shape[1], generator=torch.Generator().manual_seed(99))
    weights["embed"][-1] = ((2.0 * weights["embed"][-2].float() + own) / 5 ** 0.5).to(torch.bfloat16)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from hyperion_b200.weights import write_file

    root = tmp_path_factory.mktemp("nunivik_models")
    made = {}
    for index, (name, doc) in enumerate({**CONFIGS, **ALONE}.items()):
        folder = root / name
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(doc))
        weights = make_weights(doc, 11 + index)
        if name == "attention":
            align_keys_with_queries(doc, weights)
        write_file(folder / "model.safetensors", weights)
        made[name] = folder
    return made


_plain_cache: dict = {}


def plain_logits(folder: Path, ids) -> np.ndarray:
    key = (str(folder), tuple(ids))
    if key not in _plain_cache:
        config, weights = plain.read_model_folder(folder)
        _plain_cache[key] = plain.forward(config, weights, list(ids)).numpy()
    return _plain_cache[key]


def ids_for(seed: int, count: int, vocab: int) -> list[int]:
    return torch.randint(0, vocab, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def engine_for(folder, dtype, **options):
    from hyperion_b200.api import Engine

    options.setdefault("page_size", 16)
    options.setdefault("max_tokens", 1024)
    options.setdefault("max_requests", 4)
    return Engine.from_folder(folder, dtype=dtype, **options)


def relative_error(got: np.ndarray, want: np.ndarray) -> float:
    """The largest difference against the largest logit: the sharp measure, which a float32 run meets.  For bfloat16
    results (the engine hands float32 logits in both modes; a bfloat16 run shows in differences above 1e-3), where rounding
    of a peaked attention's scores moves single logits, the worst row's root-mean-square difference against its
    root-mean-square logit."""
    sharp = float(np.abs(got - want).max() / np.abs(want).max())
    if sharp <= TOLERANCE["float32"]:
        return sharp
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    return float((np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))).max())


def run_cut(engine, name, ids, sizes, want_all=True) -> np.ndarray:
    """One request in portions of the given sizes (cycled), every position's logits."""
    from hyperion_b200.engine.batch import StepEntry

    rows, at, k = [], 0, 0
    while at < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - at)
        k += 1
        rows.append(engine.step([StepEntry(name, ids[at:at + n], list(range(n)))]).cpu().numpy().copy())
        at += n
    engine.finish(name)
    engine.check()
    return np.concatenate(rows)


# ------------------------------------------------------------------------------------------ every mechanism alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_layer_of_each_kind(folders, name, dtype):
    """A model of one layer: the whole prompt at once, and again in portions of 5, 2, 1, 9 tokens."""
    vocab = ALONE[name]["vocab"]
    ids = ids_for(3, 75, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype)
    whole = run_cut(engine, "w", ids, [len(ids)])
    assert relative_error(whole, want) <= TOLERANCE[dtype]
    cut = run_cut(engine, "c", ids, [5, 2, 1, 9])
    assert relative_error(cut, want) <= TOLERANCE[dtype]
    if dtype == "float32":
        assert np.array_equal(whole.view(np.uint32), cut.view(np.uint32))


def test_interleaved_rotation_alone():
    """The position part by itself: pairs (2i, 2i+1) of the first dims dimensions, the rest untouched, positions stretched."""
    from hyperion_b200.parts import POSITIONS, BuildContext, PartSpec, base

    dev = torch.device("cuda", 0)
    build = BuildContext(dtype=torch.float32, device=dev, max_positions=1 << 20, shared={})
    part = base.make(POSITIONS, PartSpec("rope_interleaved", "", {"dims": 10, "base": 500.0, "factor": 1.5}), build)
    x = torch.randn(5, 3 * 14 + 6, generator=torch.Generator().manual_seed(1))
    positions = torch.tensor([0, 1, 77, 4000, 123456], dtype=torch.int32)
    xd = x.to(dev).clone()
    part.apply_(xd, 3, 14, positions.to(dev))
    want = plain.rotate_interleaved(x[:, :42].double().view(5, 3, 14), positions, 10, 500.0, 1.5).reshape(5, 42)
    # the angle is a float32 product: it is exact to half a unit in its last place, 2^-24 of the angle
    bound = (positions.double() / 1.5 * 2.0 ** -23 + 1e-6) * x.abs().max().item() * 2
    assert ((xd.cpu().double()[:, :42] - want).abs().max(dim=1).values <= bound).all()
    assert torch.equal(xd.cpu()[:, 42:], x[:, 42:])
    assert torch.equal(xd.cpu().view(5, -1)[:, 10:14], x[:, 10:14])


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_against_token_by_token_and_portions(folders, name, dtype):
    vocab = CONFIGS[name]["vocab"]
    ids = ids_for(5, 150, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=8 if name == "A" else 16)
    results = {"whole": run_cut(engine, "w", ids, [len(ids)]), "single": run_cut(engine, "s", ids, [1]),
               "pairs": run_cut(engine, "p", ids, [2]), "mixed sizes": run_cut(engine, "m", ids, [7, 2, 16, 3, 33, 1, 1, 64])}
    for how, got in results.items():
        assert relative_error(got, want) <= TOLERANCE[dtype], how
        if dtype == "float32":
            assert np.array_equal(got.view(np.uint32), results["whole"].view(np.uint32)), how


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_together_over_pages_and_slots_that_are_used_again(folders, name, dtype):
    """Six requests of unequal length through a cache of 3 state slots and too few pages for all: portions of some beside
    single tokens of others, a request sitting out now and then; as one ends, the next takes its slot and pages."""
    from hyperion_b200.engine.batch import StepEntry

    vocab = CONFIGS[name]["vocab"]
    lengths = [90, 41, 130, 17, 66, 101]
    requests = {f"r{i}": ids_for(50 + i, n, vocab) for i, n in enumerate(lengths)}
    want = {rid: plain_logits(folders[name], ids) for rid, ids in requests.items()}
    engine = engine_for(folders[name], dtype, page_size=16, max_tokens=3 * 144, max_requests=3)
    waiting, live, sizes, k, step = list(requests), {}, [5, 2, 19, 3, 8, 2, 30, 4], 0, 0
    slots_seen: dict[int, set] = {}
    worst = 0.0
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for j, rid in enumerate(list(live)):
            ids, at = requests[rid], live[rid]
            if (step + j) % 5 == 4 and len(live) > 1:
                continue
            n = 1 if at >= len(ids) - 10 else min(sizes[k % len(sizes)], len(ids) - 10 - at)
            k += 1
            entries.append(StepEntry(rid, ids[at:at + n], list(range(n))))
        logits = engine.step(entries).cpu().numpy()
        row = 0
        for entry in entries:
            at = live[entry.request]
            n = len(entry.tokens)
            worst = max(worst, relative_error(logits[row:row + n], want[entry.request][at:at + n]))
            row += n
            live[entry.request] = at + n
            slots_seen.setdefault(engine.cache.slot(entry.request), set()).add(entry.request)
            if at + n == len(requests[entry.request]):
                engine.finish(entry.request)
                del live[entry.request]
        step += 1
    engine.check()
    engine.cache.check()
    assert worst <= TOLERANCE[dtype], worst
    assert max(len(users) for users in slots_seen.values()) >= 2  # a slot served more than one request


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_window_edge_and_far_away(folders, dtype):
    """One attention layer with a window of 21 over pages of 8: a marker token stands at a chosen distance behind the
    last token and nowhere else, so its key scores high against the last query (the layer's key matrices are its query matrices).  Distances
    just inside the window (19, 20), just outside (21, 22), at page borders (8, 16) and far away (150) are each run as a
    whole prompt and with the tail decoded token by token."""
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "attention", ALONE["attention"]["vocab"]
    engine = engine_for(folders[name], dtype, page_size=8)
    for distance in (1, 7, 8, 16, 19, 20, 21, 22, 150):
        ids = ids_for(900 + distance, 200, vocab - 2)  # the last two tokens of the vocabulary are kept for the marked places
        ids[-1], ids[-1 - distance] = vocab - 2, vocab - 1
        want = plain_logits(folders[name], ids)
        whole = engine.step([StepEntry("w", ids, [len(ids) - 1])]).cpu().numpy()[0]
        engine.finish("w")
        assert relative_error(whole, want[-1]) <= TOLERANCE[dtype], distance
        head = len(ids) - 30
        engine.step([StepEntry("d", ids[:head], [])])
        for at in range(head, len(ids)):
            last = engine.step([StepEntry("d", [ids[at]], [0])]).cpu().numpy()[0]
            assert relative_error(last, want[at]) <= TOLERANCE[dtype], (distance, at)
        engine.finish("d")
    engine.check()
    # the marked key matters: the plain logits move by a hundred float32 tolerances when it is taken away or stands one place further back
    inside = ids_for(920, 200, vocab - 2)
    inside[-1], inside[-21] = vocab - 2, vocab - 1
    without = list(inside)
    without[-21] = 0
    outside = list(inside)
    outside[-21], outside[-22] = inside[-22], vocab - 1
    base = plain_logits(folders[name], inside)[-1]
    assert relative_error(plain_logits(folders[name], without)[-1], base) > 100 * TOLERANCE["float32"]
    assert relative_error(plain_logits(folders[name], outside)[-1], base) > 100 * TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(folders, dtype):
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "B", CONFIGS["B"]["vocab"]
    ids = ids_for(8, 400, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=32, max_tokens=512)
    worst = 0.0
    for at, token in enumerate(ids):  # position 0 alone, then every other one: a one-token prompt and 399 decoded tokens
        worst = max(worst, relative_error(engine.step([StepEntry("r", [token], [0])]).cpu().numpy()[0], want[at]))
    engine.finish("r")
    pair = engine.step([StepEntry("pair", ids[:2], [0, 1])]).cpu().numpy()
    engine.finish("pair")
    engine.check()
    assert relative_error(pair, want[:2]) <= TOLERANCE[dtype]
    # 400 positions of a peaked attention: in bfloat16 the worst row of the whole prompt in one step may itself pass the
    # tolerance of the shorter tests; decoding token by token must not be further off than that
    whole = relative_error(run_cut(engine, "whole", ids, [len(ids)]), want)
    assert worst <= max(TOLERANCE[dtype], 1.25 * whole), (worst, whole)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_scheduler(folders, name):
    from hyperion_b200.sampling import SamplingParams

    vocab = CONFIGS[name]["vocab"]
    prompts = [ids_for(300 + i, n, vocab) for i, n in enumerate([5, 37, 1, 80, 23])]
    config, weights = plain.read_model_folder(folders[name])

    def greedy(prompt, count):
        ids = list(prompt)
        for _ in range(count):
            ids.append(int(plain.forward(config, weights, ids)[-1].argmax()))
        return ids[len(prompt):]

    want = [greedy(prompt, 6) for prompt in prompts]
    engine = engine_for(folders[name], "float32", max_tokens=3 * 128, max_requests=3)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), max_batch_tokens=48, prefill_chunk_busy=16)
    assert got == want
    engine = engine_for(folders[name], "bfloat16", max_tokens=3 * 128, max_requests=3)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), max_batch_tokens=48, prefill_chunk_busy=16)
    for prompt, tokens in zip(prompts, got):
        logits = plain.forward(config, weights, prompt + tokens).numpy()
        for i, token in enumerate(tokens):  # on its own tokens, every choice is the plain argmax or a near tie of it
            row = logits[len(prompt) + i - 1]
            assert row.max() - row[token] <= 2 * TOLERANCE["bfloat16"] * np.abs(row).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_command(folders, dtype, tmp_path):
    """bin/trace_run on a model of this design: two requests side by side, one ends, a third takes its place."""
    name, vocab = "A", CONFIGS["A"]["vocab"]
    a, b, c = ids_for(1, 70, vocab), ids_for(2, 33, vocab), ids_for(3, 50, vocab)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [39]}, {"id": "b", "tokens": b[:31], "want": [0, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:42], "want": [0, 1]}, {"id": "b", "tokens": b[31:32], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[32:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c, "want": [49]}, {"id": "a", "tokens": a[42:], "want": [27]}], "end": ["a", "c"]}]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype", dtype, "--out", str(tmp_path),
                           "--max-tokens", "192"], input=text, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(4)]
    ref = {"a": plain_logits(folders[name], a), "b": plain_logits(folders[name], b), "c": plain_logits(folders[name], c)}
    read = lambda step: np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
    expected = {0: [ref["a"][39], ref["b"][0], ref["b"][30]], 1: [ref["a"][40], ref["a"][41], ref["b"][31]], 2: [ref["b"][32]],
                3: [ref["c"][49], ref["a"][69]]}
    for step, rows in expected.items():
        assert relative_error(read(step), np.stack(rows)) <= TOLERANCE[dtype], step


def test_the_command_line_writes_a_random_model_and_generates_with_it(tmp_path):
    """``python -m hyperion_b200 random`` from a config.json of this design, then ``generate`` on the folder it wrote:
    the tokens are the plain implementation's greedy ones."""
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["B"]))
    folder = tmp_path / "model"
    run = lambda *args: subprocess.run([sys.executable, "-m", "hyperion_b200", *args], capture_output=True, text=True, timeout=900, cwd=ROOT)
    done = run("random", "--config", str(config), "--out", str(folder), "--seed", "5", "--std", "0.3")
    assert done.returncode == 0, done.stderr[-2000:]
    prompt = ids_for(71, 19, CONFIGS["B"]["vocab"])
    done = run("generate", "-m", str(folder), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
               "--ignore-eos", "--max-batch", "2")
    assert done.returncode == 0, done.stderr[-2000:]
    got = json.loads(done.stdout.strip().splitlines()[-1])
    plain_config, weights = plain.read_model_folder(folder)
    ids = list(prompt)
    for _ in range(5):
        ids.append(int(plain.forward(plain_config, weights, ids)[-1].argmax()))
    assert got["tokens"] == ids[len(prompt):] and got["finish_reason"] == "length"
