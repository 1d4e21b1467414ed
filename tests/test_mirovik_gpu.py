"""Mirovik on the GPU against the plain implementation (``tests/plain/mirovik_plain.py``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests against each alone,
pages and state slots that are freed and taken again, keys at the edges of the distance buckets, at page borders and far
away, the first tokens, long decoding, sizes that differ in every respect between the configurations, and greedy
generation through ``Engine.generate``.

The configurations and weights are made here.  Weights are drawn so that a fault shows: query and key norm weights around 2
make the attention peaked, the distance biases are large, and where a test is about one key a marker token, whose key
points where the last query points, makes that key's score stand out.  float32 runs are held to 3e-4 of the largest
logit, which no wrong key, bucket or lost state survives; bfloat16 runs to 5e-2 of a row's root-mean-square logit.
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import mirovik_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOLERANCE = {"float32": 3e-4, "bfloat16": 5e-2}


# ------------------------------------------------------------------------------------------ configurations
def left(heads, kv_heads, dim, vdim, bias_max, buckets, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "bias_max": bias_max, "buckets": buckets}


def right(heads, dim, vdim, decay, rot=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return m


def parallel(l, r, left_scale=0.7, right_scale=1.1):
    return {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}


def selective(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(count, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": count, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def document(width, vocab, layers, loop=None, scale=3.0, eps=1e-5):
    doc = {"architecture": "Mirovik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}
    if loop:
        doc["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return doc


CONFIGS = {
    # a selective scan first; a run of two layers in the middle passed three times; keys and values of one size; two experts per
    # token plus a shared one; a layer without a feed-forward; a last layer whose every expert is used by every token, no shared one
    "A": document(96, 211, [
        layer("mamba1", selective(160, 12, 6, 3), dense(136)),
        layer("parallel", parallel(left(6, 3, 32, 32, 40, 12), right(3, 24, 20, [0.9, 0.97, 0.995], rot=16)), experts(5, 2, 40, shared=56)),
        layer("parallel", parallel(left(4, 1, 16, 40, 300, 10, scale=0.3), right(2, 36, 12, [1.0, 0.5], rot=36, base=500.0), 1.3, 0.4)),
        layer("mamba1", selective(72, 40, 3, 2), experts(3, 3, 24)),
    ], loop=(1, 3, 3)),
    # one layer passed twice; keys and values of two sizes; one query head per key head; sizes that are no multiple of 4, 8 or 32; a
    # rotation of a small part of the head; a selective scan with one step input, five taps and no feed-forward
    "B": document(64, 130, [
        layer("parallel", parallel(left(2, 2, 48, 24, 64, 8), right(4, 8, 40, [0.8, 0.9, 0.99, 0.999], rot=4)), dense(72)),
        layer("mamba1", selective(100, 5, 1, 5)),
        layer("parallel", parallel(left(3, 1, 20, 10, 17, 6), right(1, 68, 6, [0.96]), 1.0, 1.0), experts(7, 1, 36, shared=20)),
    ], loop=(1, 2, 2), scale=1.5, eps=1e-6),
    # no repeated run at all; heads of 64 for keys and values alike; experts and a shared expert whose sizes fill whole tiles
    "C": document(128, 300, [
        layer("parallel", parallel(left(4, 2, 64, 64, 128, 32), right(2, 64, 64, [0.98, 0.999], rot=32)), experts(8, 2, 128, shared=128)),
        layer("mamba1", selective(256, 16, 8, 4), dense(264)),
    ], scale=2.0),
}
ALONE = {
    "attention": document(48, 97, [layer("parallel", parallel(left(4, 2, 24, 12, 30, 8, scale=0.25), right(1, 8, 8, [0.9]), 1.0, 0.0))], scale=0.4),
    # heads of 128 for keys and values alike: in bfloat16 the tensor-core kernels read the pages, with the bias table as an argument
    "attention_wide": document(64, 97, [layer("parallel", parallel(left(2, 1, 128, 128, 40, 8), right(1, 8, 8, [0.9]), 1.0, 0.0))], scale=0.5),
    # heads of 192: the TMA-fed tile kernel serves prompt portions too; beside a retention of 6 values, so that the attention's columns
    # of the buffer both branches fill do not start rows on 16-byte pieces
    "attention_192": document(64, 97, [layer("parallel", parallel(left(2, 2, 192, 192, 40, 8), right(1, 8, 6, [0.9]), 1.0, 0.0))], scale=0.5),
    "retention": document(48, 97, [layer("parallel", parallel(left(1, 1, 8, 8, 9, 4), right(3, 20, 28, [0.9, 0.99, 0.999], rot=12), 0.0, 1.0))]),
    "retention_wide": document(40, 61, [layer("parallel", parallel(left(1, 1, 8, 8, 9, 4), right(1, 136, 8, [0.97], rot=136), 0.0, 1.0))]),
    "selective": document(48, 97, [layer("mamba1", selective(88, 24, 5, 4))]),
    "selective_wide": document(40, 61, [layer("mamba1", selective(24, 136, 2, 1))]),
    "experts": document(48, 97, [layer("mamba1", selective(16, 4, 1, 2), experts(6, 2, 28, shared=12))]),
    "dense": document(48, 97, [layer("mamba1", selective(16, 4, 1, 2), dense(100))], loop=(0, 1, 1)),
}


def make_weights(doc: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors under the design's names: matrices N(0, 1/in), the layers' norm weights near 0, query/key norms near 2,
    large distance biases, decays and step sizes spread over their useful range."""
    from hyperion_b200.models import DecoderModel, get_architecture

    entry = get_architecture("Mirovik")
    model = DecoderModel(entry.build_spec(entry.read_config(doc)), torch.float32, torch.device("meta"))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, wanted in model.expected_tensors().items():
        shape = tuple(wanted.shape)
        if name.endswith("q.norm") or name.endswith("k.norm"):
            t = 2.0 + 0.2 * torch.randn(shape, generator=g)
        elif "norm" in name.rsplit(".", 1)[-1]:
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".rel"):
            t = 1.5 * torch.randn(shape, generator=g)
        elif name.endswith("A_log"):
            t = 0.7 * torch.randn(shape, generator=g)
        elif name.endswith("dt.b"):
            t = -2.0 + torch.randn(shape, generator=g)
        elif name.endswith("conv.b") or name == "loop.step":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g) * (4.0 / shape[-1] ** 0.5)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def align_keys_with_queries(doc: dict, weights: dict[str, torch.Tensor], norm: float = 1.6) -> None:
    """Make one score stand out: every key head gets the matrix of its first query head and both norms one weight, so a key
    made from the same token as the query meets it with cosine 1 where other keys' cosines are about 1 / sqrt(dim)."""
    for index, entry in enumerate(doc["layers"]):
        if entry["type"] != "parallel":
            continue
        m, p = entry["mixer"]["left"], f"l{index}.mix.left."
        rep, d = m["heads"] // m["kv_heads"], m["dim"]
        q = weights[p + "q"].view(m["heads"], d, -1)
        weights[p + "k"] = q[::rep].reshape(m["kv_heads"] * d, -1).clone()
        weights[p + "q.norm"] = torch.full((m["heads"] * d,), norm, dtype=torch.bfloat16)
        weights[p + "k.norm"] = torch.full((m["kv_heads"] * d,), norm, dtype=torch.bfloat16)
    # the last token of the vocabulary is the marker, the one before it the query: the marker's embedding is mostly the
    # query's, so its key points where the query points, and partly its own, so its value is another
    own = torch.randn(weights["embed"].shape[1], generator=torch.Generator().manual_seed(99))
    weights["embed"][-1] = ((2.0 * weights["embed"][-2].float() + own) / 5 ** 0.5).to(torch.bfloat16)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from hyperion_b200.weights import write_file

    root = tmp_path_factory.mktemp("mirovik_models")
    made = {}
    for index, (name, doc) in enumerate({**CONFIGS, **ALONE}.items()):
        folder = root / name
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(doc))
        weights = make_weights(doc, 11 + index)
        if name == "attention":
            align_keys_with_queries(doc, weights)
        if name in ("attention_wide", "attention_192"):  # a flat attention that favours the keys of the last bucket: what the far tiles add decides the result
            weights["l0.mix.left.rel"][-1] = 4.0
            for norm in ("l0.mix.left.q.norm", "l0.mix.left.k.norm"):
                weights[norm] = (0.25 * weights[norm].float()).to(torch.bfloat16)
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
    results, where rounding of a peaked attention's scores moves single logits, the worst row's root-mean-square
    difference against its root-mean-square logit."""
    sharp = float(np.abs(got - want).max() / np.abs(want).max())
    if sharp <= TOLERANCE["float32"]:
        return sharp
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    return float((np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))).max())


def rows_over(got: np.ndarray, want: np.ndarray, tolerance: float) -> float:
    """The fraction of rows whose root-mean-square difference is more than ``tolerance`` of the row's root-mean-square logit."""
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    return float(((np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))) > tolerance).mean())


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what=None, routed: bool = False) -> None:
    """float32: every logit to the sharp measure.  bfloat16: every row to its tolerance, except in models with routed experts
    against the plain implementation: there the router reads rows that carry the rounding of everything before them, a token
    whose best experts lie close together may go to another expert than in exact arithmetic, and such a token's row is off;
    up to a tenth of the rows may be (a wrong key, a lost state or a wrong slot moves all rows behind it, not a tenth)."""
    if dtype == "bfloat16" and routed:
        assert rows_over(got, want, TOLERANCE[dtype]) <= 0.1, what
    else:
        assert relative_error(got, want) <= TOLERANCE[dtype], what


def run_cut(engine, name, ids, sizes) -> np.ndarray:
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
    assert_close(whole, want, dtype, routed=name == "experts")
    cut = run_cut(engine, "c", ids, [5, 2, 1, 9])
    assert_close(cut, want, dtype, routed=name == "experts")
    assert rows_over(cut, whole, TOLERANCE[dtype]) <= 0.03  # the same arithmetic on both sides: rows agree however the work is cut
    if dtype == "float32":
        assert np.array_equal(whole.view(np.uint32), cut.view(np.uint32))


def test_half_rotation_alone():
    """The position part by itself: dimension i with i + dims/2 over the first dims dimensions, the rest untouched."""
    from hyperion_b200.parts import POSITIONS, BuildContext, PartSpec, base

    dev = torch.device("cuda", 0)
    build = BuildContext(dtype=torch.float32, device=dev, max_positions=1 << 20, shared={})
    part = base.make(POSITIONS, PartSpec("rope_half_partial", "", {"dims": 10, "base": 500.0}), build)
    x = torch.randn(5, 3 * 14 + 6, generator=torch.Generator().manual_seed(1))
    positions = torch.tensor([0, 1, 77, 4000, 123456], dtype=torch.int32)
    xd = x.to(dev).clone()
    part.apply_(xd, 3, 14, positions.to(dev))
    want = plain.rotate_half(x[:, :42].double().view(5, 3, 14), positions, 10, 500.0).reshape(5, 42)
    bound = (positions.double() * 2.0 ** -23 + 1e-6) * x.abs().max().item() * 2  # the angle is a float32 product
    assert ((xd.cpu().double()[:, :42] - want).abs().max(dim=1).values <= bound).all()
    assert torch.equal(xd.cpu()[:, 42:], x[:, 42:])
    assert torch.equal(xd.cpu().view(5, -1)[:, 10:14], x[:, 10:14])


def test_distance_buckets_as_a_table_by_distance():
    """The bias a key n positions back gets is the row of its bucket, for every n up to and beyond the last bucket's start."""
    from hyperion_b200.parts import MIXERS, BuildContext, PartSpec, base

    dev = torch.device("cuda", 0)
    build = BuildContext(dtype=torch.float32, device=dev, max_positions=1 << 20, shared={})
    for buckets, far in ((16, 128), (6, 17), (32, 1000), (2, 5)):
        part = base.make(MIXERS, PartSpec("biased_attention", "", {"hidden_size": 8, "heads": 3, "kv_heads": 1, "head_dim": 4, "scale": 1.0,
                                                                   "bias_max": far, "eps": 1e-6}), build)
        rel = torch.randn(buckets, 3, generator=torch.Generator().manual_seed(buckets))
        part.load_core({"q.norm": torch.ones(12), "k.norm": torch.ones(4), "rel": rel.to(dev)})
        table = part.by_distance.cpu()
        assert table.shape == (3, far + 1)
        for n in range(far + 1):
            assert torch.equal(table[:, n], rel[plain.distance_bucket(n, buckets, far)]), (buckets, far, n)
        assert plain.distance_bucket(far, buckets, far) == buckets - 1 == plain.distance_bucket(50 * far, buckets, far)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_of_the_output_then_add_then_norm_of_the_sum(out_dtype):
    """h += y / rms(y) * w (+ offset); x = h / rms(h) * w': in place, with only the offset, for chosen rows only."""
    from hyperion_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(4)
    for hidden in (40, 100, 1024, 3000):
        h = torch.randn(7, hidden, generator=g) * 3
        y = (torch.randn(7, hidden, generator=g) * 0.1).to(out_dtype)
        w_post, w_next, offset = 1 + 0.2 * torch.randn(hidden, generator=g), 1 + 0.2 * torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
        for use_y, use_offset in ((True, False), (True, True), (False, True)):
            want_h = h.double()
            if use_y:
                want_h = want_h + plain.unit_rms(y.double(), 1e-5) * w_post.double()
            if use_offset:
                want_h = want_h + offset.double()
            want_x = plain.unit_rms(want_h, 1e-6) * w_next.double()
            hd = h.to(dev).clone()
            x = ops.norm_add_norm(hd, y.to(dev) if use_y else None, w_post.to(dev) if use_y else None, 1e-5, offset.to(dev) if use_offset else None,
                                  w_next.to(dev), 1e-6, out_dtype)
            assert (hd.cpu().double() - want_h).abs().max() <= 2e-6 * want_h.abs().max()
            tolerance = 1e-5 if out_dtype == torch.float32 else 1e-2
            assert (x.cpu().double() - want_x).abs().max() <= tolerance * want_x.abs().max()
            rows = torch.tensor([5, 0, 3], dtype=torch.int32)
            hd = h.to(dev).clone()
            some = ops.norm_add_norm(hd, y.to(dev) if use_y else None, w_post.to(dev) if use_y else None, 1e-5, offset.to(dev) if use_offset else None,
                                     w_next.to(dev), 1e-6, out_dtype, rows.to(dev))
            assert torch.equal(hd.cpu(), h)  # the stream stays as it was
            assert torch.equal(some.cpu(), x.cpu()[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routing_sorting_and_summing_of_experts(dtype):
    """The router's choices and weights, every pair in a slot of its expert's run, the grouped product against one product per
    expert, and the sum of a token's rows, with more experts than tokens and with experts that no token chose.  In bfloat16 the
    sizes take all three kernels of the product: tensor-core tiles (many pairs, rows of whole 16 bytes), the streaming kernel
    (few pairs) and the plain one (other sizes)."""
    from hyperion_b200.ops import moe

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    for tokens, hidden, count, top, inner in ((37, 48, 5, 2, 20), (3, 24, 9, 3, 7), (300, 64, 4, 1, 130), (1, 16, 2, 2, 5), (300, 72, 4, 1, 136),
                                              (200, 128, 3, 2, 256), (5, 64, 8, 2, 40)):
        x = torch.randn(tokens, hidden, generator=g).to(dtype)
        router = torch.randn(count, hidden, generator=g)
        router[count - 1] = -5 * x.float().mean(dim=0) if tokens > 1 else router[count - 1]  # an expert that is rarely chosen
        chosen, weights = moe.route(x.to(dev), router.to(dev), top)
        logits = x.double() @ router.double().T
        want = torch.topk(logits, top, dim=-1)
        assert torch.equal(chosen.cpu().long(), want.indices)
        assert (weights.cpu().double() - torch.sigmoid(want.values)).abs().max() <= 1e-5
        where = moe.plan(chosen, weights, count)
        slot_of, slot_token = where.slot_of.cpu().view(tokens, top), where.slot_token.cpu()
        tile_expert = where.tile_expert.cpu()
        assert len(set(slot_of.flatten().tolist())) == tokens * top  # no slot twice
        for t in range(tokens):
            for k in range(top):
                slot = int(slot_of[t, k])
                assert slot_token[slot] == t and tile_expert[slot // moe.PAD] == chosen[t, k]
        assert int((slot_token >= 0).sum()) == tokens * top == int(where.tile_rows.sum())
        assert all(int(r) == int((slot_token[i * moe.PAD:(i + 1) * moe.PAD] >= 0).sum()) and bool((slot_token[i * moe.PAD:i * moe.PAD + int(r)] >= 0).all())
                   for i, r in enumerate(where.tile_rows.cpu()))  # the taken slots of a tile come first
        rows = moe.gather(x.to(dev), where)
        w = (torch.randn(count, inner, hidden, generator=g) / hidden ** 0.5).to(dtype)
        y = moe.grouped_linear(rows, w.to(dev), where)
        back = torch.randn(count, hidden, inner, generator=g).to(dtype) / inner ** 0.5
        z = moe.grouped_linear(y, back.to(dtype).to(dev), where)
        base = torch.randn(tokens, hidden, generator=g).to(dtype)
        total = moe.combine(z, where, base.to(dev), tokens).cpu().double()
        expect = base.double().clone()
        tolerance = 1e-5 if dtype == torch.float32 else 3e-2
        for t in range(tokens):
            for k in range(top):
                e = int(chosen[t, k])
                row = (x[t].double() * float(weights[t, k])).to(dtype).double()
                mid = (w[e].double() @ row).to(dtype).double()
                assert (y[int(slot_of[t, k])].cpu().double() - mid).abs().max() <= tolerance * max(1.0, mid.abs().max())
                expect[t] += (back[e].double() @ mid).to(dtype).double()
        assert (total - expect).abs().max() <= tolerance * expect.abs().max()


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
        assert_close(got, want, dtype, how, routed=True)
        assert rows_over(got, results["whole"], TOLERANCE[dtype]) <= 0.03, how  # the same arithmetic on both sides
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
    got_rows, want_rows = [], []
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
            got_rows.append(logits[row:row + n])
            want_rows.append(want[entry.request][at:at + n])
            row += n
            live[entry.request] = at + n
            slots_seen.setdefault(engine.cache.slot(entry.request), set()).add(entry.request)
            if at + n == len(requests[entry.request]):
                engine.finish(entry.request)
                del live[entry.request]
        step += 1
    engine.check()
    engine.cache.check()
    assert_close(np.concatenate(got_rows), np.concatenate(want_rows), dtype, routed=True)
    assert max(len(users) for users in slots_seen.values()) >= 2  # a slot served more than one request


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_edges_of_the_distance_buckets_and_far_away(folders, dtype):
    """One attention with 8 buckets up to distance 30 over pages of 8: a marker token stands at a chosen distance behind the
    last token and nowhere else, so its key scores high against the last query (the layer's key matrices are its query
    matrices) and the bias of its bucket decides how high.  Distances on both sides of every bucket's edge (0 | 1 | 2 | 3 | 4,
    6 | 7, 10 | 11, 18 | 19), at page borders (8, 16), where the last bucket has long begun (30, 31) and far away (150) are
    each run as a whole prompt and with the tail decoded token by token."""
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "attention", ALONE["attention"]["vocab"]
    edges = [n for n in range(1, 31) if plain.distance_bucket(n, 8, 30) != plain.distance_bucket(n - 1, 8, 30)]
    assert len(edges) == 7
    engine = engine_for(folders[name], dtype, page_size=8)
    for distance in sorted(({1, 8, 16, 30, 31, 150} | set(edges) | {n - 1 for n in edges}) - {0}):
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
    # the marked key and its bucket matter: the plain logits move by many float32 tolerances when the key is taken away or
    # stands one place further back, in the next bucket
    inside = ids_for(920, 200, vocab - 2)
    inside[-1], inside[-1 - 10] = vocab - 2, vocab - 1
    without = list(inside)
    without[-1 - 10] = 0
    outside = list(inside)
    outside[-1 - 10], outside[-1 - 11] = inside[-1 - 11], vocab - 1
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
    rows = []
    for at, token in enumerate(ids):  # position 0 alone, then every other one: a one-token prompt and 399 decoded tokens
        rows.append(engine.step([StepEntry("r", [token], [0])]).cpu().numpy()[0].copy())
    engine.finish("r")
    pair = engine.step([StepEntry("pair", ids[:2], [0, 1])]).cpu().numpy().copy()
    engine.finish("pair")
    engine.check()
    single = np.stack(rows)
    assert_close(single, want, dtype, routed=True)
    assert_close(single[:8], want[:8], dtype, "the first tokens")
    assert_close(pair, want[:2], dtype)
    whole = run_cut(engine, "whole", ids, [len(ids)])
    assert rows_over(single, whole, TOLERANCE[dtype]) <= 0.03


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention_wide", "attention_192"])
def test_keys_far_beyond_the_last_bucket_in_the_tensor_core_kernels(folders, name, dtype):
    """Heads of 128 (and of 192) and a bias that ends at distance 40: in a prompt of 450 tokens most key tiles lie wholly in the last
    bucket (the tcgen05 prompt kernel adds their bias as one shift of the tile), the tiles near the diagonal look every score's bias
    up; the tail is decoded token by token through the split-key kernel."""
    from hyperion_b200.engine.batch import StepEntry

    vocab = ALONE[name]["vocab"]
    ids = ids_for(77, 450, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype)
    whole = run_cut(engine, "w", ids, [len(ids)])
    assert_close(whole, want, dtype, "whole")
    got = [engine.step([StepEntry("d", ids[:300], list(range(300)))]).cpu().numpy().copy()]
    got.append(engine.step([StepEntry("d", ids[300:420], list(range(120)))]).cpu().numpy().copy())
    for at in range(420, 450):
        got.append(engine.step([StepEntry("d", [ids[at]], [0])]).cpu().numpy().copy())
    engine.finish("d")
    engine.check()
    assert_close(np.concatenate(got), want, dtype, "two portions and a decoded tail")
    # the last bucket's bias matters: without it the plain logits of the late rows are off by several tolerances
    config, weights = plain.read_model_folder(folders[name])
    weights["l0.mix.left.rel"][-1] = 0
    assert rows_over(plain.forward(config, weights, ids).numpy()[-50:], want[-50:], 2 * TOLERANCE["bfloat16"]) > 0.9


@pytest.mark.parametrize("name", ["retention", "selective"])
def test_long_rows_scanned_in_segments(folders, name):
    """In bfloat16 a row of 512 tokens or more has its scan (retention, selective) cut into segments that run side by side and are
    joined: a prompt of 700 tokens, then decoded tokens that go on from the joined state, then a long portion of one request
    beside single tokens of two others whose states must stay their own."""
    from hyperion_b200.engine.batch import StepEntry

    vocab = ALONE[name]["vocab"]
    a, b, c = ids_for(41, 720, vocab), ids_for(42, 40, vocab), ids_for(43, 1300, vocab)
    want = {"a": plain_logits(folders[name], a), "b": plain_logits(folders[name], b), "c": plain_logits(folders[name], c)}
    engine = engine_for(folders[name], "bfloat16", max_tokens=4096)
    got = engine.step([StepEntry("a", a[:700], list(range(700)))]).cpu().numpy().copy()
    assert engine.runner.last_context.host["scan_segments"] == 2
    assert_close(got, want["a"][:700], "bfloat16", "a prompt in two segments")
    for at in range(700, 720):
        row = engine.step([StepEntry("a", [a[at]], [0])]).cpu().numpy()[0]
        assert_close(row, want["a"][at], "bfloat16", ("decoded after the joined state", at))
    engine.finish("a")
    engine.step([StepEntry("b", b[:30], []), StepEntry("c", c[:100], [])])
    got = engine.step([StepEntry("b", [b[30]], [0]), StepEntry("c", c[100:1299], list(range(1199))), StepEntry("a", a[:1], [0])]).cpu().numpy().copy()
    assert engine.runner.last_context.host["scan_segments"] == 1 + 4 + 1
    assert_close(got[0], want["b"][30], "bfloat16", "a single token beside a long portion")
    assert_close(got[1:1200], want["c"][100:1299], "bfloat16", "a long portion that goes on from a state")
    assert_close(got[1200], want["a"][0], "bfloat16", "a first token beside a long portion")
    got = engine.step([StepEntry("b", [b[31]], [0]), StepEntry("c", [c[1299]], [0])]).cpu().numpy()
    assert_close(got[0], want["b"][31], "bfloat16")
    assert_close(got[1], want["c"][1299], "bfloat16", "decoded after four joined segments")
    engine.check()


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
