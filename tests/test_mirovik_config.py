"""Mirovik's configuration reader and its model as data, without a GPU: every size and constant comes from the document,
a missing or malformed key is refused by name, the document is written back as it was read, the repeated run of layers
becomes schedule entries with caches of their own, and the parts ask for the design's tensor names and for the right
kinds of cache."""
from __future__ import annotations

import copy

import pytest
import torch

from hyperion_b200.config import ConfigError, MirovikConfig
from hyperion_b200.models import DecoderModel, architecture_of, get_architecture
from hyperion_b200.parts import PagedTokens, RequestState
from hyperion_b200.weights.loader import WeightsError, check_tensors

DOCUMENT = {
    "architecture": "Mirovik", "vocab": 77, "width": 40, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 56, "state": 10, "dt_rank": 3, "conv": 2}, "mlp": {"kind": "dense", "ff": 60}},
        {"type": "parallel", "mixer": {"left": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "bias_max": 50, "buckets": 10},
                                       "right": {"heads": 3, "dim": 14, "vdim": 9, "decay": [0.5, 0.9, 1.0], "rot": {"dims": 8, "base": 777.0}},
                                       "left_scale": 0.6, "right_scale": -1.25},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 16}}},
        {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2, "bias_max": 64, "buckets": 32},
                                       "right": {"heads": 1, "dim": 16, "vdim": 16, "decay": [0.99]}, "left_scale": 1.0, "right_scale": 1.0}, "mlp": None},
        {"type": "mamba1", "mixer": {"inner": 20, "state": 3, "dt_rank": 1, "conv": 4}, "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 8}}},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}


def test_the_document_is_read_and_written_back():
    entry = architecture_of(DOCUMENT)
    assert entry.name == "Mirovik"
    config = entry.read_config(DOCUMENT)
    assert entry.write_config(config) == DOCUMENT
    a = config.layers[1].mixer
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim, a.left.scale, a.left.bias_max) == (6, 2, 12, 20, 0.3, 50)
    assert (a.right.heads, a.right.decay, a.right.rot_dims, a.right.rot_base, a.left_scale, a.right_scale) == (3, (0.5, 0.9, 1.0), 8, 777.0, 0.6, -1.25)
    assert config.layers[2].mixer.right.rot_dims == 0 and config.layers[2].mlp is None
    assert (config.layers[1].mlp.experts, config.layers[1].mlp.top, config.layers[1].mlp.ff, config.layers[1].mlp.shared_ff) == (5, 2, 24, 16)
    assert config.layers[3].mlp.shared_ff is None and config.layers[0].mlp.ff == 60
    assert config.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    without = copy.deepcopy(DOCUMENT)
    del without["loop"]
    assert MirovikConfig.from_dict(without).runs() == [(0, None), (1, None), (2, None), (3, None)]


@pytest.mark.parametrize("path, value, key", [
    (("vocab",), 0, "vocab"), (("width",), None, "width"), (("norm", "eps"), -1.0, "norm.eps"), (("embedding",), None, "embedding"),
    (("layers", 0, "type"), "lstm", "layers[0].type"), (("layers", 0, "mixer", "state"), 0, "layers[0].mixer.state"),
    (("layers", 0, "mixer", "dt_rank"), None, "layers[0].mixer.dt_rank"), (("layers", 1, "mixer", "left", "kv_heads"), 4, "layers[1].mixer.left.kv_heads"),
    (("layers", 1, "mixer", "right", "rot", "dims"), 7, "layers[1].mixer.right.rot.dims"), (("layers", 1, "mixer", "right", "rot", "dims"), 16, "layers[1].mixer.right.rot.dims"),
    (("layers", 1, "mixer", "right", "decay"), [0.5, 0.9], "layers[1].mixer.right.decay"), (("layers", 1, "mixer", "left_scale"), "big", "layers[1].mixer.left_scale"),
    (("layers", 1, "mlp", "kind"), "sparse", "layers[1].mlp.kind"), (("layers", 1, "mlp", "router", "top"), 6, "layers[1].mlp.router.top"),
    (("layers", 1, "mlp", "expert"), None, "layers[1].mlp.expert"), (("layers", 2, "mixer", "left", "bias_max"), 0, "layers[2].mixer.left.bias_max"),
    (("loop", "stop"), 5, "loop.stop"), (("loop", "start"), 3, "loop.stop"), (("loop", "times"), 0, "loop.times"),
])
def test_a_bad_value_is_refused_by_name(path, value, key):
    document = copy.deepcopy(DOCUMENT)
    at = document
    for step in path[:-1]:
        at = at[step]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as refused:
        MirovikConfig.from_dict(document)
    assert refused.value.key == key


def test_the_model_as_data_asks_for_the_designs_tensors_and_caches():
    entry = get_architecture("Mirovik")
    model = DecoderModel(entry.build_spec(entry.read_config(DOCUMENT)), torch.float32, torch.device("meta"))
    expected = model.expected_tensors()
    wanted = {name: tuple(spec.shape) for name, spec in expected.items()}
    assert wanted["embed"] == (77, 40) and "head" not in wanted and wanted["final.norm"] == (40,) and wanted["loop.step"] == (3, 40)
    assert wanted["l0.mix.in"] == (112, 40) and wanted["l0.mix.conv"] == (56, 2) and wanted["l0.mix.x"] == (3 + 20, 56) and wanted["l0.mix.dt"] == (56, 3)
    assert wanted["l0.mix.A_log"] == (56, 10) and wanted["l0.mix.D"] == (56,) and wanted["l0.mix.dt.b"] == (56,) and wanted["l0.mix.o"] == (40, 56)
    assert all(wanted[f"l0.{n}"] == (40,) for n in ("norm1", "norm1b", "norm2", "norm2b")) and wanted["l0.mlp.up"] == (60, 40) and "l0.mlp.gate" not in wanted
    assert wanted["l1.mix.left.q"] == (72, 40) and wanted["l1.mix.left.k"] == (24, 40) and wanted["l1.mix.left.v"] == (40, 40)
    assert wanted["l1.mix.left.q.norm"] == (72,) and wanted["l1.mix.left.k.norm"] == (24,) and wanted["l1.mix.left.rel"] == (10, 6)
    assert wanted["l1.mix.left.g"] == (120, 40) and wanted["l1.mix.left.o"] == (40, 120)
    assert wanted["l1.mix.right.q"] == (42, 40) and wanted["l1.mix.right.v"] == (27, 40) and wanted["l1.mix.right.g"] == (27, 40) and wanted["l1.mix.right.o"] == (40, 27)
    assert wanted["l1.mlp.router"] == (5, 40) and wanted["l1.mlp.e4.gate"] == (24, 40) and wanted["l1.mlp.e0.down"] == (40, 24) and wanted["l1.mlp.shared.up"] == (16, 40)
    assert "l2.norm2" not in wanted and "l3.mlp.shared.up" not in wanted and "l3.mlp.e1.up" in wanted
    # eight schedule entries: the two repeated layers own pages and a state in each of their three passes
    assert [(run.layer, run.offset) for run in model.spec.schedule] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    users = dict(model.cache_users())
    assert set(users) == {0, (1, 0), (1, 1), (2, 0), (2, 1), (3, 0), (3, 1), (4, 0), (4, 1), (5, 0), (5, 1), (6, 0), (6, 1), 7}
    assert users[(1, 0)] == users[(3, 0)] == PagedTokens((2,), (32,), 0)  # keys of 12 and values of 20 side by side
    assert users[(2, 0)] == PagedTokens((2, 1), (32,), 0)  # keys and values of one size: the layout every attention of the package uses
    assert users[(1, 1)] == RequestState((3 * 9 * 16,), torch.float32) and users[(2, 1)] == RequestState((16 * 16,), torch.float32)
    assert isinstance(users[0], RequestState) and users[0].shape[0] >= 56 * 12 + 1 * 56 and users[7].shape[0] >= 20 * 4 + 3 * 20


def test_the_distance_bias_takes_the_checkpoints_number_of_buckets():
    """The rows of the bias tensor are the checkpoint's business; every other shape is held to the configuration."""
    from hyperion_b200.weights.safetensors_io import TensorEntry

    entry = get_architecture("Mirovik")
    model = DecoderModel(entry.build_spec(entry.read_config(DOCUMENT)), torch.float32, torch.device("meta"))
    expected = model.expected_tensors()
    fields = TensorEntry.__dataclass_fields__ if hasattr(TensorEntry, "__dataclass_fields__") else None

    def found(changes):
        out = {}
        for name, spec in expected.items():
            shape = changes.get(name, tuple(spec.shape))
            out[name] = _entry(TensorEntry, fields, shape)
        return out

    check_tensors(found({"l1.mix.left.rel": (16, 6)}), expected)
    with pytest.raises(WeightsError):
        check_tensors(found({"l1.mix.left.rel": (16, 5)}), expected)
    with pytest.raises(WeightsError):
        check_tensors(found({"l1.mix.left.q": (70, 40)}), expected)
    tolerated = found({})
    tolerated["l2.norm2"] = _entry(TensorEntry, fields, (40,))
    check_tensors(tolerated, expected, model.spec.tolerated)


def _entry(cls, fields, shape):
    values = {"shape": tuple(shape), "dtype": torch.bfloat16}
    if fields is None:
        return type("Found", (), values)()
    filled = {}
    for name in fields:
        filled[name] = values.get(name, None)
    return cls(**filled)
