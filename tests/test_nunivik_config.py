"""Nunivik's configuration reader and its model as data, without a GPU: every size and constant comes from the document,
a missing or malformed key is refused by name, the document is written back as it was read, and the parts ask for the
design's tensor names and for the right kind of cache."""
from __future__ import annotations

import copy

import pytest
import torch

from hyperion_b200.config import ConfigError, NunivikConfig
from hyperion_b200.models import DecoderModel, architecture_of, get_architecture
from hyperion_b200.parts import PagedTokens, RequestState

DOCUMENT = {
    "architecture": "Nunivik", "vocab": 77, "width": 40, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 10, "groups": 2, "norm_groups": 3, "conv": 2}, "mlp": {"kind": "dense", "ff": 56}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "softcap": 9.0, "mask": {"size": 5},
                                        "rot": {"dims": 8, "base": 777.0, "scaling": {"factor": 1.5}}, "v_mix": True}, "mlp": None},
        {"type": "delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 14, "vdim": 9, "conv": 6}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 10, "scale": 0.25, "v_mix": True}, "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2, "v_mix": False}, "mlp": None},
    ],
}


def test_the_document_is_read_and_written_back():
    entry = architecture_of(DOCUMENT)
    assert entry.name == "Nunivik"
    config = entry.read_config(DOCUMENT)
    assert entry.write_config(config) == DOCUMENT
    a = config.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.rot_dims, a.rot_base, a.rot_factor, a.softcap) == (6, 2, 12, 20, 5, 8, 777.0, 1.5, 9.0)
    b = config.layers[3].mixer
    assert (b.window, b.rot_dims, b.softcap, b.v_mix) == (0, 0, 0.0, True)
    assert config.layers[0].ff == 56 and config.layers[1].ff is None


@pytest.mark.parametrize("path, value, key", [
    (("vocab",), 0, "vocab"), (("width",), None, "width"), (("norm", "eps"), -1.0, "norm.eps"), (("embedding",), None, "embedding"),
    (("layers", 0, "type"), "lstm", "layers[0].type"), (("layers", 0, "mixer", "groups"), 3, "layers[0].mixer.groups"),
    (("layers", 0, "mixer", "norm_groups"), 5, "layers[0].mixer.norm_groups"), (("layers", 1, "mixer", "kv_heads"), 4, "layers[1].mixer.kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "layers[1].mixer.rot.dims"), (("layers", 1, "mixer", "rot", "dims"), 14, "layers[1].mixer.rot.dims"),
    (("layers", 2, "mixer", "conv"), 0, "layers[2].mixer.conv"), (("layers", 3, "mlp", "kind"), "experts", "layers[3].mlp.kind"),
    (("layers", 3, "mixer", "vdim"), 11, "layers[3].mixer.v_mix"), (("layers", 1, "mixer", "mask", "size"), 0, "layers[1].mixer.mask.size"),
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
        NunivikConfig.from_dict(document)
    assert refused.value.key == key


def test_the_model_as_data_asks_for_the_designs_tensors_and_caches():
    entry = get_architecture("Nunivik")
    model = DecoderModel(entry.build_spec(entry.read_config(DOCUMENT)), torch.float32, torch.device("meta"))
    wanted = {name: tuple(spec.shape) for name, spec in model.expected_tensors().items()}
    assert wanted["embed"] == (77, 40) and wanted["head"] == (77, 40) and wanted["final.norm"] == (40,)
    assert wanted["l0.mix.in"] == (2 * 24 + 2 * 2 * 10 + 4, 40) and wanted["l0.mix.conv"] == (24 + 40, 2) and wanted["l0.mix.conv.b"] == (64,)
    assert wanted["l0.mix.norm"] == (24,) and wanted["l0.mix.D"] == (4,) and wanted["l0.norm2"] == (40,) and wanted["l0.mlp.down"] == (40, 56)
    assert wanted["l1.mix.q"] == (72, 40) and wanted["l1.mix.k"] == (24, 40) and wanted["l1.mix.v"] == (40, 40) and wanted["l1.mix.o"] == (40, 120)
    assert wanted["l1.mix.q.norm"] == (12,) and wanted["l1.mix.vmix"] == () and "l1.norm2" not in wanted
    assert wanted["l2.mix.q"] == (14, 40) and wanted["l2.mix.v"] == (27, 40) and wanted["l2.mix.v.conv"] == (27, 6) and wanted["l2.mix.b"] == (3, 40)
    assert wanted["l2.mix.norm"] == (9,) and wanted["l2.mix.o"] == (40, 27) and "l4.mix.vmix" not in wanted
    users = dict(model.cache_users())
    assert users[1] == PagedTokens((2,), (32,), 5) and users[3] == PagedTokens((4,), (26,), 0)
    assert users[4] == PagedTokens((2, 1), (32,), 0)  # keys and values of one size: the layout every attention of the package uses
    assert isinstance(users[0], RequestState) and isinstance(users[2], RequestState)
    # the delta rule's record: heads * vdim columns of dim (rounded up to 4) entries, then conv - 1 inputs of every convolved channel
    assert users[2].shape == (3 * 9 * 16 + 5 * (14 + 14 + 27) + 1,) or users[2].shape[0] % 4 == 0
    assert users[2].shape[0] >= 3 * 9 * 16 + 5 * 55 and users[0].shape[0] >= 4 * 6 * 12 + 1 * 64
