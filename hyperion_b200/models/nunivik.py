"""Nunivik expressed as parts: a decoder whose layers differ in kind.

Every layer is the output-norm arrangement (x <- x + norm(mixer(x)); x <- x + norm(ff(x)), the sublayers reading the
stream itself) of one of three mixers: windowed attention with query/key norm, rotation of adjacent pairs, capped
scores and value mixing across layers (``capped_attention``); the gated delta rule (``delta_rule``); the state-space
mixer (``mamba2``), with a dense SiLU-gated feed-forward or none.  The embedding is scaled, the head is a matrix of its
own.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``,
``head``.  The design states no limit on positions; the engine's own limit of 2^30 stands in.
"""
from __future__ import annotations

from ..config.nunivik import ARCHITECTURE, NunivikConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from .registry import Architecture, register_architecture

NO_POSITION_LIMIT = 1 << 30


def build_spec(config: NunivikConfig) -> ModelSpec:
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        m = layer.mixer
        if layer.type == "attention":
            position = None
            if m.rot_dims:
                position = PartSpec("rope_interleaved", "", {"dims": m.rot_dims, "base": m.rot_base, "factor": m.rot_factor})
            mixer = PartSpec("capped_attention", prefix + "mix.", {
                "hidden_size": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
                "softcap": m.softcap, "window": m.window, "qk_norm": True, "eps": config.eps, "position": position,
                "v_mix": "values" if m.v_mix else None,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "v_mix": "vmix"}})
        elif layer.type == "delta":
            mixer = PartSpec("delta_rule", prefix + "mix.", {"hidden_size": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim,
                                                             "value_dim": m.vdim, "conv": m.conv, "eps": config.eps})
        else:
            mixer = PartSpec("mamba2", prefix + "mix.", {"hidden_size": config.width, "heads": m.heads, "value_dim": m.vdim, "state": m.state,
                                                         "groups": m.groups, "norm_groups": m.norm_groups, "conv": m.conv, "eps": config.eps})
        norms = {"mixer_out": PartSpec("rmsnorm", prefix, {"hidden_size": config.width, "eps": config.eps, "weight_name": "norm1"})}
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec("swiglu", prefix + "mlp.", {"hidden_size": config.width, "intermediate_size": layer.ff,
                                                                "names": {"gate": "gate", "up": "up", "down": "down"}})
            norms["feed_forward_out"] = PartSpec("rmsnorm", prefix, {"hidden_size": config.width, "eps": config.eps, "weight_name": "norm2"})
        layers.append(LayerSpec(arrangement="output_norm", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": config.vocab, "hidden_size": config.width}
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", "", {**sizes, "scale": config.embedding_scale, "weight_name": "embed"}),
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", "final.", {"hidden_size": config.width, "eps": config.eps, "weight_name": "norm"}),
        head=PartSpec("linear_head", "", {**sizes, "tied": False, "weight_name": "head"}),
    )


register_architecture(Architecture(ARCHITECTURE, NunivikConfig.from_dict, build_spec, NunivikConfig.to_dict))
