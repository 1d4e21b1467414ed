"""Mirovik expressed as parts: a decoder whose layers are normalised on both sides of every sublayer, with a run of
layers that is passed several times.

Every layer is the sandwich arrangement (x <- x + norm_b(mixer(norm_a(x))); x <- x + norm_d(ff(norm_c(x))), the norms' stored
weights kept as offsets from one) of one of two mixers: attention with a learned distance bias beside retention, summed with a scale
each (``parallel_mixers`` of ``biased_attention`` and ``retention``), or the selective scan (``mamba1``); with a feed-forward
without a gate (tanh-form GELU), one of routed experts plus a shared one, or none.  The layers ``loop.start .. loop.stop - 1``
run ``loop.times`` times in a row with the same weights; every pass is a schedule entry of its own per layer, so it has its own
pages and state, and the first entry of pass t adds row t of the tensor ``loop.step`` to the stream.  The embedding is scaled and
the head is the embedding table itself.  Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.  The design states no limit on positions; the engine's own limit of 2^30 stands in.
"""
from __future__ import annotations

from ..config.mirovik import ARCHITECTURE, DenseFF, MirovikConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from .registry import Architecture, register_architecture

NO_POSITION_LIMIT = 1 << 30


def build_spec(config: MirovikConfig) -> ModelSpec:
    width, eps = config.width, config.eps
    layers, tolerated = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        m = layer.mixer
        if layer.type == "parallel":
            position = None
            if m.right.rot_dims:
                position = PartSpec("rope_half_partial", "", {"dims": m.right.rot_dims, "base": m.right.rot_base})
            left = PartSpec("biased_attention", "left.", {"hidden_size": width, "heads": m.left.heads, "kv_heads": m.left.kv_heads, "head_dim": m.left.dim,
                                                          "value_dim": m.left.vdim, "scale": m.left.scale, "bias_max": m.left.bias_max,
                                                          "buckets": m.left.buckets, "eps": eps})
            right = PartSpec("retention", "right.", {"hidden_size": width, "heads": m.right.heads, "head_dim": m.right.dim, "value_dim": m.right.vdim,
                                                     "decay": tuple(m.right.decay), "position": position, "eps": eps})
            mixer = PartSpec("parallel_mixers", prefix + "mix.", {"hidden_size": width, "branches": ((left, m.left_scale), (right, m.right_scale))})
        else:
            mixer = PartSpec("mamba1", prefix + "mix.", {"hidden_size": width, "inner": m.inner, "state": m.state, "dt_rank": m.dt_rank, "conv": m.conv})

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", prefix, {"hidden_size": width, "eps": eps, "weight_name": name, "one_plus": True})

        norms = {"input": norm("norm1"), "mixer_out": norm("norm1b")}
        feed_forward = None
        if layer.mlp is None:  # a checkpoint may carry the feed-forward's norms all the same; nothing reads them
            tolerated += [prefix + "norm2", prefix + "norm2b"]
        else:
            norms.update({"post_mixer": norm("norm2"), "feed_forward_out": norm("norm2b")})
            if isinstance(layer.mlp, DenseFF):
                feed_forward = PartSpec("activated_mlp", prefix + "mlp.", {"hidden_size": width, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh",
                                                                           "names": {"up": "up", "down": "down"}})
            else:
                feed_forward = PartSpec("routed_experts", prefix + "mlp.", {"hidden_size": width, "experts": layer.mlp.experts, "top": layer.mlp.top,
                                                                            "expert_size": layer.mlp.ff, "shared_size": layer.mlp.shared_ff,
                                                                            "weighting": "sigmoid", "weight_on": "input"})
        layers.append(LayerSpec(arrangement="sandwich_norm", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    offsets = None
    if config.loop is not None:
        offsets = PartSpec("offset_table", "", {"count": config.loop.times, "hidden_size": width, "weight_name": "loop.step"})
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", "", {**sizes, "scale": config.embedding_scale, "weight_name": "embed"}),
        layers=tuple(layers),
        schedule=tuple(Run(layer, offset=opens) for layer, opens in config.runs()),
        final_norm=PartSpec("rmsnorm", "final.", {"hidden_size": width, "eps": eps, "weight_name": "norm", "one_plus": True}),
        head=PartSpec("linear_head", "", {**sizes, "tied": True}),
        offsets=offsets,
        tolerated=tuple(tolerated),
    )


register_architecture(Architecture(ARCHITECTURE, MirovikConfig.from_dict, build_spec, MirovikConfig.to_dict))
