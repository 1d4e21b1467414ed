"""Grouped-query attention with the options newer decoders add to it: query and key norm, rotation of a part
of each head, a smooth cap on the scores, a sliding window, values of another size than keys, and value
mixing across layers.

Per step: one fused projection to [q | k | v]; one kernel (``csrc/heads_prepare.cu``) that norms query and key
heads (RMS norm over the head, one weight for all heads, before the rotation), rotates them, mixes the values
and writes keys and values to their pages; attention of every token over its request's pages
(``csrc/attention_generic.cu``: scores (q . k) * scale, then cap * tanh(score / cap), softmax over the keys
at positions p - window < j <= p, all in float); the output projection.  Query head h reads key/value head
h // (heads / kv_heads).

Value mixing: the layers of a model that name the same ``v_mix`` key share the values of the first of them:
in every later one v <- (1 - lambda) v + lambda v_first, with v_first the first layer's values of the same
token (before any mixing) and lambda that layer's scalar tensor; the mixed v is what is cached.  The first
layer's own scalar exists in the checkpoint and is not used.

Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim`` (``head_dim`` unless stated),
``scale``, ``softcap`` (0 = none), ``window`` (0 = all keys), ``qk_norm`` (bool), ``eps``, ``position`` (a PartSpec
or None), ``v_mix`` (a key, or None), ``names`` (tensor names after the prefix: q, k, v, o, q_norm, k_norm, v_mix).
Keys and values of one size lie in pages of [2, kv_heads, page, d] like every other attention's, and in bfloat16 with
head sizes the tensor-core kernels take they are read by those kernels (``GroupedQueryAttention``'s own: tcgen05 tiles
for prompt portions, the TMA-fed split-key kernel for decoded tokens), which take the cap and the window as
arguments; of two sizes they lie in pages of [kv_heads, page, d + e] and are read by the general kernel, as is
everything in float32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import attention as fast_attention
from .attention import GroupedQueryAttention
from .base import POSITIONS, BuildContext, Mixer, PagedKV, PagedTokens, WeightSpec, make, register_mixer
from .spec import PartSpec

DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_norm": "q_norm.weight",
                 "k_norm": "k_norm.weight", "v_mix": "v_mix"}


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class CappedAttention(GroupedQueryAttention):
    """Shares the planning and the launches of the tensor-core path with its base; everything else is its own."""

    def __init__(self, spec: PartSpec, build: BuildContext):
        Mixer.__init__(self, spec, build)
        p = spec.params
        self.bias, self.shares_kv = False, False
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = int(p.get("window") or 0)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("eps", 0.0))
        self.v_mix = p.get("v_mix")
        self.names = {**DEFAULT_NAMES, **dict(p.get("names") or {})}
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.kv_heads} key/value heads do not divide {self.heads} heads")
        if max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"heads of {self.head_dim} / {self.value_dim} are above the kernels' limit of 256")
        self.position = make(POSITIONS, p["position"], build) if p.get("position") is not None else None
        if self.position is not None and not hasattr(self.position, "inv_freq"):
            raise ValueError("this attention rotates adjacent pairs: its position encoding must offer frequencies ('rope_interleaved')")
        self.q_width = self.heads * self.head_dim
        self.k_width = self.kv_heads * self.head_dim
        self.v_width = self.kv_heads * self.value_dim
        self.fast = self.dtype == torch.bfloat16 and self.value_dim == self.head_dim and fast_attention.supported(self.head_dim)

    def weights(self) -> dict[str, WeightSpec]:
        n = self.names
        wanted = {n["q"]: WeightSpec((self.q_width, self.hidden)), n["k"]: WeightSpec((self.k_width, self.hidden)),
                  n["v"]: WeightSpec((self.v_width, self.hidden)), n["o"]: WeightSpec((self.hidden, self.heads * self.value_dim))}
        if self.qk_norm:
            wanted[n["q_norm"]] = WeightSpec((self.head_dim,), init="one_plus_normal")
            wanted[n["k_norm"]] = WeightSpec((self.head_dim,), init="one_plus_normal")
        if self.v_mix is not None:
            wanted[n["v_mix"]] = WeightSpec(())
        return wanted

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        mats = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        dtype = _common_dtype(mats)
        self.w_qkv = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.q_norm = tensors[n["q_norm"]].to(torch.float32).contiguous() if self.qk_norm else None
        self.k_norm = tensors[n["k_norm"]].to(torch.float32).contiguous() if self.qk_norm else None
        self.mix = tensors[n["v_mix"]].to(torch.float32).reshape(1).contiguous() if self.v_mix is not None else None

    def cache_request(self):
        if self.value_dim == self.head_dim:
            return PagedKV(self.kv_heads, self.head_dim, self.window)
        return PagedTokens((self.kv_heads,), (self.head_dim + self.value_dim,), self.window)

    def kernel_modules(self):
        modules = [("heads_prepare", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]
        if not self.fast:
            return modules + [("attention_generic", {})]
        modules.append(("attention_bf16", {"HB_HEAD_DIM": self.head_dim}))  # which is launched depends on the page size of the cache
        if self.head_dim % 64 == 0:
            modules.append(("attention_tma", {"HB_HEAD_DIM": self.head_dim}))
        if self.head_dim in (64, 128):
            modules.append(("attention_tcgen05", {"HB_HEAD_DIM": self.head_dim}))
        return modules

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError("this attention writes a paged cache of its own; the schedule gave it none")
        qkv = ops.linear(x, self.w_qkv, None, self.dtype)
        v_first = None
        if self.v_mix is not None:
            key = ("v_mix", self.v_mix)
            v_first = step.scratch.get(key)
            if v_first is None:  # the first layer of the key: its values, as projected, stay where later layers find them
                step.scratch[key] = qkv[:, self.q_width + self.k_width:]
            elif v_first.shape[1] != self.v_width:
                raise ValueError(f"layers that mix values under the key {self.v_mix!r} must have values of one width")
        ops.heads_prepare_(qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim, step.positions, q_norm=self.q_norm, k_norm=self.k_norm,
                           eps=self.eps, inv_freq=self.position.inv_freq if self.position is not None else None,
                           rot_dims=self.position.dims if self.position is not None else 0, v_first=v_first,
                           mix=self.mix if v_first is not None else None, cache=cache.kv, block_table=cache.block_table,
                           token_row=step.token_row, page_size=cache.page_size)
        if self.fast:
            attn = self._attend_fast(qkv, step, cache)
        else:
            attn = ops.attention_general(qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim, cache.kv, cache.block_table, step.token_row,
                                         step.positions, cache.page_size, self.scale, self.softcap, self.window)
        return ops.linear(attn, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("capped_attention", CappedAttention)
