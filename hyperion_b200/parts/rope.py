"""Rotate-half rotary position encoding with a configurable base.

The table holds cos and sin of ``position * base**(-2i/d)`` for ``i < d/2``, computed in float64 and
kept in float32 (the reference computes the same angles in f64 and rounds the table to bfloat16:
helios/crates/helios-hal/src/reference.rs:71-87); the rotation is y[i] = x[i] c - x[i+d/2] s,
y[i+d/2] = x[i+d/2] c + x[i] s over the whole head (reference.rs:91-109).  Parameters: ``head_dim``,
``base``, ``max_positions``.  Tables are shared between parts with the same parameters.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import BuildContext, PositionEncoding, register_position
from .spec import PartSpec


def rotary_table(head_dim: int, base: float, max_positions: int) -> torch.Tensor:
    """[max_positions, head_dim/2, 2] float32: (cos, sin)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / head_dim)
    angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.stack([angle.cos(), angle.sin()], dim=-1).to(torch.float32).contiguous()


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.head_dim = int(spec.params["head_dim"])
        self.base = float(spec.params["base"])
        self.max_positions = int(spec.params.get("max_positions", build.max_positions))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        key = ("rotary_table", self.head_dim, self.base, self.max_positions, str(build.device))
        if key not in build.shared:
            build.shared[key] = rotary_table(self.head_dim, self.base, self.max_positions).to(build.device)
        self.table = build.shared[key]

    def kernel_modules(self):
        return [("elementwise", {})]

    def apply_(self, x, heads, head_dim, positions):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        ops.rope_(x, heads, head_dim, positions, self.table)

    def apply_and_store_(self, x, q_heads, kv_heads, head_dim, positions, cache, token_row):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        ops.rope_kv_store_(x, q_heads, kv_heads, head_dim, positions, self.table, cache.kv, cache.block_table, token_row)


register_position("rope", RotaryEncoding)


class InterleavedRotaryEncoding(PositionEncoding):
    """Rotary encoding of adjacent pairs: within the first ``dims`` dimensions of a head, dimension 2i is paired
    with 2i + 1 and the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a) with
    a = p * base**(-2i/dims) / factor; dimensions from ``dims`` on pass unchanged.  ``factor`` is a linear
    stretch of the positions (1 = none).  No table: the frequencies are computed once in float64 and kept in
    float32, the angle and its sine and cosine are float32 on the device, so there is no limit on positions.
    Parameters: ``dims``, ``base``, ``factor``."""

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.dims = int(spec.params["dims"])
        self.base = float(spec.params["base"])
        self.factor = float(spec.params.get("factor", 1.0))
        if self.dims % 2 or self.dims < 0:
            raise ValueError(f"rotary encoding of pairs needs an even number of dimensions, got {self.dims}")
        key = ("interleaved_frequencies", self.dims, self.base, self.factor, str(build.device))
        if key not in build.shared:
            i = torch.arange(self.dims // 2, dtype=torch.float64)
            freq = torch.tensor(self.base, dtype=torch.float64) ** (-2.0 * i / max(1, self.dims)) / self.factor
            build.shared[key] = freq.to(torch.float32).to(build.device)
        self.inv_freq = build.shared[key]

    def kernel_modules(self):
        return [("heads_prepare", {})]

    def apply_(self, x, heads, head_dim, positions):
        if head_dim < self.dims:
            raise ValueError(f"rotary encoding of {self.dims} dimensions, used with heads of {head_dim}")
        ops.heads_prepare_(x, heads, 0, head_dim, head_dim, positions, inv_freq=self.inv_freq, rot_dims=self.dims)


register_position("rope_interleaved", InterleavedRotaryEncoding)


class PartialHalfRotaryEncoding(InterleavedRotaryEncoding):
    """The same without a table for the other pairing: within the first ``dims`` dimensions of a head, dimension i turns
    together with dimension i + dims/2 by the angle p * base**(-2i/dims) / factor; the rest of the head passes unchanged.
    It works on float rows (recurrences keep their queries and keys in float).  Parameters: ``dims``, ``base``, ``factor``."""

    half = True

    def apply_(self, x, heads, head_dim, positions):
        if head_dim < self.dims:
            raise ValueError(f"rotary encoding of {self.dims} dimensions, used with heads of {head_dim}")
        if x.dtype != torch.float32:
            raise ValueError("this rotation works on float rows")
        width = heads * head_dim
        ops.heads_prepare_wide(x, 0, 0, 0, heads, 0, head_dim, head_dim, positions, q_out=x[:, :width], k_out=x[:, :width], inv_freq=self.inv_freq,
                               rot_dims=self.dims, rot_half=True)


register_position("rope_half_partial", PartialHalfRotaryEncoding)
