"""Mixers that run side by side on the same input, and two mixers made to be run that way.

``parallel_mixers`` holds several *branches*; all of them read the same rows x and the result is the sum of their results
times a scale each:  y = sum_b scale_b * branch_b(x).  The branches' input projections are one matrix product (their matrices
stacked, the result kept in float), every branch then works on its columns of that product and writes what its output
projection reads, times its scale, into its columns of one buffer, and one more product (the output matrices side by side)
gives the sum: two products for any number of branches.  A branch keeps what it needs between steps like any mixer; the
combination asks for all of it as a tuple.  Parameters: ``hidden_size``, ``branches``: a tuple of (PartSpec, scale).

A branch is a mixer that also offers: ``in_names`` (its input matrices' tensor names, in the order of its columns),
``in_width`` and ``core_width`` (columns it takes of the first product and gives to the second), ``out_name``, and
``core(proj, col0, step, cache, out, scale)``.  Used alone, a branch is an ordinary mixer.

``biased_attention``: causal grouped-query softmax attention without any rotation; all it knows about positions is a learned
bias per head and bucket of distance:  score(i, j) = (q_i . k_j) * scale + rel[bucket(i - j), head].  With B buckets and
D = ``bias_max``: bucket(n) = n for n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) * (B - B/2))): from distance
D on every key shares the last bucket, so the part keeps the bias as a table [heads, D + 1] by distance.  Queries and keys pass
an RMS norm over their *whole* projection (all heads at once, a weight per column); the heads' outputs are multiplied by
sigmoid(W_g x).  Keys of size ``head_dim`` and values of ``value_dim`` lie in pages; norms, scores, bias and softmax are float.
Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``bias_max``, ``buckets`` (rows of the
bias tensor when random weights are made; a checkpoint's own number of rows is taken as it comes), ``eps``.
Tensors: q, k, v, q.norm, k.norm, rel, g, o.

``retention``: a matrix-valued state per head that fades by a constant of the head and takes k v^T at every token; the output is the
state applied to the query as it is (nothing is exponentiated, nothing divided by a sum):
    S <- decay_h S + k v^T;  o = S^T q,
q and k rotated (dimension i with i + dims/2, the first ``dims`` dimensions of a head), k then times head_dim^(-1/2); each
head's o is divided by its root mean square and multiplied by silu(W_g x).  The state is one float record per request.
Parameters: ``hidden_size``, ``heads``, ``head_dim``, ``value_dim``, ``decay`` (one per head), ``position`` (a PartSpec or None), ``eps``.
Tensors: q, k, v, g, o.
"""
from __future__ import annotations

import math
from typing import Mapping

import torch

from .. import ops
from ..ops import attention as fast_attention
from ..ops import recurrent
from .attention import GroupedQueryAttention
from .base import MIXERS, POSITIONS, BuildContext, Mixer, PagedTokens, RequestState, WeightSpec, make, register_mixer
from .spec import PartSpec


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


def _round_up(value: int, step: int) -> int:
    return -(-value // step) * step


def distance_bucket(n: int, buckets: int, far: int) -> int:
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half))))


class Branch(Mixer):
    """A mixer that can run beside others on one input (see the module's text)."""

    in_names: tuple[str, ...]
    out_name: str
    in_width: int
    core_width: int
    hidden: int

    def core(self, proj: torch.Tensor, col0: int, step, cache, out: torch.Tensor, scale: float) -> None:
        """``proj`` [tokens, *] float: this branch's input projections start at column ``col0``.  Write what the output
        projection reads, times ``scale``, to ``out`` [tokens, core_width] (a view, activation type)."""
        raise NotImplementedError

    def load_core(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Everything but the input and output matrices."""

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        mats = [tensors[name] for name in self.in_names]
        dtype = _common_dtype(mats)
        self.w_in = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.w_o = tensors[self.out_name].contiguous()
        self.load_core(tensors)

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache:
            raise ValueError(f"{type(self).__name__} keeps something per request; the schedule gave it none")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        out = torch.empty((x.shape[0], self.core_width), dtype=self.dtype, device=x.device)
        self.core(proj, 0, step, cache, out, 1.0)
        return ops.linear(out, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


class BiasedAttention(Branch):
    in_names = ("q", "k", "v", "g")
    out_name = "o"

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim, self.value_dim = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale, self.bias_max, self.eps = float(p["scale"]), int(p["bias_max"]), float(p["eps"])
        self.buckets = int(p.get("buckets") or 32)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.kv_heads} key/value heads do not divide {self.heads} heads")
        if max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"heads of {self.head_dim} / {self.value_dim} are above the kernels' limit of 256")
        self.q_width, self.k_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_width, self.core_width = self.kv_heads * self.value_dim, self.heads * self.value_dim
        self.in_width = self.q_width + self.k_width + self.v_width + self.core_width
        # keys and values of one size that the TMA-fed kernels take, in bfloat16: the tensor-core kernels of the package's other
        # attentions read the pages (tcgen05 tiles for prompt portions, split keys for decoded tokens), with the bias as an argument
        self.window, self.softcap = 0, 0.0
        self.fast = self.dtype == torch.bfloat16 and self.value_dim == self.head_dim and self.head_dim % 64 == 0

    def weights(self) -> dict[str, WeightSpec]:
        h = self.hidden
        return {"q": WeightSpec((self.q_width, h)), "k": WeightSpec((self.k_width, h)), "v": WeightSpec((self.v_width, h)),
                "q.norm": WeightSpec((self.q_width,), init="one_plus_normal"), "k.norm": WeightSpec((self.k_width,), init="one_plus_normal"),
                "rel": WeightSpec((self.buckets, self.heads), any_extent=(0,)), "g": WeightSpec((self.core_width, h)),
                "o": WeightSpec((h, self.core_width))}

    def load_core(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.q_norm = tensors["q.norm"].to(torch.float32).contiguous()
        self.k_norm = tensors["k.norm"].to(torch.float32).contiguous()
        rel = tensors["rel"].to(torch.float32)
        buckets = rel.shape[0]
        if buckets < 2 or self.bias_max <= buckets // 2:
            raise ValueError(f"a distance bias of {buckets} buckets needs bias_max above {buckets // 2}, got {self.bias_max}")
        index = torch.tensor([distance_bucket(n, buckets, self.bias_max) for n in range(self.bias_max + 1)], dtype=torch.long, device=rel.device)
        self.by_distance = rel[index].t().contiguous()  # [heads, bias_max + 1]
        self.by_distance_log2 = (self.by_distance * math.log2(math.e)).contiguous() if self.fast else None  # the fast kernels' softmax is in base 2

    def cache_request(self):
        if self.value_dim == self.head_dim:
            return PagedTokens((2, self.kv_heads), (self.head_dim,), 0)
        return PagedTokens((self.kv_heads,), (self.head_dim + self.value_dim,), 0)

    def kernel_modules(self):
        modules = [("heads_prepare", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]
        if not self.fast:
            return modules + [("attention_generic", {})]
        modules += [("elementwise", {}), ("attention_tma", {"HB_HEAD_DIM": self.head_dim})]  # which is launched depends on the page size of the cache
        if self.head_dim in (64, 128):
            modules.append(("attention_tcgen05", {"HB_HEAD_DIM": self.head_dim}))
        return modules

    step_plans = GroupedQueryAttention.step_plans  # the rows of a step cut into tiles and single tokens, as for every attention of the package
    _attend_fast = GroupedQueryAttention._attend_fast
    _longest_short_row = staticmethod(GroupedQueryAttention._longest_short_row)

    def core(self, proj, col0, step, cache, out, scale):
        q = torch.empty((proj.shape[0], self.q_width), dtype=self.dtype, device=proj.device)
        k_off = col0 + self.q_width
        v_off = k_off + self.k_width
        ops.heads_prepare_wide(proj, col0, k_off, v_off, self.heads, self.kv_heads, self.head_dim, self.value_dim, step.positions, q_out=q,
                               q_norm=self.q_norm, k_norm=self.k_norm, norm_whole=True, eps=self.eps, cache=cache.kv, block_table=cache.block_table,
                               token_row=step.token_row, page_size=cache.page_size)
        if self.fast and fast_attention.takes_distance_bias(self.head_dim, cache.page_size):
            # the tensor-core kernels store rows in 16-byte pieces: columns of a wider buffer whose rows do not start on such a piece
            # are filled through a buffer of their own
            direct = out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
            target = out if direct else torch.empty((proj.shape[0], self.core_width), dtype=self.dtype, device=proj.device)
            self._attend_fast(q, step, cache, out=target, bias=self.by_distance_log2)
            if not direct:
                out.copy_(target)
            ops.sigmoid_gate_(out, proj, v_off + self.v_width, scale)
            return
        ops.attention_general(q, self.heads, self.kv_heads, self.head_dim, self.value_dim, cache.kv, cache.block_table, step.token_row, step.positions,
                              cache.page_size, self.scale, distance_bias=self.by_distance, gate=proj, gate_off=v_off + self.v_width, out_scale=scale, out=out)


class Retention(Branch):
    in_names = ("q", "k", "v", "g")
    out_name = "o"

    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.n, self.e, self.eps = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"]), float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        if self.n > 256:
            raise ValueError(f"a state of {self.n} per column is above the scan kernel's limit of 256")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(build.device)
        self.position = make(POSITIONS, p["position"], build) if p.get("position") is not None else None
        if self.position is not None and not (hasattr(self.position, "inv_freq") and getattr(self.position, "half", False)):
            raise ValueError("retention rotates dimension i with i + dims / 2: its position encoding must be 'rope_half_partial'")
        if self.position is not None and self.position.dims > self.n:
            raise ValueError(f"a rotation of {self.position.dims} dimensions in heads of {self.n}")
        self.qk_width, self.core_width = self.heads * self.n, self.heads * self.e
        self.in_width = 2 * self.qk_width + 2 * self.core_width
        self.n_padded = _round_up(self.n, 4)
        self.record = self.heads * self.e * self.n_padded

    def weights(self) -> dict[str, WeightSpec]:
        h = self.hidden
        return {"q": WeightSpec((self.qk_width, h)), "k": WeightSpec((self.qk_width, h)), "v": WeightSpec((self.core_width, h)),
                "g": WeightSpec((self.core_width, h)), "o": WeightSpec((h, self.core_width))}

    def cache_request(self):
        return RequestState((self.record,), torch.float32)

    def kernel_modules(self):
        return [("heads_prepare", {}), ("recurrent", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def step_plans(self):
        return recurrent.segment_planner(self.dtype)

    def core(self, proj, col0, step, cache, out, scale):
        k_off, v_off = col0 + self.qk_width, col0 + 2 * self.qk_width
        ops.heads_prepare_wide(proj, col0, k_off, v_off, self.heads, self.heads, self.n, self.e, step.positions, q_out=proj[:, col0:k_off],
                               k_out=proj[:, k_off:v_off], inv_freq=self.position.inv_freq if self.position is not None else None,
                               rot_dims=self.position.dims if self.position is not None else 0, rot_half=True, k_scale=self.n ** -0.5)
        # Segments pay while one pass leaves the GPU mostly idle: a row's walk is a chain of dependent steps (0.23 us a token on a
        # B200) that few blocks share, and cutting it doubles the arithmetic.  Measured at heads of 128 x 128: 64 blocks 482 -> 290 us for
        # 2,048 tokens, 128 blocks 487 -> 509 us.
        blocks = self.heads * -(-self.e // 32)
        segments = step.host.get("scan_segments", 0) if self.dtype == torch.bfloat16 and blocks <= 100 else 0
        if segments:
            o = recurrent.retention_in_segments(proj, k_off, col0, v_off, self.decay, cache.state, cache.slots, step.extra["scan_seg_start"],
                                                step.extra["scan_seg_row"], segments, self.heads, self.n, self.n_padded, self.e)
        else:
            o = recurrent.state_scan(recurrent.MODE_RETENTION, proj, k_off, col0, v_off, proj, 0, 0, self.decay, self.decay, None, cache.state, 0, cache.slots,
                                     step.row_start, step.n_rows, self.heads, self.heads, self.n, self.n_padded, self.e)
        recurrent.gated_group_norm(o, proj, v_off + self.core_width, None, self.e, False, self.eps, self.dtype, scale=scale, out=out)


class ParallelMixers(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.branches: list[Branch] = []
        self.scales: list[float] = []
        self.prefixes: list[str] = []
        for branch_spec, scale in spec.params["branches"]:
            branch = make(MIXERS, branch_spec, build)
            if not isinstance(branch, Branch):
                raise ValueError(f"a mixer of kind {branch_spec.kind!r} cannot run beside others (it is no Branch)")
            if branch.hidden != self.hidden:
                raise ValueError("branches read and write rows of the combination's width")
            self.branches.append(branch)
            self.scales.append(float(scale))
            self.prefixes.append(branch_spec.prefix)  # relative to the combination's own prefix
        if not self.branches:
            raise ValueError("parallel mixers need at least one branch")
        self.core_width = sum(b.core_width for b in self.branches)

    def weights(self) -> dict[str, WeightSpec]:
        return {prefix + name: wanted for prefix, branch in zip(self.prefixes, self.branches) for name, wanted in branch.weights().items()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        ins, outs = [], []
        for prefix, branch in zip(self.prefixes, self.branches):
            own = {name: tensors[prefix + name] for name in branch.weights()}
            branch.load_core(own)
            ins += [own[name] for name in branch.in_names]
            outs.append(own[branch.out_name])
        dtype = _common_dtype(ins + outs)
        self.w_in = torch.cat([m.to(dtype) for m in ins], dim=0).contiguous()
        self.w_o = torch.cat([m.to(dtype) for m in outs], dim=1).contiguous()

    def cache_request(self):
        return tuple(branch.cache_request() for branch in self.branches)

    def kernel_modules(self):
        return [module for branch in self.branches for module in branch.kernel_modules()]

    def step_plans(self):
        plans = {}
        for branch in self.branches:
            plans.update(getattr(branch, "step_plans", lambda: {})())
        return plans

    def forward(self, x, step, cache, own_cache):
        if cache is None or not own_cache or len(cache) != len(self.branches):
            raise ValueError("parallel mixers keep what their branches keep; the schedule gave them something else")
        proj = ops.linear(x, self.w_in, None, torch.float32)
        out = torch.empty((x.shape[0], self.core_width), dtype=self.dtype, device=x.device)
        col = at = 0
        for branch, scale, view in zip(self.branches, self.scales, cache):
            branch.core(proj, col, step, view, out[:, at : at + branch.core_width], scale)
            col += branch.in_width
            at += branch.core_width
        return ops.linear(out, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_mixer("biased_attention", BiasedAttention)
register_mixer("retention", Retention)
register_mixer("parallel_mixers", ParallelMixers)
