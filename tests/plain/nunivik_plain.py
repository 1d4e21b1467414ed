"""A plain, slow implementation of the Nunivik decoder: whole sequences, no cache, no batching, one
function per mechanism, torch on the CPU in float64 (or the dtype asked for).

It shares no code with the package: it reads the model folder with its own safetensors reader and
walks every recurrence token by token.  Notation: T tokens, W the model width, H heads, G key/value
(or q/k) heads, d the query/key size of a head, e the value size of a head, N the state size of a
state-space head.  Weights are stored [out, in].

A layer adds the *normalised output* of each sublayer to the stream, and each sublayer reads the
stream itself:  x <- x + rms(mixer(x)) * w1;  x <- x + rms(ff(x)) * w2  (the second only when the
layer has a feed-forward).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    blob = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + length])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        begin, end = meta["data_offsets"]
        raw = bytearray(blob[8 + length + begin : 8 + length + end])
        out[name] = torch.frombuffer(raw, dtype=DTYPES[meta["dtype"]]).reshape(meta["shape"]).clone() if raw else torch.zeros(meta["shape"], dtype=DTYPES[meta["dtype"]])
    return out


def read_model_folder(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ------------------------------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* weight) over the last dimension."""
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y * weight if weight is not None else y


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y[t, c] = sum_j weight[c, taps-1-j] * x[t-j, c] (+ bias[c]), x before the start being zero.
    x [T, C], weight [C, taps]: the last column multiplies the current token."""
    tokens, channels = x.shape
    taps = weight.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        if j < tokens:
            y[j:] += weight[:, taps - 1 - j] * x[: tokens - j]
    return y + bias if bias is not None else y


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float) -> torch.Tensor:
    """x [T, heads, d]: the pairs (2i, 2i+1), i < dims/2, turn by the angle p * base^(-2i/dims) / factor;
    dimensions from ``dims`` on pass unchanged."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)) / float(factor)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = angle.cos().to(x.dtype)[:, None, :], angle.sin().to(x.dtype)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------ the mixers
def attention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, shared: dict) -> torch.Tensor:
    """Windowed grouped-query attention with query/key norm, partial interleaved rotation, capped
    scores and value mixing.  ``shared`` carries the first value-mixing layer's values."""
    tokens = h.shape[0]
    heads, groups, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t()).view(tokens, heads, d)
    k = (h @ w[p + "k"].t()).view(tokens, groups, d)
    v = (h @ w[p + "v"].t()).view(tokens, groups, e)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    positions = torch.arange(tokens)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_interleaved(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_interleaved(k, positions, rot["dims"], rot["base"], factor)
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = w[p + "vmix"]
            v = (1 - lam) * v + lam * shared["v_first"]
    rep = heads // groups
    out = torch.zeros(tokens, heads, e, dtype=h.dtype)
    window = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    for head in range(heads):
        g = head // rep
        s = (q[:, head] @ k[:, g].t()) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        i, j = positions[:, None], positions[None, :]
        visible = (j <= i) if not window else ((i - j >= 0) & (i - j < window))
        s = s.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(tokens, heads * e) @ w[p + "o"].t()


def delta_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Gated delta rule, token by token.  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    tokens = h.shape[0]
    heads, groups, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].t(), w[p + "q.conv"])).view(tokens, groups, d)
    k = silu(causal_conv(h @ w[p + "k"].t(), w[p + "k.conv"])).view(tokens, groups, d)
    v = silu(causal_conv(h @ w[p + "v"].t(), w[p + "v.conv"])).view(tokens, heads, e)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].t())
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].t() + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].t()).view(tokens, heads, e)
    rep = heads // groups
    out = torch.zeros(tokens, heads, e, dtype=h.dtype)
    for head in range(heads):
        g = head // rep
        state = torch.zeros(d, e, dtype=h.dtype)
        for t in range(tokens):
            state = decay[t, head] * state
            u = beta[t, head] * (v[t, head] - state.t() @ k[t, g])
            state = state + torch.outer(k[t, g], u)
            out[t, head] = state.t() @ q[t, g]
    out = rms_norm(out, w[p + "norm"], eps) * gate
    return out.reshape(tokens, heads * e) @ w[p + "o"].t()


def mamba2_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """State-space mixer: S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T;  y_t = S_t^T C_t + D x_t."""
    tokens = h.shape[0]
    heads, e, n, groups, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = heads * e
    z, xbc, dt = torch.split(h @ w[p + "in"].t(), [inner, inner + 2 * groups * n, heads], dim=-1)
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(tokens, heads, e)
    b = xbc[:, inner : inner + groups * n].view(tokens, groups, n)
    c = xbc[:, inner + groups * n :].view(tokens, groups, n)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    rep = heads // groups
    y = torch.zeros(tokens, heads, e, dtype=h.dtype)
    for head in range(heads):
        g = head // rep
        state = torch.zeros(n, e, dtype=h.dtype)
        for t in range(tokens):
            state = decay[t, head] * state + dt[t, head] * torch.outer(b[t, g], x[t, head])
            y[t, head] = state.t() @ c[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(tokens, inner) * silu(z)
    y = rms_norm(y.view(tokens, parts, inner // parts), None, eps).reshape(tokens, inner) * w[p + "norm"]
    return y @ w[p + "o"].t()


def feed_forward(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


# ------------------------------------------------------------------------------------------ the model
def forward(config: dict, weights: dict, ids, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(ids).long()] * float(config["embedding"]["scale"])
    shared: dict = {}
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            a = attention_mixer(x, w, p + "mix.", m, eps, shared)
        elif kind == "delta":
            a = delta_mixer(x, w, p + "mix.", m, eps)
        elif kind == "mamba2":
            a = mamba2_mixer(x, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + rms_norm(a, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].t()
