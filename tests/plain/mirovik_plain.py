"""A plain, slow implementation of the Mirovik decoder: whole sequences, no cache, no batching, one
function per mechanism, torch on the CPU in float64 (or the dtype asked for).

It shares no code with the package: it reads the model folder with its own safetensors reader and
walks every recurrence token by token.  Notation: T tokens, W the model width, H heads, G key/value
heads, d the query/key size of a head, e the value size of a head, N the state size of a channel.
Weights are stored [out, in].

A layer normalises what each sublayer reads and what it returns:
    x <- x + norm1b(mixer(norm1(x)));  x <- x + norm2b(ff(norm2(x)))
with norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  A run of layers may be passed several times with
the same weights; a vector of its own is added to the stream before every pass.
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
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms: the tensor holds the weight's offset from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, c] = bias[c] + sum_j weight[c, taps-1-j] * x[t-j, c], x before the start being zero."""
    tokens = x.shape[0]
    taps = weight.shape[1]
    y = torch.zeros_like(x)
    for j in range(min(taps, tokens)):
        y[j:] += weight[:, taps - 1 - j] * x[: tokens - j]
    return y + bias


def distance_bucket(n: int, buckets: int, far: int) -> int:
    """Distances below half the number of buckets have a bucket each; beyond, buckets widen
    logarithmically up to the distance ``far``, from which on everything lies in the last bucket."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half))))


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: dimension i turns together with dimension i + dims/2 (i < dims/2) by the angle
    p * base^(-2i/dims); dimensions from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = angle.cos().to(x.dtype)[:, None, :], angle.sin().to(x.dtype)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------ mixers
def selective_scan_mixer(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """The state-space mixer with one decay per channel and state entry."""
    inner, n, rank = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"]))
    dbc = x @ w[p + "x"].T
    dt = softplus(dbc[:, :rank] @ w[p + "dt"].T + w[p + "dt.b"])  # [T, inner]
    b, c = dbc[:, rank : rank + n], dbc[:, rank + n : rank + 2 * n]
    a = -torch.exp(w[p + "A_log"])  # [inner, n]
    state = torch.zeros(inner, n, dtype=h.dtype)
    ys = []
    for t in range(h.shape[0]):
        state = torch.exp(dt[t][:, None] * a) * state + (dt[t] * x[t])[:, None] * b[t][None, :]
        ys.append(state @ c[t] + w[p + "D"] * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ w[p + "o"].T


def biased_attention(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Causal softmax attention whose only knowledge of positions is a learned bias per head and
    bucket of distance; queries and keys are normalised over their whole projection; the heads'
    outputs pass a sigmoid gate."""
    tokens = h.shape[0]
    heads, groups, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = unit_rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    q, k, v = q.view(tokens, heads, d), k.view(tokens, groups, d), v.view(tokens, groups, e)
    rel = w[p + "rel"]
    buckets = rel.shape[0]
    bucket = torch.tensor([[distance_bucket(i - j, buckets, m["bias_max"]) if j <= i else 0 for j in range(tokens)] for i in range(tokens)])
    seen = torch.tril(torch.ones(tokens, tokens, dtype=torch.bool))
    out = torch.zeros(tokens, heads, e, dtype=h.dtype)
    for head in range(heads):
        g = head // (heads // groups)
        score = (q[:, head] @ k[:, g].T) * m["scale"] + rel[:, head][bucket]
        score = score.masked_fill(~seen, float("-inf"))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, g]
    gated = out.reshape(tokens, heads * e) * torch.sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T


def retention(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """A state per head that fades by the head's constant and takes k v^T at every token: S <- decay S + k v^T, o = S^T q."""
    tokens = h.shape[0]
    heads, d, e = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(tokens)
    q = (h @ w[p + "q"].T).view(tokens, heads, d)
    k = (h @ w[p + "k"].T).view(tokens, heads, d)
    v = (h @ w[p + "v"].T).view(tokens, heads, e)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate_half(q, positions, rot["dims"], rot["base"]), rotate_half(k, positions, rot["dims"], rot["base"])
    k = k * d ** -0.5
    out = torch.zeros(tokens, heads, e, dtype=h.dtype)
    for head in range(heads):
        state = torch.zeros(d, e, dtype=h.dtype)
        for t in range(tokens):
            state = m["decay"][head] * state + k[t, head][:, None] * v[t, head][None, :]
            out[t, head] = state.T @ q[t, head]
    out = unit_rms(out, eps).reshape(tokens, heads * e) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    return m["left_scale"] * biased_attention(h, w, p + "left.", m["left"], eps) + m["right_scale"] * retention(h, w, p + "right.", m["right"], eps)


# ------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h: torch.Tensor, w: dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def gated_expert(h: torch.Tensor, w: dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """Every token goes through its ``top`` best experts, scaled on the way *in* by the sigmoid of its
    router logit (not renormalised), and through the shared expert."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    score = torch.sigmoid(h @ w[p + "router"].T)
    out = gated_expert(h, w, p + "shared.") if mlp.get("shared") is not None else torch.zeros_like(h)
    chosen = torch.topk(score, top, dim=-1).indices
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += gated_expert((score[t, e] * h[t])[None, :], w, f"{p}e{e}.")[0]
    assert experts == score.shape[1]
    return out


# ------------------------------------------------------------------------------------------ the model
def layer_runs(config: dict) -> list[tuple[int, int | None]]:
    """(layer, pass number if the layer opens a pass of the repeated run) in the order they run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, None) for i in range(count)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], count)]


def forward(config: dict, weights: dict[str, torch.Tensor], tokens: list[int], dtype=torch.float64, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``, if a list, receives the stream after every layer run."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    for index, opens in layer_runs(config):
        layer, p = config["layers"][index], f"l{index}."
        if opens is not None:
            x = x + w["loop.step"][opens]
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "mamba1":
            y = selective_scan_mixer(h, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_one_plus(x, w[p + "norm2"], eps)
            y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
            x = x + norm_one_plus(y, w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps) @ w["embed"].T
