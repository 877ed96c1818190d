"""A plain, slow Kegizen: whole sequences, no cache, one function per mechanism.

Kegizen is a decoder whose layers each have one of two mixers (a gated delta-rule
recurrence with short convolutions, or softmax attention with a sliding window that
keeps the first tokens, a score soft-cap, a norm over the whole q and k projections
and partly rotated heads with YaRN-scaled frequencies), a gated feed-forward, four
weight-only layer norms per layer, and a run of layers that is repeated with the
embedding fed in again at the start of every pass.

This file shares no code with `liteinfer_b200`: it parses config.json with `json`,
reads tensors with `safetensors` and computes with stock torch ops in one dtype
(float64 by default), token by token where the mechanism is a recurrence.
Notation: T tokens, D width, H heads, G key heads, d key size, e value size.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


def read_model(model_dir: str | Path, dtype: torch.dtype = torch.float64) -> tuple[dict, dict[str, torch.Tensor]]:
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    tensors = load_file(str(model_dir / "model.safetensors"))
    return config, {name: t.to(dtype) for name, t in tensors.items()}


# ------------------------------------------------------------------ small pieces
def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w over the last axis, var = mean of squared deviations; no bias."""
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * weight


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time per channel.  x [T, C], taps [C, K]; the last column multiplies the
    current token, the one before it the previous token, and so on; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([x.new_zeros(K - 1, C), x])
    out = x.new_zeros(T, C)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def gated_feed_forward(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


# ------------------------------------------------------------------ rotary
def yarn_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """(frequency of each of the dims/2 pairs, the factor that multiplies cos and sin)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_partly(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, mult: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: the first `dims` dimensions of each head are rotated (i with i + dims/2), the rest pass."""
    half = dims // 2
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = (torch.cos(angle) * mult).to(x.dtype)[:, None, :], (torch.sin(angle) * mult).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ mixers
def visible(i: int, j: int, size: int | None, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    return size is None or i - j < size or j < keep_first


def attention_mixer(h: torch.Tensor, w: dict[str, torch.Tensor], p: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = rms_unit(h @ w["q"].T, eps) * w["q.norm"]          # over all H*d entries at once
    k = rms_unit(h @ w["k"].T, eps) * w["k.norm"]
    v = (h @ w["v"].T).view(T, G, e)
    q, k = q.view(T, H, d), k.view(T, G, d)
    rot = p.get("rot")
    if rot:
        freq, mult = yarn_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
        positions = torch.arange(T)
        q = rotate_partly(q, positions, freq, mult, rot["dims"])
        k = rotate_partly(k, positions, freq, mult, rot["dims"])
    mask = p.get("mask") or {}
    size, keep_first = mask.get("size"), int(mask.get("keep_first") or 0)
    allowed = torch.tensor([[visible(i, j, size, keep_first) for j in range(T)] for i in range(T)])
    cap = p.get("softcap")
    out = h.new_zeros(T, H, e)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * p["scale"]
        if cap:
            score = cap * torch.tanh(score / cap)
        score = score.masked_fill(~allowed, float("-inf"))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, g]
    return out.reshape(T, H * e) @ w["o"].T


def delta_mixer(h: torch.Tensor, w: dict[str, torch.Tensor], p: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                       # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    gate = silu(h @ w["g"].T).view(T, H, e)
    out = h.new_zeros(T, H, e)
    for head in range(H):
        g = head // (H // G)
        S = h.new_zeros(d, e)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w["norm"] * gate
    return out.reshape(T, H * e) @ w["o"].T


MIXERS = {"attention": attention_mixer, "delta": delta_mixer}


# ------------------------------------------------------------------ the model
def layer_runs(config: dict) -> list[tuple[int, bool]]:
    """(layer, whether the stream is re-mixed with the embedding before it) for every layer run, in order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for _ in range(times):
        runs += [(i, i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def part(tensors: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int], trace: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `trace` collects the stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x0 = tensors["embed"][torch.tensor(tokens)]
    x = x0
    for index, remix in layer_runs(config):
        if remix:
            x = torch.cat([x, x0], dim=-1) @ tensors["loop.in"].T
        layer, name = config["layers"][index], f"l{index}."
        mixed = MIXERS[layer["type"]](layer_norm(x, tensors[name + "norm1"], eps), part(tensors, name + "mix."),
                                      layer["mixer"], eps)
        x = x + layer_norm(mixed, tensors[name + "norm1b"], eps)
        if layer.get("mlp"):
            assert layer["mlp"]["kind"] == "dense"
            fed = gated_feed_forward(layer_norm(x, tensors[name + "norm2"], eps), tensors[name + "mlp.gate"],
                                     tensors[name + "mlp.up"], tensors[name + "mlp.down"])
            x = x + layer_norm(fed, tensors[name + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
