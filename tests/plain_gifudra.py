"""A plain, slow Gifudra: whole sequences, no cache, one function per mechanism.

Gifudra is a decoder whose layers each have a latent attention (queries through a low-rank latent, keys and
values expanded per head from one shared normalised latent per token, one rotated key part shared by all heads,
a learned sink in the softmax's denominator, a sigmoid output gate; a layer may read an earlier layer's latent
and rotated key part instead of making its own) and an optional squared-relu feed-forward.  Sublayer outputs
are scaled per channel, and the residual is kept as several streams that every sublayer reads as a weighted
sum and rewrites through a small mixing matrix.

This file shares no code with `liteinfer_b200`: it parses config.json with `json`, reads tensors with
`safetensors` and computes with stock torch ops in one dtype (float64 by default).
Notation: T tokens, D width, H heads, d unrotated and r rotated key size, e value size, c latent size, S streams.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import load_file


def read_model(model_dir: str | Path, dtype: torch.dtype = torch.float64) -> tuple[dict, dict[str, torch.Tensor]]:
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    tensors = load_file(str(model_dir / "model.safetensors"))
    return config, {name: t.to(dtype) for name, t in tensors.items()}


# ------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def squared_relu_feed_forward(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    a = torch.relu(h @ up.T)
    return (a * a) @ down.T


def rotate_half_split(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotates the first `dims` entries of the last axis of x [T, ..., n]: entry i pairs with entry i + dims/2,
    by the angle position * base^(-2i/dims); the other entries pass."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    angle = positions.to(torch.float64)[:, None] * freq                      # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(angle).to(x.dtype).reshape(shape), torch.sin(angle).to(x.dtype).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                           sink: torch.Tensor | None) -> torch.Tensor:
    """q [H, T, n], k [H, T, n], v [H, T, e] -> [H, T, e].  Causal.  The softmax's denominator also holds
    exp(sink[h]), which belongs to no key and no value and is not scaled."""
    H, T, _ = q.shape
    scores = torch.einsum("hik,hjk->hij", q, k) * scale
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    scores = scores.masked_fill(~visible, float("-inf"))
    if sink is not None:
        scores = torch.cat([scores, sink.to(scores.dtype)[:, None, None].expand(H, T, 1)], dim=-1)
    weights = torch.softmax(scores, dim=-1)[..., :T]
    return torch.einsum("hij,hje->hie", weights, v)


# ------------------------------------------------------------------ the mixer
def latent_and_rotated_key(h: torch.Tensor, w: dict[str, torch.Tensor], m: dict, eps: float,
                           positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """What a layer remembers of a token: the normalised latent [T, c] and the rotated shared key part [T, r]."""
    c, r = m["kv_rank"], m["rot_dim"]
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :c], w["dkv.norm"], eps)
    shared = rotate_half_split(down[:, c:c + r], positions, m["rot"]["dims"], m["rot"]["base"])
    return latent, shared


def latent_attention(h: torch.Tensor, w: dict[str, torch.Tensor], m: dict, eps: float, positions: torch.Tensor,
                     latent: torch.Tensor, shared: torch.Tensor) -> torch.Tensor:
    """The mixer on h [T, D], given the latent and the rotated key part it attends over (its own or another layer's)."""
    T = h.shape[0]
    H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (rms_norm(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T).reshape(T, H, d + r)
    q_rot = rotate_half_split(q[..., d:], positions, m["rot"]["dims"], m["rot"]["base"])
    q = torch.cat([q[..., :d], q_rot], dim=-1).transpose(0, 1)                           # [H, T, d + r]
    k_plain = (latent @ w["uk"].T).reshape(T, H, d)
    k = torch.cat([k_plain, shared[:, None, :].expand(T, H, r)], dim=-1).transpose(0, 1)
    v = (latent @ w["uv"].T).reshape(T, H, e).transpose(0, 1)
    heads = sink_softmax_attention(q, k, v, m["scale"], w.get("sink"))                   # [H, T, e]
    joined = heads.transpose(0, 1).reshape(T, H * e) * torch.sigmoid(h @ w["g"].T)
    return joined @ w["o"].T


# ------------------------------------------------------------------ the residual streams
def streams_read(streams: torch.Tensor, read: torch.Tensor) -> torch.Tensor:
    """streams [S, T, D], read [S] -> sum_s read[s] streams[s]."""
    return torch.einsum("s,std->td", read, streams)


def streams_write(streams: torch.Tensor, mix: torch.Tensor, write: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """New stream t = sum_s mix[s, t] old stream s + write[t] y, all from the old streams."""
    return torch.einsum("sk,std->ktd", mix, streams) + write[:, None, None] * y[None]


# ------------------------------------------------------------------ the model
def _part(tensors: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int], trace: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `trace` collects the residual (the sum of the streams) after every layer."""
    dtype = tensors["embed"].dtype
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = tensors["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    S = config.get("streams")
    streams = x[None].repeat(S, 1, 1) if S else None
    kept: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    def sublayer(i: int, q: int, fn):
        nonlocal x, streams
        norm_w, scale = tensors[f"l{i}.norm{q}"], tensors[f"l{i}.ls{q}"]
        if streams is None:
            x = x + scale * fn(rms_norm(x, norm_w, eps))
            return
        hc = _part(tensors, f"l{i}.hc{q}.")
        y = scale * fn(rms_norm(streams_read(streams, hc["in"]), norm_w, eps))
        streams = streams_write(streams, hc["mix"], hc["out"], y)

    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "latent_attention"
        m, w = layer["mixer"], _part(tensors, f"l{i}.mix.")

        def mixer(h, i=i, m=m, w=w):
            if m.get("kv_from") is None:
                kept[i] = latent_and_rotated_key(h, w, m, eps, positions)
                latent, shared = kept[i]
            else:
                latent, shared = kept[m["kv_from"]]
            return latent_attention(h, w, m, eps, positions, latent, shared)

        sublayer(i, 1, mixer)
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            mlp = _part(tensors, f"l{i}.mlp.")
            sublayer(i, 2, lambda h, mlp=mlp: squared_relu_feed_forward(h, mlp["up"], mlp["down"]))
        if trace is not None:
            trace.append(x.clone() if streams is None else streams.sum(0))
    if streams is not None:
        x = streams.sum(0)
    return (rms_norm(x, tensors["final.norm"], eps) @ tensors["embed"].T * config["logit_scale"]).to(dtype)
