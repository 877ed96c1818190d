"""Typed configuration of the Gifudra decoder, read from its config.json.

    {"architecture": "Gifudra", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": a},
     "logit_scale": b, "streams": S,
     "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A `latent_attention` mixer gives `heads, dim, rot_dim, vdim, q_rank, kv_rank, scale`, `rot: {dims, base}` and
optionally `kv_from: j`, the layer whose cache entries it reads instead of making its own.  Sizes have no defaults:
a missing size is a `ConfigError`.  `streams` absent or null: one residual with the plain sum; `embedding.scale` and
`logit_scale` absent: 1.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from liteinfer_b200.config.kegizen_config import _need
from liteinfer_b200.config.model_config import ConfigError

MIXER_TYPES = ("latent_attention",)


@dataclass(frozen=True)
class GifudraMixer:
    heads: int
    dim: int                 # unrotated query/key numbers per head
    rot_dim: int             # rotated query/key numbers per head; the key's are shared by all heads
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int            # how many of the rot_dim numbers turn (pairs i, i + rot_dims / 2)
    rot_base: float
    kv_from: int | None = None

    def __post_init__(self) -> None:
        for name in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            if getattr(self, name) < 1:
                raise ConfigError(f"mixer {name} must be >= 1, got {getattr(self, name)}")
        if self.rot_dims < 2 or self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ConfigError(f"rot.dims={self.rot_dims} must be even and within the {self.rot_dim} rotated numbers")
        if not self.rot_base > 0:
            raise ConfigError("rot.base must be > 0")

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str) -> GifudraMixer:
        sizes = {name: _need(raw, name, int, where) for name in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")}
        rot = raw.get("rot") if isinstance(raw, dict) else None
        kv_from = raw.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
            raise ConfigError(f"config.json {where} 'kv_from' must be a layer's index, got {kv_from!r}")
        return cls(scale=_need(raw, "scale", float, where), rot_dims=_need(rot, "dims", int, where + ".rot"),
                   rot_base=_need(rot, "base", float, where + ".rot"), kv_from=kv_from, **sizes)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale,
                               "rot": {"dims": self.rot_dims, "base": self.rot_base}}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class GifudraLayer:
    mixer: GifudraMixer
    ff: int | None           # width of the feed-forward; None = the layer has none


@dataclass(frozen=True)
class GifudraConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[GifudraLayer, ...]
    streams: int | None = None
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    eos_token_id: tuple[int, ...] = ()
    architecture: str = "Gifudra"

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1:
            raise ConfigError("vocab and width must be >= 1")
        if not self.layers:
            raise ConfigError("config.json names no layer")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be > 0")
        if self.streams is not None and self.streams < 1:
            raise ConfigError("streams must be >= 1")
        for i, layer in enumerate(self.layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i:
                raise ConfigError(f"layers[{i}] reads the entries of layer {j}, which is not an earlier layer")
            owner, m = self.layers[j].mixer, layer.mixer
            if owner.kv_from is not None:
                raise ConfigError(f"layers[{i}] reads the entries of layer {j}, which makes none of its own")
            if (owner.kv_rank, owner.rot_dim, owner.rot_dims, owner.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                raise ConfigError(f"layers[{i}] reads the entries of layer {j}, whose latent size or rotation differs")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> GifudraConfig:
        if not isinstance(raw.get("layers"), list):
            raise ConfigError("config.json has no 'layers' list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if entry.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json {where} has type {entry.get('type')!r}; known: {list(MIXER_TYPES)}")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json {where}.mlp has kind {mlp.get('kind')!r}; known: ['dense']")
            layers.append(GifudraLayer(GifudraMixer.from_dict(entry.get("mixer"), where + ".mixer"),
                                       None if mlp is None else _need(mlp, "ff", int, where + ".mlp")))
        streams = raw.get("streams")
        if streams is not None and (isinstance(streams, bool) or not isinstance(streams, int)):
            raise ConfigError(f"config.json 'streams' must be an integer, got {streams!r}")
        embedding = raw.get("embedding") or {}
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_need(raw, "vocab", int, ""), hidden_size=_need(raw, "width", int, ""),
                   norm_eps=_need(raw.get("norm"), "eps", float, "norm"), layers=tuple(layers), streams=streams,
                   embedding_scale=float(embedding.get("scale", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
                   eos_token_id=eos_ids, architecture=str(raw.get("architecture", "Gifudra")))

    def to_dict(self) -> dict[str, Any]:
        """config.json contents that `from_dict` reads back to an equal config."""
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "logit_scale": self.logit_scale, "streams": self.streams,
            "layers": [{"type": "latent_attention", "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}} for layer in self.layers],
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
