"""Typed configuration of the Kegizen decoder, read from its config.json.

A Kegizen config.json names everything per layer:

    {"architecture": "Kegizen", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "delta" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n} | null}

`delta` mixers give `heads, kv_heads, dim, vdim, conv`; `attention` mixers give `heads, kv_heads, dim, vdim, scale`
and optionally `softcap`, `mask: {size, keep_first}` and `rot: {dims, base, scaling: {factor, original, fast,
slow} | null}`.  Sizes have no defaults: a missing size is a `ConfigError`.  An option that is absent or null is
off (no soft-cap, every earlier key visible, no rotation, no frequency scaling, no feed-forward, no repeated run).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from liteinfer_b200.config.model_config import ConfigError

MIXER_TYPES = ("delta", "attention")


def _need(raw: dict[str, Any], key: str, kind: type, where: str) -> Any:
    if not isinstance(raw, dict) or raw.get(key) is None:
        raise ConfigError(f"config.json {where} has no {key!r}")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float) if kind is float else int):
        raise ConfigError(f"config.json {where} {key!r} must be {'a number' if kind is float else 'an integer'}, got {value!r}")
    return kind(value)


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: YarnScaling | None = None


@dataclass(frozen=True)
class KegizenMixer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int = 0                    # delta: taps of the short convolutions
    scale: float = 0.0               # attention: what a score is multiplied by
    softcap: float = 0.0             # attention: 0 = scores are not capped
    window: int | None = None        # attention: None = every earlier key is visible
    keep_first: int = 0              # attention: the first tokens stay visible behind the window
    rot: Rotation | None = None

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"mixer type {self.type!r} is not supported; known: {list(MIXER_TYPES)}")
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) < 1:
                raise ConfigError(f"mixer {name} must be >= 1, got {getattr(self, name)}")
        if self.heads % self.kv_heads:
            raise ConfigError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
        if self.type == "delta" and self.conv < 1:
            raise ConfigError("a delta mixer needs conv >= 1")
        if self.window is not None and self.window < 1:
            raise ConfigError("mask.size must be >= 1")
        if self.keep_first < 0:
            raise ConfigError("mask.keep_first must be >= 0")
        if self.rot is not None and (self.rot.dims < 2 or self.rot.dims % 2 or self.rot.dims > self.dim):
            raise ConfigError(f"rot.dims={self.rot.dims} must be even and within the head's {self.dim} dimensions")

    @classmethod
    def from_dict(cls, kind: str, raw: dict[str, Any], where: str) -> KegizenMixer:
        sizes = {name: _need(raw, name, int, where) for name in ("heads", "kv_heads", "dim", "vdim")}
        if kind == "delta":
            return cls(kind, conv=_need(raw, "conv", int, where), **sizes)
        mask = raw.get("mask") or {}
        rot = None
        if raw.get("rot"):
            r = raw["rot"]
            scaling = None
            if r.get("scaling"):
                s = r["scaling"]
                scaling = YarnScaling(*(_need(s, k, float, where + " rot.scaling") for k in ("factor", "original", "fast", "slow")))
            rot = Rotation(_need(r, "dims", int, where + " rot"), _need(r, "base", float, where + " rot"), scaling)
        return cls(kind, scale=_need(raw, "scale", float, where), softcap=float(raw.get("softcap") or 0.0),
                   window=int(mask["size"]) if mask.get("size") is not None else None,
                   keep_first=int(mask.get("keep_first") or 0), rot=rot, **sizes)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "delta":
            out["conv"] = self.conv
            return out
        out["scale"] = self.scale
        if self.softcap:
            out["softcap"] = self.softcap
        if self.window is not None or self.keep_first:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            s = self.rot.scaling
            out["rot"] = {"dims": self.rot.dims, "base": self.rot.base,
                          "scaling": None if s is None else {"factor": s.factor, "original": s.original,
                                                             "fast": s.fast, "slow": s.slow}}
        return out


@dataclass(frozen=True)
class KegizenLayer:
    mixer: KegizenMixer
    ff: int | None                   # width of the gated feed-forward; None = the layer has none


@dataclass(frozen=True)
class KegizenLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class KegizenConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[KegizenLayer, ...]
    loop: KegizenLoop | None = None
    eos_token_id: tuple[int, ...] = ()
    architecture: str = "Kegizen"

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1:
            raise ConfigError("vocab and width must be >= 1")
        if not self.layers:
            raise ConfigError("config.json names no layer")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be > 0")
        if self.loop is not None:
            if not 0 <= self.loop.start <= self.loop.stop <= len(self.layers) or self.loop.times < 0:
                raise ConfigError(f"loop {self.loop} does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> KegizenConfig:
        layers = []
        if not isinstance(raw.get("layers"), list):
            raise ConfigError("config.json has no 'layers' list")
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json {where} has type {kind!r}; known: {list(MIXER_TYPES)}")
            mixer = KegizenMixer.from_dict(kind, entry.get("mixer"), where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json {where}.mlp has kind {mlp.get('kind')!r}; known: ['dense']")
            layers.append(KegizenLayer(mixer, None if mlp is None else _need(mlp, "ff", int, where + ".mlp")))
        loop = None
        if raw.get("loop"):
            loop = KegizenLoop(*(_need(raw["loop"], k, int, "loop") for k in ("start", "stop", "times")))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_need(raw, "vocab", int, ""), hidden_size=_need(raw, "width", int, ""),
                   norm_eps=_need(raw.get("norm"), "eps", float, "norm"), layers=tuple(layers), loop=loop,
                   eos_token_id=eos_ids, architecture=str(raw.get("architecture", "Kegizen")))

    def to_dict(self) -> dict[str, Any]:
        """config.json contents that `from_dict` reads back to an equal config."""
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": layer.mixer.type, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}} for layer in self.layers],
            "loop": None if self.loop is None else {"start": self.loop.start, "stop": self.loop.stop,
                                                    "times": self.loop.times},
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
