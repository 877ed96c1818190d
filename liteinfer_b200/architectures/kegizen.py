"""The Kegizen decoder as a `ModelSpec`.

Every layer is a sandwich-norm block (weight-only layer norms before and after each sublayer) around one of two
mixers, a gated delta-rule recurrence or a softmax attention with a sliding window that keeps the first tokens, and
an optional gated feed-forward.  The residual stream is summed in 32-bit.  A run of layers [start, stop) may be
repeated `times` times with the same weights; every pass keeps caches and states of its own, and before its first
layer the stream is mixed with the embedding's output through one product.  Tensor names: `embed`, `loop.in`,
`l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`, `final.norm`, `head`.
"""

from __future__ import annotations

from liteinfer_b200.config.kegizen_config import KegizenConfig, KegizenMixer
from liteinfer_b200.config.registry import register_architecture
from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_BARE = {"weight": ""}      # a tensor stored under the part's prefix itself
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"}
_DELTA_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                "b_proj.weight": "b", "a_proj.weight": "a", "o_proj.weight": "o", "q_conv.weight": "q.conv",
                "k_conv.weight": "k.conv", "v_conv.weight": "v.conv", "norm.weight": "norm"}
_MLP_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def _mixer(config: KegizenConfig, mixer: KegizenMixer) -> tuple[PartSpec, dict[str, str]]:
    sizes = {"hidden_size": config.hidden_size, "heads": mixer.heads, "kv_heads": mixer.kv_heads}
    if mixer.type == "delta":
        return PartSpec("gated_delta_rule", {**sizes, "dim": mixer.dim, "vdim": mixer.vdim, "conv": mixer.conv,
                                             "norm_eps": config.norm_eps}), _DELTA_NAMES
    if mixer.rot is None:
        position = PartSpec("none", {})
    elif mixer.rot.scaling is None:
        position = PartSpec("rotary", {"head_dim": mixer.dim, "rotary_dim": mixer.rot.dims, "theta": mixer.rot.base})
    else:
        s = mixer.rot.scaling
        position = PartSpec("rotary", {"head_dim": mixer.dim, "rotary_dim": mixer.rot.dims, "theta": mixer.rot.base,
                                       "rope_type": "yarn", "factor": s.factor,
                                       "original_max_position_embeddings": s.original, "fast": s.fast, "slow": s.slow})
    return PartSpec("attention", {**sizes, "head_dim": mixer.dim, "v_head_dim": mixer.vdim, "position": position,
                                  "scale": mixer.scale, "softcap": mixer.softcap, "window": mixer.window,
                                  "keep_first": mixer.keep_first, "qk_norm": "projection",
                                  "qk_norm_eps": config.norm_eps}), _ATTENTION_NAMES


def schedule_of(config: KegizenConfig) -> tuple[ScheduleEntry, ...]:
    """Layers before the repeated run once, the run `times` times (each pass re-enters at its first layer), the rest."""
    n = len(config.layers)
    if config.loop is None:
        return tuple(ScheduleEntry(i) for i in range(n))
    start, stop, times = config.loop.start, config.loop.stop, config.loop.times
    stops = [ScheduleEntry(i) for i in range(start)]
    for _ in range(times):
        stops += [ScheduleEntry(i, reenter=i == start) for i in range(start, stop)]
    return tuple(stops + [ScheduleEntry(i) for i in range(stop, n)])


def kegizen_spec(config: KegizenConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"size": config.hidden_size, "eps": config.norm_eps})
    layers, ignored = [], []
    for i, layer in enumerate(config.layers):
        mixer, mixer_names = _mixer(config, layer.mixer)
        parts = {"mixer_norm": norm, "mixer": mixer, "mixer_post_norm": norm}
        prefixes = {"mixer_norm": f"l{i}.norm1", "mixer": f"l{i}.mix.", "mixer_post_norm": f"l{i}.norm1b"}
        renames = {"mixer_norm": _BARE, "mixer": mixer_names, "mixer_post_norm": _BARE}
        if layer.ff is not None:
            parts.update({"feed_forward_norm": norm, "feed_forward_post_norm": norm, "feed_forward": PartSpec(
                "gated_mlp", {"hidden_size": config.hidden_size, "intermediate_size": layer.ff, "activation": "silu"})})
            prefixes.update({"feed_forward_norm": f"l{i}.norm2", "feed_forward": f"l{i}.mlp.",
                             "feed_forward_post_norm": f"l{i}.norm2b"})
            renames.update({"feed_forward_norm": _BARE, "feed_forward": _MLP_NAMES, "feed_forward_post_norm": _BARE})
        else:
            ignored += [f"l{i}.norm2", f"l{i}.norm2b"]      # norms of a feed-forward that the layer does not have
        layers.append(LayerSpec("sandwich_norm" if layer.ff is not None else "sandwich_norm_mixer_only", parts,
                                prefixes, renames))
    schedule = schedule_of(config)
    if not schedule:
        raise ValueError("the configuration runs no layer")
    loops = config.loop is not None
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        embedding=PartSpec("token_embedding", sizes), embedding_prefix="embed",
        layers=tuple(layers), schedule=schedule,
        final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", sizes), head_prefix="head",
        stream_dtype="float32",
        reentry=PartSpec("embedding_remix", {"hidden_size": config.hidden_size}) if loops else None,
        reentry_prefix="loop.in",
        renames={"embedding": _BARE, "final_norm": _BARE, "head": _BARE, "reentry": _BARE},
        ignored=tuple(ignored) + (() if loops else ("loop.in",)),
    )


register_architecture("Kegizen", KegizenConfig, kegizen_spec, replace=True)
