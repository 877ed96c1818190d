"""The Gifudra decoder as a `ModelSpec`.

Every layer is a pre-norm block around a latent attention (parts/latent_attention.py) and an optional
squared-relu feed-forward.  The residual is `streams` 32-bit copies that every sublayer reads as a weighted sum
and rewrites through a small matrix, its output scaled per channel (parts/connection.py); all norms are RMS norms
computed in 32-bit.  A layer may read an earlier layer's cache entries instead of making its own (`kv_from`): its
schedule entry names that stop as `cache_of`.  The embedding's rows are multiplied by `embedding.scale`; the head
is the embedding's table, and `logit_scale` is folded into the last norm.  Tensor names: `embed`,
`l<i>.norm1|norm2`, `l<i>.ls1|ls2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|g|o`,
`l<i>.mlp.up|down`, `final.norm`.
"""

from __future__ import annotations

from liteinfer_b200.config.gifudra_config import GifudraConfig, GifudraMixer
from liteinfer_b200.config.registry import register_architecture
from liteinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_BARE = {"weight": ""}      # a tensor stored under the part's prefix itself
_MIXER_NAMES = {"dq.weight": "dq", "dq_norm.weight": "dq.norm", "uq.weight": "uq", "dkv.weight": "dkv",
                "dkv_norm.weight": "dkv.norm", "uk.weight": "uk", "uv.weight": "uv", "g.weight": "g", "o.weight": "o"}
_MLP_NAMES = {"up_proj.weight": "up", "down_proj.weight": "down"}


def _connection_names(q: int) -> dict[str, str]:
    return {"in": f"hc{q}.in", "out": f"hc{q}.out", "mix": f"hc{q}.mix", "gain": f"ls{q}"}


def _mixer(config: GifudraConfig, m: GifudraMixer) -> PartSpec:
    position = PartSpec("rotary", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base, "exact": True})
    return PartSpec("latent_attention", {
        "hidden_size": config.hidden_size, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
        "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": config.norm_eps, "position": position,
        "own_kv": m.kv_from is None})


def gifudra_spec(config: GifudraConfig) -> ModelSpec:
    streams = config.streams or 1
    norm = PartSpec("stream_rmsnorm", {"size": config.hidden_size, "eps": config.norm_eps, "streams": streams})
    connection = PartSpec("stream_mix", {"streams": streams, "width": config.hidden_size,
                                         "learned": config.streams is not None})
    layers, ignored = [], []
    for i, layer in enumerate(config.layers):
        parts = {"mixer_norm": norm, "mixer": _mixer(config, layer.mixer), "mixer_connection": connection}
        prefixes = {"mixer_norm": f"l{i}.norm1", "mixer": f"l{i}.mix.", "mixer_connection": f"l{i}."}
        renames = {"mixer_norm": _BARE, "mixer": _MIXER_NAMES, "mixer_connection": _connection_names(1)}
        if layer.ff is not None:
            parts.update({"feed_forward_norm": norm, "feed_forward_connection": connection, "feed_forward": PartSpec(
                "dense_mlp", {"hidden_size": config.hidden_size, "intermediate_size": layer.ff,
                              "activation": "relu_squared"})})
            prefixes.update({"feed_forward_norm": f"l{i}.norm2", "feed_forward": f"l{i}.mlp.",
                             "feed_forward_connection": f"l{i}."})
            renames.update({"feed_forward_norm": _BARE, "feed_forward": _MLP_NAMES,
                            "feed_forward_connection": _connection_names(2)})
        else:   # what belongs to a feed-forward that the layer does not have may still be in the file
            ignored += [f"l{i}.norm2", f"l{i}.ls2", f"l{i}.hc2.in", f"l{i}.hc2.out", f"l{i}.hc2.mix"]
        layers.append(LayerSpec("stream_mixed" if layer.ff is not None else "stream_mixed_mixer_only", parts,
                                prefixes, renames))
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        embedding=PartSpec("token_embedding", {**sizes, "scale": config.embedding_scale}), embedding_prefix="embed",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, cache_of=layer.mixer.kv_from) for i, layer in enumerate(config.layers)),
        final_norm=PartSpec("stream_rmsnorm", {"size": config.hidden_size, "eps": config.norm_eps, "streams": streams,
                                               "out_scale": config.logit_scale}),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", sizes), head_prefix="head", tied={"head": "embed"},
        stream_dtype="float32", stream_copies=streams,
        renames={"embedding": _BARE, "final_norm": _BARE, "head": _BARE},
        ignored=tuple(ignored),
    )


register_architecture("Gifudra", GifudraConfig, gifudra_spec, replace=True)
