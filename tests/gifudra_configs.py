"""Tiny Gifudra configurations for the tests: they differ in every size, option and layer order.

GIF_A: two residual streams, layers that read an earlier layer's cache entries (one right behind its owner, one
further back), two owners of different sizes, a layer without feed-forward, a shared key part of which only a
part turns, scales that are no powers of two.
GIF_B: ONE stream that still has its read, write and mixing coefficients, one head, sizes that are multiples of
nothing (pages of 4).
GIF_C: no `streams` key at all (one residual, the plain sum), five heads, no scales in the file, every layer its
own entries.
GIF_D: four streams on sizes that the tensor-core attention takes (latent 64, rotated part 32), a reader of the
first layer's entries at the end.
"""

import random


def _mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, dims=None, base=10000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"dims": rot_dim if dims is None else dims, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, ff):
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


GIF_A = {
    "architecture": "Gifudra", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.7},
    "logit_scale": 0.6, "streams": 2,
    "layers": [
        _layer(_mixer(4, 16, 8, 24, 40, 48, 0.21, dims=4, base=500.0), 112),
        _layer(_mixer(2, 24, 8, 16, 24, 48, 0.17, dims=4, base=500.0, kv_from=0), 64),
        _layer(_mixer(3, 8, 16, 8, 32, 24, 0.3), None),
        _layer(_mixer(4, 16, 8, 24, 40, 48, 0.21, dims=4, base=500.0, kv_from=0), 48),
        _layer(_mixer(3, 8, 16, 40, 16, 24, 0.25, kv_from=2), 80),
    ],
}

GIF_B = {
    "architecture": "Gifudra", "vocab": 257, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "logit_scale": 1.0, "streams": 1,
    "layers": [
        _layer(_mixer(1, 12, 6, 20, 24, 40, 0.3, base=100.0), 56),
        _layer(_mixer(1, 12, 6, 20, 24, 40, 0.3, base=100.0), 56),
    ],
}

GIF_C = {
    "architecture": "Gifudra", "vocab": 120, "width": 48, "norm": {"eps": 1e-4},
    "layers": [
        _layer(_mixer(5, 8, 4, 8, 16, 16, 0.35, base=1000.0), 40),
        _layer(_mixer(5, 4, 2, 12, 8, 20, 0.5, base=50.0), None),
        _layer(_mixer(2, 20, 10, 6, 12, 36, 0.2, dims=6), 40),
    ],
}

GIF_D = {
    "architecture": "Gifudra", "vocab": 200, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "logit_scale": 1.5, "streams": 4,
    "layers": [
        _layer(_mixer(8, 32, 32, 32, 64, 64, 0.125, base=5000.0), 96),
        _layer(_mixer(16, 16, 32, 48, 32, 128, 0.14, base=5000.0), 96),
        _layer(_mixer(4, 64, 32, 16, 64, 64, 0.1, base=5000.0, kv_from=0), None),
    ],
}

# name -> (config, seed, page size)
ALL = {"gif_a": (GIF_A, 21, 16), "gif_b": (GIF_B, 22, 4), "gif_c": (GIF_C, 23, 8), "gif_d": (GIF_D, 24, 32)}


def prompt(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]


# Largest absolute difference of float32 logits from the float64 plain implementation that rounding alone explains,
# and the same for bfloat16 (the stand-in kernels, run in bfloat16 on a CPU, set the scale).
FLOAT32_TOLERANCE = {"gif_a": 5e-5, "gif_b": 5e-5, "gif_c": 5e-5, "gif_d": 1e-4}
BFLOAT16_TOLERANCE = {"gif_a": 0.06, "gif_b": 0.06, "gif_c": 0.06, "gif_d": 0.1}
