"""Tiny Kegizen configurations for the tests: they differ in every size, option and layer order.

KEG_A: a repeated run of two layers (attention first), a window of 20 that keeps 3 tokens, half-rotated heads with
YaRN scaling, a soft-cap, values narrower than keys, a plain full attention, a layer without feed-forward.
KEG_B: no repeated run, one key head for three query heads, a window shorter than a page with nothing kept, a
rotation without scaling over a fifth of the head, five taps, head sizes that are no powers of two.
KEG_C: a run that "repeats" once, kept tokens that fill more than a page, convolutions of one tap (none at all),
an attention without rotation and without window, values wider than keys.
"""

import random

KEG_A = {
    "architecture": "Kegizen", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 112},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 24, "scale": 0.2, "softcap": 10.0,
                   "mask": {"size": 20, "keep_first": 3},
                   "rot": {"dims": 16, "base": 10000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}}},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 48},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25,
                   "rot": {"dims": 16, "base": 500.0, "scaling": None}}},
        {"type": "delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 40, "conv": 2}},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

KEG_B = {
    "architecture": "Kegizen", "vocab": 257, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "delta", "mlp": {"kind": "dense", "ff": 80},
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 48, "vdim": 20, "conv": 5}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 80},
         "mixer": {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 48, "scale": 0.3, "softcap": 5.0,
                   "mask": {"size": 9, "keep_first": 0}, "rot": {"dims": 8, "base": 100.0, "scaling": None}}},
    ],
    "loop": None,
}

KEG_C = {
    "architecture": "Kegizen", "vocab": 120, "width": 48, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.5, "softcap": 30.0,
                   "mask": {"size": 33, "keep_first": 17},
                   "rot": {"dims": 12, "base": 1000.0, "scaling": {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 0.5}}}},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 1}},
        {"type": "attention", "mlp": None, "mixer": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 16, "scale": 0.35}},
    ],
    "loop": {"start": 1, "stop": 2, "times": 1},
}

# name -> (config, seed, page size)
ALL = {"keg_a": (KEG_A, 11, 16), "keg_b": (KEG_B, 12, 4), "keg_c": (KEG_C, 13, 8)}


def prompt(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]
