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

# Sizes that the tensor-core attention kernels and the staged recurrence kernel take (keys and values of 64, a state
# of 64 x 32), with a window, kept tokens, a cap and scaled rotation on them; two passes over both layers.
KEG_D = {
    "architecture": "Kegizen", "vocab": 200, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "delta", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 32, "conv": 3}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 12.0,
                   "mask": {"size": 70, "keep_first": 5},
                   "rot": {"dims": 64, "base": 5000.0, "scaling": {"factor": 3.0, "original": 64, "fast": 16.0, "slow": 2.0}}}},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

# name -> (config, seed, page size)
ALL = {"keg_a": (KEG_A, 11, 16), "keg_b": (KEG_B, 12, 4), "keg_c": (KEG_C, 13, 8), "keg_d": (KEG_D, 14, 16)}


def prompt(vocab: int, length: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]

# Largest absolute difference of float32 logits from the float64 plain implementation that rounding alone explains
# (the plain implementation itself, run in float32, differs from its float64 run by 4e-5 on KEG_D: two passes of
# layer norms over small sublayer outputs amplify the last bits).
FLOAT32_TOLERANCE = {"keg_a": 5e-5, "keg_b": 5e-5, "keg_c": 5e-5, "keg_d": 2e-4}
# The same for bfloat16 (the plain stand-in kernels, run in bfloat16 on a CPU, come to 0.05 and 0.04).  How far
# rounding carries depends on the sizes: with one q/k head for four value heads in KEG_D's recurrence the same
# stand-ins differ from float64 by 0.47, every head repeating the same rounded q and k.
BFLOAT16_TOLERANCE = {"keg_a": 0.06, "keg_b": 0.06, "keg_c": 0.06, "keg_d": 0.1}
