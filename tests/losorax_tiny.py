"""Tiny Losorax configurations for the tests; they differ in every size, order and option."""
import numpy as np


def _att(heads, kv, dim, vdim, taps, rows, far, coef, every, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps,
         "bias_rows": rows, "bias_max": far, "q_temp": {"coef": coef, "every": every},
         "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, dim, rank):
    return {"heads": heads, "dim": dim, "decay_rank": rank}


def _ff(n):
    return {"kind": "dense", "ff": n}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


# grouped heads with values wider than keys, a layer that reads the first layer's keys and
# values, two experts a token, a delta layer in the middle
L_A = {
    "architecture": "Losorax", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 16, 24, 3, 12, 40, 0.5, 7, 0.3), "mlp": _ff(96)},
        {"type": "general_delta", "mixer": _delta(2, 16, 8), "mlp": _moe(6, 2, 32)},
        {"type": "attention", "mixer": _att(4, 2, 16, 24, 3, 12, 40, 0.5, 7, 0.3, kv_from=0),
         "mlp": _moe(6, 2, 32)},
    ],
}
# a delta layer first and without feed-forward, one tap (no saved inputs), an odd number of
# bias rows, values narrower than keys, three of five experts, a gain that grows every token,
# a reader whose queries have four taps where the writer has one
L_B = {
    "architecture": "Losorax", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "general_delta", "mixer": _delta(3, 24, 5), "mlp": None},
        {"type": "attention", "mixer": _att(2, 1, 32, 16, 1, 7, 100, 0.2, 1, 0.2), "mlp": _moe(5, 3, 40)},
        {"type": "attention", "mixer": _att(2, 1, 32, 16, 4, 9, 33.5, 1.0, 50, 0.25, kv_from=1),
         "mlp": _ff(64)},
        {"type": "general_delta", "mixer": _delta(1, 32, 3), "mlp": _moe(5, 3, 40)},
    ],
}
# everything that can be one is one: one head, one expert, two bias rows, rank one
L_C = {
    "architecture": "Losorax", "vocab": 70, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(1, 1, 8, 8, 2, 2, 3, 0.0, 1, 1.0), "mlp": _moe(1, 1, 48)},
        {"type": "general_delta", "mixer": _delta(1, 8, 1), "mlp": None},
    ],
}
# sizes that are multiples of nothing in particular: head sizes 12, 20 and 10, five taps, an odd
# vocabulary, a width of 40, as many key/value heads as query heads, far more rows than distances
L_D = {
    "architecture": "Losorax", "vocab": 77, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(3, 3, 12, 20, 5, 64, 500, 0.3, 16, 0.29), "mlp": _moe(7, 2, 24)},
        {"type": "general_delta", "mixer": _delta(3, 10, 4), "mlp": _ff(56)},
        {"type": "attention", "mixer": _att(3, 3, 12, 20, 2, 6, 90, 0.3, 64, 0.29, kv_from=0), "mlp": None},
    ],
}
CONFIGS = {"A": L_A, "B": L_B, "C": L_C, "D": L_D}
SEEDS = {"A": 111, "B": 222, "C": 333, "D": 444}


def one_layer(kind: str, mixer=None, mlp=None):
    """A model of a single layer of one mixer: the mechanism alone."""
    if mixer is None:
        mixer = {"attention": _att(4, 2, 16, 8, 3, 10, 60, 0.4, 5, 0.4),
                 "general_delta": _delta(2, 16, 6)}[kind]
    return {"architecture": "Losorax", "vocab": 80, "width": 64, "norm": {"eps": 1e-5},
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


def tokens(name: str, length: int, seed: int):
    rng = np.random.default_rng(9000 * seed + length)
    return rng.integers(0, CONFIGS[name]["vocab"], size=length).tolist()
