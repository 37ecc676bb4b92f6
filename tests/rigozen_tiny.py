"""Tiny Rigozen configurations for the tests; they differ in every size, order and option."""
import numpy as np


def _att(heads, kv, dim, window, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
            "mask": {"size": window}}


def _lat(heads, dim, vdim, rank, window, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
            "mask": {"size": window}}


def _delta(heads, kv, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}


def _ff(n):
    return {"kind": "dense", "ff": n}


# delta first (grouped q/k heads, value size unlike key size, three taps), an attention layer
# without feed-forward that is run twice (the second time on a cache of its own), a latent layer
R_A = {
    "architecture": "Rigozen", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "delta", "mixer": _delta(4, 2, 16, 24, 3), "mlp": _ff(96)},
        {"type": "attention", "mixer": _att(4, 2, 16, 9, 0.3), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(3, 16, 8, 40, 21, 0.2), "mlp": _ff(80)},
        {"type": "attention", "mixer": _att(4, 2, 16, 9, 0.3), "mlp": None, "weights_of": 1},
    ],
}
# windows that cross cache blocks (70, 130), a delta layer run twice, two taps, one q/k head
R_B = {
    "architecture": "Rigozen", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": _lat(2, 24, 32, 64, 70, 0.25), "mlp": _ff(64)},
        {"type": "delta", "mixer": _delta(2, 1, 32, 16, 2), "mlp": _ff(128)},
        {"type": "delta", "mixer": _delta(2, 1, 32, 16, 2), "mlp": _ff(128), "weights_of": 1},
        {"type": "attention", "mixer": _att(2, 1, 32, 130, 0.2), "mlp": _ff(64)},
    ],
}
# everything that can be one is one: one head, one tap (no convolution state), a window that
# shows a query nothing but itself, a window of two
R_C = {
    "architecture": "Rigozen", "vocab": 70, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "delta", "mixer": _delta(1, 1, 8, 8, 1), "mlp": None},
        {"type": "attention", "mixer": _att(1, 1, 8, 1, 1.0), "mlp": _ff(48)},
        {"type": "latent_attention", "mixer": _lat(1, 8, 16, 8, 2, 0.5), "mlp": None},
    ],
}
# sizes that are multiples of nothing in particular: head sizes 12 and 20, a latent of 20, an
# odd vocabulary, a width of 40; a window longer than any test sequence
R_D = {
    "architecture": "Rigozen", "vocab": 77, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(3, 1, 12, 500, 0.29), "mlp": _ff(56)},
        {"type": "delta", "mixer": _delta(3, 1, 12, 6, 5), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(2, 20, 6, 20, 5, 0.3), "mlp": _ff(24)},
    ],
}
CONFIGS = {"A": R_A, "B": R_B, "C": R_C, "D": R_D}
SEEDS = {"A": 101, "B": 202, "C": 303, "D": 404}


def one_layer(kind: str, window: int = 12):
    """A model of a single layer of one mixer and no feed-forward: the mechanism alone."""
    mixer = {"attention": _att(4, 2, 16, window, 0.4),
             "latent_attention": _lat(3, 16, 24, 32, window, 0.4),
             "delta": _delta(4, 2, 16, 8, 4)}[kind]
    return {"architecture": "Rigozen", "vocab": 80, "width": 64, "norm": {"eps": 1e-5},
            "layers": [{"type": kind, "mixer": mixer, "mlp": None}]}


def tokens(name: str, length: int, seed: int):
    rng = np.random.default_rng(7000 * seed + length)
    return rng.integers(0, CONFIGS[name]["vocab"], size=length).tolist()
