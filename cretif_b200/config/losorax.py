"""Typed configuration of the Losorax decoder, read from config.json, and its ModelSpec.

A Losorax checkpoint's config.json names its class with ``"architecture": "Losorax"`` and
describes the model as a list of layers, each with a mixer of its own kind and sizes:

=====================  ========================================================================
key                    meaning
=====================  ========================================================================
vocab, width           vocabulary and residual width
norm.eps               eps of the RMS divisions inside the mixers (the block's norm has none)
layers[i].type         ``attention`` | ``general_delta``
layers[i].mixer        attention: heads, kv_heads, dim, vdim, scale, conv (taps), bias_max,
                       q_temp {coef, every}, kv_from (optional: the layer whose keys and values
                       this layer reads instead of projecting its own);
                       general_delta: heads, dim
layers[i].mlp          ``{"kind": "dense", "ff": F}``, ``{"kind": "moe", "expert": {"ff": F},
                       "router": {"experts": E, "top": k}}``, or null for no feed-forward
max_positions          (optional) longest sequence; the design itself has no limit
=====================  ========================================================================

Two sizes are not in config.json but in the tensors' shapes: the rows of an attention layer's
distance-bias table and the low rank of a delta layer's decay.  ``mixer.bias_rows`` and
``mixer.decay_rank`` (optional, this library's own keys) say what the random-weights mode
draws.

The block norms before and after each sublayer with Dynamic Tanh, scales the normed result
per channel and blends the mixer's input with the previous token's:
``x += ls1 * dyt(mixer(shift(dyt(x))))``, ``x += ls2 * dyt(ff(dyt(x)))``.  Tensors are named
``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.norm1/1b/2/2b`` (``.b``, ``.alpha`` beside them),
``l<i>.ls1/ls2``, ``l<i>.shift``, ``embed``, ``final.norm`` and ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .registry import ConfigError, register_architecture
from .spec import BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("attention", "general_delta")
DEFAULT_MAX_POSITIONS = 1 << 20
UNIT_EPS = 1e-6                          # under the root of the delta rule's key length
DECAY_SCALE = math.exp(-0.5)             # the decay is exp(-DECAY_SCALE * sigmoid(.))
SINK_SCORE = 0.0                         # the softmax's denominator has exp(0) added
DEFAULT_BIAS_ROWS = 64                   # what the random-weights mode draws where config.json
DEFAULT_DECAY_RANK = 32                  # is silent; a checkpoint's tensors decide


@dataclass
class LosoraxConfig:
    vocab: int
    width: int
    eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Losorax"

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                             "width": self.width, "norm": {"eps": self.eps},
                             "layers": [dict(l) for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d


def _positive_int(where: str, d: Dict[str, Any], key: str) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {v!r}")
    return v


def _number(where: str, d: Dict[str, Any], key: str, positive: bool = False) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{where}: {key} must be a {'positive ' if positive else ''}number, "
                          f"got {v!r}")
    return float(v)


def _check_attention(i: int, m: Dict[str, Any], layers: List[Any]) -> None:
    where = f"layers[{i}].mixer"
    heads = _positive_int(where, m, "heads")
    g = _positive_int(where, m, "kv_heads")
    if heads % g:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({g})")
    for key in ("dim", "vdim", "conv"):
        _positive_int(where, m, key)
    _number(where, m, "scale", positive=True)
    _number(where, m, "bias_max", positive=True)
    qt = m.get("q_temp")
    if not isinstance(qt, dict):
        raise ConfigError(f"{where}: q_temp must be an object with coef and every")
    _number(where + ".q_temp", qt, "coef")
    _positive_int(where + ".q_temp", qt, "every")
    if m.get("bias_rows") is not None:
        _positive_int(where, m, "bias_rows")
    j = m.get("kv_from")
    if j is not None:
        if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
            raise ConfigError(f"{where}: kv_from must name an earlier layer, got {j!r}")
        other = layers[j]
        om = other.get("mixer") if isinstance(other, dict) else None
        if (not isinstance(other, dict) or other.get("type") != "attention"
                or not isinstance(om, dict) or om.get("kv_from") is not None):
            raise ConfigError(f"{where}: kv_from = {j}: that layer stores no keys and values of "
                              "its own")
        for key in ("kv_heads", "dim", "vdim"):
            if om.get(key) != m.get(key):
                raise ConfigError(f"{where}: kv_from = {j}: {key} differs ({om.get(key)!r} there, "
                                  f"{m.get(key)!r} here)")


def _check_mlp(i: int, mlp: Any) -> None:
    where = f"layers[{i}].mlp"
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}.kind must be 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        _positive_int(where, mlp, "ff")
        return
    _positive_int(where + ".expert", mlp.get("expert"), "ff")
    n = _positive_int(where + ".router", mlp.get("router"), "experts")
    top = _positive_int(where + ".router", mlp.get("router"), "top")
    if top > n:
        raise ConfigError(f"{where}.router: top ({top}) exceeds experts ({n})")


def losorax_config_from_dict(raw: Dict[str, Any]) -> LosoraxConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError(f"config.json lacks required keys: {missing}")
    vocab = _positive_int("config", raw, "vocab")
    width = _positive_int("config", raw, "width")
    eps = _number("norm", raw["norm"], "eps", positive=True)
    layers = raw["layers"]
    if not isinstance(layers, list) or not layers:
        raise ConfigError("layers must be a non-empty list")
    for i, layer in enumerate(layers):
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"layers[{i}].type must be one of {MIXER_TYPES}, got "
                              f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"layers[{i}].mixer must be an object")
        if layer["type"] == "attention":
            _check_attention(i, m, layers)
        else:
            _positive_int(f"layers[{i}].mixer", m, "heads")
            _positive_int(f"layers[{i}].mixer", m, "dim")
            if m.get("decay_rank") is not None:
                _positive_int(f"layers[{i}].mixer", m, "decay_rank")
        _check_mlp(i, layer.get("mlp"))
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"max_positions must be a positive integer, got {max_positions!r}")
    return LosoraxConfig(vocab=vocab, width=width, eps=eps, layers=[dict(l) for l in layers],
                         max_positions=max_positions,
                         architecture=str(raw.get("architecture", "Losorax")))


def _mixer_spec(kind: str, m: Dict[str, Any], eps: float) -> PartSpec:
    if kind == "attention":
        own = m.get("kv_from") is None
        return PartSpec("attention", {
            "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "scale": float(m["scale"]), "window": 0,
            "position": {"kind": "none"}, "own_kv": own,
            "conv": {"taps": m["conv"], "q": "mix.q.conv", "k": "mix.k.conv", "v": "mix.v.conv"},
            "head_norm": {"eps": eps},
            "query_gain": {"coef": float(m["q_temp"]["coef"]), "every": int(m["q_temp"]["every"])},
            "distance_bias": {"name": "mix.rel", "far": float(m["bias_max"]),
                              "rows": int(m.get("bias_rows", DEFAULT_BIAS_ROWS))},
            "fixed_sink": SINK_SCORE,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o"}})
    return PartSpec("general_delta_rule", {
        "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["dim"], "eps": eps,
        "unit_eps": UNIT_EPS, "decay_scale": DECAY_SCALE,
        "decay_rank": int(m.get("decay_rank", DEFAULT_DECAY_RANK)),
        "names": {"r": "mix.r", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "a": "mix.a",
                  "a_bias": "mix.a.b", "w1": "mix.w1", "w2": "mix.w2", "w0": "mix.w0",
                  "norm": "mix.norm", "o": "mix.o"}})


def _mlp_spec(mlp: Dict[str, Any]) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp["ff"], "activation": "silu",
                                      "names": {"gate": "mlp.gate", "up": "mlp.up",
                                                "down": "mlp.down"}})
    return PartSpec("routed_experts", {
        "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "intermediate_size": mlp["expert"]["ff"], "activation": "silu", "weight_on": "input",
        "renormalize": False,
        "names": {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up",
                  "down": "mlp.e{e}.down"}})


def build_losorax_spec(cfg: LosoraxConfig) -> ModelSpec:
    def dyt(name: str, gain: str = None) -> PartSpec:
        return PartSpec("dynamic_tanh", {"name": name, **({"gain": gain} if gain else {})})

    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        branches = [BranchSpec("mixer", _mixer_spec(layer["type"], layer["mixer"], cfg.eps),
                               norm=dyt("norm1"), post_norm=dyt("norm1b", "ls1"),
                               shift=PartSpec("token_shift", {"name": "shift"}))]
        if layer.get("mlp") is not None:
            branches.append(BranchSpec("feed_forward", _mlp_spec(layer["mlp"]),
                                       norm=dyt("norm2"), post_norm=dyt("norm2b", "ls2")))
        layers.append(LayerSpec(f"l{i}.", tuple(branches)))
        schedule.append(ScheduleEntry(i, cache=layer["mixer"].get("kv_from")))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {"name": "embed"}),
        layers=layers, schedule=schedule, final_norm=dyt("final.norm"),
        head=PartSpec("linear_head", {"tied": False, "name": "head"}),
        max_positions=cfg.max_positions)


register_architecture("Losorax", losorax_config_from_dict, build_losorax_spec)
