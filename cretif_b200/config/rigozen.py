"""Typed configuration of the Rigozen decoder, read from config.json, and its ModelSpec.

A Rigozen checkpoint's config.json names its class with ``"architecture": "Rigozen"`` and
describes the model as a list of layers, each with a mixer of its own kind and sizes:

=====================  ========================================================================
key                    meaning
=====================  ========================================================================
vocab, width           vocabulary and residual width
norm.eps               eps of every RMS norm of the model
layers[i].type         ``attention`` | ``latent_attention`` | ``delta``
layers[i].mixer        the mixer's sizes: heads, kv_heads, dim, vdim, scale, mask.size (window),
                       kv_rank (latent), conv (taps of the delta rule's convolutions)
layers[i].mlp          ``{"kind": "dense", "ff": F}`` or null for a layer without feed-forward
layers[i].weights_of   j: the layer has no tensors, it runs layer j's once more with a cache
                       or state of its own
max_positions          (optional) longest sequence; the design itself has no limit
=====================  ========================================================================

The block norms its sublayers' OUTPUTS, ``x += norm(mixer(x))`` then ``x += norm(ff(x))``, with
weights stored around zero (factor 1 + w); the sublayers read the stream itself.  Tensors are
named ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.norm1/2``, ``embed`` (also the output matrix) and
``final.norm``.  The three mixers map to the parts ``attention`` (with the norm over whole
projections and the keys as values), ``latent_attention`` and ``gated_delta_rule``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import BranchSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_TYPES = ("attention", "latent_attention", "delta")
DEFAULT_MAX_POSITIONS = 1 << 20         # the design has no limit; this bounds the cache's tables
UNIT_EPS = 1e-6                         # under the root of the delta rule's q/k lengths


@dataclass
class RigozenConfig:
    vocab: int
    width: int
    eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Rigozen"

    def source_of(self, i: int) -> int:
        """The layer whose tensors layer ``i`` uses (itself unless it borrows)."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                             "width": self.width, "norm": {"eps": self.eps},
                             "layers": [dict(l) for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d


def _positive_int(where: str, d: Dict[str, Any], key: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: {key} must be a positive integer, got {v!r}")
    return v


def _check_mixer(i: int, kind: str, m: Dict[str, Any]) -> None:
    where = f"layers[{i}].mixer"
    if not isinstance(m, dict):
        raise ConfigError(f"{where} must be an object")
    heads = _positive_int(where, m, "heads")
    _positive_int(where, m, "dim")
    _positive_int(where, m, "vdim")
    if kind in ("attention", "delta"):
        g = _positive_int(where, m, "kv_heads")
        if heads % g:
            raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({g})")
    if kind in ("attention", "latent_attention"):
        if m.get("mask") is not None:               # no mask: every earlier key is seen
            if not isinstance(m["mask"], dict):
                raise ConfigError(f"{where}: mask must be an object with a size")
            _positive_int(where + ".mask", m["mask"], "size")
        if m.get("scale") is not None and (not isinstance(m["scale"], (int, float))
                                           or isinstance(m["scale"], bool) or not m["scale"] > 0):
            raise ConfigError(f"{where}: scale must be a positive number, got {m['scale']!r}")
    if kind == "attention" and m["vdim"] != m["dim"]:
        raise ConfigError(f"{where}: the values of this mixer are its keys, so vdim "
                          f"({m['vdim']}) must equal dim ({m['dim']})")
    if kind == "latent_attention":
        _positive_int(where, m, "kv_rank")
    if kind == "delta":
        _positive_int(where, m, "conv")


def rigozen_config_from_dict(raw: Dict[str, Any]) -> RigozenConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError(f"config.json lacks required keys: {missing}")
    vocab = _positive_int("config", raw, "vocab")
    width = _positive_int("config", raw, "width")
    norm = raw["norm"]
    if not isinstance(norm, dict) or not isinstance(norm.get("eps"), (int, float)) \
            or not norm["eps"] > 0:
        raise ConfigError(f"norm.eps must be a positive number, got {norm!r}")
    layers = raw["layers"]
    if not isinstance(layers, list) or not layers:
        raise ConfigError("layers must be a non-empty list")
    for i, layer in enumerate(layers):
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"layers[{i}].type must be one of {MIXER_TYPES}, got "
                              f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
        _check_mixer(i, layer["type"], layer.get("mixer"))
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"layers[{i}].mlp.kind must be 'dense', got {mlp!r}")
            _positive_int(f"layers[{i}].mlp", mlp, "ff")
        j = layer.get("weights_of")
        if j is not None:
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(layers) or j == i:
                raise ConfigError(f"layers[{i}].weights_of must name another layer, got {j!r}")
            other = layers[j]
            if not isinstance(other, dict) or other.get("weights_of") is not None:
                raise ConfigError(f"layers[{i}].weights_of = {j}: that layer has no tensors of "
                                  "its own")
            if layer.get("type") != other.get("type"):
                raise ConfigError(f"layers[{i}] uses the tensors of layer {j} but describes "
                                  "another layer")
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"max_positions must be a positive integer, got {max_positions!r}")
    return RigozenConfig(vocab=vocab, width=width, eps=float(norm["eps"]),
                         layers=[dict(l) for l in layers], max_positions=max_positions,
                         architecture=str(raw.get("architecture", "Rigozen")))


def _mixer_spec(kind: str, m: Dict[str, Any], eps: float) -> PartSpec:
    if kind != "delta":
        m = dict(m)
        m["mask"] = {"size": (m.get("mask") or {}).get("size", 0)}       # 0: all keys
        if m.get("scale") is None:
            m["scale"] = m["dim"] ** -0.5
    if kind == "attention":
        return PartSpec("attention", {
            "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "scale": float(m["scale"]), "window": m["mask"]["size"],
            "position": {"kind": "none"}, "values": "keys",
            "qk_norm": {"eps": eps, "q": "mix.q.norm", "k": "mix.k.norm"},
            "names": {"q": "mix.q", "k": "mix.k", "o": "mix.o"}})
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
            "latent_rank": m["kv_rank"], "scale": float(m["scale"]),
            "window": m["mask"]["size"], "eps": eps,
            "names": {"q": "mix.q", "down": "mix.dkv", "down_norm": "mix.dkv.norm",
                      "up_k": "mix.uk", "up_v": "mix.uv", "sink": "mix.sink", "o": "mix.o"}})
    return PartSpec("gated_delta_rule", {
        "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "conv_taps": m["conv"], "eps": eps, "unit_eps": UNIT_EPS,
        "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "q_conv": "mix.q.conv",
                  "k_conv": "mix.k.conv", "v_conv": "mix.v.conv", "beta": "mix.b",
                  "decay": "mix.a", "A_log": "mix.A_log", "dt_bias": "mix.dt_bias",
                  "gate": "mix.g", "norm": "mix.norm", "o": "mix.o"}})


def build_rigozen_spec(cfg: RigozenConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"eps": cfg.eps, "name": name, "offset": 1.0})

    layers: List[LayerSpec] = []
    index_of: Dict[int, int] = {}            # config layer -> index among the layers with tensors
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        branches = [BranchSpec("mixer", _mixer_spec(layer["type"], layer["mixer"], cfg.eps),
                               post_norm=norm("norm1"))]
        mlp: Optional[Dict[str, Any]] = layer.get("mlp")
        if mlp is not None:
            ff = PartSpec("gated_mlp", {"intermediate_size": mlp["ff"], "activation": "silu",
                                        "names": {"gate": "mlp.gate", "up": "mlp.up",
                                                  "down": "mlp.down"}})
            branches.append(BranchSpec("feed_forward", ff, post_norm=norm("norm2")))
        index_of[i] = len(layers)
        layers.append(LayerSpec(f"l{i}.", tuple(branches)))
    schedule = [ScheduleEntry(index_of[cfg.source_of(i)]) for i in range(len(cfg.layers))]
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {"name": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"tied": True, "name": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions)


register_architecture("Rigozen", rigozen_config_from_dict, build_rigozen_spec)
