"""A plain, slow Losorax: whole sequences, no cache, one function per mechanism.

The yardstick for the engine's Losorax parts.  It shares no code with the package: config.json
is read with ``json``, the weights with the ``safetensors`` library, and everything is
elementary torch arithmetic on the CPU in float64 (or float32).

Notation: ``x`` [S, D] is the residual stream of one sequence of S tokens; a linear map is
stored [out, in] and applied as ``x @ W.T``; ``unit(x) = x / sqrt(mean(x**2) + eps)`` over the
last axis.

* norm: ``dyt(x) = tanh(alpha x) * w + b`` (no statistics);
* block: ``x += ls1 * dyt_1b(mixer(mix(dyt_1(x))))`` then ``x += ls2 * dyt_2b(ff(dyt_2(x)))``
  where ``mix(h)_t = h_t + (h_{t-1} - h_t) * shift`` blends each row with the row before it
  (zeros before the first);
* two mixers -- causal attention behind short convolutions with a bucketed distance bias, a
  position-dependent query gain and a softmax whose denominator has one added, and a
  generalized delta rule whose state is a matrix per head;
* feed-forward: SwiGLU, dense or routed over small experts whose INPUT is scaled by the
  router's sigmoid score;
* logits: ``dyt_final(x) @ head.T``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def read_model_folder(model_dir: str):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(torch.float64)
    return cfg, weights


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dyt(x, W, name):
    """tanh(alpha x) * w + b with the scalar and the offset stored beside the weight."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def blend_with_previous(h, shift):
    """Row t becomes h_t + (h_{t-1} - h_t) * shift, with the rows as they were before."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * shift


def causal_conv(z, taps_w):
    """z [S, C], taps_w [C, K]: y_t = sum_j taps_w[:, j] * z_{t-K+1+j}, zeros before the start."""
    S, C = z.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=z.dtype), z], dim=0)
    y = torch.zeros_like(z)
    for j in range(K):
        y = y + padded[j:j + S] * taps_w[:, j]
    return y


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Distances below rows/2 have a row each; beyond, rows are spaced by the logarithm up to
    ``far``, and the last row takes everything farther."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half)
                                               * (rows - half))))


def query_gain(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def attention_scores_to_output(q, k, v, scale, rel, far, gains):
    """q [S, H, d], k [S, G, d], v [S, G, e]; rel [rows, H].  Causal; the softmax's denominator
    has one added (a slot with score 0 and no value)."""
    S, H, d = q.shape
    G = k.shape[1]
    rows = rel.shape[0]
    out = torch.zeros(S, H, v.shape[2], dtype=q.dtype)
    bucket = torch.tensor([distance_bucket(n, rows, far) for n in range(S)])
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] * gains[:, None]) @ k[:, g].T * scale                  # [S, S]
        i = torch.arange(S)
        dist = i[:, None] - i[None, :]
        s = s + rel[bucket[dist.clamp(min=0)], h]
        s = s.masked_fill(dist < 0, float("-inf"))
        m = torch.clamp(s.max(dim=1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(dim=1, keepdim=True))
        out[:, h] = p @ v[:, g]
    return out


def attention_keys_values(x, W, p, m, eps):
    """What a layer caches: keys after convolution and unit norm, values after convolution."""
    S = x.shape[0]
    G, d, e = m["kv_heads"], m["dim"], m["vdim"]
    k = causal_conv(x @ W[p + "k"].T, W[p + "k.conv"]).reshape(S, G, d)
    v = causal_conv(x @ W[p + "v"].T, W[p + "v.conv"]).reshape(S, G, e)
    return unit(k, eps), v


def mixer_attention(x, W, p, m, eps, kv=None):
    S = x.shape[0]
    H, d = m["heads"], m["dim"]
    q = unit(causal_conv(x @ W[p + "q"].T, W[p + "q.conv"]).reshape(S, H, d), eps)
    k, v = kv if kv is not None else attention_keys_values(x, W, p, m, eps)
    gains = torch.tensor([query_gain(t, m["q_temp"]["coef"], m["q_temp"]["every"])
                          for t in range(S)], dtype=x.dtype)
    o = attention_scores_to_output(q, k, v, m["scale"], W[p + "rel"], m["bias_max"], gains)
    return o.reshape(S, -1) @ W[p + "o"].T


def general_delta_rule(r, k, v, w, a):
    """r, k, w, a [S, H, d], v [S, H, e].  Per head, with u the key at unit length:
    M <- diag(w) M - (a u)(u^T M) + k v^T (both products of the old M);  o = M^T r."""
    S, H, d = k.shape
    e = v.shape[2]
    M = torch.zeros(H, d, e, dtype=k.dtype)
    out = torch.zeros(S, H, e, dtype=k.dtype)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    for t in range(S):
        uM = torch.einsum("hd,hde->he", u[t], M)
        M = (w[t][:, :, None] * M - (a[t] * u[t])[:, :, None] * uM[:, None, :]
             + k[t][:, :, None] * v[t][:, None, :])
        out[t] = torch.einsum("hde,hd->he", M, r[t])
    return out


def mixer_general_delta(x, W, p, m, eps):
    S = x.shape[0]
    H, d = m["heads"], m["dim"]
    r = (x @ W[p + "r"].T).reshape(S, H, d)
    k = (x @ W[p + "k"].T).reshape(S, H, d)
    v = (x @ W[p + "v"].T).reshape(S, H, d)
    w = torch.exp(-math.exp(-0.5) * sigmoid(torch.tanh(x @ W[p + "w1"].T) @ W[p + "w2"].T
                                            + W[p + "w0"])).reshape(S, H, d)
    a = sigmoid(x @ W[p + "a"].T + W[p + "a.b"]).reshape(S, H, d)
    o = unit(general_delta_rule(r, k, v, w, a), eps).reshape(S, H * d)
    return (o * W[p + "norm"] * sigmoid(x @ W[p + "g"].T)) @ W[p + "o"].T


def swiglu(x, W, p):
    return (silu(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def routed_experts(x, W, p, mlp):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(x @ W[p + "router"].T)                                     # [S, n]
    best = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for score, e in zip(best.values[t], best.indices[t]):
            out[t] += swiglu((score * x[t])[None], W, f"{p}e{int(e)}.")[0]
    return out


def feed_forward(x, W, p, mlp):
    if mlp["kind"] == "dense":
        return swiglu(x, W, p)
    return routed_experts(x, W, p, mlp)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [S, vocab] of one sequence; ``streams`` collects the residual after each layer."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(ids, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = blend_with_previous(dyt(x, W, p + "norm1"), W[p + "shift"])
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, W, p + "mix.", m, eps)
            y = mixer_attention(h, W, p + "mix.", m, eps, kv=kept[i if src is None else src])
        else:
            y = mixer_general_delta(h, W, p + "mix.", m, eps)
        x = x + W[p + "ls1"] * dyt(y, W, p + "norm1b")
        if layer.get("mlp") is not None:
            y = feed_forward(dyt(x, W, p + "norm2"), W, p + "mlp.", layer["mlp"])
            x = x + W[p + "ls2"] * dyt(y, W, p + "norm2b")
        if streams is not None:
            streams.append(x.clone())
    return dyt(x, W, "final.norm") @ W["head"].T


def greedy(cfg, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, weights, ids, dtype)[-1].argmax()))
    return ids[len(prompt):]
