"""A plain, slow Rigozen: whole sequences, no cache, one function per mechanism.

The yardstick for the engine's Rigozen parts.  It shares no code with the package: config.json
is read with ``json``, the weights with the ``safetensors`` library, and everything is
elementary torch arithmetic on the CPU in float64 (or float32).

Notation: ``x`` [S, D] is the residual stream of one sequence of S tokens; a linear map is
stored [out, in] and applied as ``x @ W.T``; ``unit(x) = x / sqrt(mean(x**2) + eps)`` over the
last axis.

* block:  ``x += unit(mixer(x)) * (1 + n1)``, then ``x += unit(ff(x)) * (1 + n2)`` -- the
  sublayers read the stream itself and only their outputs are normed;
* three mixers -- windowed attention whose values are its un-normed keys, windowed attention
  over a low-rank latent with a per-head sink in the softmax's denominator, and a gated delta
  rule (a matrix-valued recurrence) behind short causal convolutions;
* feed-forward: ``down(silu(gate x) * (up x))``;
* a layer entry with ``weights_of: j`` runs layer j's tensors once more;
* logits: ``unit(x) * (1 + final) @ embed.T``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List

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
    """x / sqrt(mean(x^2) + eps) over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The block's and the model's norm: the stored weight is an offset from one."""
    return unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit(x, eps) * w


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def window_mask(S: int, size: int) -> torch.Tensor:
    """visible[i, j]: 0 <= i - j < size."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    return (i - j >= 0) & (i - j < size)


def windowed_softmax_attention(q, k, v, scale, size, sink=None):
    """q [S, H, d], k [S, G, d], v [S, G, e] -> [S, H, e].  Head h reads group h // (H/G).
    ``sink`` [H]: an extra term exp(sink_h) in the denominator, with no key, no value and no
    scale."""
    S, H, _ = q.shape
    G = k.shape[1]
    vis = window_mask(S, size)
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~vis, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def mixer_attention(x, W, p, m, eps):
    """Keys double as values; queries and keys are normed over the whole projection."""
    S = x.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = x @ W[p + "q"].T
    k = x @ W[p + "k"].T
    v = k.reshape(S, G, d)                                   # as projected, before the norm
    q = norm_plain(q, W[p + "q.norm"], eps).reshape(S, H, d)
    kn = norm_plain(k, W[p + "k.norm"], eps).reshape(S, G, d)
    o = windowed_softmax_attention(q, kn, v, m["scale"], m["mask"]["size"])
    return o.reshape(S, H * d) @ W[p + "o"].T


def mixer_latent_attention(x, W, p, m, eps):
    S = x.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = (x @ W[p + "q"].T).reshape(S, H, d)
    c = norm_plain(x @ W[p + "dkv"].T, W[p + "dkv.norm"], eps)     # [S, rank]
    k = (c @ W[p + "uk"].T).reshape(S, H, d)
    v = (c @ W[p + "uv"].T).reshape(S, H, e)
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], sink=W[p + "sink"])
    return o.reshape(S, H * e) @ W[p + "o"].T


def causal_conv(z, taps_w):
    """z [S, C], taps_w [C, K]: y[t, c] = sum_i taps_w[c, K-1-i] * z[t-i, c], zeros before 0."""
    S, C = z.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(z)
    for i in range(K):
        shifted = torch.zeros_like(z)
        if i < S:
            shifted[i:] = z[:S - i]
        y = y + shifted * taps_w[:, K - 1 - i]
    return y


def delta_rule(q, k, v, beta, decay):
    """q, k [S, H, d], v [S, H, e], beta, decay [S, H] -> o [S, H, e]; state M [d, e] per head,
    zero at the start: M <- decay M; u = beta (v - M^T k); M <- M + k u^T; o = M^T q."""
    S, H, d = q.shape
    e = v.shape[-1]
    o = torch.zeros(S, H, e, dtype=q.dtype)
    for h in range(H):
        M = torch.zeros(d, e, dtype=q.dtype)
        for t in range(S):
            M = decay[t, h] * M
            u = beta[t, h] * (v[t, h] - M.T @ k[t, h])
            M = M + torch.outer(k[t, h], u)
            o[t, h] = M.T @ q[t, h]
    return o


def mixer_delta(x, W, p, m, eps):
    S = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(x @ W[p + "q"].T, W[p + "q.conv"])).reshape(S, G, d)
    k = silu(causal_conv(x @ W[p + "k"].T, W[p + "k.conv"])).reshape(S, G, d)
    v = silu(causal_conv(x @ W[p + "v"].T, W[p + "v.conv"])).reshape(S, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)                      # head h uses group h // rep
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(x @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(x @ W[p + "a"].T + W[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    o = unit(o, eps) * W[p + "norm"]                         # per head, over e
    o = o * silu(x @ W[p + "g"].T).reshape(S, H, e)
    return o.reshape(S, H * e) @ W[p + "o"].T


MIXERS = {"attention": mixer_attention, "latent_attention": mixer_latent_attention,
          "delta": mixer_delta}


def feed_forward(x, W, p):
    return (silu(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            streams=None) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence.  ``streams``, a list, receives the residual
    stream after every layer run."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = torch.stack([W["embed"][i] for i in ids])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        y = MIXERS[layer["type"]](x, W, p + "mix.", layer["mixer"], eps)
        x = x + norm_around_zero(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(x, W, p + "mlp.")
            x = x + norm_around_zero(y, W[p + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return norm_around_zero(x, W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        logits = forward(cfg, weights, ids, dtype)[-1]
        best = int(torch.nonzero(logits == logits.max())[0])
        out.append(best)
        ids.append(best)
    return out
