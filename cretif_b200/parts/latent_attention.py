"""Attention over a cached low-rank latent, with a sliding window and a softmax sink.

Per token the layer projects queries ``q = W_q x`` (heads × dim) and a latent
``c = rmsnorm(W_down x)`` of ``latent_rank`` numbers; head h's keys and values are
``k = W_uk[h] c`` and ``v = W_uv[h] c``.  Only ``c`` is cached.  The kernels never expand it:

    score  = q_h · (W_uk[h] c) = (W_uk[h]ᵀ q_h) · c        -> the query is moved into latent space
    out_h  = Σ p (W_uv[h] c)   = W_uv[h] (Σ p c)           -> the values are expanded once, after

so the attention itself is multi-query attention with ONE key/value head of size
``latent_rank`` whose keys and values are the same cached rows, and every attention kernel
of the library serves it as it is.  The two per-head products around it are one batched launch
each.  The softmax's denominator holds one more term ``exp(sink_h)`` per head, unscaled, with
no key and no value; there is no position encoding.
"""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..csrc import ops
from ..weights.loader import WeightSpec
from .attention import run_attention
from .base import Part, register_part
from .linear import linear_few as linear


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: ``num_heads``, ``head_dim`` (query/key size per head), ``value_dim``,
    ``latent_rank``, ``scale``, ``window`` (0 = all keys), ``eps`` (of the latent's norm),
    ``names`` (q, down, down_norm, up_k, up_v, o and, optionally, sink)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.hd = int(params["head_dim"])
        self.vd = int(params["value_dim"])
        self.rank = int(params["latent_rank"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        self.eps = float(params["eps"])
        if min(self.nh, self.hd, self.vd, self.rank) <= 0:
            raise ValueError("latent_attention: sizes must be positive")
        if self.rank > 512:
            raise ValueError(f"latent_attention: latent_rank {self.rank} is above 512; the "
                             "attention kernels take no larger head")
        self.sink = None

    @classmethod
    def weight_specs(cls, params, hidden_size):
        H, d, e, r = (params["num_heads"], params["head_dim"], params["value_dim"],
                      params["latent_rank"])
        n = params["names"]
        out = {"q": (n["q"], WeightSpec((H * d, hidden_size))),
               "down": (n["down"], WeightSpec((r, hidden_size))),
               "down_norm": (n["down_norm"], WeightSpec((r,), init=(1.0, 0.1))),
               "up_k": (n["up_k"], WeightSpec((H * d, r))),
               "up_v": (n["up_v"], WeightSpec((H * e, r))),
               "o": (n["o"], WeightSpec((hidden_size, H * e)))}
        if n.get("sink"):
            out["sink"] = (n["sink"], WeightSpec((H,), init=(0.0, 1.0)))
        return out

    def load(self, tensors):
        H, d, e, r = self.nh, self.hd, self.vd, self.rank
        self.w_in = self._matrix(torch.cat([tensors["q"], tensors["down"]], dim=0))  # [q | c]
        # W_uk[h] is [d, r]; the query goes to latent space through its transpose [r, d]
        self.w_q_latent = self._matrix(tensors["up_k"].reshape(H, d, r).transpose(1, 2))
        self.w_up_v = self._matrix(tensors["up_v"].reshape(H, e, r))
        self.w_o = self._matrix(tensors["o"])
        self.down_norm = self._vector32(tensors["down_norm"])
        if "sink" in tensors:
            self.sink = self._vector32(tensors["sink"])

    def cache_request(self):
        return KVRequest(1, self.rank, self.window, shared_values=True)

    def forward(self, x, ctx, cache):
        H, d, e, r, T = self.nh, self.hd, self.vd, self.rank, ctx.T
        kv = cache.kv
        qc = linear(x, self.w_in)                                   # [T, H d + r]
        # the latent is normed and stored as the one key/value head; q is left as it is
        ops.proj_norm_kv_append(qc, H * d, None, 1, r, self.down_norm, self.eps, ctx.tok_pos,
                                ctx.tok_seq, ctx.seq_slot, kv.table, kv.k, None, kv.block_tokens,
                                cache.writes, ctx.fault)
        q_lat = torch.empty((T, H, r), dtype=self.dtype, device=x.device)
        ops.gemm_batched(qc[:, :H * d].unflatten(1, (H, d)), self.w_q_latent, q_lat)
        o_lat = torch.empty((T, H * r), dtype=self.dtype, device=x.device)
        run_attention(q_lat.view(T, H * r), o_lat, ctx, kv, H, 1, r, self.scale, self.window,
                      self.dtype, self.sink)
        o = torch.empty((T, H, e), dtype=self.dtype, device=x.device)
        ops.gemm_batched(o_lat.view(T, H, r), self.w_up_v, o)
        return linear(o.view(T, H * e), self.w_o, out_dtype=torch.float32)

    def weight_bytes(self):
        n = (self.w_in.numel() + self.w_q_latent.numel() + self.w_up_v.numel()
             + self.w_o.numel())
        return n * self.w_o.element_size()
