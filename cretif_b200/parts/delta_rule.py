"""The gated delta rule: a linear-attention mixer whose memory is a matrix per head.

Per token, with ``x`` the mixer's input: ``q = W_q x`` and ``k = W_k x`` (kv_heads × dim),
``v = W_v x`` (heads × value_dim); each channel of q, k and v passes a short causal
convolution over time (``taps`` weights, the last one for the present token, zeros before
the sequence's start) and SiLU; q and k are brought to unit length per head and q is scaled
by dim^-1/2.  ``beta = sigmoid(W_b x)`` and ``g = exp(-exp(A_log) · softplus(W_a x + dt_bias))``
are one number per head.  Head h (with the q/k of group h // (heads / kv_heads)) keeps
``M`` [dim, value_dim]:

    M <- g M;   u = beta (v - Mᵀ k);   M <- M + k uᵀ;   o = Mᵀ q

``o`` is RMS-normed per head over value_dim (weight shared by the heads), multiplied by
``silu(W_g x)`` and projected by ``W_o``.  Between steps a sequence keeps M (32-bit) and the
last ``taps - 1`` inputs of every convolved channel: one fixed-size state per cache slot,
zeroed when the slot is handed out.  All six projections are one product whose result stays
in 32-bit, as does everything after it up to the normed output.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear_few as linear


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Part):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``, ``conv_taps``,
    ``eps`` (of the output norm), ``unit_eps`` (under the root of the q/k lengths), ``names``
    (q, k, v, q_conv, k_conv, v_conv, beta, decay, A_log, dt_bias, gate, norm, o)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.vd = int(params["value_dim"])
        self.taps = int(params["conv_taps"])
        self.eps = float(params["eps"])
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        if min(self.nh, self.nkv, self.hd, self.vd, self.taps) <= 0 or self.nh % self.nkv:
            raise ValueError(f"gated_delta_rule: {self.nh} heads cannot share {self.nkv} "
                             "query/key heads, or a size is not positive")
        self.conv_channels = 2 * self.nkv * self.hd + self.nh * self.vd
        self.matrix_floats = self.nh * self.hd * self.vd

    @classmethod
    def weight_specs(cls, params, hidden_size):
        H, G, d, e, K = (params["num_heads"], params["num_kv_heads"], params["head_dim"],
                         params["value_dim"], params["conv_taps"])
        n = params["names"]
        conv = dict(init=(0.0, 0.5))
        return {"q": (n["q"], WeightSpec((G * d, hidden_size))),
                "k": (n["k"], WeightSpec((G * d, hidden_size))),
                "v": (n["v"], WeightSpec((H * e, hidden_size))),
                "gate": (n["gate"], WeightSpec((H * e, hidden_size))),
                "beta": (n["beta"], WeightSpec((H, hidden_size))),
                "decay": (n["decay"], WeightSpec((H, hidden_size))),
                "q_conv": (n["q_conv"], WeightSpec((G * d, K), **conv)),
                "k_conv": (n["k_conv"], WeightSpec((G * d, K), **conv)),
                "v_conv": (n["v_conv"], WeightSpec((H * e, K), **conv)),
                "A_log": (n["A_log"], WeightSpec((H,), init=(0.0, 0.5))),
                "dt_bias": (n["dt_bias"], WeightSpec((H,), init=(0.0, 0.5))),
                "norm": (n["norm"], WeightSpec((e,), init=(1.0, 0.1))),
                "o": (n["o"], WeightSpec((hidden_size, H * e)))}

    def load(self, tensors):
        t = tensors
        # one product: [q | k | v | gate | beta | decay]
        self.w_in = self._matrix(torch.cat([t["q"], t["k"], t["v"], t["gate"], t["beta"],
                                            t["decay"]], dim=0))
        self.conv_w = self._vector32(torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], dim=0))
        self.a_log = self._vector32(t["A_log"])
        self.dt_bias = self._vector32(t["dt_bias"])
        self.norm_w = self._vector32(t["norm"])
        self.w_o = self._matrix(t["o"])

    def cache_request(self):
        return StateRequest((self.matrix_floats + self.conv_channels * (self.taps - 1),),
                            torch.float32)

    def forward(self, x, ctx, cache):
        H, G, d, e, C = self.nh, self.nkv, self.hd, self.vd, self.conv_channels
        T = ctx.T
        proj = linear(x, self.w_in, out_dtype=torch.float32)          # [T, C + H e + 2 H]
        matrices = cache.state[:, :self.matrix_floats]
        inputs = cache.state[:, self.matrix_floats:]
        prep = torch.empty((T, C + 2 * H), dtype=torch.float32, device=x.device)
        ops.delta_prepare(proj, prep, self.conv_w, inputs, self.a_log, self.dt_bias, ctx.tok_pos,
                          ctx.tok_seq, ctx.seq_slot, ctx.seq_start, H, G, d, e, self.unit_eps)
        out = torch.empty((T, H * e), dtype=self.dtype, device=x.device)
        ops.delta_recurrence(prep, proj[:, C:C + H * e], matrices, ctx.cu_seqlens, ctx.seq_slot,
                             ctx.B, H, G, d, e, self.norm_w, self.eps, out,
                             write_state=cache.writes)
        if cache.writes:
            ops.delta_conv_state(proj, inputs, self.taps, C, ctx.cu_seqlens, ctx.seq_slot, ctx.B)
        return linear(out, self.w_o, out_dtype=torch.float32)

    def weight_bytes(self):
        return ((self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()
                + 4 * (self.conv_w.numel() + 2 * self.nh + self.vd))
