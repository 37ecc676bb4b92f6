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


@register_part("mixer", "general_delta_rule")
class GeneralDeltaRule(Part):
    """The generalized delta rule: decay and removal rate per head AND key channel.

    Per token, with ``x`` the mixer's input: ``r = W_r x``, ``k = W_k x`` (heads × dim),
    ``v = W_v x`` (heads × value_dim); decay ``w = exp(-decay_scale · sigmoid(W_w2 tanh(W_w1 x)
    + w0))`` through a low rank (the rank is the stored matrices' shape); removal rate
    ``a = sigmoid(W_a x + a_b)``.  With ``u`` the key of a head at unit length,
    ``u = k / sqrt(|k|² + unit_eps)``, the head keeps ``M`` [dim, value_dim]:

        M <- diag(w) M - (a ⊙ u)(uᵀ M) + k vᵀ      (both products of the old M);   o = Mᵀ r

    ``o`` is divided by its root mean square per head, multiplied by a weight of all heads'
    size and by ``sigmoid(W_g x)``, and projected by ``W_o``.  ``M`` lives in 32-bit per cache
    slot (one ``StateRequest``, zeroed when the slot is handed out).  All six projections are
    one product whose result stays in 32-bit, as does everything after it up to the normed
    output.

    params: ``num_heads``, ``head_dim``, ``value_dim`` (default head_dim), ``eps`` (of the
    output norm), ``unit_eps``, ``decay_scale``, ``decay_rank`` (what the random-weights mode
    draws; a checkpoint's tensors decide), ``names`` (r, k, v, gate, a, a_bias, w1, w2, w0,
    norm, o)."""

    graph_safe = True

    def __init__(self, params, hidden_size, dtype, device):
        super().__init__(params, hidden_size, dtype, device)
        self.nh = int(params["num_heads"])
        self.hd = int(params["head_dim"])
        self.vd = int(params.get("value_dim") or self.hd)
        self.eps = float(params["eps"])
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        self.decay_scale = float(params["decay_scale"])
        if min(self.nh, self.hd, self.vd) <= 0:
            raise ValueError("general_delta_rule: sizes must be positive")
        if self.hd > 256:
            raise ValueError(f"general_delta_rule: head_dim {self.hd} exceeds 256 (a head's "
                             "channels stay in one warp's registers)")
        self.matrix_floats = self.nh * self.hd * self.vd

    @classmethod
    def weight_specs(cls, params, hidden_size):
        H, d = params["num_heads"], params["head_dim"]
        e = params.get("value_dim") or d
        R = int(params.get("decay_rank", 32))
        n = params["names"]
        return {"r": (n["r"], WeightSpec((H * d, hidden_size))),
                "k": (n["k"], WeightSpec((H * d, hidden_size))),
                "v": (n["v"], WeightSpec((H * e, hidden_size))),
                "gate": (n["gate"], WeightSpec((H * e, hidden_size))),
                "a": (n["a"], WeightSpec((H * d, hidden_size))),
                "a_bias": (n["a_bias"], WeightSpec((H * d,), init=(0.0, 0.5))),
                "w1": (n["w1"], WeightSpec((R, hidden_size), free=(0,))),
                "w2": (n["w2"], WeightSpec((H * d, R), init=(0.0, 0.3), free=(1,))),
                "w0": (n["w0"], WeightSpec((H * d,), init=(0.0, 1.0))),
                "norm": (n["norm"], WeightSpec((H * e,), init=(1.0, 0.1))),
                "o": (n["o"], WeightSpec((hidden_size, H * e)))}

    def load(self, tensors):
        t = tensors
        if t["w1"].shape[0] != t["w2"].shape[1]:
            raise ValueError(f"general_delta_rule: the decay's low rank is {t['w1'].shape[0]} in "
                             f"one matrix and {t['w2'].shape[1]} in the other")
        self.rank = int(t["w1"].shape[0])
        # one product: [r | k | v | gate | a | w1]
        self.w_in = self._matrix(torch.cat([t["r"], t["k"], t["v"], t["gate"], t["a"], t["w1"]],
                                           dim=0))
        self.a_bias = self._vector32(t["a_bias"])
        self.w2 = self._matrix(t["w2"])                  # the expanding product's matrix
        self.w0 = self._vector32(t["w0"])
        self.norm_w = self._vector32(t["norm"])
        self.w_o = self._matrix(t["o"])

    def cache_request(self):
        return StateRequest((self.matrix_floats,), torch.float32)

    def forward(self, x, ctx, cache):
        H, d, e = self.nh, self.hd, self.vd
        T = ctx.T
        proj = linear(x, self.w_in, out_dtype=torch.float32)     # [T, 3Hd + 2He + rank]
        prep = torch.empty((T, 3 * H * d), dtype=torch.float32, device=x.device)
        # the decay's low rank: tanh of the narrow projection, expanded by a product of its own
        low = torch.empty((T, self.rank), dtype=self.dtype, device=x.device)
        ops.tanh_cols(proj[:, 3 * H * d + 2 * H * e:], low)
        z = linear(low, self.w2, out_dtype=torch.float32)
        ops.general_delta_prepare(proj, prep, self.a_bias, z, self.w0, H, d, e,
                                  self.unit_eps, self.decay_scale)
        out = torch.empty((T, H * e), dtype=self.dtype, device=x.device)
        gate = proj[:, 2 * H * d + H * e:2 * H * d + 2 * H * e]
        ops.general_delta_recurrence(proj, prep, gate, cache.state, ctx.cu_seqlens, ctx.seq_slot,
                                     ctx.B, H, d, e, self.norm_w, self.eps, out,
                                     per_head_weight=True, gate_sigmoid=True, write_state=True)
        return linear(out, self.w_o, out_dtype=torch.float32)

    def weight_bytes(self):
        return ((self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()
                + self.w2.numel() * self.w2.element_size()
                + 4 * (3 * self.nh * self.hd + self.nh * self.vd))
