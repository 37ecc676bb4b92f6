"""Token shift: what a sublayer reads is blended, channel by channel, with what the token
before it read.

``x_t = n_t + (n_{t-1} - n_t) * shift`` where ``n`` are the normed rows as they were before the
blend and ``shift`` is a learned vector; before a sequence's first token stands a row of zeros.
The last normed row of a sequence is kept per cache slot between steps (one ``StateRequest`` of
the residual width, zeroed when the slot is handed out), so a step that continues a sequence —
a further portion of a prompt or a single token — starts from the row the step before left.

The part stands between a branch's norm and its part (``BranchSpec.shift``).  With a norm that
offers ``pointwise_params()`` the norm and the blend are one kernel that reads the residual
stream; with any other norm the normed rows are computed first (in 32-bit) and blended then.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part


@register_part("shift", "token_shift")
class TokenShift(Part):
    """params: ``name`` (the blend vector, relative to the layer's prefix)."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        return {"shift": (params["name"], WeightSpec((hidden_size,), init=(0.5, 0.25)))}

    def load(self, tensors):
        self.shift = self._vector32(tensors["shift"])

    def cache_request(self):
        return StateRequest((self.hidden_size,), torch.float32)

    def forward(self, h, norm, ctx, state):
        """``h`` [T, H]: the float32 residual stream (with ``norm``) or rows that are normed
        already (``norm`` None); returns the blended rows in the compute type and leaves each
        sequence's last normed row in ``state``."""
        out = torch.empty(h.shape, dtype=self.dtype, device=h.device)
        point = getattr(norm, "pointwise_params", None)
        point = point() if point is not None else None
        if norm is not None and point is None:
            # any other norm: its rows in 32-bit first
            if norm.dtype != torch.float32:
                raise ValueError("token_shift: a norm that is not pointwise must run in float32 "
                                 "in front of the shift")
            h, point = norm.forward(h, None), None
        w, b, alpha = point if point is not None else (None, None, None)
        ops.shift_rows(h, self.shift, state, ctx.tok_seq, ctx.seq_slot, ctx.cu_seqlens, out,
                       weight=w, bias=b, alpha=alpha)
        return out

    def weight_bytes(self):
        return 4 * self.shift.numel()
