"""RMSNorm, fused with the residual addition that precedes it.

``forward(h, delta)`` performs ``h ← h + delta`` in place on the 32-bit residual
stream and returns ``norm(h)`` in the compute dtype, which is the reference's fused
kernel (src/kernels/elementwise.cu:463-506; the plain norm is :30-72).  The weight
multiplies directly unless ``offset`` is given: a checkpoint that stores its norm weights
around zero is read with ``offset = 1`` (the factor is ``offset + w``, added once at loading in
32-bit).  All arithmetic is 32-bit.

``add_into(h, y)`` is the norm on a sublayer's OUTPUT: ``h += norm(y)`` in one kernel, the
normed rows never leaving 32-bit.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: ``eps``; ``name`` (tensor name relative to the prefix); ``offset`` (default 0:
    added to the stored weight)."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        mean = 1.0 - float(params.get("offset", 0.0))
        return {"weight": (params["name"], WeightSpec((hidden_size,), init=(mean, 0.02)))}

    def load(self, tensors):
        self.weight = self._vector32(tensors["weight"])
        offset = float(self.params.get("offset", 0.0))
        if offset:
            self.weight = (self.weight + offset).contiguous()
        self.eps = float(self.params["eps"])

    def rms_params(self):
        """(weight, eps): offered so that a kernel may apply this norm in its own prologue.  A
        norm that offers it promises that its ``forward`` is exactly this RMSNorm."""
        return self.weight, self.eps

    def forward(self, h, delta=None, rows=None, write_h=True):
        R = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((R, h.shape[1]), dtype=self.dtype, device=h.device)
        ops.add_rmsnorm(h, delta, self.weight, out, self.eps, rows=rows,
                        write_h=write_h and rows is None and delta is not None)
        return out

    def add_into(self, h, y, emit: bool = False):
        """``h += norm(y)``: ``y`` [T, H] in float32 or bfloat16, ``h`` the residual stream.
        With ``emit`` (and a compute type other than float32) the new rows are also returned in
        the compute type, for the sublayer that reads the stream next."""
        x = None
        if emit and self.dtype == torch.bfloat16:
            x = torch.empty(h.shape, dtype=self.dtype, device=h.device)
        ops.rmsnorm_add(h, y, self.weight, self.eps, x_out=x)
        return x

    def weight_bytes(self):
        return self.weight.numel() * 4
