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


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Part):
    """A norm without statistics: ``tanh(alpha x) * w + b`` element by element, with one learned
    scalar ``alpha``.  params: ``name`` (the weight; the offset and the scalar are stored beside
    it as ``<name>.b`` and ``<name>.alpha``); ``gain`` (optional: name of a per-channel factor
    on the result, a layer scale).  It has ``forward`` and ``add_into`` like the RMS norm, and
    offers ``pointwise_params()``: a promise that every element is normed on its own, so that a
    kernel may apply the norm to single rows wherever it reads them."""

    graph_safe = True

    @classmethod
    def weight_specs(cls, params, hidden_size):
        n = params["name"]
        out = {"weight": (n, WeightSpec((hidden_size,), init=(1.0, 0.1))),
               "bias": (n + ".b", WeightSpec((hidden_size,), init=(0.0, 0.1))),
               "alpha": (n + ".alpha", WeightSpec((), init=(0.7, 0.1)))}
        if params.get("gain"):
            out["gain"] = (params["gain"], WeightSpec((hidden_size,), init=(0.5, 0.1)))
        return out

    def load(self, tensors):
        self.weight = self._vector32(tensors["weight"])
        self.bias = self._vector32(tensors["bias"])
        self.alpha = self._vector32(tensors["alpha"].reshape(1))
        self.gain = self._vector32(tensors["gain"]) if "gain" in tensors else None

    def pointwise_params(self):
        """(weight, bias, alpha) when nothing else is applied (no gain), else None."""
        return None if self.gain is not None else (self.weight, self.bias, self.alpha)

    def forward(self, h, delta=None, rows=None, write_h=True):
        R = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((R, h.shape[1]), dtype=self.dtype, device=h.device)
        ops.dyt_rows(h, delta, self.weight, self.bias, self.alpha, out, gain=self.gain, rows=rows,
                     write_h=write_h)
        return out

    def add_into(self, h, y, emit: bool = False):
        """``h += norm(y)`` in one 32-bit kernel.  Nothing is returned: the next reader of the
        stream stands behind a norm of its own."""
        ops.dyt_add(h, y, self.weight, self.bias, self.alpha, gain=self.gain)
        return None

    def weight_bytes(self):
        return 4 * (2 + (self.gain is not None)) * self.weight.numel() + 4
