"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in 32 bits
(reference: crates/ferrox-core/src/matmul.rs:62-69,121-123)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Norm, register_part


class RmsNorm(Norm):
    """``one_plus``: the stored weight lies around zero and the norm multiplies by 1 + w (added once, in 32 bits,
    when the weights are loaded)."""

    graph_safe = True

    def _name(self):
        return getattr(self.spec, "name", None) or self.spec.prefix + "weight"

    def tensor_decls(self):
        one_plus = getattr(self.spec, "one_plus", False)
        return [TensorDecl(self._name(), (self.spec.size,), init="normal" if one_plus else "ones")]

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self._name())
        if getattr(self.spec, "one_plus", False):
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def forward(self, h, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.spec.size)
        return ops.rmsnorm(h, self.weight, self.spec.eps, out, rows=rows)


    def as_rms(self):
        return self.weight, self.spec.eps


class LayerNorm(Norm):
    """(x - mean) / sqrt(variance + eps) * w (+ b), the variance being the mean of the squared deviations; a weight
    and, where the spec names one, a bias; statistics in 32 bits."""

    graph_safe = True

    def _bias_name(self):
        return getattr(self.spec, "bias_name", None)

    def tensor_decls(self):
        d = [TensorDecl(self.spec.name, (self.spec.size,), init="ones")]
        if self._bias_name():
            d.append(TensorDecl(self._bias_name(), (self.spec.size,)))
        return d

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self.spec.name)
        self.bias = src.get(self._bias_name()) if self._bias_name() else None

    def forward(self, h, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.spec.size)
        return ops.layernorm(h, self.weight, self.spec.eps, out, rows=rows, bias=self.bias)

    def forward_in_place(self, h):
        """The 32-bit stream normed where it lies."""
        return ops.layernorm(h, self.weight, self.spec.eps, h, bias=self.bias)

    def as_layer_norm(self):
        """(weight, eps) for a kernel that applies the norm itself; None with a bias, which those kernels lack."""
        return (self.weight, self.spec.eps) if self.bias is None else None


register_part("rms_norm", RmsNorm, replace=True)
register_part("layer_norm", LayerNorm, replace=True)
