"""Dense feed-forwards.  SwiGLU: down( silu(gate x) * (up x) ), with or without biases; plain: down( relu(up x)^2 )
(reference: crates/ferrox-moe/src/lib.rs:655-658; decoder.rs:2902-2913)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, register_part


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows ; up rows]: one product yields [gate | up] per token."""
    dt = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
    return torch.cat([gate.to(dt), up.to(dt)], dim=0).contiguous()


class SwigluMlp(FeedForward):
    """down( act(gate x) * (up x) ); ``spec.activation`` names act (SiLU unless the spec says ReLU).  With
    ``spec.bias_names`` every projection has a bias: down( act(gate x + bg) * (up x + bu) ) + bd; the products'
    epilogues add them."""

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.activation = getattr(spec, "activation", "silu")
        ops.gate_code(self.activation)   # an unknown activation fails here, by name
        names = getattr(spec, "tensor_names", None) or ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        self._gate, self._up, self._down = (spec.prefix + n for n in names)
        biases = getattr(spec, "bias_names", None)
        self._biases = tuple(spec.prefix + n for n in biases) if biases else None

    def tensor_decls(self):
        s = self.spec
        d = [
            TensorDecl(self._gate, (s.intermediate, s.hidden)),
            TensorDecl(self._up, (s.intermediate, s.hidden)),
            TensorDecl(self._down, (s.hidden, s.intermediate)),
        ]
        if self._biases:
            d += [TensorDecl(self._biases[0], (s.intermediate,)), TensorDecl(self._biases[1], (s.intermediate,)),
                  TensorDecl(self._biases[2], (s.hidden,))]
        return d

    def load(self, src, rt):
        super().load(src, rt)
        self.w_gu = pack_gate_up(src.get(self._gate), src.get(self._up))
        self.w_down = src.get(self._down)
        self.b_gu = self.b_down = None
        if self._biases:
            bg, bu = src.get(self._biases[0]), src.get(self._biases[1])
            dt = torch.float32 if torch.float32 in (bg.dtype, bu.dtype) else bg.dtype
            self.b_gu = torch.cat([bg.to(dt), bu.to(dt)]).contiguous()
            self.b_down = src.get(self._biases[2])

    def forward_add(self, x, h, batch):
        self.forward_into(x, h, batch, accumulate=True)

    def forward_into(self, x, out, batch, accumulate=False):
        T, I = x.shape[0], self.spec.intermediate
        act = self.rt.empty(T, I)
        # act(gate (+ bias)) * (up (+ bias)) in the epilogue
        ops.gated_linear(x, self.w_gu, act, status=batch.status, stream=batch.stream, activation=self.activation,
                         bias=self.b_gu)
        ops.linear(act, self.w_down, out, bias=self.b_down, accumulate=accumulate, status=batch.status,
                   stream=batch.stream)


class PlainMlp(FeedForward):
    """down(act(up x)) without a gate; act = the square of ReLU, in the first product's epilogue where its kernel has
    one (in place on the rows it wrote otherwise)."""

    graph_safe = True
    ACTIVATIONS = ("relu_square",)

    def __init__(self, spec):
        super().__init__(spec)
        if spec.activation not in self.ACTIVATIONS:
            raise ValueError(f"plain_mlp activation {spec.activation!r}: known: {', '.join(self.ACTIVATIONS)}")
        names = getattr(spec, "tensor_names", None) or ("up", "down")
        self._up, self._down = (spec.prefix + n for n in names)

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(self._up, (s.intermediate, s.hidden)), TensorDecl(self._down, (s.hidden, s.intermediate))]

    def load(self, src, rt):
        super().load(src, rt)
        self.w_up = src.get(self._up)
        self.w_down = src.get(self._down)

    def forward_add(self, x, h, batch):
        self.forward_into(x, h, batch, accumulate=True)

    def forward_into(self, x, out, batch, accumulate=False):
        act = self.rt.empty(x.shape[0], self.spec.intermediate)
        ops.linear(x, self.w_up, act, status=batch.status, stream=batch.stream, activation=self.spec.activation)
        ops.linear(act, self.w_down, out, accumulate=accumulate, status=batch.status, stream=batch.stream)


register_part("swiglu_mlp", SwigluMlp, replace=True)
register_part("plain_mlp", PlainMlp, replace=True)
