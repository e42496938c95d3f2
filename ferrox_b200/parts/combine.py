"""Mixers made of mixers.  ``input_conv``: a mixer behind a short causal convolution of its input (see
:class:`InputConv`).  ``mixer_sum``: several mixers side by side: all read the same input and the result is the
weighted sum of their outputs,

    y = sum_i scales[i] * mixers[i](x)

Each keeps its own cache needs: at most one of them may ask for pages (the layer has one block table), and the
states of all are named tensors of the layer's one state block, under ``<index>.<name>``.  The sum itself is not
made here when the block norms the mixer's output before adding it: the block's norm kernel takes the outputs
and their scales (:meth:`MixerSum.forward_parts`); ``forward_add`` serves blocks that add directly.
"""
from __future__ import annotations

from dataclasses import replace

import torch

from ..cache.specs import CacheSpec, StateSpec
from ..kernels import ops
from .base import Mixer, build_part, register_part


class MixerSum(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        if len(spec.mixers) != len(spec.scales) or not spec.mixers:
            raise ValueError("mixer_sum: one scale per mixer, at least one mixer")
        self.mixers = [build_part(m) for m in spec.mixers]
        self.scales = [float(x) for x in spec.scales]

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.mixers)

    def tensor_decls(self):
        return [d for m in self.mixers for d in m.tensor_decls()]

    def load(self, src, rt):
        super().load(src, rt)
        for m in self.mixers:
            m.load(src, rt)

    def reset_after_fault(self):
        for m in self.mixers:
            m.reset_after_fault()

    def cache_spec(self):
        paged, parts, dtype = None, [], torch.float32
        for i, m in enumerate(self.mixers):
            cs = m.cache_spec()
            if cs is None:
                continue
            if cs.paged is not None:
                if paged is not None:
                    raise ValueError("mixer_sum: only one of the mixers may keep pages")
                paged = cs.paged
            if cs.state is not None:
                own = cs.state.parts or (("state", cs.state.shape),)
                parts += [(f"{i}.{name}", shape) for name, shape in own]
                dtype = cs.state.dtype
        if paged is None and not parts:
            return None
        return CacheSpec(paged=paged, state=StateSpec(parts=tuple(parts), dtype=dtype) if parts else None)

    def _view(self, i, cache):
        """The layer's cache as mixer i sees it: its own state tensors under their own names."""
        pre = f"{i}."
        own = {n[len(pre):]: t for n, t in (cache.states or {}).items() if n.startswith(pre)}
        return replace(cache, states=own or None, state=own.get("state"))

    def forward_parts(self, x, batch, cache):
        """[(32-bit output of mixer i, scale i)]: for a caller that sums them itself."""
        outs = []
        for i, m in enumerate(self.mixers):
            y = self.rt.empty(x.shape[0], self.spec_hidden(m), dtype=torch.float32)
            m.forward_into(x, y, batch, self._view(i, cache), accumulate=False)
            outs.append((y, self.scales[i]))
        return outs

    @staticmethod
    def spec_hidden(m):
        return m.spec.hidden

    def forward_add(self, x, h, batch, cache):
        for i, m in enumerate(self.mixers):
            if self.scales[i] == 1.0:
                m.forward_add(x, h, batch, self._view(i, cache))
            else:
                y = self.rt.empty(x.shape[0], h.shape[1], dtype=torch.float32)
                m.forward_into(x, y, batch, self._view(i, cache), accumulate=False)
                ops.scale_(y, self.scales[i], stream=batch.stream)
                ops.residual_add(h, y, stream=batch.stream)


class InputConv(Mixer):
    """A mixer that reads x + conv(x) instead of x,

        conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j)        (zeros before the request's start)

    a causal convolution over time on every channel of the mixer's input.  The last taps - 1 inputs of a request
    are a state tensor of the layer (``input_conv.tail``, 32-bit) beside whatever the inner mixer keeps, so that a
    request may be cut into steps anywhere; the inner mixer sees its own cache needs only."""

    TAIL = "input_conv.tail"

    def __init__(self, spec):
        super().__init__(spec)
        if not 1 <= spec.taps <= 16:
            raise ValueError(f"input convolution of {spec.taps} taps: between 1 and 16")
        self.inner = build_part(spec.mixer)

    @property
    def graph_safe(self):
        return self.inner.graph_safe

    def tensor_decls(self):
        from ..weights.loader import TensorDecl

        return [TensorDecl(self.spec.name, (self.spec.channels, self.spec.taps))] + self.inner.tensor_decls()

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self.spec.name)
        self.inner.load(src, rt)

    def reset_after_fault(self):
        self.inner.reset_after_fault()

    def cache_spec(self):
        s = self.spec
        cs = self.inner.cache_spec()
        parts, paged = [], None
        if cs is not None:
            paged = cs.paged
            if cs.state is not None:
                if cs.state.dtype != torch.float32:
                    raise ValueError("input_conv: the inner mixer's state shares a 32-bit block with the tail")
                parts = list(cs.state.parts or (("state", cs.state.shape),))
        if any(n == self.TAIL for n, _ in parts):
            raise ValueError("input_conv: the inner mixer already keeps a tail of that name")
        parts.append((self.TAIL, (max(1, s.taps - 1), s.channels)))
        return CacheSpec(paged=paged, state=StateSpec(parts=tuple(parts), dtype=torch.float32))

    def _inner_view(self, cache):
        own = {n: t for n, t in (cache.states or {}).items() if n != self.TAIL}
        return replace(cache, states=own or None, state=own.get("state"))

    def _convolved(self, x, batch, cache):
        s = self.spec
        tail = cache.states[self.TAIL]
        xc = self.rt.empty(x.shape[0], x.shape[1], dtype=x.dtype)
        single = batch.max_new == 1      # a decode step: the kernel that reads a channel's tail also moves it on
        ops.input_conv(x, self.weight, s.taps, tail, batch.token_seq, batch.seq_slot, xc, update_tail=single,
                       stream=batch.stream)
        if not single and s.taps > 1:
            ops.conv_tail_update(x, s.channels, s.taps, tail, batch.token_seq, batch.seq_slot, batch.n_seqs,
                                 stream=batch.stream)
        return xc

    def forward_add(self, x, h, batch, cache):
        self.inner.forward_add(self._convolved(x, batch, cache), h, batch, self._inner_view(cache))

    def forward_into(self, x, out, batch, cache, accumulate=False):
        self.inner.forward_into(self._convolved(x, batch, cache), out, batch, self._inner_view(cache), accumulate)


register_part("mixer_sum", MixerSum, replace=True)
register_part("input_conv", InputConv, replace=True)
