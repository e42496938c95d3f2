"""Arrangement of a layer's parts: pre-norm with two residual additions,

    h += mixer(norm1(h));  h += ffn(norm2(h))

(reference: crates/ferrox-models/src/decoder.rs:2054-2173).  The block asks its
mixer what cache it needs and passes the step's batch through; it is built from
whatever norm, mixer and feed-forward its spec names.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, build_part, register_part


class PreNormBlock(Block):
    def __init__(self, spec):
        super().__init__(spec)
        self.norm1 = build_part(spec.norm1)
        self.mixer = build_part(spec.mixer)
        # (a layer without a feed-forward ends after its mixer and has no second norm)
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self.norm2 = build_part(spec.norm2) if self.ffn is not None else None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def tensor_decls(self):
        from ..weights.loader import TensorDecl

        d = [x for p in self._parts() for x in p.tensor_decls()]
        # tensors a checkpoint may hold for this layer although nothing reads them
        d += [TensorDecl(n, tuple(shape), optional=True) for n, shape in getattr(self.spec, "unused_tensors", ())]
        return d

    def load(self, src, rt):
        super().load(src, rt)
        for part in self._parts():
            part.load(src, rt)

    def reset_after_fault(self):
        for part in self._parts():
            part.reset_after_fault()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    passes_norm = True

    def forward(self, h, batch, cache, x=None, then_norm=None):
        """``x``: norm1(h) if the block before has computed it.  ``then_norm``: the first norm of the block that runs
        next; its output on the new h is returned if the feed-forward's last kernel applied it, else None."""
        if x is None:
            with ops.trace_scope("norm"):
                x = self.norm1.forward(h)
        with ops.trace_scope("mixer"):
            self.mixer.forward_add(x, h, batch, cache)
        if self.ffn is None:
            return None
        with ops.trace_scope("norm"):
            x2 = self.norm2.forward(h)
        with ops.trace_scope("feed-forward"):
            if then_norm is not None and self.ffn.fuses_norm:
                return self.ffn.forward_add(x2, h, batch, then_norm=then_norm)
            self.ffn.forward_add(x2, h, batch)
        return None


class ParallelBlock(Block):
    """One norm, two sublayers that read it, one residual addition each:

        x = norm1(h);  h += mixer(x);  h += ffn(x)

    (``ffn`` None: the layer ends after the mixer.)  The sum h + (mixer + ffn) is made in 32 bits in the stream.

    ``residual_mult`` m other than 1:  h += m (mixer(x) + ffn(x)).  Both sublayers then add into a 32-bit buffer of
    the stream's shape, and one kernel multiplies it, adds it to the stream and, where the next block starts with an
    RMS norm, applies that to the new rows as well."""

    passes_norm = True

    def __init__(self, spec):
        super().__init__(spec)
        self.norm1 = build_part(spec.norm1)
        self.mixer = build_part(spec.mixer)
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        self.mult = float(getattr(spec, "residual_mult", 1.0))

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.ffn) if p is not None]

    def tensor_decls(self):
        return [d for p in self._parts() for d in p.tensor_decls()]

    def load(self, src, rt):
        super().load(src, rt)
        for part in self._parts():
            part.load(src, rt)

    def reset_after_fault(self):
        for part in self._parts():
            part.reset_after_fault()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    def forward(self, h, batch, cache, x=None, then_norm=None):
        if x is None:
            with ops.trace_scope("norm"):
                x = self.norm1.forward(h)
        if self.mult != 1.0:
            return self._forward_scaled(h, x, batch, cache, then_norm)
        with ops.trace_scope("mixer"):
            self.mixer.forward_add(x, h, batch, cache)
        if self.ffn is None:
            return None
        with ops.trace_scope("feed-forward"):
            if then_norm is not None and self.ffn.fuses_norm:
                return self.ffn.forward_add(x, h, batch, then_norm=then_norm)
            self.ffn.forward_add(x, h, batch)
        return None

    def _forward_scaled(self, h, x, batch, cache, then_norm):
        y = self.rt.empty(h.shape[0], h.shape[1], dtype=torch.float32)
        with ops.trace_scope("mixer"):
            self.mixer.forward_into(x, y, batch, cache, accumulate=False)
        if self.ffn is not None:
            with ops.trace_scope("feed-forward"):
                self.ffn.forward_add(x, y, batch)
        with ops.trace_scope("norm"):
            rms = then_norm.as_rms() if then_norm is not None else None
            if rms is not None:
                out = self.rt.empty(h.shape[0], h.shape[1])
                return ops.scaled_add_norm(h, y, self.mult, norm=(rms[0], rms[1], out), stream=batch.stream)
            ops.scaled_add_norm(h, y, self.mult, stream=batch.stream)
        return None


class SandwichNormBlock(Block):
    """A norm before and after each sublayer,

        h += post1(mixer(norm1(h)));   h += post2(ffn(norm2(h)))

    (``ffn`` None: the layer ends after the mixer).  The sublayer's output is a 32-bit buffer; one kernel norms it,
    adds it to the stream and, where the norm that comes next is a layer norm too, applies that to the new row as
    well (the mixer's post-norm with norm2, the feed-forward's post-norm with the next block's norm1).  A mixer
    that is a weighted sum of mixers hands its parts over, and the same kernel takes the sum."""

    passes_norm = True

    def __init__(self, spec):
        super().__init__(spec)
        self.norm1 = build_part(spec.norm1)
        self.mixer = build_part(spec.mixer)
        self.post1 = build_part(spec.post1)
        self.has_ffn = spec.ffn is not None
        self.norm2 = build_part(spec.norm2) if self.has_ffn else None
        self.ffn = build_part(spec.ffn) if self.has_ffn else None
        self.post2 = build_part(spec.post2) if self.has_ffn else None

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.post1, self.norm2, self.ffn, self.post2) if p is not None]

    def tensor_decls(self):
        return [d for p in self._parts() for d in p.tensor_decls()]

    def load(self, src, rt):
        super().load(src, rt)
        for part in self._parts():
            part.load(src, rt)

    def reset_after_fault(self):
        for part in self._parts():
            part.reset_after_fault()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    def _add_normed(self, h, outs, post, then_norm, batch):
        """h += post(sum of scale * y over ``outs``); returns then_norm(h) if the same kernel made it, else None."""
        ln = post.as_layer_norm()
        nxt = then_norm.as_layer_norm() if then_norm is not None else None
        if ln is not None and len(outs) <= 2:
            (y, sc), (y2, sc2) = outs[0], (outs[1] if len(outs) == 2 else (None, 1.0))
            then = None
            if nxt is not None:
                then = (nxt[0], nxt[1], self.rt.empty(h.shape[0], h.shape[1]))
            return ops.layernorm_residual(h, y, ln[0], ln[1], scale=sc, y2=y2, scale2=sc2, then=then,
                                          stream=batch.stream)
        # any other norm: sum the parts, norm the sum as a stream of its own, add
        total = outs[0][0]
        if outs[0][1] != 1.0:
            ops.scale_(total, outs[0][1], stream=batch.stream)
        for y, sc in outs[1:]:
            if sc != 1.0:
                ops.scale_(y, sc, stream=batch.stream)
            ops.residual_add(total, y, stream=batch.stream)
        ops.residual_add(h, post.forward(total), stream=batch.stream)
        return None

    def forward(self, h, batch, cache, x=None, then_norm=None):
        if x is None:
            with ops.trace_scope("norm"):
                x = self.norm1.forward(h)
        with ops.trace_scope("mixer"):
            if hasattr(self.mixer, "forward_parts"):
                outs = self.mixer.forward_parts(x, batch, cache)
            else:
                y = self.rt.empty(h.shape[0], h.shape[1], dtype=torch.float32)
                self.mixer.forward_into(x, y, batch, cache, accumulate=False)
                outs = [(y, 1.0)]
        with ops.trace_scope("norm"):
            x2 = self._add_normed(h, outs, self.post1, self.norm2 if self.has_ffn else then_norm, batch)
        if not self.has_ffn:
            return x2
        if x2 is None:
            with ops.trace_scope("norm"):
                x2 = self.norm2.forward(h)
        with ops.trace_scope("feed-forward"):
            y = self.rt.empty(h.shape[0], h.shape[1], dtype=torch.float32)
            self.ffn.forward_into(x2, y, batch, accumulate=False)
        with ops.trace_scope("norm"):
            return self._add_normed(h, [(y, 1.0)], self.post2, then_norm, batch)


register_part("pre_norm", PreNormBlock, replace=True)
register_part("sandwich_norm", SandwichNormBlock, replace=True)
register_part("parallel", ParallelBlock, replace=True)
