"""Attention over one latent vector a position.

    q      = Wq x                       (or  Wuq . rmsnorm(Wdq x)  when the queries pass a latent of their own)
    c, kr  = split(Wdkv x);  c <- rmsnorm(c);  kr <- rotate(kr)          cached: [c | kr], one row a position
    head h:  score(i, j) = scale * ( q_plain[i, h] . (Wuk_h c_j)  +  rotate(q_rot[i, h]) . kr_j )
             out[i, h]   = Wuv_h . sum_j softmax_j(score) c_j
    y      = Wo . (concat(heads) * sigmoid(Wg x))                        (the gate only if the mixer has one)

The read-out matrices never touch the cache: the plain query part is taken through Wuk_h first
(q'[i, h] = Wuk_h^T q_plain[i, h], as wide as the latent), so that a score is one dot product of rank + rot_dim
elements against a cached row, every head reads the same rows, and the attention's result stays in the latent
space until Wuv_h is applied to it.  Queries and results are laid out head by head ([head][token][..]) in
between, so that both per-head products are one grouped product with the heads as groups.

Prompt portions in bfloat16 may take the other order (:meth:`LatentAttention._forward_expanded`): the cached rows
that the step's queries can see are copied out of the pages, ONE product with the matrix [Wuk_h, 0; 0, I] per head
over [Wuv_h, 0] turns them into per-head keys [k_plain | k_rot] and values, and the attention runs per head over
rows of head_dim + rot_dim and value_dim elements instead of rank + rot_dim and rank: a score costs a third or less
of the latent-space form's when the latent is much wider than a head, at the price of one product over the visible
rows.  ``expanded_gain`` estimates both; decoding always reads the latent rows (nothing is expanded for one token).

Rotation: neighbouring pairs (2i, 2i + 1) of the first ``rotary_dims`` elements of the rot_dim part, pair i at
base^(-2i / rotary_dims); angles, norms and scores are 32-bit.  ``rotary_pairing="halves"`` pairs element i with
element i + rotary_dims / 2 instead, and ``rotary_scaling`` stretches the frequencies (``ScaledRotarySpec``).

``sink``: a learned number per head whose exponential joins the softmax's denominator (no key, no value, counted
once).  ``gate_per_head``: the output gate is one number a head, sigmoid(g_h . x).
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.specs import CacheSpec, PagedSpec, PagedTensorSpec
from ..kernels import ops
from ..weights.loader import TensorDecl
from .attention import _common_dtype, general_attention
from .base import Mixer, build_part, register_part
from .specs import AdjacentRotarySpec, ScaledRotarySpec


# The expanded form of a prompt step is taken when its estimated cost is below this share of the latent-space form's
# (tests set 0 and a large number to force either).
EXPANDED_MAX_COST_RATIO = 0.8
# Its product runs on tcgen05 at several times the rate of the attention's mma.sync tiles: the weight of one of its
# multiply-adds against one of the attention's.
EXPANSION_FLOP_WEIGHT = 0.25


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.rotary_dims % 2 or not 0 <= s.rotary_dims <= s.rot_dim:
            raise ValueError(f"rotary_dims={s.rotary_dims}: even and at most rot_dim={s.rot_dim}")
        if s.window is not None and s.window < 1:
            raise ValueError(f"window={s.window}: a window holds at least the query's own position")
        if s.kv_rank + s.rot_dim > ops.ATTENTION_MAX_KEY_DIM or s.kv_rank > ops.ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"kv_rank={s.kv_rank}, rot_dim={s.rot_dim}: a cached row holds at most "
                             f"{ops.ATTENTION_MAX_KEY_DIM} elements, a latent at most {ops.ATTENTION_MAX_VALUE_DIM}")
        self.q_width = s.n_heads * (s.head_dim + s.rot_dim)
        self.row = s.kv_rank + s.rot_dim
        self.o_size = s.n_heads * s.value_dim
        pairing = getattr(s, "rotary_pairing", "adjacent")
        scaling = getattr(s, "rotary_scaling", None)
        if pairing not in ("adjacent", "halves"):
            raise ValueError(f"rotary_pairing={pairing!r}: adjacent or halves")
        if pairing == "adjacent":
            if scaling is not None:
                raise ValueError("latent attention: stretched frequencies come with the halves pairing")
            self.rotary = build_part(AdjacentRotarySpec(rotary_dim=max(2, s.rotary_dims), theta=s.rotary_base))
        else:
            f, o, fa, sl = scaling if scaling is not None else (None, 0.0, 0.0, 0.0)
            self.rotary = build_part(ScaledRotarySpec(rotary_dim=max(2, s.rotary_dims), theta=s.rotary_base, factor=f,
                                                      original=o, fast=fa, slow=sl))
        self.pairing = ops.PAIR_ADJACENT if pairing == "adjacent" else ops.PAIR_HALVES
        self.gate_per_head = bool(getattr(s, "gate_per_head", False)) and s.output_gate
        self.gate_rows = (s.n_heads if self.gate_per_head else self.o_size) if s.output_gate else 0
        self.sink_name = getattr(s, "sink", None)
        self._groups = {}

    def cache_spec(self):
        return CacheSpec(paged=PagedSpec((PagedTensorSpec("kv", (self.row,), lead_dims=0),), self.spec.window))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = []
        if s.q_rank:
            d += [TensorDecl(p + "dq", (s.q_rank, s.hidden)), TensorDecl(p + "dq.norm", (s.q_rank,), init="ones"),
                  TensorDecl(p + "uq", (self.q_width, s.q_rank))]
        else:
            d.append(TensorDecl(p + "q", (self.q_width, s.hidden)))
        d += [TensorDecl(p + "dkv", (self.row, s.hidden)), TensorDecl(p + "dkv.norm", (s.kv_rank,), init="ones"),
              TensorDecl(p + "uk", (s.n_heads * s.head_dim, s.kv_rank)),
              TensorDecl(p + "uv", (s.n_heads * s.value_dim, s.kv_rank))]
        if s.output_gate:
            d.append(TensorDecl(p + "g", (self.gate_rows, s.hidden)))
        if self.sink_name:
            d.append(TensorDecl(p + self.sink_name, (s.n_heads,)))
        d.append(TensorDecl(p + "o", (s.hidden, self.o_size)))
        return d

    def load(self, src, rt):
        super().load(src, rt)
        s, p = self.spec, self.spec.prefix
        H, D, V, C = s.n_heads, s.head_dim, s.value_dim, s.kv_rank
        # one product for everything that reads the mixer's input: [q or dq | dkv | g]
        first = [src.get(p + ("dq" if s.q_rank else "q")), src.get(p + "dkv")]
        if s.output_gate:
            first.append(src.get(p + "g"))
        dt = _common_dtype(first)
        rows = sum(w.shape[0] for w in first)
        if rows % 8:
            # (a gate of one row a head: rows of zeros behind it keep the product's rows 16 bytes apart in 16 bits)
            first.append(torch.zeros(8 - rows % 8, s.hidden, dtype=dt, device=first[0].device))
        self.w_in = torch.cat([w.to(dt) for w in first], dim=0).contiguous()
        self.sink = src.get(p + self.sink_name).to(torch.float32).contiguous() if self.sink_name else None
        self.w_uq = src.get(p + "uq") if s.q_rank else None
        self.q_norm = src.get(p + "dq.norm") if s.q_rank else None
        self.c_norm = src.get(p + "dkv.norm")
        # groups = heads: [H, C, D] takes a head's plain query part into the latent space (Wuk_h transposed),
        # [H, V, C] takes a head's result out of it
        self.w_uk_t = src.get(p + "uk").view(H, D, C).transpose(1, 2).contiguous()
        self.w_uv = src.get(p + "uv").view(H, V, C).contiguous()
        self.w_o = src.get(p + "o")
        self.rotary.load(src, rt)
        # the expanded form's matrix: per head [Wuk_h, 0; 0, I] (rows: head_dim + rot_dim), then [Wuv_h, 0] per head
        self.w_exp = None
        R = s.rot_dim
        ldq = self.q_width if s.q_rank else self.w_in.shape[0]      # row stride of the queries as projected
        if (rt.dtype == torch.bfloat16 and rt.device.type == "cuda" and (D + R) % 16 == 0 and V % 16 == 0 and self.row % 8 == 0
                and ldq % 8 == 0 and self.w_in.dtype == torch.bfloat16 and ops.general_attention_fits(D + R, V)):
            uk, uv = src.get(p + "uk").view(H, D, C), src.get(p + "uv").view(H, V, C)
            wk = torch.zeros(H, D + R, self.row, dtype=uk.dtype, device=uk.device)
            wk[:, :D, :C] = uk
            wk[:, D:, C:] = torch.eye(R, dtype=uk.dtype, device=uk.device)
            wv = torch.zeros(H, V, self.row, dtype=uk.dtype, device=uk.device)
            wv[:, :, :C] = uv
            self.w_exp = torch.cat([wk.view(H * (D + R), self.row), wv.view(H * V, self.row)], dim=0).contiguous()

    def _head_groups(self, T: int):
        """Where each head's rows begin when rows lie head by head, and the list of heads (the grouped products'
        group offsets and active groups).  Made once per step size, outside graph captures."""
        g = self._groups.get(T)
        if g is None:
            H, dev = self.spec.n_heads, self.rt.device
            g = ((torch.arange(H + 1, dtype=torch.int32, device=dev) * T).to(torch.int32),
                 torch.cat([torch.arange(H, dtype=torch.int32, device=dev),
                            torch.full((1,), -1, dtype=torch.int32, device=dev)]))
            if not (dev.type == "cuda" and torch.cuda.is_current_stream_capturing()):
                self._groups[T] = g
        return g

    def forward_add(self, x, h, batch, cache):
        self.forward_into(x, h, batch, cache, accumulate=True)

    def _visible_pages(self, batch, cache):
        """Per entry of a prompt step: (first, one past the last) logical page its queries can see."""
        W, ps = self.spec.window, cache.page_size
        return [((max(0, e.start - W + 1) if W else 0) // ps, (e.start + len(e.tokens) - 1) // ps + 1) for e in batch.entries]

    def expanded_gain(self, batch, cache) -> float:
        """Estimated cost of the expanded form over that of the latent-space form for this step (below 1: cheaper):
        per head, (query, key) pairs times the row widths of either form, plus the product over the visible rows."""
        s = self.spec
        W, ps = s.window, cache.page_size
        pairs = rows = 0
        for e, (p0, p1) in zip(batch.entries, self._visible_pages(batch, cache)):
            n = len(e.tokens)
            seen = e.start + (n + 1) / 2
            pairs += n * (min(W, seen) if W else seen)
            rows += (p1 - p0) * ps
        wide, narrow = 2 * s.kv_rank + s.rot_dim, s.head_dim + s.rot_dim + s.value_dim
        return (pairs * narrow + EXPANSION_FLOP_WEIGHT * rows * self.row * narrow) / max(1.0, pairs * wide)

    def _use_expanded(self, batch, cache) -> bool:
        return (self.w_exp is not None and batch.max_new > 1 and cache.table_host is not None and cache.writes
                and self.expanded_gain(batch, cache) < EXPANDED_MAX_COST_RATIO)

    def _expanded_plan(self, batch, cache):
        """What the expanded form needs from the host for this step, made once and shared by the layers with the same
        window: the pages to copy (their ids in the layer's group), a block table over the copies (row = entry), the
        entries' rows of that table, and the attention's work list (every head its own kv head)."""
        key = ("latent attention expanded", self.spec.window, self.spec.n_heads)
        plan = batch.shared.get(key)
        if plan is None:
            spans = self._visible_pages(batch, cache)
            width = max(p1 for _, p1 in spans)
            table = np.full((len(spans), width), -1, dtype=np.int32)
            src, n = [], 0
            for b, (e, (p0, p1)) in enumerate(zip(batch.entries, spans)):
                ids = cache.table_host[e.slot, p0:p1]
                src.append(ids)
                table[b, p0:p1] = np.arange(n, n + (p1 - p0), dtype=np.int32)
                n += p1 - p0
            items = ops.general_attention_items([len(e.tokens) for e in batch.entries], self.spec.n_heads, self.spec.n_heads)
            flat = np.concatenate([np.concatenate(src).astype(np.int32), table.reshape(-1),
                                   np.arange(len(spans), dtype=np.int32), items.reshape(-1)])
            dev = torch.from_numpy(flat).to(self.rt.device)
            a, b2, c = n, n + table.size, n + table.size + len(spans)
            plan = (dev[:a], dev[a:b2].view(len(spans), width), dev[b2:c], dev[c:].view(-1, 5), n)
            batch.shared[key] = plan
        return plan

    def _forward_expanded(self, x, out, batch, cache, accumulate):
        s, rt, st = self.spec, self.rt, batch.stream
        T, H, D, R, V, C = x.shape[0], s.n_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        row, ps = self.row, cache.page_size
        proj = rt.empty(T, self.w_in.shape[0])
        ops.linear(x, self.w_in, proj, status=batch.status, stream=st, after_short_kernel=True)
        if s.q_rank:
            cq = rt.empty(T, s.q_rank)
            ops.rmsnorm_rows(proj[:, :s.q_rank], self.q_norm, s.norm_eps, cq, stream=st)
            q = rt.empty(T, self.q_width)
            ops.linear(cq, self.w_uq, q, status=batch.status, stream=st)
            rest = s.q_rank
        else:
            q = proj[:, :self.q_width]
            rest = self.q_width
        dkv = proj[:, rest:rest + row]
        gate = proj[:, rest + row:rest + row + self.gate_rows] if s.output_gate else None
        pages = cache.pages["kv"]
        cos_sin = self.rotary.table(batch) if s.rotary_dims > 0 else None
        # cache write; the queries' rotated parts turned where they lie
        ops.latent_prep(q, dkv, batch.positions, batch.token_seq, batch.seq_slot, self.c_norm, s.norm_eps, cos_sin,
                        s.rotary_dims, None, None, pages, cache.block_table, ps, H, D, R, C, write_cache=True,
                        status=batch.status, stream=st, pairing=self.pairing)
        src_pages, table, rows_of, items, n_copies = self._expanded_plan(batch, cache)
        seen = rt.empty(n_copies, ps * row)
        ops.gather_rows(pages.view(pages.shape[0], ps * row), src_pages, seen, stream=st)
        wide = H * (D + R) + H * V
        kv = rt.empty(n_copies * ps, wide)
        ops.linear(seen.view(n_copies * ps, row), self.w_exp, kv, status=batch.status, stream=st)
        attn = rt.empty(T, self.o_size)
        k_view, v_view = kv, kv[:, H * (D + R):]
        ops.general_attention(q, q.stride(0), D + R, k_view, v_view, wide, wide, table, ps, batch.positions, batch.token_seq,
                              rows_of, items, attn, attn.stride(0), V, H, H, D + R, V, s.window, s.scale, stream=st,
                              kv_strides=(ps * wide, D + R, ps * wide, V), sinks=self.sink)
        if gate is not None:
            ops.gate_heads_(attn, gate, H, stream=st, gate_per_head=self.gate_per_head)
        ops.linear(attn, self.w_o, out, accumulate=accumulate, status=batch.status, stream=st, after_short_kernel=True)

    def forward_into(self, x, out, batch, cache, accumulate=False):
        if self._use_expanded(batch, cache):
            return self._forward_expanded(x, out, batch, cache, accumulate)
        s, rt, st = self.spec, self.rt, batch.stream
        T, H, D, R, V, C = x.shape[0], s.n_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        row = self.row
        proj = rt.empty(T, self.w_in.shape[0])
        ops.linear(x, self.w_in, proj, status=batch.status, stream=st, after_short_kernel=True)
        if s.q_rank:
            cq = rt.empty(T, s.q_rank)
            ops.rmsnorm_rows(proj[:, :s.q_rank], self.q_norm, s.norm_eps, cq, stream=st)
            q = rt.empty(T, self.q_width)
            ops.linear(cq, self.w_uq, q, status=batch.status, stream=st)
            rest = s.q_rank
        else:
            q = proj[:, :self.q_width]
            rest = self.q_width
        dkv = proj[:, rest:rest + row]
        gate = proj[:, rest + row:rest + row + self.gate_rows] if s.output_gate else None
        pages = cache.pages["kv"]
        q_plain = rt.empty(H, T, D)
        q_full = rt.empty(H, T, row)
        cos_sin = self.rotary.table(batch) if s.rotary_dims > 0 else None
        ops.latent_prep(q, dkv, batch.positions, batch.token_seq, batch.seq_slot, self.c_norm, s.norm_eps, cos_sin,
                        s.rotary_dims, q_plain, q_full, pages, cache.block_table, cache.page_size, H, D, R, C,
                        write_cache=cache.writes, status=batch.status, stream=st, pairing=self.pairing)
        offsets, heads = self._head_groups(T)
        ops.grouped_linear(q_plain.view(H * T, D), self.w_uk_t, q_full.view(H * T, row)[:, :C], offsets, heads, T,
                           status=batch.status, stream=st)
        o_lat = rt.empty(H, T, C)
        general_attention(q_full, row, T * row, pages, pages, row, row, o_lat, C, T * C, batch, cache, H, 1, row, C,
                          s.window, s.scale, None, rt, sinks=self.sink)
        o_heads = rt.empty(H, T, V)
        ops.grouped_linear(o_lat.view(H * T, C), self.w_uv, o_heads.view(H * T, V), offsets, heads, T,
                           status=batch.status, stream=st)
        attn = rt.empty(T, self.o_size)
        ops.heads_to_tokens(o_heads, attn, gate=gate, stream=st, gate_per_head=self.gate_per_head)
        ops.linear(attn, self.w_o, out, accumulate=accumulate, status=batch.status, stream=st, after_short_kernel=True)


register_part("latent_attention", LatentAttention, replace=True)
