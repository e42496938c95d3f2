"""Grouped-query attention over paged keys and values.

    q = Wq x + bq, k = Wk x + bk, v = Wv x + bv     (one fused product, [q|k|v] rows)
    q, k rotated at the token's absolute position; k, v written to the cache pages
    head h attends with kv head h / (n_heads / n_kv_heads), scale 1/sqrt(head_dim),
    over positions max(0, p-W+1)..p of its own request
    h += Wo . concat(heads)

Reference: crates/ferrox-models/src/decoder.rs:2075-2157 (one token), :3230-3549 (a
batch), attention in crates/ferrox-core/src/attention.rs:402-524.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..cache.specs import CacheSpec, KvCacheSpec, PagedSpec, PagedTensorSpec, StateSpec
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, build_part, register_part
from .specs import NoPositionSpec


RANGE_COUNTERS = 16384            # (token, block of heads) pairs of a decode step whose key ranges one kernel merges
DECODE_ATTENTION_MAX_NEW = 8  # entries that bring at most this many tokens use the split-key kernel
# A decode step of up to this many requests leaves the rotary kernel's work to the attention kernel (measured on a
# B200, 16 heads of 128: 2 us a layer gained at 1 request, 4 at 8, 1.5 lost at 64, where every one of a thousand
# blocks pays for what one short kernel did).
ROTARY_IN_DECODE_KERNEL_MAX_TOKENS = 32


def _common_dtype(tensors):
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


def query_tiles(batch, rows: int) -> torch.Tensor:
    """The work list of a prompt-attention kernel that takes ``rows`` queries of one request at a time: int32
    [n_tiles, 4] rows of (first flat token, rows in the tile, entry index, absolute position of the first row).
    Made once a step for each tile size and shared by the layers (``batch.shared``)."""
    key = ("attention query tiles", rows)
    t = batch.shared.get(key)
    if t is None:
        out, flat = [], 0
        for b, e in enumerate(batch.entries):
            n = len(e.tokens)
            for i in range(0, n, rows):
                out.append((flat + i, min(rows, n - i), b, e.start + i))
            flat += n
        t = torch.from_numpy(np.asarray(out, dtype=np.int32).reshape(-1, 4)).to(batch.token_ids.device)
        batch.shared[key] = t
    return t


def prefill_tc_plan(batch, window, n_heads: int):
    """This step's work items for the tcgen05 prompt attention kernel (``ops.prefill_tc_plan``) on the device: made
    once a step for each window and shared by the layers that have it."""
    key = ("attention tcgen05 items", window, n_heads)
    plan = batch.shared.get(key)
    if plan is None:
        items, merges, parts = ops.prefill_tc_plan([(len(e.tokens), e.start) for e in batch.entries], window, n_heads)
        both = torch.from_numpy(np.concatenate([items.reshape(-1), merges.reshape(-1)])).to(batch.token_ids.device)
        plan = (both[:items.size].view(-1, 8), both[items.size:].view(-1, 4) if merges.size else None, parts)
        batch.shared[key] = plan
    return plan


class GqaAttention(Mixer):
    @property
    def graph_safe(self):
        # this mixer only enqueues kernels; whether its position part does is that part's word
        return self.position.graph_safe

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.head_dim % 2 or s.head_dim > 256:
            raise ValueError(f"head_dim={s.head_dim}: must be even and at most 256")
        if s.window is not None and s.window < 1:
            raise ValueError(f"window={s.window}: a window holds at least the query's own position")
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        # the position encoding is a part of its own: it rotates q and k and stores k and v (no encoding: it only stores)
        self.position = build_part(s.position if s.position is not None else NoPositionSpec())
        self.q_size = s.n_heads * s.head_dim
        self.kv_size = s.n_kv_heads * s.head_dim
        # Queries and keys normed per head, a query temperature, a distance bias, or values of another width than
        # the keys: the general form (its own step between projection and attention, its own attention kernels).
        self.value_dim = int(getattr(s, "value_dim", None) or s.head_dim)
        self.qk_norm = getattr(s, "qk_norm", None)
        self.temperature = getattr(s, "query_temperature", None)
        self.slopes_spec = getattr(s, "distance_slopes", None)
        self.value_norm_eps = getattr(s, "value_norm_eps", None)
        self.keep_first = int(getattr(s, "keep_first", 0) or 0) if s.window is not None else 0
        self.gate_name = getattr(s, "output_gate", None)
        if int(getattr(s, "keep_first", 0) or 0) < 0:
            raise ValueError(f"keep_first={s.keep_first}: a number of positions")
        self.general = bool(self.qk_norm or self.temperature or self.slopes_spec or self.value_dim != s.head_dim
                            or self.value_norm_eps is not None or self.keep_first or self.gate_name)
        self.v_size = s.n_kv_heads * self.value_dim
        self.o_size = s.n_heads * self.value_dim
        if self.general:
            if s.position is not None and not isinstance(s.position, NoPositionSpec):
                raise ValueError("attention with normed queries, keys or values, a query temperature, a distance bias, "
                                 "kept first positions, an output gate or its own value width takes no rotary "
                                 "position encoding")
            if s.tied_values or s.softcap:
                raise ValueError("the general attention form has neither tied values nor a soft cap")
            if self.slopes_spec is not None and len(self.slopes_spec) != s.n_heads:
                raise ValueError("distance_slopes: one slope per head")
            if self.temperature is not None and int(self.temperature[1]) < 1:
                raise ValueError("query_temperature: 'every' is a positive number of positions")
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(s.head_dim)
        self.softcap = float(s.softcap) if s.softcap else None
        if self.softcap is not None and self.softcap < 0:
            raise ValueError(f"softcap={s.softcap}: the cap of the scores is positive")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                     q_bias="q_proj.bias", k_bias="k_proj.bias", v_bias="v_proj.bias")
        names.update(dict(s.tensor_names or ()))
        self._names = {key: s.prefix + n for key, n in names.items()}
        # tied values: the v rows of the fused product are the k rows once more, so that every kernel after it
        # finds [q | k | v] rows as ever and the position part rotates the k copy only
        self._qkv_keys = ("q", "k", "k") if s.tied_values else ("q", "k", "v")

    def cache_spec(self):
        s = self.spec
        if self.value_dim != s.head_dim:
            return CacheSpec(paged=PagedSpec((PagedTensorSpec("k", (s.n_kv_heads, s.head_dim), lead_dims=1),
                                              PagedTensorSpec("v", (s.n_kv_heads, self.value_dim), lead_dims=1)), s.window,
                                             self.keep_first))
        return CacheSpec(paged=KvCacheSpec(s.n_kv_heads, s.head_dim, s.window, self.keep_first))

    def tensor_decls(self):
        s, n = self.spec, self._names
        sizes = dict(q=self.q_size, k=self.kv_size, v=self.v_size)
        keys = sorted(set(self._qkv_keys))
        d = [TensorDecl(n[key], (sizes[key], s.hidden)) for key in keys]
        d.append(TensorDecl(n["o"], (s.hidden, self.o_size)))
        if self.qk_norm:
            d += [TensorDecl(s.prefix + self.qk_norm[0], (s.head_dim,), init="ones"),
                  TensorDecl(s.prefix + self.qk_norm[1], (s.head_dim,), init="ones")]
        if s.qkv_bias:
            d += [TensorDecl(n[key + "_bias"], (sizes[key],)) for key in keys]
        if self.gate_name:
            d.append(TensorDecl(s.prefix + self.gate_name, (self.o_size, s.hidden)))
        return d

    def load(self, src, rt):
        super().load(src, rt)
        n = self._names
        ws = [src.get(n[key]) for key in self._qkv_keys]
        if self.gate_name:
            # the output gate reads the same input as q, k and v: its rows follow theirs in the fused product
            ws.append(src.get(self.spec.prefix + self.gate_name))
        dt = _common_dtype(ws)
        self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.b_qkv = None
        if self.spec.qkv_bias:
            bs = [src.get(n[key + "_bias"]) for key in self._qkv_keys]
            if self.gate_name:
                bs.append(torch.zeros(self.o_size, dtype=bs[0].dtype, device=bs[0].device))    # (the gate has no bias)
            bdt = _common_dtype(bs)
            self.b_qkv = torch.cat([b.to(bdt) for b in bs]).contiguous()
        self.w_o = src.get(n["o"])
        self.position.load(src, rt)
        self.q_norm_w = self.k_norm_w = self.slopes = None
        if self.qk_norm:
            ws = [src.get(self.spec.prefix + self.qk_norm[0]), src.get(self.spec.prefix + self.qk_norm[1])]
            dt = _common_dtype(ws)
            self.q_norm_w, self.k_norm_w = (w.to(dt).contiguous() for w in ws)
        if self.slopes_spec is not None:
            self.slopes = torch.tensor([float(x) for x in self.slopes_spec], dtype=torch.float32, device=rt.device)
        # zeroed scratch of the decode attention kernel that merges its own key ranges (it leaves it zeroed)
        self._range_counters = (torch.zeros(RANGE_COUNTERS, dtype=torch.int32, device=rt.device)
                                if rt.device.type == "cuda" else None)

    def reset_after_fault(self):
        # blocks that gave up never counted themselves: the counters of the merge must start at zero again
        if self._range_counters is not None:
            self._range_counters.zero_()
        self.position.reset_after_fault()

    def forward_add(self, x, h, batch, cache):
        self.forward_into(x, h, batch, cache, accumulate=True)

    def forward_into(self, x, out, batch, cache, accumulate=False):
        """out (+)= Wo . attention: ``out`` is the residual stream (accumulate) or a 32-bit buffer of its shape."""
        if self.general:
            return self._forward_general(x, out, batch, cache, accumulate)
        h = out
        s = self.spec
        T = x.shape[0]
        qkv = self.rt.empty(T, self.q_size + 2 * self.kv_size)
        # (what runs before a block's first product is a norm or the combination before it: short kernels)
        ops.linear(x, self.w_qkv, qkv, bias=self.b_qkv, status=batch.status, stream=batch.stream, after_short_kernel=True)
        # A decode step of one token a request: where the attention kernel can, it rotates the queries and rotates and
        # stores the keys and values itself (one launch less on every layer's path); else the position part does.
        in_kernel = None
        capped = self.softcap is not None
        if (batch.max_new == 1 and T <= ROTARY_IN_DECODE_KERNEL_MAX_TOKENS and not capped
                and ops.decode_store_ok(qkv, cache.k, s.head_dim, cache.page_size)):
            in_kernel = self.position.in_decode_kernel(batch, s.head_dim)
        if in_kernel is None:
            self.position.rotate_and_store(qkv, batch, cache, s.n_heads, s.n_kv_heads, s.head_dim)
        attn = self.rt.empty(T, self.q_size)
        if batch.max_new <= DECODE_ATTENTION_MAX_NEW and ops.decode_ok(qkv, s.head_dim):
            # few query tokens: split each request's keys over many blocks
            group = s.n_heads // s.n_kv_heads
            # (capped scores: not the kernel that streams pages by TMA)
            per_sm = 0 if capped else ops.decode_tma_blocks_per_sm(qkv.dtype, s.head_dim, cache.page_size)
            # blocks per token: the tensor-core kernels take 16 query heads of a kv head at a time, the CUDA-core one 8
            kv_blocks = s.n_kv_heads * -(-group // (16 if qkv.dtype == torch.bfloat16 else 8))
            # the most keys a token reads: the context limit, or a window (with the 64-key blocks it straddles)
            reach = cache.block_table.shape[1] * cache.page_size
            if s.window is not None:
                reach = min(reach, (s.window + 63) // 64 * 64 + 64)
            split_len, n_splits = ops.decode_split_plan(
                T, kv_blocks, reach, per_sm or 3, single_is_final=per_sm > 0,
                run_latency=ops.DECODE_RUN_LATENCY if per_sm else 0.0)
            part_acc = self.rt.empty(T, s.n_heads, n_splits, s.head_dim, dtype=torch.float32)
            part_ml = self.rt.empty(T, s.n_heads, n_splits, 2, dtype=torch.float32)
            ops.decode_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, batch.positions, batch.token_seq,
                batch.seq_slot, attn, s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, split_len, n_splits,
                part_acc, part_ml, status=batch.status, counters=self._range_counters, stream=batch.stream,
                # the kernel just before (the position part's, or the projection) wrote these rows' q and at most the
                # k, v of the step's own positions, max_new of a request
                fresh_positions=batch.max_new,
                store_new=in_kernel is not None, write_pages=cache.writes, cos_sin=in_kernel[0] if in_kernel else None,
                softcap=self.softcap,
            )
        elif not capped and ops.prefill_tc_ok(qkv, attn, cache.k, cache.page_size, s.head_dim):
            # prompt portions: tiles of 256 queries (long ones cut into runs of key blocks), tcgen05
            items, merges, parts = prefill_tc_plan(batch, s.window, s.n_heads)
            part_o = part_ml = None
            if parts:
                part_o = self.rt.empty(parts, s.n_heads, ops.WIDE_PREFILL_TILE, s.head_dim, dtype=torch.float32)
                part_ml = self.rt.empty(parts, s.n_heads, ops.WIDE_PREFILL_TILE, 2, dtype=torch.float32)
            ops.prefill_attention_tc(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, items, batch.seq_slot, attn,
                s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, status=batch.status, stream=batch.stream,
                merges=merges, part_o=part_o, part_ml=part_ml,
            )
        elif ops.prefill_ok(qkv, attn, cache.k, s.head_dim):
            # prompt portions, other head and page sizes: tiles of 64 queries, mma.sync
            ops.prefill_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, query_tiles(batch, ops.PREFILL_TILE),
                batch.seq_slot, attn,
                s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, stream=batch.stream, softcap=self.softcap,
            )
        else:
            # 32-bit, and head sizes that are no multiple of 16: a warp per (token, head)
            ops.paged_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, batch.positions, batch.token_seq,
                batch.seq_slot, attn, s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, stream=batch.stream,
                softcap=self.softcap,
            )
        # (the attention's last blocks only add up key ranges: the memory system is idle under them)
        ops.linear(attn, self.w_o, h, accumulate=accumulate, status=batch.status, stream=batch.stream,
                   after_short_kernel=True)


    def _forward_general(self, x, out, batch, cache, accumulate):
        """The form with normed queries, keys or values, a query temperature, a distance bias, kept first positions,
        an output gate, values of their own width: fused [q | k | v (| gate)] product; one kernel norms q and k (and
        v) per head, applies the temperature and stores k and v; attention with the bias and the mask; the gate;
        output product."""
        s = self.spec
        T, D, V = x.shape[0], s.head_dim, self.value_dim
        qkv_width = self.q_size + self.kv_size + self.v_size
        qkv = self.rt.empty(T, qkv_width + (self.o_size if self.gate_name else 0))
        ops.linear(x, self.w_qkv, qkv, bias=self.b_qkv, status=batch.status, stream=batch.stream, after_short_kernel=True)
        eps = self.qk_norm[2] if self.qk_norm else 0.0
        ops.qk_norm_store(qkv, batch.positions, batch.token_seq, batch.seq_slot, self.q_norm_w, self.k_norm_w, eps,
                          self.temperature, cache.k, cache.v, cache.block_table, cache.page_size, s.n_heads, s.n_kv_heads,
                          D, V, write_cache=cache.writes, status=batch.status, stream=batch.stream,
                          value_norm_eps=self.value_norm_eps)
        attn = self.rt.empty(T, self.o_size)
        general_attention(qkv, qkv.stride(0), D, cache.k, cache.v, D, V, attn, attn.stride(0), V, batch, cache,
                          s.n_heads, s.n_kv_heads, D, V, s.window, self.scale, self.slopes, self.rt,
                          keep_first=self.keep_first)
        if self.gate_name:
            ops.gate_heads_(attn, qkv[:, qkv_width:], s.n_heads, stream=batch.stream)
        ops.linear(attn, self.w_o, out, accumulate=accumulate, status=batch.status, stream=batch.stream,
                   after_short_kernel=True)


def general_attention(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, out, ldo, ldoh, batch, cache, n_heads, n_kv_heads,
                      key_dim, value_dim, window, scale, slopes, rt, keep_first=0, softcap=None, sinks=None,
                      value_share=1):
    """Attention over pages in its general form (keys and values of different widths, strided queries and outputs, an
    optional distance bias, a window that may keep the request's first positions visible, capped scores, a learned
    number per head in the softmax's denominator, key heads that share value heads), by the kernel that fits
    the step: tiles of (token, head) pairs on the tensor cores
    in bfloat16, a warp per (token, head) on the CUDA cores in 32-bit and for widths that are no multiple of 16."""
    per_sm = ops.general_attention_ok(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, out, ldo, ldoh, key_dim, value_dim)
    if per_sm:
        items, n_splits, part_o, part_ml = None, 1, None, None
        if batch.max_new == 1:
            # one token a request: cut every token's keys into runs, so that few tokens fill the machine (the number
            # of runs is a function of the step's size and the context limit only: a captured step keeps its grid)
            T = batch.n_tokens
            tiles = n_kv_heads * -(-(n_heads // n_kv_heads) // ops.GENERAL_TILE_ROWS)
            reach = cache.block_table.shape[1] * cache.page_size
            if window is not None:
                reach = min(reach, (window + 63) // 64 * 64 + 64 + (keep_first + 63) // 64 * 64)
            _, n_splits = ops.decode_split_plan(T, tiles, reach, per_sm, single_is_final=True)
            if n_splits > 1:
                part_o = rt.empty(T, n_heads, n_splits, value_dim, dtype=torch.float32)
                part_ml = rt.empty(T, n_heads, n_splits, 2, dtype=torch.float32)
        if batch.max_new > 1:
            key = ("general attention items", n_heads, n_kv_heads)
            items = batch.shared.get(key)
            if items is None:
                items = torch.from_numpy(ops.general_attention_items([len(e.tokens) for e in batch.entries], n_heads,
                                                                     n_kv_heads)).to(batch.token_ids.device)
                batch.shared[key] = items
        return ops.general_attention(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, cache.block_table, cache.page_size,
                                     batch.positions, batch.token_seq, batch.seq_slot, items, out, ldo, ldoh, n_heads,
                                     n_kv_heads, key_dim, value_dim, window, scale, slopes=slopes, stream=batch.stream,
                                     n_splits=n_splits, part_o=part_o, part_ml=part_ml, keep_first=keep_first,
                                     softcap=softcap, sinks=sinks, value_share=value_share)
    ops.paged_attention_ex(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, cache.block_table, cache.page_size, batch.positions,
                           batch.token_seq, batch.seq_slot, out, ldo, ldoh, n_heads, n_kv_heads, key_dim, value_dim,
                           window, scale, slopes=slopes, stream=batch.stream, keep_first=keep_first, softcap=softcap,
                           sinks=sinks, value_share=value_share)


class DifferentialAttention(Mixer):
    """Two attention maps a head over the same values, the second taken off the first:

        q = Wq x (H heads of [map 1 | map 2]),  k = Wk x (G kv heads likewise),  v = Wv x (G heads)
        a short causal convolution on every channel of q, k and v; the maps' first rotary_dim elements rotated
        a_j = softmax(cap(scale q_j . k_j)) v                                   (j = 1, 2; causal)
        o   = rms(a_1 - lambda a_2) (1 - diff),   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
        y   = Wo . concat(heads)

    The attention kernels see 2H query heads on 2G key heads whose pairs read one value head (``value_share``).
    So that a key head's query heads lie side by side, the rows of Wq (and of its convolution) are reordered when
    they are loaded: kv head by kv head, map by map, then the heads of the group.  One kernel does the convolution,
    the rotation and the cache write (``ops.conv_rotary_store``), one the combination of the maps with its norm
    (``ops.diff_combine``).  The convolution's last inputs are a 32-bit state of the request."""

    TAIL = "conv_tail"

    @property
    def graph_safe(self):
        return self.position is None or self.position.graph_safe

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if s.head_dim > ops.ATTENTION_MAX_KEY_DIM or s.value_dim > ops.ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"head_dim={s.head_dim}, value_dim={s.value_dim}: at most {ops.ATTENTION_MAX_KEY_DIM} "
                             f"and {ops.ATTENTION_MAX_VALUE_DIM}")
        self.taps = int(s.conv_taps or 1)
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv_taps={s.conv_taps}: between 1 and 16")
        self.position = build_part(s.position) if s.position is not None else None
        if self.position is not None and not hasattr(self.position, "table"):
            raise ValueError("differential attention rotates by a table of cos and sin: a rotary position part or none")
        self.group = s.n_heads // s.n_kv_heads
        self.nq, self.nk = 2 * s.n_heads, 2 * s.n_kv_heads
        self.q_size, self.k_size = self.nq * s.head_dim, self.nk * s.head_dim
        self.v_size, self.o_size = s.n_kv_heads * s.value_dim, s.n_heads * s.value_dim
        self.channels = self.q_size + self.k_size + self.v_size
        if s.softcap is not None and s.softcap <= 0:
            raise ValueError(f"softcap={s.softcap}: the cap of the scores is positive")

    def cache_spec(self):
        s = self.spec
        paged = PagedSpec((PagedTensorSpec("k", (self.nk, s.head_dim), lead_dims=1),
                           PagedTensorSpec("v", (s.n_kv_heads, s.value_dim), lead_dims=1)), None)
        state = StateSpec(parts=((self.TAIL, (self.taps - 1, self.channels)),)) if self.taps > 1 else None
        return CacheSpec(paged=paged, state=state)

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = [TensorDecl(p + "q", (self.q_size, s.hidden)), TensorDecl(p + "k", (self.k_size, s.hidden)),
             TensorDecl(p + "v", (self.v_size, s.hidden))]
        if s.conv_taps:
            d += [TensorDecl(p + "q.conv", (self.q_size, self.taps)), TensorDecl(p + "k.conv", (self.k_size, self.taps)),
                  TensorDecl(p + "v.conv", (self.v_size, self.taps))]
        d += [TensorDecl(p + n, (s.head_dim,)) for n in ("lq1", "lk1", "lq2", "lk2")]
        d.append(TensorDecl(p + "o", (s.hidden, self.o_size)))
        return d

    def _query_row_order(self):
        """Row r of the reordered Wq is row order[r] of the stored one: (kv head, map, head of the group, element)
        from (head, map, element)."""
        s = self.spec
        g, j, hg, e = torch.meshgrid(torch.arange(s.n_kv_heads), torch.arange(2), torch.arange(self.group),
                                     torch.arange(s.head_dim), indexing="ij")
        return (((g * self.group + hg) * 2 + j) * s.head_dim + e).reshape(-1)

    def load(self, src, rt):
        super().load(src, rt)
        s, p = self.spec, self.spec.prefix
        order = self._query_row_order().to(rt.device)
        ws = [src.get(p + "q")[order], src.get(p + "k"), src.get(p + "v")]
        dt = _common_dtype(ws)
        self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        if s.conv_taps:
            cs = [src.get(p + "q.conv")[order], src.get(p + "k.conv"), src.get(p + "v.conv")]
            self.conv_w = torch.cat([c.to(torch.float32) for c in cs], dim=0).contiguous()
        else:
            self.conv_w = torch.ones(self.channels, 1, dtype=torch.float32, device=rt.device)
        lam = [src.get(p + n).to(torch.float32).cpu() for n in ("lq1", "lk1", "lq2", "lk2")]
        # one number for the layer, worked out once in 32 bits
        self.lam = float(torch.exp((lam[0] * lam[1]).sum()) - torch.exp((lam[2] * lam[3]).sum()) + torch.tensor(float(s.diff)))
        self.w_o = src.get(p + "o")
        if self.position is not None:
            self.position.load(src, rt)

    def reset_after_fault(self):
        if self.position is not None:
            self.position.reset_after_fault()

    def forward_add(self, x, h, batch, cache):
        self.forward_into(x, h, batch, cache, accumulate=True)

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt, st = self.spec, self.rt, batch.stream
        T, D, V = x.shape[0], s.head_dim, s.value_dim
        proj = rt.empty(T, self.channels)
        ops.linear(x, self.w_qkv, proj, status=batch.status, stream=st, after_short_kernel=True)
        tail = cache.states[self.TAIL] if self.taps > 1 else None
        single = batch.max_new == 1      # a decode step: the kernel that reads the tail also moves it on
        cos_sin = self.position.table(batch) if self.position is not None else None
        rot = self.position.rotary_dim if self.position is not None else 0
        pairing = self.position.pairing if self.position is not None else ops.PAIR_HALVES
        q = rt.empty(T, self.q_size)
        ops.conv_rotary_store(proj, self.conv_w, self.taps, tail, batch.positions, batch.token_seq, batch.seq_slot, cos_sin,
                              rot, pairing, q, cache.k, cache.v, cache.block_table, cache.page_size, self.nq, self.nk, D,
                              s.n_kv_heads, V, write_cache=cache.writes, update_tail=single and self.taps > 1,
                              status=batch.status, stream=st)
        if self.taps > 1 and not single:
            ops.conv_tail_update(proj, self.channels, self.taps, tail, batch.token_seq, batch.seq_slot, batch.n_seqs,
                                 stream=st)
        maps = rt.empty(T, self.nq * V)
        general_attention(q, q.stride(0), D, cache.k, cache.v, D, V, maps, maps.stride(0), V, batch, cache, self.nq,
                          self.nk, D, V, None, s.scale, None, rt, softcap=s.softcap, value_share=2)
        attn = rt.empty(T, self.o_size)
        ops.diff_combine(maps, attn, s.n_heads, self.group, V, self.lam, s.norm_eps, 1.0 - float(s.diff), stream=st)
        ops.linear(attn, self.w_o, out, accumulate=accumulate, status=batch.status, stream=st, after_short_kernel=True)


register_part("gqa_attention", GqaAttention, replace=True)
register_part("differential_attention", DifferentialAttention, replace=True)
