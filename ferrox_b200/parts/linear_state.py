"""Mixers that carry a matrix state per head from token to token instead of reading old keys.

``gated_delta_rule``:  per head a state S [head_dim, value_dim];  for every token

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

with q, k, v after a short causal convolution and SiLU, q and k of unit length (q times head_dim^-1/2),
beta = sigmoid(Wb x), g = exp(-exp(A_log) softplus(Wa x + dt_bias)); each head's o is RMS-normed, weighted, and
gated by SiLU(Wg x) before the output projection.  The convolution's last taps - 1 inputs are state as well.

``decayed_linear_attention``:  S <- d_h S + k v^T, o = S^T q on SiLU(q, k, v) with one fixed decay per head; the
heads' read-outs are RMS-normed together, weighted, and gated by sigmoid(Wg x).

``general_delta_rule``:  per head a state S [head_dim, head_dim] with a decay w and a removal rate a per key channel,

    u = k / sqrt(sum k^2 + 1e-6);   S <- diag(w) S - (a u) (u^T S) + k v^T;   o = S^T r

(both terms read the state of the token before), w = exp(-rate sigmoid(W2 tanh(W1 x) + w0)), a = sigmoid(Wa x + ba);
each head's o is RMS-normed, the concatenated heads weighted and gated by sigmoid(Wg x).

``mlstm``:  per head a state S [head_dim, value_dim], a normaliser n [head_dim] and the running maximum m of the
gates' logarithms (m starts at 0),

    i = cap tanh((Wi x + bi) / cap);   f = logsigmoid(cap tanh((Wf x + bf) / cap));   m' = max(f + m, i)
    S <- exp(f + m - m') S + exp(i - m') k v^T;   n likewise with k alone;   o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)

with q = Wq x head_dim^(-1/2); each head's o is RMS-normed, the concatenated heads weighted and gated by sigmoid(Wg x).

The states live in the cache manager's slots as 32-bit tensors; the recurrences, the gates and the norms are
32-bit (``csrc/linear_state.cu``); the projections run in the engine's dtype.  Tokens of a request are taken in
order whatever the step looks like, so a position's output does not depend on how the request was cut.
"""
from __future__ import annotations

import torch

from ..cache.specs import CacheSpec, StateSpec
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, register_part


def _cat_rows(tensors):
    dt = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype
    return torch.cat([t.to(dt) for t in tensors], dim=0).contiguous()


class _StateMixer(Mixer):
    graph_safe = True

    def forward_add(self, x, h, batch, cache):
        self.forward_into(x, h, batch, cache, accumulate=True)


class GatedDeltaRule(_StateMixer):
    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if s.conv_taps < 1 or s.conv_taps > 16:
            raise ValueError(f"conv_taps={s.conv_taps}: between 1 and 16")
        if s.head_dim > 256:
            raise ValueError(f"head_dim={s.head_dim}: the recurrence kernel holds at most 256 rows of a state column")
        self.qk = s.n_kv_heads * s.head_dim
        self.vv = s.n_heads * s.value_dim
        self.channels = 2 * self.qk + self.vv

    def cache_spec(self):
        s = self.spec
        return CacheSpec(state=StateSpec(parts=(
            ("matrix", (s.n_heads, s.value_dim, s.head_dim)),           # S, column by column
            ("conv_tail", (max(1, s.conv_taps - 1), self.channels)),    # the convolution's last inputs, oldest first
        )))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = []
        for n, rows in (("q", self.qk), ("k", self.qk), ("v", self.vv)):
            d.append(TensorDecl(p + n, (rows, s.hidden)))
            d.append(TensorDecl(p + n + ".conv", (rows, s.conv_taps)))
        d += [
            TensorDecl(p + "b", (s.n_heads, s.hidden)), TensorDecl(p + "a", (s.n_heads, s.hidden)),
            TensorDecl(p + "A_log", (s.n_heads,)), TensorDecl(p + "dt_bias", (s.n_heads,)),
            TensorDecl(p + "norm", (s.value_dim,), init="ones"),
            TensorDecl(p + "g", (self.vv, s.hidden)), TensorDecl(p + "o", (s.hidden, self.vv)),
        ]
        return d

    def load(self, src, rt):
        super().load(src, rt)
        p = self.spec.prefix
        # one product for everything the mixer reads from its input: rows [q | k | v | gate | b | a]; its output is
        # written in 32 bits, because b and a feed the gates of the recurrence
        self.w_in = _cat_rows([src.get(p + n) for n in ("q", "k", "v", "g", "b", "a")])
        self.conv_w = torch.cat([src.get(p + n + ".conv").float() for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = src.get(p + "A_log").float().contiguous()
        self.dt_bias = src.get(p + "dt_bias").float().contiguous()
        self.norm_w = src.get(p + "norm").float().contiguous()
        self.w_o = src.get(p + "o")

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt = self.spec, self.rt
        T, H, G, D, V = x.shape[0], s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim
        f32 = torch.float32
        proj = rt.empty(T, self.channels + self.vv + 2 * H, dtype=f32)
        ops.linear(x, self.w_in, proj, status=batch.status, stream=batch.stream)
        ba = proj[:, self.channels + self.vv:]
        qkv = rt.empty(T, self.channels, dtype=f32)
        beta, g = rt.empty(T, H, dtype=f32), rt.empty(T, H, dtype=f32)
        tail, state = cache.states["conv_tail"], cache.states["matrix"]
        single = batch.max_new == 1      # a decode step: the kernel that reads a channel's tail also moves it on
        ops.delta_prep(proj, self.conv_w, s.conv_taps, tail, ba, self.a_log, self.dt_bias, batch.token_seq,
                       batch.seq_slot, qkv, beta, g, G, D, H, V, stream=batch.stream, update_tail=single)
        if not single:
            ops.conv_tail_update(proj, self.channels, s.conv_taps, tail, batch.token_seq, batch.seq_slot, batch.n_seqs,
                                 stream=batch.stream)
        read = rt.empty(T, self.vv, dtype=f32)
        ops.state_scan(qkv[:, :self.qk], qkv[:, self.qk:2 * self.qk], qkv[:, 2 * self.qk:], g, H, beta, state, read,
                       batch.token_seq, batch.seq_slot, batch.n_seqs, H, G, D, V, stream=batch.stream)
        y = rt.empty(T, self.vv)
        ops.gated_group_norm(read, proj[:, self.channels:self.channels + self.vv], self.norm_w, s.norm_eps, "silu", y, H, V, stream=batch.stream)
        ops.linear(y, self.w_o, out, accumulate=accumulate, status=batch.status, stream=batch.stream)


class DecayedLinearAttention(_StateMixer):
    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if len(s.decay) != s.n_heads:
            raise ValueError(f"decay lists {len(s.decay)} values for {s.n_heads} heads")
        if s.head_dim > 256:
            raise ValueError(f"head_dim={s.head_dim}: the recurrence kernel holds at most 256 rows of a state column")
        self.qk = s.n_heads * s.head_dim
        self.vv = s.n_heads * s.value_dim

    def cache_spec(self):
        s = self.spec
        return CacheSpec(state=StateSpec(parts=(("matrix", (s.n_heads, s.value_dim, s.head_dim)),)))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        return [
            TensorDecl(p + "q", (self.qk, s.hidden)), TensorDecl(p + "k", (self.qk, s.hidden)),
            TensorDecl(p + "v", (self.vv, s.hidden)), TensorDecl(p + "g", (self.vv, s.hidden)),
            TensorDecl(p + "o", (s.hidden, self.vv)), TensorDecl(p + "norm", (self.vv,), init="ones"),
        ]

    def load(self, src, rt):
        super().load(src, rt)
        p = self.spec.prefix
        self.w_in = _cat_rows([src.get(p + n) for n in ("q", "k", "v", "g")])          # rows [q | k | v | gate]
        self.norm_w = src.get(p + "norm").float().contiguous()
        self.w_o = src.get(p + "o")
        self.decay = torch.tensor([float(d) for d in self.spec.decay], dtype=torch.float32, device=rt.device)

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt = self.spec, self.rt
        T, H, D, V = x.shape[0], s.n_heads, s.head_dim, s.value_dim
        proj = rt.empty(T, 2 * self.qk + 2 * self.vv)
        ops.linear(x, self.w_in, proj, status=batch.status, stream=batch.stream)
        read = rt.empty(T, self.vv, dtype=torch.float32)
        # SiLU of q, k, v where the recurrence reads them
        ops.state_scan(proj[:, :self.qk], proj[:, self.qk:2 * self.qk], proj[:, 2 * self.qk:2 * self.qk + self.vv],
                       self.decay, 0, None, cache.states["matrix"], read, batch.token_seq, batch.seq_slot, batch.n_seqs,
                       H, H, D, V, silu_on_load=True, stream=batch.stream)
        y = rt.empty(T, self.vv)
        ops.gated_group_norm(read, proj[:, 2 * self.qk + self.vv:], self.norm_w, s.norm_eps, "sigmoid", y, 1, self.vv,
                             stream=batch.stream)
        ops.linear(y, self.w_o, out, accumulate=accumulate, status=batch.status, stream=batch.stream)


class GeneralDeltaRule(_StateMixer):
    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.head_dim > 256:
            raise ValueError(f"head_dim={s.head_dim}: the recurrence kernel holds at most 256 rows of a state column")
        if s.decay_rank < 1:
            raise ValueError(f"decay_rank={s.decay_rank}: the decay's inner width is positive")
        self.hd = s.n_heads * s.head_dim

    def cache_spec(self):
        s = self.spec
        return CacheSpec(state=StateSpec(parts=(("matrix", (s.n_heads, s.head_dim, s.head_dim)),)))   # column by column

    def tensor_decls(self):
        s, p, hd = self.spec, self.spec.prefix, self.hd
        d = [TensorDecl(p + n, (hd, s.hidden)) for n in ("r", "k", "v", "g", "a")]
        d += [
            TensorDecl(p + "a.b", (hd,)), TensorDecl(p + "w1", (s.decay_rank, s.hidden)),
            TensorDecl(p + "w2", (hd, s.decay_rank)), TensorDecl(p + "w0", (hd,)),
            TensorDecl(p + "norm", (hd,), init="ones"), TensorDecl(p + "o", (s.hidden, hd)),
        ]
        return d

    def load(self, src, rt):
        super().load(src, rt)
        p = self.spec.prefix
        # one product for everything the mixer reads from its input: rows [r | k | v | gate | a | w1]; its output is
        # written in 32 bits, because all but the gate enters the recurrence
        self.w_in = _cat_rows([src.get(p + n) for n in ("r", "k", "v", "g", "a", "w1")])
        self.w2 = src.get(p + "w2")
        self.w0 = src.get(p + "w0")
        self.a_bias = src.get(p + "a.b")
        self.norm_w = src.get(p + "norm")
        self.w_o = src.get(p + "o")

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt = self.spec, self.rt
        T, H, D, hd = x.shape[0], s.n_heads, s.head_dim, self.hd
        f32 = torch.float32
        proj = rt.empty(T, 5 * hd + s.decay_rank, dtype=f32)
        ops.linear(x, self.w_in, proj, status=batch.status, stream=batch.stream)
        r, k, v, gate = (proj[:, i * hd:(i + 1) * hd] for i in range(4))
        u, au, w = rt.empty(T, hd, dtype=f32), rt.empty(T, hd, dtype=f32), rt.empty(T, hd, dtype=f32)
        ops.general_delta_prep(k, proj[:, 4 * hd:5 * hd], proj[:, 5 * hd:], self.w2, self.w0, self.a_bias, s.decay_rate,
                               u, au, w, H, D, stream=batch.stream)
        read = rt.empty(T, hd, dtype=f32)
        ops.general_delta_scan(r, k, v, u, au, w, cache.states["matrix"], read, batch.token_seq, batch.seq_slot,
                               batch.n_seqs, H, D, stream=batch.stream)
        y = rt.empty(T, hd)
        ops.gated_group_norm(read, gate, self.norm_w, s.norm_eps, "sigmoid", y, H, D, stream=batch.stream)
        ops.linear(y, self.w_o, out, accumulate=accumulate, status=batch.status, stream=batch.stream)


class Mlstm(_StateMixer):
    """One product for everything the mixer reads from its input, rows [q | k | v | gate | i | f], written in 32 bits
    (all but the gate enters the recurrence); ``ops.mlstm_scan`` (gates, running maximum, state, read-out);
    ``ops.gated_group_norm`` (per-head RMS, weight, sigmoid gate); output product."""

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if not s.gate_cap > 0:
            raise ValueError(f"gate_cap={s.gate_cap}: the cap of the gates is positive")
        self.qk = s.n_heads * s.head_dim
        self.vv = s.n_heads * s.value_dim
        self.copies = None      # copies of the normaliser and the maximum the state keeps (asked of the kernels once)

    def _copies(self):
        if self.copies is None:
            self.copies = ops.mlstm_column_blocks(self.spec.head_dim, self.spec.value_dim)
        return self.copies

    def cache_spec(self):
        s, z = self.spec, self._copies()
        return CacheSpec(state=StateSpec(parts=(
            ("matrix", (s.n_heads, s.value_dim, s.head_dim)),       # S, column by column
            ("normalizer", (s.n_heads, z, s.head_dim)),             # n, one copy for each block of columns
            ("log_max", (s.n_heads, z)),                            # m, likewise
        )))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        return [
            TensorDecl(p + "q", (self.qk, s.hidden)), TensorDecl(p + "k", (self.qk, s.hidden)),
            TensorDecl(p + "v", (self.vv, s.hidden)), TensorDecl(p + "g", (self.vv, s.hidden)),
            TensorDecl(p + "o", (s.hidden, self.vv)), TensorDecl(p + "norm", (self.vv,), init="ones"),
            TensorDecl(p + "i", (s.n_heads, s.hidden)), TensorDecl(p + "i.b", (s.n_heads,)),
            TensorDecl(p + "f", (s.n_heads, s.hidden)), TensorDecl(p + "f.b", (s.n_heads,)),
        ]

    def load(self, src, rt):
        super().load(src, rt)
        s, p = self.spec, self.spec.prefix
        ws = [src.get(p + n) for n in ("q", "k", "v", "g", "i", "f")]
        rows = sum(w.shape[0] for w in ws)
        if rows % 8:     # (rows of zeros keep the product's output rows a multiple of 32 bytes wide)
            ws.append(torch.zeros(8 - rows % 8, s.hidden, dtype=ws[0].dtype, device=ws[0].device))
        self.w_in = _cat_rows(ws)
        self.i_bias = src.get(p + "i.b").to(torch.float32).contiguous()
        self.f_bias = src.get(p + "f.b").to(torch.float32).contiguous()
        self.norm_w = src.get(p + "norm")
        self.w_o = src.get(p + "o")

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt = self.spec, self.rt
        T, H, D, V = x.shape[0], s.n_heads, s.head_dim, s.value_dim
        f32 = torch.float32
        proj = rt.empty(T, self.w_in.shape[0], dtype=f32)
        ops.linear(x, self.w_in, proj, status=batch.status, stream=batch.stream)
        q, k = proj[:, :self.qk], proj[:, self.qk:2 * self.qk]
        v = proj[:, 2 * self.qk:2 * self.qk + self.vv]
        gate = proj[:, 2 * self.qk + self.vv:2 * self.qk + 2 * self.vv]
        gates = proj[:, 2 * self.qk + 2 * self.vv:]       # [i | f] as projected
        read = rt.empty(T, self.vv, dtype=f32)
        ops.mlstm_scan(q, k, v, gates, self.i_bias, self.f_bias, s.gate_cap, float(D) ** -0.5, cache.states["matrix"],
                       cache.states["normalizer"], cache.states["log_max"], read, batch.token_seq, batch.seq_slot,
                       batch.n_seqs, H, D, V, stream=batch.stream)
        y = rt.empty(T, self.vv)
        ops.gated_group_norm(read, gate, self.norm_w, s.norm_eps, "sigmoid", y, H, V, stream=batch.stream)
        ops.linear(y, self.w_o, out, accumulate=accumulate, status=batch.status, stream=batch.stream)


register_part("mlstm", Mlstm, replace=True)
register_part("gated_delta_rule", GatedDeltaRule, replace=True)
register_part("general_delta_rule", GeneralDeltaRule, replace=True)
register_part("decayed_linear_attention", DecayedLinearAttention, replace=True)
