"""A plain, slow statement of the Sesuzen design in torch on the CPU: one function per mechanism, whole sequences
at a time, no cache, no batches.  It shares no code with the engine; the tests compare the engine with it.

``cfg`` is the parsed ``config.json`` (a dict), ``W`` maps tensor names to tensors of one floating type (32-bit,
or 64-bit where a test wants a reference that rounding does not reach).
"""
from __future__ import annotations

import contextlib
import math

import torch

_round = lambda t: t


@contextlib.contextmanager
def rounded_to(dtype):
    """Within the block, everything that the design allows in reduced precision (the inputs and outputs of matrix
    products, activations between them) is rounded to ``dtype`` and back; what it wants in 32-bit is not.  The
    distance of such a run from the exact one is what rounding alone costs a model: the measure for an engine that
    computes in ``dtype``."""
    global _round
    old, _round = _round, (lambda t: t.to(dtype).to(t.dtype))
    try:
        yield
    finally:
        _round = old


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of the squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis; no weight."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def input_convolution(x, w):
    """x [n, C], w [C, taps]: x_t + sum_j w[:, j] x_(t - taps + 1 + j), zeros before the sequence."""
    n, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    out = x.clone()
    for j in range(taps):
        out = out + padded[j:j + n] * w[:, j]
    return out


def visible(n, size=None, keep_first=0):
    """[n, n] bool: query i (rows) sees key j (columns) when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def mixer_attention(x, m, W, p, eps):
    """Grouped-query attention without rotation: biased projections, values of unit RMS per head, a sliding
    window that keeps the first tokens, softmax, a sigmoid gate on the heads' outputs."""
    n = x.shape[0]
    H, D = m["heads"], m["dim"]
    G, V = m.get("kv_heads", H), m.get("vdim", D)
    q = _round(x @ W[p + "q"].T + W[p + "q.b"]).view(n, H, D)
    k = _round(x @ W[p + "k"].T + W[p + "k.b"]).view(n, G, D)
    v = _round(x @ W[p + "v"].T + W[p + "v.b"]).view(n, G, V)
    v = _round(unit_rms(v, eps))
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    mask = m.get("mask")
    ok = visible(n, mask["size"], mask.get("keep_first", 0)) if mask else visible(n)
    s = s.masked_fill(~ok[None], float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = _round(torch.einsum("hij,jhd->ihd", a, vv).reshape(n, H * V))
    o = _round(o * torch.sigmoid(_round(x @ W[p + "g"].T)))
    return o @ W[p + "o"].T


DECAY_RATE = math.exp(-0.5)


def delta_inputs(x, m, W, p):
    """What the generalized delta rule reads per token: r, k, v [n, H, D], decay w and removal rate a [n, H, D]."""
    n = x.shape[0]
    H, D = m["heads"], m["dim"]
    r = (x @ W[p + "r"].T).view(n, H, D)
    k = (x @ W[p + "k"].T).view(n, H, D)
    v = (x @ W[p + "v"].T).view(n, H, D)
    z = torch.tanh(x @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]
    w = torch.exp(-DECAY_RATE * torch.sigmoid(z)).view(n, H, D)
    a = torch.sigmoid(x @ W[p + "a"].T + W[p + "a.b"]).view(n, H, D)
    return r, k, v, w, a


def delta_recurrence(r, k, v, w, a, S=None):
    """S_t = diag(w_t) S_(t-1) - (a_t u_t) (u_t^T S_(t-1)) + k_t v_t^T with u = k / sqrt(sum k^2 + 1e-6);
    o_t = S_t^T r_t.  All [n, H, D]; S [H, D(key), D(value)].  Returns (o [n, H, D], S)."""
    n, H, D = r.shape
    if S is None:
        S = torch.zeros(H, D, D, dtype=r.dtype)
    out = []
    for t in range(n):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(dim=-1, keepdim=True) + 1e-6)
        uS = torch.einsum("hi,hij->hj", u, S)
        S = w[t][:, :, None] * S - (a[t] * u)[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hij,hi->hj", S, r[t]))
    return torch.stack(out), S


def mixer_general_delta(x, m, W, p, eps):
    n = x.shape[0]
    r, k, v, w, a = delta_inputs(x, m, W, p)
    o, _ = delta_recurrence(r, k, v, w, a)
    o = unit_rms(o, eps).reshape(n, -1) * W[p + "norm"]
    o = _round(o * torch.sigmoid(x @ W[p + "g"].T))
    return o @ W[p + "o"].T


def ffn_dense(x, W, p):
    z = torch.relu(_round(x @ W[p + "up"].T))
    return _round(z * z) @ W[p + "down"].T


def route(x, f, W, p):
    """(chosen experts [n, top], their weights [n, top], router logits [n, experts])."""
    z = x @ W[p + "router"].T
    top = f["router"]["top"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1), z


def ffn_moe(x, f, W, p, chosen=None):
    idx, wt, _ = route(x, f, W, p) if chosen is None else chosen
    out = torch.zeros(x.shape[0], W[p + "e0.down"].shape[0], dtype=x.dtype)
    for e in range(f["router"]["experts"]):
        hit = idx == e
        rows = hit.any(dim=-1)
        if not rows.any():
            continue
        xe = x[rows]
        g = xe @ W[p + f"e{e}.gate"].T
        y = _round(g * torch.sigmoid(g) * (xe @ W[p + f"e{e}.up"].T)) @ W[p + f"e{e}.down"].T
        out[rows] += y * (wt * hit)[rows].sum(dim=-1, keepdim=True)
    return out


def layer_runs(cfg):
    """The order in which the layers run: layers start .. stop - 1 'times' times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def run_layer(h, i, cfg, W, margins=None):
    layer, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    x = _round(layer_norm(h, W[p + "norm1"], W[p + "norm1.b"], eps))
    x = _round(input_convolution(x, W[p + "canon1"]))
    if layer["type"] == "attention":
        h = h + mixer_attention(x, layer["mixer"], W, p + "mix.", eps)
    elif layer["type"] == "general_delta":
        h = h + mixer_general_delta(x, layer["mixer"], W, p + "mix.", eps)
    else:
        raise ValueError(layer["type"])
    f = layer.get("mlp")
    if f is None:
        return h
    x = _round(layer_norm(h, W[p + "norm2"], W[p + "norm2.b"], eps))
    if f["kind"] == "dense":
        return h + ffn_dense(x, W, p + "mlp.")
    if margins is not None:
        _, _, z = route(x, f, W, p + "mlp.")
        srt = torch.sort(z, dim=-1, descending=True).values
        top = f["router"]["top"]
        if top < z.shape[-1]:
            margins.append((srt[:, top - 1] - srt[:, top]) / z.abs().max(dim=-1).values.clamp_min(1e-30))
    return h + ffn_moe(x, f, W, p + "mlp.")


def forward(cfg, W, tokens, return_layers=False, return_margins=False):
    """Logits [n, vocab] of one sequence.  ``return_layers``: also the residual stream after every layer run.
    ``return_margins``: also, per position, the smallest relative gap at a router's cut over all layer runs."""
    dt = W["embed"].dtype
    t = torch.as_tensor(tokens, dtype=torch.long)
    h = W["embed"][t] + W["pos"][: len(t)]
    streams, margins = [], []
    for i in layer_runs(cfg):
        h = run_layer(h, i, cfg, W, margins if return_margins else None)
        streams.append(h)
    x = _round(layer_norm(h, W["final.norm"], W["final.norm.b"], cfg["norm"]["eps"]))
    z = x @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * torch.tanh(z / cap)
    out = [z]
    if return_layers:
        out.append(torch.stack(streams))
    if return_margins:
        out.append(torch.stack(margins).min(dim=0).values if margins else torch.full((len(t),), float("inf"), dtype=dt))
    return out[0] if len(out) == 1 else tuple(out)
