"""A plain, slow statement of the Zanezen design in torch on the CPU: one function per mechanism, whole sequences
at a time, no cache, every recurrence an explicit loop over the tokens.  It shares no code with the engine; the
tests compare the engine with it.

``cfg`` is the parsed ``config.json`` (a dict), ``W`` maps tensor names to tensors of the working precision
(float32, or float64 for a sharper oracle).
"""
from __future__ import annotations

import contextlib
import math

import torch

_ROUND = None      # an element type that everything the design allows in 16 bits is rounded to (None: nothing is)


@contextlib.contextmanager
def rounded_to(dtype):
    """Inside: the products' inputs and outputs that an engine may keep in ``dtype`` are rounded to it, so that the
    distance to the unrounded result shows what rounding alone does."""
    global _ROUND
    old, _ROUND = _ROUND, dtype
    try:
        yield
    finally:
        _ROUND = old


def _r(x):
    return x.to(_ROUND).to(x.dtype) if _ROUND is not None else x


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def causal(n):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return j <= i


def short_conv(u, w):
    """u [n, channels], w [channels, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            y[back:] += w[:, j][None, :] * u[:n - back]
    return y


def rotary_frequencies(dims, base, scaling=None, dtype=torch.float64):
    """[dims / 2] frequencies and the factor on cos and sin.  ``scaling`` (factor, original, fast, slow): the
    interpolation between f_i and f_i / factor by a ramp over the pair index."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    mag = 1.0
    if scaling is not None:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def pair_of(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
        ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), mag


def rotate_halves(x, dims, freqs, mag=1.0):
    """x [n, ..., d]: element i of the first ``dims`` is paired with element i + dims/2 and the pair turned by
    position * freqs[i]; position = index along axis 0; cos and sin times ``mag``; the rest passes unchanged."""
    n, half = x.shape[0], dims // 2
    pos = torch.arange(n, dtype=torch.float32)                      # positions and angles are 32-bit
    ang = pos[:, None] * freqs.to(torch.float32)[None, :]
    shape = [n] + [1] * (x.dim() - 2) + [half]
    c = (torch.cos(ang) * mag).reshape(shape).to(x.dtype)
    s = (torch.sin(ang) * mag).reshape(shape).to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def capped(x, cap):
    return cap * torch.tanh(x / cap)


def mlstm(m, W, p, h, eps):
    """Matrix memory with an input and a forget gate in the logarithm and a running maximum that starts at 0."""
    n = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m.get("vdim", m["dim"]), float(m["gate_cap"])
    q = (h @ W[p + "q"].T).view(n, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).view(n, H, D)
    v = (h @ W[p + "v"].T).view(n, H, V)
    gi = capped(h @ W[p + "i"].T + W[p + "i.b"], cap)
    gf = torch.nn.functional.logsigmoid(capped(h @ W[p + "f"].T + W[p + "f.b"], cap))
    out = torch.zeros(n, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        z = torch.zeros(D, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(n):
            m_new = torch.maximum(gf[t, a] + mx, gi[t, a])
            keep, take = torch.exp(gf[t, a] + mx - m_new), torch.exp(gi[t, a] - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            z = keep * z + take * k[t, a]
            mx = m_new
            den = torch.maximum(torch.abs(z @ q[t, a]), torch.exp(-mx)) + 1e-6
            out[t, a] = (S.T @ q[t, a]) / den
    y = rms(out, eps).reshape(n, H * V) * W[p + "norm"]
    y = y * torch.sigmoid(h @ W[p + "g"].T)
    return _r(y) @ W[p + "o"].T


def differential_attention(m, W, p, h, eps):
    """Two attention maps a head over the same values; the second is taken off the first, times lambda."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = _r(h @ W[p + "q"].T), _r(h @ W[p + "k"].T), _r(h @ W[p + "v"].T)
    if m.get("conv"):
        q, k, v = short_conv(q, W[p + "q.conv"]), short_conv(k, W[p + "k.conv"]), short_conv(v, W[p + "v.conv"])
    q, k, v = q.view(n, H, 2, D), k.view(n, G, 2, D), _r(v).view(n, G, V)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        f, mag = rotary_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
        q, k = rotate_halves(q, rot["dims"], f, mag), rotate_halves(k, rot["dims"], f, mag)
    q, k = _r(q), _r(k)
    lam = (torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum())
           + float(m["diff"]))
    ok = causal(n)
    out = torch.zeros(n, H, V, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for j in range(2):
            s = (q[:, a, j] @ k[:, g, j].T) * float(m["scale"])
            if m.get("softcap"):
                s = capped(s, float(m["softcap"]))
            s = s.masked_fill(~ok, float("-inf"))
            maps.append(_r(torch.softmax(s, dim=-1) @ v[:, g]))
        out[:, a] = rms(maps[0] - lam * maps[1], eps) * (1.0 - float(m["diff"]))
    return _r(out.reshape(n, H * V)) @ W[p + "o"].T


def latent_attention(m, W, p, h, eps):
    """Keys and values read out of one normed latent vector a position; one rotated key part for all heads; a
    learned number per head in the softmax's denominator; a gate per head."""
    n = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = _r(h @ W[p + "q"].T).view(n, H, D + R)
    dkv = _r(h @ W[p + "dkv"].T)
    c = _r(rms(dkv[:, :C], eps) * W[p + "dkv.norm"])
    kr = dkv[:, C:]
    rot = m["rot"]
    f, mag = rotary_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
    q_rot = rotate_halves(q[:, :, D:], rot["dims"], f, mag)
    q_rot, kr = _r(q_rot), _r(rotate_halves(kr, rot["dims"], f, mag))
    k = (c @ W[p + "uk"].T).view(n, H, D)
    v = (c @ W[p + "uv"].T).view(n, H, V)
    gate = torch.sigmoid(_r(h @ W[p + "g"].T))                 # [n, H]
    ok = causal(n)
    out = torch.zeros(n, H, V, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :D] @ k[:, a].T + q_rot[:, a] @ kr.T) * float(m["scale"])
        s = s.masked_fill(~ok, float("-inf"))
        sink = W[p + "sink"][a]
        mx = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        w = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - mx))
        out[:, a] = (w @ v[:, a]) * gate[:, a:a + 1]
    return _r(out.reshape(n, H * V)) @ W[p + "o"].T


def dense_mlp(W, p, h):
    g = _r(h @ W[p + "gate"].T + W[p + "gate.b"])
    u = _r(h @ W[p + "up"].T + W[p + "up.b"])
    return _r(torch.nn.functional.silu(g) * u) @ W[p + "down"].T + W[p + "down.b"]


def expert(W, p, h):
    return _r(_r(torch.relu(h @ W[p + "up"].T) ** 2) @ W[p + "down"].T)


def choose_experts(f, W, p, h):
    """(indices [n, top], weights [n, top], scores [n, experts])."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    pick = torch.topk(s + W[p + "correction"], f["router"]["top"], dim=-1).indices
    w = torch.gather(s, 1, pick)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20) * float(f["router"]["scale"])
    return pick, w, s


def moe(f, W, p, h):
    pick, w, _ = choose_experts(f, W, p, h)
    y = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(pick.shape[1]):
            e = int(pick[t, j])
            y[t] += w[t, j] * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
    if f.get("shared"):
        y = y + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(W, p + "shared.", h)
    return y


def router_margins(f, W, p, h):
    """Per token, the gap between the last chosen and the first rejected choice score."""
    s = torch.sigmoid(h @ W[p + "router"].T) + W[p + "correction"]
    top = f["router"]["top"]
    if top >= s.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    srt = torch.sort(s, dim=-1, descending=True).values
    return srt[:, top - 1] - srt[:, top]


MIXERS = {"mlstm": mlstm, "attention": differential_attention, "latent_attention": latent_attention}


def forward(cfg, W, tokens, return_layers=False, return_margins=False):
    """Logits [n, vocab] of one sequence (and the residual stream after every layer, the routers' smallest margins)."""
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    layers, margins = [], torch.full((len(tokens),), float("inf"), dtype=x.dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _r(rms(x, eps) * W[p + "norm1"])
        y = MIXERS[layer["type"]](layer["mixer"], W, p + "mix.", h, eps)
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                y = y + dense_mlp(W, p + "mlp.", h)
            else:
                y = y + moe(f, W, p + "mlp.", h)
                margins = torch.minimum(margins, router_margins(f, W, p + "mlp.", h))
        x = x + mult * y
        layers.append(x)
    logits = _r(rms(x, eps) * W["final.norm"]) @ W["head"].T
    out = (logits,)
    if return_layers:
        out += (torch.stack(layers),)
    if return_margins:
        out += (margins,)
    return out[0] if len(out) == 1 else out
