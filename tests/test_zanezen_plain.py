"""Zanezen without a GPU: the configuration reader, the description made of parts, the cache needs of its layers,
and the plain implementation against restatements of its mechanisms as explicit loops or in other algebra."""
import copy
import math

import pytest
import torch

import plain_zanezen as pz
from zanezen_configs import ZANEZEN_A, ZANEZEN_B, ZANEZEN_C


def resolve(cfg):
    import ferrox_b200  # noqa: F401  (registers the architectures)
    from ferrox_b200.config.registry import resolve as r

    return r(cfg)


def test_configuration_is_read_layer_by_layer():
    cfg, spec = resolve(ZANEZEN_A)
    assert [l.type for l in cfg.layers] == ["attention", "mlstm", "latent_attention", "attention", "mlstm"]
    assert cfg.norm_eps == 1e-5 and cfg.embedding_scale == 3.0 and cfg.residual_mult == 0.5
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.diff, a.softcap, a.conv) == (4, 2, 32, 48, 0.2, 0.3, 20.0, 4)
    assert a.rot.dims == 16 and a.rot.base == 500.0 and a.rot.scaling == (4.0, 64.0, 8.0, 1.0)
    assert cfg.layers[3].mixer.rot.scaling is None and cfg.layers[3].mixer.softcap is None
    m = cfg.layers[1].mixer
    assert (m.heads, m.dim, m.vdim, m.gate_cap) == (2, 16, 32, 10.0)
    f = cfg.layers[0].mlp
    assert (f.experts, f.top, f.scale, f.ff, f.shared_ff) == (6, 2, 1.5, 32, 64) and cfg.layers[3].mlp.shared_ff == 0
    assert cfg.layers[1].mlp.ff == 96
    assert [(e.layer, e.cache) for e in spec.schedule] == [(i, i) for i in range(5)]
    assert spec.embedding_scale == 3.0 and all(b.residual_mult == 0.5 for b in spec.layers)
    cfgB, specB = resolve(ZANEZEN_B)
    assert cfgB.embedding_scale == 1.0 and cfgB.residual_mult == 1.0
    b = cfgB.layers[3].mixer
    assert b.conv is None and b.rot is None and b.softcap is None and b.kv_heads == 1
    assert cfgB.layers[1].mlp is None and cfgB.layers[4].mlp is None
    assert specB.layers[3].mixer.position is None and specB.layers[3].mixer.conv_taps is None


def test_defaults_of_keys_that_may_be_absent():
    c = copy.deepcopy(ZANEZEN_B)
    del c["layers"][1]["mixer"]["kv_heads"], c["layers"][1]["mixer"]["vdim"], c["layers"][2]["mixer"]["vdim"]
    del c["residual_mult"]
    cfg, _ = resolve(c)
    assert cfg.layers[1].mixer.kv_heads == 3 and cfg.layers[1].mixer.vdim == 20 and cfg.layers[2].mixer.vdim == 12
    assert cfg.residual_mult == 1.0


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="ring"), "not implemented"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=40), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "empty"),
])
def test_configurations_that_are_refused(change, text):
    from ferrox_b200 import ConfigError

    cfg = copy.deepcopy(ZANEZEN_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        resolve(cfg)


def test_description_declares_the_tensors_and_the_cache_needs():
    from ferrox_b200.parts.build import build_model

    _, spec = resolve(ZANEZEN_A)
    model = build_model(spec)
    decls = {d.name: d.shape for d in model.tensor_decls()}
    assert decls["embed"] == (211, 64) and decls["head"] == (211, 64) and decls["final.norm"] == (64,)
    assert decls["l0.mix.q"] == (4 * 2 * 32, 64) and decls["l0.mix.k"] == (2 * 2 * 32, 64) and decls["l0.mix.v"] == (2 * 48, 64)
    assert decls["l0.mix.q.conv"] == (256, 4) and decls["l0.mix.v.conv"] == (96, 4) and decls["l0.mix.lk2"] == (32,)
    assert decls["l0.mix.o"] == (64, 4 * 48)
    assert decls["l0.mlp.router"] == (6, 64) and decls["l0.mlp.correction"] == (6,) and decls["l0.mlp.e5.down"] == (64, 32)
    assert decls["l0.mlp.shared.up"] == (64, 64) and decls["l0.mlp.shared.sg"] == (1, 64) and "l0.mlp.e0.gate" not in decls
    assert decls["l1.mix.q"] == (32, 64) and decls["l1.mix.v"] == (64, 64) and decls["l1.mix.norm"] == (64,)
    assert decls["l1.mix.i"] == (2, 64) and decls["l1.mix.f.b"] == (2,) and decls["l1.mix.o"] == (64, 64)
    assert decls["l1.mlp.gate.b"] == (96,) and decls["l1.mlp.down.b"] == (64,) and decls["l1.mlp.up"] == (96, 64)
    assert decls["l2.mix.q"] == (4 * 48, 64) and decls["l2.mix.dkv"] == (80, 64) and decls["l2.mix.dkv.norm"] == (48,)
    assert decls["l2.mix.g"] == (4, 64) and decls["l2.mix.sink"] == (4,) and decls["l2.mix.uv"] == (64, 48)
    assert "l3.mlp.shared.up" not in decls and "l3.mlp.shared.sg" not in decls
    caches = model.cache_specs()
    assert [t.token_shape for t in caches[0].paged.tensors] == [(4, 32), (2, 48)] and caches[0].paged.window is None
    assert dict(caches[0].state.parts) == {"conv_tail": (3, 256 + 128 + 96)}
    assert caches[1].paged is None and dict(caches[1].state.parts)["matrix"] == (2, 32, 16)
    z = dict(caches[1].state.parts)["normalizer"][1]
    assert dict(caches[1].state.parts) == {"matrix": (2, 32, 16), "normalizer": (2, z, 16), "log_max": (2, z)}
    assert [t.token_shape for t in caches[2].paged.tensors] == [(80,)] and caches[2].state is None
    _, specB = resolve(ZANEZEN_B)
    cachesB = build_model(specB).cache_specs()
    assert cachesB[3].state is None          # an attention without convolution keeps no tail
    assert dict(cachesB[1].state.parts) == {"conv_tail": (2, 3 * 2 * 20 * 2 + 3 * 12)}


def test_query_rows_are_reordered_key_head_by_key_head():
    from ferrox_b200.parts.base import build_part
    from ferrox_b200.parts import build  # noqa: F401

    _, spec = resolve(ZANEZEN_A)
    part = build_part(spec.layers[0].mixer)          # 4 heads on 2 kv heads, maps of 32
    order = part._query_row_order().view(2, 2, 2, 32)    # [kv head, map, head of the group, element]
    for g in range(2):
        for j in range(2):
            for hg in range(2):
                h = g * 2 + hg
                assert order[g, j, hg].tolist() == list(range((h * 2 + j) * 32, (h * 2 + j) * 32 + 32))


# ------------------------------------------------------------------ the plain implementation against restatements
def test_short_convolution_against_an_explicit_loop():
    g = torch.Generator().manual_seed(0)
    for n, taps in ((1, 4), (3, 4), (9, 1), (20, 5)):
        u, w = torch.randn(n, 6, generator=g), torch.randn(6, taps, generator=g)
        want = torch.zeros(n, 6)
        for t in range(n):
            for j in range(taps):
                s = t - taps + 1 + j
                if s >= 0:
                    want[t] += w[:, j] * u[s]
        assert torch.allclose(pz.short_conv(u, w), want, atol=1e-6)


def test_stretched_frequencies():
    plain, mag = pz.rotary_frequencies(16, 500.0)
    assert mag == 1.0 and plain[0] == 1.0 and abs(float(plain[1]) - 500.0 ** (-2 / 16)) < 1e-12
    # a factor of 1 changes nothing
    same, mag = pz.rotary_frequencies(16, 500.0, dict(factor=1.0, original=64, fast=8.0, slow=1.0))
    assert mag == 1.0 and torch.equal(same, plain)
    f, mag = pz.rotary_frequencies(16, 500.0, dict(factor=4.0, original=64, fast=8.0, slow=1.0))
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    pair = lambda t: 16 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(500.0))
    lo, hi = max(math.floor(pair(8.0)), 0), min(math.ceil(pair(1.0)), 15)
    assert 0 <= lo < hi < 8           # the ramp lies inside the pairs of this configuration
    for i in range(8):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(float(f[i]) - float(plain[i]) * (r / 4.0 + 1 - r)) < 1e-12
    assert f[lo] == plain[lo] and abs(float(f[7]) - float(plain[7]) / 4) < 1e-12


def test_rotation_turns_pairs_of_halves_and_leaves_the_rest():
    x = torch.randn(5, 3, 10, generator=torch.Generator().manual_seed(1))
    f = torch.tensor([0.5, 0.25, 0.1], dtype=torch.float64)
    y = pz.rotate_halves(x, 6, f, 1.2)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0, :, :6], 1.2 * x[0, :, :6])
    for p in range(5):
        for i in range(3):
            a = p * float(f[i])
            u, v = x[p, :, i], x[p, :, i + 3]
            assert torch.allclose(y[p, :, i], 1.2 * (u * math.cos(a) - v * math.sin(a)), atol=1e-5)
            assert torch.allclose(y[p, :, i + 3], 1.2 * (v * math.cos(a) + u * math.sin(a)), atol=1e-5)


def mlstm_weights(hidden, H, D, V, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    shapes = {"q": (H * D, hidden), "k": (H * D, hidden), "v": (H * V, hidden), "g": (H * V, hidden), "o": (hidden, H * V),
              "i": (H, hidden), "f": (H, hidden), "i.b": (H,), "f.b": (H,)}
    w = {"m." + n: torch.randn(*s, generator=g, dtype=torch.float64) * std for n, s in shapes.items()}
    w["m.norm"] = 1 + 0.1 * torch.randn(H * V, generator=g, dtype=torch.float64)
    return w


def test_mlstm_against_the_sums_it_stands_for():
    """Without the running maximum: S_t = sum_s exp(i_s + f_(s+1) + .. + f_t) k_s v_s^T, and the read-out's floor
    exp(-m_t) in the same units.  The plain loop carries the maximum; in 64 bits both agree."""
    hidden, H, D, V, cap, n = 24, 2, 6, 5, 3.0, 40
    w = mlstm_weights(hidden, H, D, V, 2)
    h = torch.randn(n, hidden, generator=torch.Generator().manual_seed(3), dtype=torch.float64)
    m = dict(heads=H, dim=D, vdim=V, gate_cap=cap)
    got = pz.mlstm(m, w, "m.", h, 1e-6)
    q = (h @ w["m.q"].T).view(n, H, D) * D ** -0.5
    k, v = (h @ w["m.k"].T).view(n, H, D), (h @ w["m.v"].T).view(n, H, V)
    gi = cap * torch.tanh((h @ w["m.i"].T + w["m.i.b"]) / cap)
    gf = torch.log(torch.sigmoid(cap * torch.tanh((h @ w["m.f"].T + w["m.f.b"]) / cap)))
    out = torch.zeros(n, H, V, dtype=torch.float64)
    for a in range(H):
        mx = torch.zeros((), dtype=torch.float64)
        for t in range(n):
            mx = torch.maximum(gf[t, a] + mx, gi[t, a])
            logw = torch.stack([gi[s, a] + gf[s + 1:t + 1, a].sum() for s in range(t + 1)])      # unstabilised weights
            wt = torch.exp(logw)
            num = (wt[:, None] * v[:t + 1, a] * (k[:t + 1, a] @ q[t, a])[:, None]).sum(0)
            den = (wt * (k[:t + 1, a] @ q[t, a])).sum()
            # the design divides by max(|n . q|, exp(-m)) + 1e-6 in units scaled by exp(-m)
            out[t, a] = num * torch.exp(-mx) / (torch.maximum(torch.abs(den) * torch.exp(-mx), torch.exp(-mx)) + 1e-6)
    want = (pz.rms(out, 1e-6).reshape(n, H * V) * w["m.norm"] * torch.sigmoid(h @ w["m.g"].T)) @ w["m.o"].T
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-9)
    # the maximum starts at 0, not at minus infinity: with strongly negative input gates the floor exp(-m) = 1 rules
    low = dict(w)
    low["m.i.b"] = w["m.i.b"] - 50.0
    a = pz.mlstm(dict(m, gate_cap=60.0), low, "m.", h[:3], 1e-6)
    assert torch.isfinite(a).all()


def diff_weights(hidden, H, G, D, V, taps, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    shapes = {"q": (H * 2 * D, hidden), "k": (G * 2 * D, hidden), "v": (G * V, hidden), "o": (hidden, H * V),
              "q.conv": (H * 2 * D, taps), "k.conv": (G * 2 * D, taps), "v.conv": (G * V, taps),
              "lq1": (D,), "lk1": (D,), "lq2": (D,), "lk2": (D,)}
    return {"m." + n: torch.randn(*s, generator=g, dtype=torch.float64) * std for n, s in shapes.items()}


def test_differential_attention_token_by_token():
    hidden, H, G, D, V, taps, n = 20, 4, 2, 6, 5, 3, 17
    w = diff_weights(hidden, H, G, D, V, taps, 4)
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=0.4, diff=0.3, softcap=2.0, conv=taps,
             rot={"dims": 4, "base": 50.0, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}})
    h = torch.randn(n, hidden, generator=torch.Generator().manual_seed(5), dtype=torch.float64)
    got = pz.differential_attention(m, w, "m.", h, 1e-6)
    f, mag = pz.rotary_frequencies(4, 50.0, m["rot"]["scaling"])
    lam = math.exp(float(w["m.lq1"] @ w["m.lk1"])) - math.exp(float(w["m.lq2"] @ w["m.lk2"])) + 0.3

    def row(name, t):      # the projected, convolved row of token t
        u = h @ w["m." + name].T
        c = w[f"m.{name}.conv"]
        return sum(c[:, j] * u[t - taps + 1 + j] for j in range(taps) if t - taps + 1 + j >= 0)

    def turn(x, t):
        y = x.clone()
        for i in range(2):
            a = float(torch.tensor(t, dtype=torch.float32) * f[i].to(torch.float32))
            y[i] = mag * (x[i] * math.cos(a) - x[i + 2] * math.sin(a))
            y[i + 2] = mag * (x[i + 2] * math.cos(a) + x[i] * math.sin(a))
        return y

    want = torch.zeros(n, H * V, dtype=torch.float64)
    for t in range(n):
        for a in range(H):
            g = a // (H // G)
            maps = []
            for j in range(2):
                qt = turn(row("q", t)[(a * 2 + j) * D:(a * 2 + j + 1) * D], t)
                s = torch.stack([qt @ turn(row("k", u)[(g * 2 + j) * D:(g * 2 + j + 1) * D], u) for u in range(t + 1)]) * 0.4
                p = torch.softmax(2.0 * torch.tanh(s / 2.0), dim=0)
                maps.append(sum(p[u] * row("v", u)[g * V:(g + 1) * V] for u in range(t + 1)))
            o = maps[0] - lam * maps[1]
            want[t, a * V:(a + 1) * V] = o / torch.sqrt((o * o).mean() + 1e-6) * 0.7
    assert torch.allclose(got, want @ w["m.o"].T, rtol=1e-6, atol=1e-6)      # (cos and sin are 32-bit in the plain code)


def test_latent_attention_against_keys_and_values_per_head_and_the_sink_counts_once():
    hidden, H, D, R, V, C, n = 20, 3, 6, 4, 5, 8, 15
    g = torch.Generator().manual_seed(6)
    shapes = {"q": (H * (D + R), hidden), "dkv": (C + R, hidden), "uk": (H * D, C), "uv": (H * V, C), "g": (H, hidden),
              "o": (hidden, H * V), "sink": (H,)}
    w = {"m." + k: torch.randn(*s, generator=g, dtype=torch.float64) * 0.4 for k, s in shapes.items()}
    w["m.dkv.norm"] = 1 + 0.1 * torch.randn(C, generator=g, dtype=torch.float64)
    m = dict(heads=H, dim=D, rot_dim=R, vdim=V, kv_rank=C, scale=0.3, rot={"dims": 4, "base": 100.0})
    h = torch.randn(n, hidden, generator=g, dtype=torch.float64)
    got = pz.latent_attention(m, w, "m.", h, 1e-6)
    f, _ = pz.rotary_frequencies(4, 100.0)
    dkv = h @ w["m.dkv"].T
    c = dkv[:, :C] / torch.sqrt((dkv[:, :C] ** 2).mean(-1, keepdim=True) + 1e-6) * w["m.dkv.norm"]
    kr = pz.rotate_halves(dkv[:, C:], 4, f)
    q = (h @ w["m.q"].T).view(n, H, D + R)
    want = torch.zeros(n, H, V, dtype=torch.float64)
    for t in range(n):
        for a in range(H):
            qa = q[t, a]
            qr = pz.rotate_halves(q[:, a, D:], 4, f)[t]
            ks = torch.cat([c[:t + 1] @ w["m.uk"][a * D:(a + 1) * D].T, kr[:t + 1]], dim=1)       # [t+1, D+R]
            s = ks @ torch.cat([qa[:D], qr]) * 0.3
            e = torch.exp(s)
            p = e / (e.sum() + torch.exp(w["m.sink"][a]))
            o = (p[:, None] * (c[:t + 1] @ w["m.uv"][a * V:(a + 1) * V].T)).sum(0)
            want[t, a] = o * torch.sigmoid(h[t] @ w["m.g"][a])
    assert torch.allclose(got, want.reshape(n, H * V) @ w["m.o"].T, rtol=1e-8, atol=1e-9)
    # at the first position the only key shares the denominator with the sink: the weight is below 1 by exactly that
    big = dict(w)
    big["m.sink"] = w["m.sink"] + 30.0
    assert float(pz.latent_attention(m, big, "m.", h, 1e-6).abs().max()) < 1e-6 * float(got.abs().max())


def moe_weights(hidden, E, I, shared, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    w = {"f.router": torch.randn(E, hidden, generator=g) * std, "f.correction": torch.randn(E, generator=g) * 0.5}
    for e in range(E):
        w[f"f.e{e}.up"], w[f"f.e{e}.down"] = torch.randn(I, hidden, generator=g) * std, torch.randn(hidden, I, generator=g) * std
    if shared:
        w["f.shared.up"], w["f.shared.down"] = torch.randn(shared, hidden, generator=g) * std, torch.randn(hidden, shared, generator=g) * std
        w["f.shared.sg"] = torch.randn(1, hidden, generator=g) * std
    return w


def test_experts_are_chosen_with_the_correction_and_weighted_without_it():
    hidden, E, I = 16, 6, 8
    w = moe_weights(hidden, E, I, 12, 7)
    f = {"router": {"experts": E, "top": 2, "scale": 1.5}, "shared": {"ff": 12}}
    h = torch.randn(30, hidden, generator=torch.Generator().manual_seed(8))
    pick, wt, s = pz.choose_experts(f, w, "f.", h)
    assert torch.allclose(wt.sum(-1), torch.full((30,), 1.5), atol=1e-5)         # divided by their sum, times the scale
    plain_pick = torch.topk(s, 2, dim=-1).indices
    assert (pick.sort(-1).values != plain_pick.sort(-1).values).any()              # the correction changes choices
    assert torch.allclose(wt, torch.gather(s, 1, pick) / torch.gather(s, 1, pick).sum(-1, keepdim=True) * 1.5)
    y = pz.moe(f, w, "f.", h)
    t = 3
    want = sum(wt[t, j] * (torch.relu(w[f"f.e{int(pick[t, j])}.up"] @ h[t]) ** 2) @ w[f"f.e{int(pick[t, j])}.down"].T
               for j in range(2))
    want = want + torch.sigmoid(w["f.shared.sg"] @ h[t]) * ((torch.relu(w["f.shared.up"] @ h[t]) ** 2) @ w["f.shared.down"].T)
    assert torch.allclose(y[t], want, atol=1e-5)


def test_a_prefix_of_a_sequence_gives_the_same_logits_and_every_layer_kind_matters():
    import tempfile
    import pathlib

    import plain_qwen2moe as reader
    from zanezen_configs import make_folder

    folder = make_folder(pathlib.Path(tempfile.mkdtemp()), "B")
    cfg, w = reader.load_model(folder, torch.float32)
    toks = [5, 17, 3, 90, 41, 7, 7, 60, 2, 33, 18, 4]
    full, layers = pz.forward(cfg, w, toks, return_layers=True)
    assert layers.shape == (6, len(toks), 72)
    assert torch.allclose(pz.forward(cfg, w, toks[:7]), full[:7], atol=1e-5)
    # no multiplier on the residual sum in this configuration; with one, everything moves
    half = dict(cfg, residual_mult=0.5)
    assert float((pz.forward(half, w, toks) - full).abs().max()) > 1e-2
    for i in range(6):       # every layer's mixer shows in the logits
        w2 = dict(w)
        w2[f"l{i}.mix.o"] = w[f"l{i}.mix.o"] * 0
        assert float((pz.forward(cfg, w2, toks) - full).abs().max()) > 1e-3, i
