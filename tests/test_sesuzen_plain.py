"""Sesuzen without a GPU: the configuration reader, the description made of parts (the loop's schedule, the size that
only a checkpoint's shapes give), the cache needs of its layers, and the plain implementation against restatements
of its mechanisms as explicit loops."""
import copy
import math

import pytest
import torch

import plain_sesuzen as pz
from sesuzen_configs import CONFIGS, SESUZEN_A, SESUZEN_B, SESUZEN_C


def resolve(cfg, shapes=None):
    import ferrox_b200  # noqa: F401  (registers the architectures)
    from ferrox_b200.config.registry import resolve as r

    return r(cfg, shapes) if shapes is not None else r(cfg)


def test_configuration_is_read_layer_by_layer():
    cfg, spec = resolve(SESUZEN_A)
    assert [l.type for l in cfg.layers] == ["general_delta", "attention", "general_delta", "attention"]
    assert cfg.taps == 3 and cfg.norm_eps == 1e-5 and cfg.logit_softcap == 12.0 and cfg.loop == (1, 3, 2)
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first) == (4, 2, 32, 48, 0.21, 21, 5)
    assert cfg.layers[1].mlp.top == 2 and cfg.layers[0].mlp.ff == 96 and cfg.layers[2].mlp is None
    # four blocks own weights; six schedule entries, each run of a layer with a cache of its own
    assert len(spec.layers) == 4
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (3, 5)]
    cfgB, specB = resolve(SESUZEN_B)
    assert cfgB.loop is None and cfgB.logit_softcap is None and cfgB.taps == 1
    assert [(e.layer, e.cache) for e in specB.schedule] == [(i, i) for i in range(5)]
    assert cfgB.layers[0].mixer.keep_first == 0 and cfgB.layers[3].mixer.window is None
    assert cfgB.layers[0].mixer.kv_heads == 3
    cfgC, specC = resolve(SESUZEN_C)
    assert [(e.layer, e.cache) for e in specC.schedule] == [(0, 0), (0, 1), (0, 2), (1, 3), (2, 4)]


def test_loop_that_changes_nothing_is_no_loop():
    for loop in ({"start": 2, "stop": 2, "times": 5}, {"start": 0, "stop": 3, "times": 1}, None):
        c = copy.deepcopy(SESUZEN_A)
        c["loop"] = loop
        cfg, spec = resolve(c)
        assert cfg.layer_runs() == (0, 1, 2, 3) and len(spec.schedule) == 4
    c = copy.deepcopy(SESUZEN_A)
    c["loop"] = {"start": 0, "stop": 4, "times": 3}
    assert resolve(c)[0].layer_runs() == (0, 1, 2, 3) * 3
    c["loop"] = {"start": 3, "stop": 4, "times": 2}
    assert resolve(c)[0].layer_runs() == (0, 1, 2, 3, 3)
    assert pz.layer_runs(c) == [0, 1, 2, 3, 3]


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="ring"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "not implemented"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3, stop=2), "loop"),
    (lambda c: c["canon"].update(taps=0), "taps"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c.update(layers=[]), "empty"),
])
def test_configurations_that_are_refused(change, text):
    from ferrox_b200 import ConfigError

    cfg = copy.deepcopy(SESUZEN_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        resolve(cfg)


def test_description_declares_the_tensors_and_the_cache_needs():
    from ferrox_b200.parts.build import build_model

    _, spec = resolve(SESUZEN_A)
    model = build_model(spec)
    decls = {d.name: d.shape for d in model.tensor_decls()}
    assert decls["embed"] == (211, 64) and decls["pos"] == (512, 64) and "head" not in decls
    assert decls["final.norm"] == (64,) and decls["final.norm.b"] == (64,)
    assert decls["l0.norm1.b"] == (64,) and decls["l0.canon1"] == (64, 3)
    assert decls["l0.mix.r"] == (2 * 16, 64) and decls["l0.mix.w1"] == (16, 64) and decls["l0.mix.w2"] == (32, 16)
    assert decls["l0.mix.a.b"] == (32,) and decls["l0.mix.norm"] == (32,) and decls["l0.mlp.up"] == (96, 64)
    assert decls["l1.mix.q"] == (4 * 32, 64) and decls["l1.mix.v"] == (2 * 48, 64) and decls["l1.mix.v.b"] == (96,)
    assert decls["l1.mix.g"] == (4 * 48, 64) and decls["l1.mix.o"] == (64, 4 * 48) and "l1.mix.g.b" not in decls
    assert decls["l1.mlp.router"] == (6, 64) and decls["l1.mlp.e5.down"] == (64, 32)
    assert decls["l2.mix.w1"] == (8, 64) and not any(n.startswith("l2.mlp.") for n in decls)
    caches = model.cache_specs()
    assert len(caches) == 6
    assert [(c.paged.window, c.paged.keep_first) if c.paged else None for c in caches] == \
        [None, (21, 5), None, (21, 5), None, (9, 9)]
    names = [[n for n, _ in c.state.parts] for c in caches]
    assert names[0] == ["matrix", "input_conv.tail"] and names[1] == ["input_conv.tail"]
    assert dict(caches[0].state.parts)["matrix"] == (2, 16, 16) and dict(caches[1].state.parts)["input_conv.tail"] == (2, 64)
    assert [t.token_shape for t in caches[1].paged.tensors] == [(2, 32), (2, 48)]


def test_a_checkpoint_s_shapes_give_the_decay_s_inner_width():
    from ferrox_b200.parts.build import build_model

    cfg = copy.deepcopy(SESUZEN_B)
    del cfg["layers"][1]["mixer"]["decay_rank"]
    _, spec = resolve(cfg, {"l1.mix.w1": (7, 72), "l4.mix.w1": (2, 72)})
    decls = {d.name: d.shape for d in build_model(spec).tensor_decls()}
    assert decls["l1.mix.w1"] == (7, 72) and decls["l1.mix.w2"] == (36, 7) and decls["l4.mix.w2"] == (40, 2)


def _weights(cfg, seed, dtype=torch.float32):
    from ferrox_b200.parts.build import build_model
    from ferrox_b200.weights.random_init import random_tensors

    _, spec = resolve(cfg)
    return {n: t.to(dtype) for n, t in random_tensors(build_model(spec).tensor_decls(), seed, torch.bfloat16, 0.15, "around_one")}


def test_plain_layer_norm_and_convolution_against_loops():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 10, generator=g, dtype=torch.float64) * 3 + 1
    w, b = torch.randn(10, generator=g, dtype=torch.float64), torch.randn(10, generator=g, dtype=torch.float64)
    got = pz.layer_norm(x, w, b, 1e-3)
    for t in range(9):
        mu = sum(float(v) for v in x[t]) / 10
        var = sum((float(v) - mu) ** 2 for v in x[t]) / 10
        for c in range(10):
            assert abs(float(got[t, c]) - ((float(x[t, c]) - mu) / math.sqrt(var + 1e-3) * float(w[c]) + float(b[c]))) < 1e-12
    for taps in (1, 2, 4, 6):
        cw = torch.randn(10, taps, generator=g, dtype=torch.float64)
        got = pz.input_convolution(x, cw)
        for t in range(9):
            for c in range(10):
                s = float(x[t, c])
                for j in range(taps):
                    src = t - taps + 1 + j
                    if src >= 0:
                        s += float(cw[c, j]) * float(x[src, c])       # (the last tap weighs the token itself)
                assert abs(float(got[t, c]) - s) < 1e-12
    assert float((pz.unit_rms(x, 1e-3) - x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3)).abs().max()) == 0


def test_plain_attention_against_loops():
    """Visibility, the norm of the values, the scale and the gate written out query by query and key by key."""
    for cfg, li in ((SESUZEN_A, 1), (SESUZEN_B, 2), (SESUZEN_B, 0), (SESUZEN_B, 3)):
        w = _weights(cfg, 3, torch.float64)
        m, p = cfg["layers"][li]["mixer"], f"l{li}.mix."
        n = 40
        h = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(1), dtype=torch.float64)
        eps = cfg["norm"]["eps"]
        want = pz.mixer_attention(h, m, w, p, eps)
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        mask = m.get("mask")
        out = torch.zeros(n, H * V, dtype=torch.float64)
        vals = []
        for j in range(n):
            v = (w[p + "v"] @ h[j] + w[p + "v.b"]).view(G, V)
            vals.append(torch.stack([v[g] / torch.sqrt((v[g] * v[g]).sum() / V + eps) for g in range(G)]))
        for i in range(n):
            for hd in range(H):
                q = w[p + "q"][hd * D:(hd + 1) * D] @ h[i] + w[p + "q.b"][hd * D:(hd + 1) * D]
                kv = hd // (H // G)
                seen = [j for j in range(i + 1)
                        if mask is None or i - j < mask["size"] or j < mask.get("keep_first", 0)]
                sc = torch.stack([(q @ (w[p + "k"][kv * D:(kv + 1) * D] @ h[j] + w[p + "k.b"][kv * D:(kv + 1) * D])) * m["scale"]
                                  for j in seen])
                pr = torch.softmax(sc, 0)
                out[i, hd * V:(hd + 1) * V] = sum(pj * vals[j][kv] for pj, j in zip(pr, seen))
        out = out * torch.sigmoid(h @ w[p + "g"].T)
        assert float((out @ w[p + "o"].T - want).abs().max()) < 1e-10


def test_plain_visibility_at_the_edges():
    ok = pz.visible(12, size=4, keep_first=2)
    assert ok[7].tolist() == [True, True, False, False, True, True, True, True, False, False, False, False]
    assert ok[3].tolist()[:5] == [True, True, True, True, False]
    assert pz.visible(5, size=1)[4].tolist() == [False, False, False, False, True]
    assert pz.visible(5)[4].all() and not pz.visible(5)[2, 3]
    big = pz.visible(6, size=2, keep_first=50)        # more kept than the sequence has: all earlier ones
    assert torch.equal(big, pz.visible(6))


def test_plain_delta_rule_against_loops_and_from_a_carried_state():
    g = torch.Generator().manual_seed(4)
    n, H, D = 11, 2, 5
    r, k, v = (torch.randn(n, H, D, generator=g, dtype=torch.float64) for _ in range(3))
    w = torch.rand(n, H, D, generator=g, dtype=torch.float64) * 0.4 + 0.6
    a = torch.rand(n, H, D, generator=g, dtype=torch.float64)
    got, S_end = pz.delta_recurrence(r, k, v, w, a)
    S = [[[0.0] * D for _ in range(D)] for _ in range(H)]
    for t in range(n):
        for hd in range(H):
            kk = [float(x) for x in k[t, hd]]
            ln = math.sqrt(sum(x * x for x in kk) + 1e-6)
            u = [x / ln for x in kk]
            old = S[hd]
            d = [sum(u[i] * old[i][j] for i in range(D)) for j in range(D)]
            new = [[float(w[t, hd, i]) * old[i][j] - float(a[t, hd, i]) * u[i] * d[j] + kk[i] * float(v[t, hd, j])
                    for j in range(D)] for i in range(D)]
            S[hd] = new
            for j in range(D):
                o = sum(new[i][j] * float(r[t, hd, i]) for i in range(D))
                assert abs(o - float(got[t, hd, j])) < 1e-10
    assert float((torch.tensor(S, dtype=torch.float64) - S_end).abs().max()) < 1e-10
    # a request cut in two: the second part starts from the state the first left
    first, S_mid = pz.delta_recurrence(r[:6], k[:6], v[:6], w[:6], a[:6])
    second, S_two = pz.delta_recurrence(r[6:], k[6:], v[6:], w[6:], a[6:], S_mid)
    assert float((torch.cat([first, second]) - got).abs().max()) < 1e-12 and float((S_two - S_end).abs().max()) < 1e-12


def test_plain_delta_inputs_are_decays_and_rates_between_their_bounds():
    cfg = SESUZEN_A
    wt = _weights(cfg, 5, torch.float64)
    h = torch.randn(30, cfg["width"], generator=torch.Generator().manual_seed(2), dtype=torch.float64) * 4
    r, k, v, w, a = pz.delta_inputs(h, cfg["layers"][0]["mixer"], wt, "l0.mix.")
    assert float(w.min()) > math.exp(-math.exp(-0.5)) and float(w.max()) < 1.0
    assert float(a.min()) > 0.0 and float(a.max()) < 1.0
    z = torch.tanh(h @ wt["l0.mix.w1"].T) @ wt["l0.mix.w2"].T + wt["l0.mix.w0"]
    assert float((w.reshape(30, -1) - torch.exp(-0.6065306597126334 / (1 + torch.exp(-z)))).abs().max()) < 1e-12


def test_plain_experts_against_loops():
    for cfg, li in ((SESUZEN_A, 1), (SESUZEN_B, 0), (SESUZEN_B, 1)):
        wt = _weights(cfg, 6, torch.float64)
        f, p = cfg["layers"][li]["mlp"], f"l{li}.mlp."
        x = torch.randn(17, cfg["width"], generator=torch.Generator().manual_seed(3), dtype=torch.float64)
        got = pz.ffn_moe(x, f, wt, p)
        E, top = f["router"]["experts"], f["router"]["top"]
        for t in range(17):
            z = [float(wt[p + "router"][e] @ x[t]) for e in range(E)]
            chosen = sorted(range(E), key=lambda e: -z[e])[:top]
            mx = max(z[e] for e in chosen)
            den = sum(math.exp(z[e] - mx) for e in chosen)
            y = torch.zeros(cfg["width"], dtype=torch.float64)
            for e in chosen:
                gt = wt[p + f"e{e}.gate"] @ x[t]
                up = wt[p + f"e{e}.up"] @ x[t]
                y += math.exp(z[e] - mx) / den * (wt[p + f"e{e}.down"] @ (gt / (1 + torch.exp(-gt)) * up))
            assert float((y - got[t]).abs().max()) < 1e-10
    x = torch.randn(5, 64, dtype=torch.float64)
    wt = _weights(SESUZEN_A, 6, torch.float64)
    z = torch.clamp(x @ wt["l0.mlp.up"].T, min=0)
    assert float((pz.ffn_dense(x, wt, "l0.mlp.") - (z * z) @ wt["l0.mlp.down"].T).abs().max()) < 1e-12


def test_plain_whole_model_equals_its_prefixes_and_the_loop_unrolled():
    """Causal: the logits of a prefix do not change when tokens follow.  A loop equals the same model with the looped
    layers written out under names of their own; the cap bounds the logits."""
    for name, (cfg, seed) in CONFIGS.items():
        w = _weights(cfg, seed)
        toks = [(7 * i + 3) % cfg["vocab"] for i in range(45)]
        full, layers = pz.forward(cfg, w, toks, return_layers=True)
        assert layers.shape[0] == len(pz.layer_runs(cfg))
        assert float((pz.forward(cfg, w, toks[:20]) - full[:20]).abs().max()) < 1e-4, name
        if cfg.get("logit_softcap"):
            assert float(full.abs().max()) <= cfg["logit_softcap"]
        if cfg.get("loop"):
            runs = pz.layer_runs(cfg)
            flat = copy.deepcopy(cfg)
            flat["loop"] = None
            flat["layers"] = [copy.deepcopy(cfg["layers"][i]) for i in runs]
            w2 = {k: v for k, v in w.items() if not k.startswith("l")}
            for new, old in enumerate(runs):
                for k, v in w.items():
                    if k.startswith(f"l{old}."):
                        w2[f"l{new}." + k[len(f"l{old}."):]] = v
            assert float((pz.forward(flat, w2, toks) - full).abs().max()) < 1e-5, name


def test_plain_positions_enter_through_the_table_only():
    """The same token at two positions differs by the position rows alone (before the first layer)."""
    cfg = SESUZEN_B
    w = _weights(cfg, 2)
    one = pz.forward(cfg, w, [5])
    w2 = dict(w)
    w2["pos"] = torch.roll(w["pos"], 1, dims=0)
    other = pz.forward(cfg, w2, [9, 5])      # token 5 now sits at position 1 and reads the row that was row 0
    assert float((one[0] - other[1]).abs().max()) > 1e-3      # ... but it also reads the token before it
    w3 = dict(w)
    w3["pos"] = torch.zeros_like(w["pos"])
    assert float((pz.forward(cfg, w3, [5])[0] - one[0]).abs().max()) > 1e-3
