"""The engine's Zanezen model against the plain implementation: every mechanism alone, then whole models under every
way of cutting the work (whole prompts, a decoded tail, portions down to two tokens, mixed batches with pages and
slots used again, long decoding, generation through the scheduler), in 32-bit and in bfloat16, on configurations
that differ in every size, constant and in the order of layers."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_zanezen as pz
import replay_util as ru
from test_safepel_gpu import CUTS, MixerHarness, load_part, random_tensors, rel, run_in_cuts
from zanezen_configs import CONFIGS, make_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": (torch.float32, 5e-5), "bfloat16": (torch.bfloat16, 3e-2)}


def inputs(hidden, lens, seed, dt, loud=None, by=None):
    """Rows for each request, rounded to the engine's element type; ``loud`` = (request, position): that row several
    times as large, so that whether a later query sees its key shows in the result."""
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(n, hidden, generator=g) for n in lens]
    if loud is not None:
        xs[loud[0]][loud[1]] *= by or (20.0 if dt == torch.float32 else 4.0)
    return [x.to(dt).float() for x in xs]


def floats(w):
    return {k: v.float() for k, v in w.items()}


# ------------------------------------------------------------------ mechanisms alone
def mlstm_spec(hidden, H, D, V, cap, eps=1e-5):
    from ferrox_b200.parts.specs import MlstmSpec

    return MlstmSpec(hidden=hidden, n_heads=H, head_dim=D, value_dim=V, gate_cap=cap, norm_eps=eps, prefix="m.")


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("H,D,V,cap", [(2, 16, 32, 10.0), (3, 12, 20, 15.0), (1, 40, 8, 2.0), (4, 64, 64, 15.0),
                                       (2, 128, 64, 6.0), (5, 4, 4, 1.0), (1, 100, 130, 15.0), (1, 300, 16, 15.0)])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_mlstm_alone(dtype, H, D, V, cap, cut):
    """The recurrence with its three states carried over every cut, two requests side by side, against the plain loop
    over tokens; the slots are then used again by requests that must start from empty states and a maximum of 0."""
    dt, tol = DTYPES[dtype]
    hidden = 64
    spec = mlstm_spec(hidden, H, D, V, cap)
    w = random_tensors(spec, seed=H + D, std=0.25)
    g = torch.Generator().manual_seed(D)
    w["m.i.b"] = (torch.randn(H, generator=g) * 2).to(torch.bfloat16)           # gates spread over their range
    w["m.f.b"] = (torch.randn(H, generator=g) * 2 + 2).to(torch.bfloat16)
    part, rt = load_part(spec, w, dt)
    xs = inputs(hidden, (150, 37), 3, dt)
    m = dict(heads=H, dim=D, vdim=V, gate_cap=cap)
    want = [pz.mlstm(m, floats(w), "m.", x, 1e-5) for x in xs]
    h = MixerHarness(part, rt, hidden, page_size=4, n_pages=8)
    got = run_in_cuts(h, xs, CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol
    got = run_in_cuts(h, xs[::-1], CUTS[cut])
    for a, b in zip(got, want[::-1]):
        assert rel(a, b) < tol


def test_mlstm_keeps_an_early_token_and_every_term_shows():
    """Forget gates near 1 (a large bias) and one early token made loud: it is still read four hundred tokens later.
    The plain implementation with a maximum that starts at minus infinity, without the cap, or without the floor of
    the denominator gives something else, so the comparison with the engine means each of them."""
    hidden, H, D, V = 64, 2, 16, 16
    spec = mlstm_spec(hidden, H, D, V, 8.0)
    w = random_tensors(spec, seed=9, std=0.25)
    w["m.f.b"] = torch.full((H,), 7.0).to(torch.bfloat16)
    w["m.i.b"] = torch.full((H,), -1.0).to(torch.bfloat16)
    wf = floats(w)
    m = dict(heads=H, dim=D, vdim=V, gate_cap=8.0)
    xs = inputs(hidden, (450,), 5, torch.float32, loud=(0, 3), by=6.0)
    want = pz.mlstm(m, wf, "m.", xs[0], 1e-5)
    quiet = xs[0].clone()
    quiet[3] /= 6.0
    assert rel(pz.mlstm(m, wf, "m.", quiet, 1e-5)[400:], want[400:]) > 0.02          # the early token is still read
    assert rel(pz.mlstm(dict(m, gate_cap=2.0), wf, "m.", xs[0], 1e-5), want) > 0.02  # the cap shows
    neg = dict(wf)
    neg["m.i.b"] = wf["m.i.b"] - 6.0                                                   # gates below the maximum's start
    a = pz.mlstm(m, neg, "m.", xs[0][:20], 1e-5)
    part, rt = load_part(spec, {k: v.to(torch.bfloat16) for k, v in neg.items()}, torch.float32)
    got = run_in_cuts(MixerHarness(part, rt, hidden, page_size=4, n_pages=8), [xs[0][:20]], [(7,), (1,), (12,)])
    assert rel(got[0], a) < 5e-5                                                       # m starts at 0: the floor is exp(-0)
    part, rt = load_part(spec, w, torch.float32)
    got = run_in_cuts(MixerHarness(part, rt, hidden, page_size=4, n_pages=8, max_positions=1024), xs,
                      [(300,), (3,)] + [(1,)] * 147)
    assert rel(got[0], want) < 5e-5


def diff_spec(hidden, H, G, D, V, scale, diff, taps=None, rotary=None, softcap=None, eps=1e-5):
    from ferrox_b200.parts.specs import DifferentialAttentionSpec, ScaledRotarySpec

    pos = None
    if rotary:
        sc = rotary.get("scaling")
        f, o, fa, sl = (sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else (None, 0.0, 0.0, 0.0)
        pos = ScaledRotarySpec(rotary_dim=rotary["dims"], theta=rotary["base"], factor=f, original=o, fast=fa, slow=sl)
    return DifferentialAttentionSpec(hidden=hidden, n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, diff=diff,
                                     scale=scale, softcap=softcap, conv_taps=taps, position=pos, norm_eps=eps, prefix="m.")


def diff_mixer(H, G, D, V, scale, diff, taps, rotary, softcap):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=scale, diff=diff)
    if taps:
        m["conv"] = taps
    if rotary:
        m["rot"] = rotary
    if softcap:
        m["softcap"] = softcap
    return m


SCALED = {"dims": 16, "base": 500.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
# beside the cuts of the other mixers' tests: portions of two requests in one step that are long enough for the
# prompt form of the convolution kernel, the second request beginning in the middle of a run of tokens
DIFF_CUTS = dict(CUTS, **{"large portions": [(70, 30), (50, 7), (30, 0)]})


@pytest.mark.parametrize("cut", list(DIFF_CUTS))
@pytest.mark.parametrize("H,G,D,V,taps,rotary,softcap,page", [
    (4, 2, 32, 48, 4, SCALED, 20.0, 4), (3, 3, 20, 12, 3, {"dims": 8, "base": 1000.0}, 5.0, 8), (6, 1, 24, 40, None, None, None, 16),
    (8, 1, 64, 128, 5, {"dims": 32, "base": 20000.0, "scaling": {"factor": 2.0, "original": 256, "fast": 32.0, "slow": 1.0}}, 30.0, 64),
    (2, 2, 16, 16, 2, {"dims": 16, "base": 10000.0}, None, 8), (1, 1, 40, 80, 16, {"dims": 2, "base": 10.0}, 50.0, 16),
    (40, 1, 16, 16, 1, None, 3.0, 16)])      # (the last: more query rows on a kv head than a tile has)
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_differential_attention_alone(dtype, H, G, D, V, taps, rotary, softcap, page, cut):
    """Convolution tails, rotation and both maps over shared values under every cut, two requests side by side; then
    the slots and pages are used again."""
    dt, tol = DTYPES[dtype]
    hidden = 64
    spec = diff_spec(hidden, H, G, D, V, 0.3, 0.35, taps, rotary, softcap)
    w = random_tensors(spec, seed=H + D, std=0.25)
    part, rt = load_part(spec, w, dt)
    xs = inputs(hidden, (150, 37), 3, dt)
    m = diff_mixer(H, G, D, V, 0.3, 0.35, taps, rotary, softcap)
    want = [pz.differential_attention(m, floats(w), "m.", x, 1e-5) for x in xs]
    if dtype == "bfloat16":
        with pz.rounded_to(torch.bfloat16):     # the difference of two rounded maps, normed: rounding is amplified
            tol = max(tol, 4 * max(rel(pz.differential_attention(m, floats(w), "m.", x, 1e-5), b) for x, b in zip(xs, want)))
    h = MixerHarness(part, rt, hidden, page_size=page, n_pages=256 // page + 8)
    got = run_in_cuts(h, xs, DIFF_CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol
    got = run_in_cuts(h, xs[::-1], [(b, a) for a, b in DIFF_CUTS[cut]] if cut == "large portions" else DIFF_CUTS[cut])
    for a, b in zip(got, want[::-1]):
        assert rel(a, b) < tol


def test_differential_attention_every_term_shows_and_a_far_key_is_read():
    """The plain implementation against variants with one term changed (no second map, no cap, plain frequencies, no
    factor on cos and sin, another lambda, the convolution's earlier taps dropped): each gives something else.  Then
    seven hundred positions with the key of position 5 made to stand out in both maps' first map only: far queries
    read it, across many pages, in a prompt's portion and decoded one by one."""
    hidden, H, G, D, V = 64, 4, 2, 32, 32
    m = diff_mixer(H, G, D, V, 0.3, 0.35, 4, SCALED, 20.0)
    spec = diff_spec(hidden, H, G, D, V, 0.3, 0.35, 4, SCALED, 20.0)
    w = random_tensors(spec, seed=11, std=0.25)
    wf = floats(w)
    x = inputs(hidden, (90,), 2, torch.float32)[0] * 1.5
    want = pz.differential_attention(m, wf, "m.", x, 1e-5)
    plain = lambda mm, ww=wf: pz.differential_attention(mm, ww, "m.", x, 1e-5)
    assert rel(plain(dict(m, softcap=None)), want) > 1e-3
    assert rel(plain(dict(m, rot={"dims": 16, "base": 500.0})), want) > 1e-3
    assert rel(plain(dict(m, rot=dict(SCALED, scaling=dict(SCALED["scaling"], factor=1.0)))), want) > 1e-3
    assert rel(plain(dict(m, diff=0.2)), want) > 1e-3
    for name in ("q.conv", "k.conv", "v.conv"):
        cut = dict(wf)
        cut["m." + name] = wf["m." + name].clone()
        cut["m." + name][:, :-1] = 0
        assert rel(plain(m, cut), want) > 1e-3
    one = dict(wf)
    one["m.lq2"] = wf["m.lq2"] * 0 + 1.0          # lambda moves with the four small vectors
    assert rel(plain(m, one), want) > 1e-3
    # a far key: queries of map 1 follow their key head's weights, so that one loud row wins the softmax from far away
    for h in range(H):
        g = h // (H // G)
        w["m.q"][(h * 2) * D:(h * 2 + 1) * D] = (w["m.k"][(g * 2) * D:(g * 2 + 1) * D].float()
                                                 + 0.3 * w["m.q"][(h * 2) * D:(h * 2 + 1) * D].float()).to(torch.bfloat16)
    for name in ("q.conv", "k.conv"):              # the convolution hands the newest input on, so that keys stay apart
        w["m." + name][:, :-1] = (w["m." + name][:, :-1].float() * 0.1).to(torch.bfloat16)
    wf = floats(w)
    m2 = dict(m, rot=None, softcap=None)
    spec2 = diff_spec(hidden, H, G, D, V, 0.3, 0.35, 4, None, None)
    xs = inputs(hidden, (700, 9), 4, torch.float32, loud=(0, 5), by=5.0)
    want = [pz.differential_attention(m2, wf, "m.", x, 1e-5) for x in xs]
    quiet = xs[0].clone()
    quiet[5] /= 5.0
    assert rel(pz.differential_attention(m2, wf, "m.", quiet, 1e-5)[600:], want[0][600:]) > 0.02
    for dtype, (dt, tol) in DTYPES.items():
        part, rt = load_part(spec2, w, dt)
        got = run_in_cuts(MixerHarness(part, rt, hidden, page_size=16, n_pages=64, max_positions=1024),
                          [x.to(dt).float() for x in xs], [(560, 0), (3, 9)] + [(1, 0)] * 137)
        if dtype == "float32":
            for a, b in zip(got, want):
                assert rel(a, b) < tol
        else:
            assert torch.isfinite(got[0]).all() and rel(got[0][600:], want[0][600:]) < 0.25


def latent_spec(hidden, H, D, R, V, C, scale, rotary, eps=1e-5):
    from ferrox_b200.parts.specs import LatentAttentionSpec

    sc = rotary.get("scaling")
    return LatentAttentionSpec(
        hidden=hidden, n_heads=H, head_dim=D, rot_dim=R, value_dim=V, kv_rank=C, q_rank=None, rotary_dims=rotary["dims"],
        rotary_base=rotary["base"], window=None, scale=scale, output_gate=True, norm_eps=eps, prefix="m.",
        rotary_pairing="halves", rotary_scaling=(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None,
        gate_per_head=True, sink="sink")


@pytest.mark.parametrize("form", ["latent", "expanded"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("H,D,R,V,C,rotary,page", [
    (4, 16, 32, 16, 48, {"dims": 16, "base": 10000.0}, 4), (3, 12, 6, 20, 40, {"dims": 4, "base": 77.0,
     "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}, 8),
    (8, 64, 64, 64, 192, {"dims": 64, "base": 250000.0}, 64), (1, 24, 8, 28, 36, {"dims": 8, "base": 1000.0}, 16),
    (5, 48, 32, 64, 80, {"dims": 32, "base": 100000.0}, 16)])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_latent_attention_with_a_sink_and_a_gate_per_head_alone(dtype, H, D, R, V, C, rotary, page, cut, form, monkeypatch):
    from ferrox_b200.parts import latent_attention as la

    if form == "expanded" and (dtype != "bfloat16" or (D + R) % 16 or V % 16 or C % 8):
        pytest.skip("prompt portions read out of the latent first only in bfloat16 at sizes in steps of 16")
    monkeypatch.setattr(la, "EXPANDED_MAX_COST_RATIO", 1e9 if form == "expanded" else 0.0)
    dt, tol = DTYPES[dtype]
    hidden = 64
    scale = round(0.12 / math.sqrt(D + R), 4)      # scores of the order of one, so that the sink weighs in everywhere
    spec = latent_spec(hidden, H, D, R, V, C, scale, rotary)
    w = random_tensors(spec, seed=H + D, std=0.25)
    w["m.sink"] = (torch.randn(H, generator=torch.Generator().manual_seed(C)) * 1.5 + 5.0).to(torch.bfloat16)
    part, rt = load_part(spec, w, dt)
    xs = inputs(hidden, (150, 37), 3, dt)
    m = dict(heads=H, dim=D, rot_dim=R, vdim=V, kv_rank=C, scale=scale, rot=rotary)
    wf = floats(w)
    want = [pz.latent_attention(m, wf, "m.", x, 1e-5) for x in xs]
    gone = dict(wf)
    gone["m.sink"] = wf["m.sink"] - 40.0
    assert rel(pz.latent_attention(m, gone, "m.", xs[0], 1e-5), want[0]) > 0.05        # the sink shows, also far back
    assert rel(pz.latent_attention(m, gone, "m.", xs[0], 1e-5)[120:], want[0][120:]) > 0.05
    h = MixerHarness(part, rt, hidden, page_size=page, n_pages=256 // page + 8)
    got = run_in_cuts(h, xs, CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol
    got = run_in_cuts(h, xs[::-1], CUTS[cut])
    for a, b in zip(got, want[::-1]):
        assert rel(a, b) < tol


@pytest.mark.parametrize("E,top,shared", [(6, 2, 64), (3, 3, 24), (5, 1, 0), (8, 3, 128), (1, 1, 8)])
@pytest.mark.parametrize("tokens", [1, 5, 40, 300])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_experts_chosen_with_a_correction_alone(dtype, tokens, E, top, shared):
    from ferrox_b200.engine.batch import StepEntry, flatten
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.specs import MoeSpec

    dt, tol = DTYPES[dtype]
    hidden, I = 64, 32
    spec = MoeSpec(hidden=hidden, n_experts=E, top_k=top, expert_intermediate=I, shared_intermediate=shared,
                   norm_topk_prob=True, shared_gate=shared > 0, prefix="f.", scores="sigmoid",
                   tensor_names=("router", "e{e}.{part}", "shared.{part}"), plain_activation="relu_square",
                   choice_bias="correction", weight_scale=1.7, renorm_eps=1e-20, shared_gate_name="shared.sg")
    w = random_tensors(spec, seed=tokens + top, std=0.2)
    w["f.correction"] = (torch.randn(E, generator=torch.Generator().manual_seed(E)) * 0.4).to(torch.bfloat16)
    part, rt = load_part(spec, w, dt)
    x = (inputs(hidden, [tokens], 5, dt)[0] * 2.0).to(dt).float()
    f = {"router": {"experts": E, "top": top, "scale": 1.7}, "expert": {"ff": I}, "shared": {"ff": shared} if shared else None}
    wf = floats(w)
    want = pz.moe(f, wf, "f.", x)
    if 1 < top < E and tokens >= 40:
        # the test can tell: without the correction other experts are chosen; with it in the weights they differ
        flat = dict(wf)
        flat["f.correction"] = wf["f.correction"] * 0
        assert rel(pz.moe(f, flat, "f.", x), want) > 0.05
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = flatten([StepEntry(0, [0] * tokens, start=0)], torch.device(DEV), status, ops.stream_ptr())
    h = torch.zeros(tokens, hidden, dtype=torch.float32, device=DEV)
    part.forward_add(x.to(DEV).to(dt), h, batch)
    torch.cuda.synchronize()
    if dtype == "bfloat16" and top < E:
        # a position whose choice scores separate the last chosen expert from the next by less than bfloat16 rounding
        # may rightly choose the other one: leave those rows out, and require them to be few
        clear = pz.router_margins(f, wf, "f.", x) > 0.02
        assert tokens < 40 or clear.float().mean() > 0.5
        if clear.any():
            assert rel(h.cpu()[clear], want[clear]) < tol
    else:
        assert rel(h, want) < tol


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_gated_feed_forward_with_biases_alone(dtype):
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.specs import DenseMlpSpec

    dt, tol = DTYPES[dtype]
    for hidden, ff in ((96, 160), (72, 50), (256, 448)):
        spec = DenseMlpSpec(hidden=hidden, intermediate=ff, prefix="f.", tensor_names=("gate", "up", "down"),
                            bias_names=("gate.b", "up.b", "down.b"))
        w = random_tensors(spec, std=0.2)
        for n in ("gate.b", "up.b", "down.b"):
            w["f." + n] = (w["f." + n].float() * 5).to(torch.bfloat16)
        part, rt = load_part(spec, w, dt)
        wf = floats(w)
        for T in (1, 3, 20, 70, 300, 2304):     # the decode-sized and the prompt-sized kernels, pairs of SMs
            x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(T)).to(dt)
            batch = SimpleNamespace(status=None, stream=ops.stream_ptr())
            out = torch.full((T, hidden), float("nan"), device=DEV)
            part.forward_into(x.to(DEV), out, batch, accumulate=False)
            want = pz.dense_mlp(wf, "f.", x.float())
            assert rel(out, want) < tol
            part.forward_into(x.to(DEV), out, batch, accumulate=True)       # added to what is there, the bias once more
            assert rel(out, 2 * want) < tol
            for n in ("gate.b", "up.b", "down.b"):                           # (the test can tell a missing bias)
                less = dict(wf)
                less["f." + n] = wf["f." + n] * 0
                assert rel(pz.dense_mlp(less, "f.", x.float()), want) > 0.01


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_residual_sum_with_a_multiplier_and_the_next_norm(dtype):
    from ferrox_b200.kernels import ops

    dt, tol = DTYPES[dtype]
    g = torch.Generator().manual_seed(1)
    for rows, hidden in ((1, 64), (7, 72), (300, 200), (5, 2048), (3, 5000)):
        h, y = torch.randn(rows, hidden, generator=g), torch.randn(rows, hidden, generator=g) * 3
        w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        hd, out = h.to(DEV), torch.empty(rows, hidden, dtype=dt, device=DEV)
        got = ops.scaled_add_norm(hd, y.to(DEV), 0.7, norm=(w.to(DEV), 3e-6, out))
        new = h + 0.7 * y
        assert got is out and rel(hd, new) < 1e-6
        assert rel(out, pz.rms(new, 3e-6) * w.float()) < (1e-5 if dt == torch.float32 else 1e-2)
        hd = h.to(DEV)
        assert ops.scaled_add_norm(hd, y.to(DEV), -1.25) is None and rel(hd, h - 1.25 * y) < 1e-6


def test_stretched_rotary_table_on_the_device():
    from ferrox_b200.parts.base import Runtime, build_part
    from ferrox_b200.parts import build  # noqa: F401
    from ferrox_b200.parts.specs import ScaledRotarySpec

    for dims, base, sc in ((16, 500.0, (4.0, 64.0, 8.0, 1.0)), (32, 20000.0, (2.0, 256.0, 32.0, 1.0)), (8, 1000.0, None),
                           (2, 10.0, (3.0, 8.0, 2.0, 1.0))):
        f, o, fa, sl = sc if sc else (None, 0.0, 0.0, 0.0)
        part = build_part(ScaledRotarySpec(rotary_dim=dims, theta=base, factor=f, original=o, fast=fa, slow=sl))
        part.load(None, Runtime(torch.device(DEV), torch.float32))
        want, mag = pz.rotary_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None)
        assert torch.equal(part.inv_freq.cpu(), want.to(torch.float32)) and abs(part.magnitude - mag) < 1e-12
        pos = torch.tensor([0, 1, 5, 1000, 70000], dtype=torch.int32, device=DEV)
        t = part.table(SimpleNamespace(shared={}, positions=pos, n_tokens=5, stream=None))
        ang = pos.cpu().float()[:, None] * want.to(torch.float32)[None, :]
        assert torch.allclose(t[..., 0].cpu(), torch.cos(ang) * mag, atol=2e-6)
        assert torch.allclose(t[..., 1].cpu(), torch.sin(ang) * mag, atol=2e-6)


# ------------------------------------------------------------------ whole models
def prompts_for(name, n=5, hi=150, seed=0):
    cfg = CONFIGS[name][0]
    rng = random.Random(seed)
    lens = [1, 2, hi] + [rng.randint(3, hi) for _ in range(max(0, n - 3))]
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(L)] for i, L in enumerate(lens)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zanezen_models")
    return {name: make_folder(tmp, name) for name in CONFIGS}


def position_errors(got, want):
    return (got - want).abs().amax(dim=-1) / want.abs().max()


def rounding_alone(cfg, w, tokens, want):
    """Per position: how far the plain implementation's logits move when everything that may be computed in bfloat16
    is rounded to it (a choice of experts that falls the other way under rounding moves a position by much more than
    the rounding itself: the measure of an engine in bfloat16 is this distribution, not a bound for every position)."""
    with pz.rounded_to(torch.bfloat16):
        return position_errors(pz.forward(cfg, w, tokens), want)


@pytest.fixture(scope="module")
def expected(folders):
    import plain_qwen2moe as reader

    out = {}
    for name in CONFIGS:
        cfg, w = reader.load_model(folders[name], torch.float32)
        want = {rid: pz.forward(cfg, w, t) for rid, t in prompts_for(name).items()}
        out[name] = (cfg, w, want, {rid: rounding_alone(cfg, w, t, want[rid]) for rid, t in prompts_for(name).items()})
    return out


def engine(folder, dtype, **kw):
    from ferrox_b200 import Engine

    kw.setdefault("page_size", 64 if folder.endswith("_C") else 8)     # C: the page size of serving
    kw.setdefault("n_pages", 64)
    kw.setdefault("max_slots", 4)
    return Engine.from_folder(folder, dtype=dtype, **kw)


def compare(got, want, tol, what, noise=None):
    """32-bit: every position within ``tol``.  bfloat16 (``noise``: what rounding alone does to the plain
    implementation at every position): the median and the ninth decile of the engine's distances over all positions
    lie within three times those of rounding alone, plus a hundredth and two."""
    errs = []
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        assert torch.isfinite(got[rid]).all(), (what, rid)
        e = position_errors(got[rid], want[rid])
        if noise is None:
            assert float(e.max()) < tol, (what, rid, float(e.max()), int(e.argmax()))
        errs.append(e)
    if noise is not None:
        e, n = torch.cat(errs), torch.cat([noise[rid] for rid in want])
        for q, slack in ((0.5, 1e-2), (0.9, 2e-2)):
            assert float(e.quantile(q)) <= 3 * float(n.quantile(q)) + slack, (what, q, float(e.quantile(q)), float(n.quantile(q)))


RUNS = {
    "whole": lambda eng, p: ru.run_whole(eng, p),
    "decoded tail": lambda eng, p: ru.run_tail_decode(eng, p, tail=50),
    "portions": lambda eng, p: ru.run_portions(eng, p),
    "decoding together": lambda eng, p: ru.run_decode_together(eng, p, tail=9),
    "mixed": lambda eng, p: ru.run_mixed(eng, p, seed=3, max_live=3),
}


@pytest.mark.parametrize("run", list(RUNS))
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_model_under_every_cut(folders, expected, dtype, name, run):
    _, tol = DTYPES[dtype]
    eng = engine(folders[name], dtype)
    got = RUNS[run](eng, prompts_for(name))
    compare(got, expected[name][2], tol, f"{name} {dtype} {run}", expected[name][3] if dtype == "bfloat16" else None)
    eng.cache.check_invariants()
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())   # all given back


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_agree_with_each_other_to_rounding(folders, name):
    eng = engine(folders[name], "float32")
    p = prompts_for(name)
    whole, mixed = ru.run_whole(eng, p), ru.run_mixed(eng, p, seed=5, max_live=4)
    for rid in p:
        assert float((whole[rid] - mixed[rid]).abs().max() / whole[rid].abs().max()) < 2e-5


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_residual_stream_after_every_layer(folders, expected, name):
    from ferrox_b200.engine.batch import StepEntry

    cfg, w = expected[name][:2]
    toks = prompts_for(name)["r3"]
    want_logits, after = pz.forward(cfg, w, toks, return_layers=True)
    eng = engine(folders[name], "float32")
    seen = []
    for i, block in enumerate(eng.model.layers):
        inner = block.forward

        def spy(h, batch, cache, _inner=inner, _i=i, **kw):
            out = _inner(h, batch, cache, **kw)
            seen.append((_i, h.detach().clone().cpu()))
            return out
        block.forward = spy
    slot = eng.open_request()
    got = eng.step([StepEntry(slot, toks, want=list(range(len(toks))))]).cpu()
    assert [i for i, _ in seen] == list(range(len(cfg["layers"])))
    for n, (_, h) in enumerate(seen):
        assert rel(h, after[n]) < 2e-5, n
    assert rel(got, want_logits) < 5e-5


@pytest.mark.parametrize("name", ["A", "C"])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding(folders, dtype, name):
    """A few tokens of prompt, then hundreds decoded one by one, across many pages, the recurrent states and the
    convolutions' tails moved on by every step."""
    import plain_qwen2moe as reader

    _, tol = DTYPES[dtype]
    cfg, w = reader.load_model(folders[name], torch.float32)
    rng = random.Random(9)
    n = 303 if name == "A" else 420
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    want = pz.forward(cfg, w, toks)
    eng = engine(folders[name], dtype, n_pages=40 if name == "A" else 8, max_slots=2)
    c = ru.Collector(eng)
    c.step({"x": toks[:3]})
    for t in toks[3:]:
        c.step({"x": [t]})
    compare({"x": c.stacked("x")}, {"x": want}, tol, "long decoding",
            {"x": rounding_alone(cfg, w, toks, want)} if dtype == "bfloat16" else None)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_scheduler(folders, name):
    import plain_qwen2moe as reader

    cfg, w = reader.load_model(folders[name], torch.float32)
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (5, 1, 23)]

    def greedy(p, n):
        toks = list(p)
        for _ in range(n):
            toks.append(int(pz.forward(cfg, w, toks)[-1].argmax()))
        return toks[len(p):]

    want = [greedy(p, 12) for p in prompts]
    eng = engine(folders[name], "float32")
    assert eng.graphs is not None            # every part of the model can be captured: decode steps replay graphs
    got = eng.generate(prompts, max_new_tokens=12, max_batch_tokens=16)     # prompts go in portions
    assert got == want
    again = eng.generate(prompts[::-1], max_new_tokens=12)                  # slots and pages used again
    assert again == want[::-1]
    bf = engine(folders[name], "bfloat16").generate(prompts, max_new_tokens=12)
    assert all(len(g) == 12 for g in bf)
    for p, g in zip(prompts, bf):
        logits = pz.forward(cfg, w, (p + g)[:-1])
        close = sum(float(logits[len(p) - 1 + i].max() - logits[len(p) - 1 + i][tok]) <= 2 * 6e-2 * float(logits.abs().max())
                    for i, tok in enumerate(g))
        assert close >= 10      # (a choice of experts within rounding may differ at a position or two)


def test_trace_replay_and_command_line_with_a_zanezen_folder(folders, tmp_path):
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    import plain_qwen2moe as reader

    cfg, w = reader.load_model(folders["B"], torch.float32)
    toks = [3, 90, 7, 7, 45, 21, 9, 81]
    want = pz.forward(cfg, w, toks)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks[:5], "want": [0, 4]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks[5:6], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": toks[6:], "want": [1]}, {"id": "b", "tokens": toks[:2], "want": [1]}],
         "end": ["a", "b"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1))
    assert rel(s0, want[[0, 4]]) < 5e-5 and rel(s2, want[[7, 1]]) < 5e-5
    nxt = [int(pz.forward(cfg, w, toks[:4])[-1].argmax())]
    nxt.append(int(pz.forward(cfg, w, toks[:4] + nxt)[-1].argmax()))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "ferrox"), "-m", folders["B"], "--tokens", "3,90,7,7",
                        "-n", "2", "--temp", "0", "--dtype", "float32", "--ignore-eos", "--repeat-penalty", "1.0"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == nxt


def test_preemption_and_decoding_ahead(folders):
    """A request that is preempted gives its pages and slot back and is recomputed (its states, its maximum and its
    convolution tails start again from zeros); greedy decode steps are replayed graphs issued one ahead of the host."""
    import plain_qwen2moe as reader

    cfg, w = reader.load_model(folders["B"], torch.float32)
    prompts = [[i + 1, i + 3, i + 7, 90, 4, 8, 15, 16] for i in range(4)]

    def greedy(p, n):
        toks = list(p)
        for _ in range(n):
            toks.append(int(pz.forward(cfg, w, toks)[-1].argmax()))
        return toks[len(p):]

    want = [greedy(p, 20) for p in prompts]
    small = engine(folders["B"], "float32", page_size=4, n_pages=14, max_slots=4)     # 4 x 28 positions do not fit 56
    outs, stats = small.generate(prompts, max_new_tokens=20, return_stats=True)
    assert stats["preemptions"] >= 1 and outs == want
    small.cache.check_invariants()
    roomy = engine(folders["B"], "float32", n_pages=64)
    outs, stats = roomy.generate(prompts, max_new_tokens=20, return_stats=True)
    assert outs == want and stats["ahead_steps"] >= 8 and stats["preemptions"] == 0
