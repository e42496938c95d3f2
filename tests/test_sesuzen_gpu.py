"""The engine's Sesuzen model against the plain implementation: every mechanism alone, then whole models under every
way of cutting the work (whole prompts, a decoded tail, portions down to two tokens, mixed batches with pages and
slots used again, long decoding, generation through the scheduler), in 32-bit and in bfloat16, on configurations
that differ in every size, constant, in the order of layers and in how they loop."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_sesuzen as pz
import replay_util as ru
from sesuzen_configs import CONFIGS, make_folder
from test_safepel_gpu import CUTS, MixerHarness, load_part, random_tensors, rel, run_in_cuts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": (torch.float32, 5e-5), "bfloat16": (torch.bfloat16, 3e-2)}
RATE = math.exp(-0.5)


def attention_spec(hidden, H, G, D, V, scale, window=None, keep_first=0, eps=1e-5):
    from ferrox_b200.parts.specs import AttentionSpec

    return AttentionSpec(hidden=hidden, n_heads=H, n_kv_heads=G, head_dim=D, qkv_bias=True, position=None, window=window,
                         prefix="m.", softmax_scale=scale, value_dim=V,
                         tensor_names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_bias", "q.b"),
                                       ("k_bias", "k.b"), ("v_bias", "v.b")),
                         value_norm_eps=eps, keep_first=keep_first, output_gate="g")


def delta_spec(hidden, H, D, rank, eps=1e-5):
    from ferrox_b200.parts.specs import GeneralDeltaSpec

    return GeneralDeltaSpec(hidden=hidden, n_heads=H, head_dim=D, decay_rank=rank, decay_rate=RATE, norm_eps=eps, prefix="m.")


def loudness(dt):
    """How much larger the loud row is: 20 times in 32-bit; 4 times in bfloat16, where scores of a hundred would be
    rounded by whole units."""
    return 20.0 if dt == torch.float32 else 4.0


def inputs(hidden, lens, seed, dt, loud=None):
    """Rows for each request, rounded to the engine's element type; ``loud`` = (request, position): that row
    several times as large, so that whether a later query sees its key shows in the result."""
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(n, hidden, generator=g) for n in lens]
    if loud is not None:
        xs[loud[0]][loud[1]] *= loudness(dt)
    return [x.to(dt).float() for x in xs]


def mask_of(window, keep):
    return {"size": window, "keep_first": keep} if window else None


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_layer_norm_with_weight_and_bias(dtype):
    from ferrox_b200.parts.specs import LayerNormSpec

    dt, tol = DTYPES[dtype]
    g = torch.Generator().manual_seed(0)
    for H in (72, 300, 1024):
        spec = LayerNormSpec(size=H, eps=3e-6, name="n", bias_name="n.b")
        w = random_tensors(spec, std=0.3)
        assert float(w["n.b"].float().abs().max()) > 0
        part, rt = load_part(spec, w, dt)
        h = torch.randn(7, H, generator=g) * 4 + 2.5
        want = pz.layer_norm(h, w["n"].float(), w["n.b"].float(), 3e-6)
        got = part.forward(h.to(DEV))
        assert got.dtype == dt and rel(got, want) < tol
        rows = torch.tensor([6, 1], dtype=torch.int32, device=DEV)
        assert torch.equal(part.forward(h.to(DEV), rows=rows), got[[6, 1]])


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_squared_relu_feed_forward_alone(dtype):
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.specs import PlainMlpSpec

    dt, tol = DTYPES[dtype]
    for hidden, ff in ((96, 160), (72, 50)):
        spec = PlainMlpSpec(hidden=hidden, intermediate=ff, prefix="f.")
        w = random_tensors(spec, std=0.2)
        part, rt = load_part(spec, w, dt)
        wf = {k: v.float() for k, v in w.items()}
        for T in (3, 70, 300):  # the decode-sized and the prompt-sized kernels
            x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(T)).to(dt)
            out = torch.full((T, hidden), float("nan"), device=DEV)
            part.forward_into(x.to(DEV), out, SimpleNamespace(status=None, stream=ops.stream_ptr()), accumulate=False)
            want = pz.ffn_dense(x.float(), wf, "f.")
            assert rel(out, want) < tol
            z = x.float() @ wf["f.up"].T
            assert rel(torch.relu(z) @ wf["f.down"].T, want) > 0.05       # (the test can tell a missing square)


@pytest.mark.parametrize("E,top", [(6, 2), (3, 3), (5, 1), (8, 4)])
@pytest.mark.parametrize("tokens", [1, 5, 40, 300])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_experts_weighted_by_the_softmax_over_the_chosen_logits(dtype, tokens, E, top):
    from ferrox_b200.engine.batch import StepEntry, flatten
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.specs import MoeSpec

    dt, tol = DTYPES[dtype]
    hidden, I = 64, 32
    spec = MoeSpec(hidden=hidden, n_experts=E, top_k=top, expert_intermediate=I, shared_intermediate=0, norm_topk_prob=True,
                   shared_gate=False, prefix="f.", tensor_names=("router", "e{e}.{part}", "shared.{part}"))
    w = random_tensors(spec, seed=tokens + top, std=0.2)
    part, rt = load_part(spec, w, dt)
    x = (inputs(hidden, [tokens], 5, dt)[0] * 2.0).to(dt).float()
    f = {"router": {"experts": E, "top": top}, "expert": {"ff": I}}
    wf = {k: v.float() for k, v in w.items()}
    want = pz.ffn_moe(x, f, wf, "f.")
    idx, wt, z = pz.route(x, f, wf, "f.")
    if top > 1 and top < E and tokens >= 40:
        # the test can tell: weights taken from the softmax over ALL logits without renormalising give something else
        full = torch.softmax(z, -1).gather(1, idx)
        assert rel(pz.ffn_moe(x, f, wf, "f.", chosen=(idx, full, z)), want) > 0.05
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = flatten([StepEntry(0, [0] * tokens, start=0)], torch.device(DEV), status, ops.stream_ptr())
    h = torch.zeros(tokens, hidden, dtype=torch.float32, device=DEV)
    part.forward_add(x.to(DEV).to(dt), h, batch)
    torch.cuda.synchronize()
    if dtype == "bfloat16" and top < E:
        # a position whose router separates the last chosen expert from the next by less than bfloat16 rounding may
        # rightly choose the other one: leave those rows out, and require them to be few
        s = z.sort(dim=-1, descending=True).values
        clear = (s[:, top - 1] - s[:, top]) > 0.02 * z.abs().amax(dim=-1)
        assert tokens < 40 or clear.float().mean() > 0.5
        if clear.any():
            assert rel(h.cpu()[clear], want[clear]) < tol
    else:
        assert rel(h, want) < tol


class ConvOnly:
    """An inner mixer that hands its input on: what the input convolution made of the rows, seen alone."""

    graph_safe = True

    def __init__(self, hidden):
        self.hidden = hidden

    def cache_spec(self):
        return None

    def tensor_decls(self):
        return []

    def load(self, src, rt):
        pass

    def forward_into(self, x, out, batch, cache, accumulate=False):
        assert not accumulate
        out.copy_(x.float())


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("taps,hidden", [(1, 40), (2, 72), (4, 64), (5, 200), (16, 24)])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_input_convolution_alone(dtype, taps, hidden, cut):
    """x + conv(x) under every cut: the last taps - 1 rows of a request are carried in its state slot, also over
    portions shorter than the taps, and a request that starts reads zeros before its first row."""
    from ferrox_b200.parts import build  # noqa: F401  (registers the built-in parts)
    from ferrox_b200.parts.base import Runtime, build_part
    from ferrox_b200.parts.specs import InputConvSpec, PlainMlpSpec
    from ferrox_b200.weights import loader as wl

    dt, tol = DTYPES[dtype]
    spec = InputConvSpec(mixer=PlainMlpSpec(hidden=hidden, intermediate=8, prefix="unused."), channels=hidden, taps=taps,
                         name="c")
    part = build_part(spec)
    part.inner = ConvOnly(hidden)
    g = torch.Generator().manual_seed(taps)
    w = {"c": (torch.randn(hidden, taps, generator=g) * 0.5).to(torch.bfloat16)}
    rt = Runtime(torch.device(DEV), dt)
    part.load(wl.from_dict(w, part.tensor_decls(), DEV, dt), rt)
    xs = inputs(hidden, (150, 37), 11, dt)
    want = [pz.input_convolution(x, w["c"].float()) for x in xs]
    assert taps == 1 or rel(want[0], xs[0] * (1 + w["c"].float()[:, -1])) > 0.05     # (earlier rows matter)
    h = MixerHarness(part, rt, hidden, page_size=4, n_pages=8)
    got = run_in_cuts(h, xs, CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol
    # the slots are used again: the next requests start from zeros, not from the last ones' tails
    got = run_in_cuts(h, xs[::-1], CUTS[cut])
    for a, b in zip(got, want[::-1]):
        assert rel(a, b) < tol


def attention_mixer(H, G, D, V, scale, window, keep):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=scale)
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return m


def keys_that_stand_out(w, H, G, D, hidden, n, seed, dt):
    """Weights and rows made so that one key can dominate: every query head's weights are its key head's plus half of
    its own random ones, and every row is a common direction z plus noise, so that the score of a query with the key
    of a row L z grows with L in every head.  Returns (the rows [n, hidden], z)."""
    rep = H // G
    for h in range(H):
        g = h // rep
        w["m.q"][h * D:(h + 1) * D] = (w["m.k"][g * D:(g + 1) * D].float() + 0.5 * w["m.q"][h * D:(h + 1) * D].float()).to(torch.bfloat16)
        w["m.q.b"][h * D:(h + 1) * D] = (w["m.k.b"][g * D:(g + 1) * D].float() + 0.5 * w["m.q.b"][h * D:(h + 1) * D].float()).to(torch.bfloat16)
    gen = torch.Generator().manual_seed(seed)
    z = torch.randn(hidden, generator=gen) * math.sqrt(2.0 / D)
    x = torch.randn(n, hidden, generator=gen) * 0.3 + z
    return x.to(dt).float(), z


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("H,G,D,V,window,keep,page", [
    (4, 2, 32, 48, 21, 5, 4), (3, 3, 20, 12, 1, 0, 8), (6, 1, 24, 40, 4, 11, 16), (8, 1, 128, 64, 70, 60, 64),
    (4, 4, 64, 64, 65, 3, 64), (2, 2, 36, 36, None, 0, 8), (2, 1, 16, 16, 9, 9, 4), (4, 2, 32, 32, 16, 1, 16),
    (72, 1, 16, 16, 33, 2, 16)])      # (the last: more heads on a kv head than a tile has rows)
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_attention_alone_at_the_edges_of_its_window_and_of_the_kept_positions(dtype, H, G, D, V, window, keep, page, cut):
    """A key that stands out at the last kept position and one at the first position that is not kept: the plain
    implementation tells that the first stays visible for good while the second is seen by the queries up to
    window - 1 later and by none after; the engine agrees with it at every position under every cut."""
    dt, tol = DTYPES[dtype]
    hidden = 64
    spec = attention_spec(hidden, H, G, D, V, 0.3, window=window, keep_first=keep)
    w = random_tensors(spec, seed=H + D, std=0.25)
    assert float(w["m.v.b"].float().abs().max()) > 0 and float(w["m.q.b"].float().abs().max()) > 0
    x0, z = keys_that_stand_out(w, H, G, D, hidden, 150, 3, dt)
    part, rt = load_part(spec, w, dt)
    xs = [x0, inputs(hidden, (37,), 3, dt)[0]]
    wf = {k: v.float() for k, v in w.items()}
    m = attention_mixer(H, G, D, V, 0.3, window, keep)
    plain = lambda x: pz.mixer_attention(x, m, wf, "m.", 1e-5)
    if window:
        b = plain(x0)
        for row, kept in ((keep - 1, True), (keep, False)):
            if row < 0:
                continue
            loud = x0.clone()
            loud[row] = (4 * z).to(dt).float()
            a = plain(loud)
            last = row + window - 1
            if kept:
                assert rel(a[last + 1:], b[last + 1:]) > 5e-2                    # kept: seen ever after
            else:
                assert rel(a[last], b[last]) > 5e-2                              # the last query of the window sees it
                assert float((a[last + 1:] - b[last + 1:]).abs().max()) == 0.0   # not kept: gone
        for row in {max(keep - 1, 0), keep}:
            x0[row] = (4 * z).to(dt).float()
    want = [plain(x) for x in xs]
    got = run_in_cuts(MixerHarness(part, rt, hidden, page_size=page, n_pages=256 // page + 8), xs, CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_attention_reads_a_kept_position_far_back_and_norms_its_values(dtype):
    """Seven hundred positions, a window of 40 that keeps 6: the query and key of position 4 are made to stand out, so
    that far queries put their weight on it; with that row's value changed every far output changes.  Values 20 times
    as large give the same output (each head's value is divided by its root mean square); without that division the
    plain implementation itself gives something else."""
    dt, tol = DTYPES[dtype]
    hidden, H, G, D, V = 64, 8, 2, 32, 32
    spec = attention_spec(hidden, H, G, D, V, 0.4, window=40, keep_first=6)
    w = random_tensors(spec, seed=1, std=0.25)
    part, rt = load_part(spec, w, dt)
    xs = inputs(hidden, (700, 9), 4, dt, loud=(0, 4))
    wf = {k: v.float() for k, v in w.items()}
    m = attention_mixer(H, G, D, V, 0.4, 40, 6)
    want = [pz.mixer_attention(x, m, wf, "m.", 1e-5) for x in xs]
    quiet = xs[0].clone()
    quiet[4] /= loudness(dt)
    assert rel(pz.mixer_attention(quiet, m, wf, "m.", 1e-5)[600:], want[0][600:]) > 0.02       # the far key matters
    not_kept = attention_mixer(H, G, D, V, 0.4, 40, 4)
    assert rel(pz.mixer_attention(xs[0], not_kept, wf, "m.", 1e-5)[600:], want[0][600:]) > 0.02
    big = dict(wf)
    big["m.v"], big["m.v.b"] = wf["m.v"] * 20, wf["m.v.b"] * 20
    assert rel(pz.mixer_attention(xs[0], m, big, "m.", 1e-5), want[0]) < 1e-3
    got = run_in_cuts(MixerHarness(part, rt, hidden, page_size=16, n_pages=64, max_positions=1024), xs,
                      [(560, 0), (3, 9)] + [(1, 0)] * 137)
    for a, b in zip(got, want):
        assert rel(a, b) < tol


def plain_delta(x, H, D, wf, eps=1e-5):
    return pz.mixer_general_delta(x, dict(heads=H, dim=D), wf, "m.", eps)


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("H,D,rank", [(2, 16, 8), (3, 12, 5), (1, 40, 3), (4, 64, 16), (2, 128, 24), (5, 4, 1),
                                      (1, 100, 2)])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_general_delta_rule_alone(dtype, H, D, rank, cut):
    """The recurrence with its state carried over every cut, two requests side by side, against the plain loop over
    tokens; the slots are then used again by requests that must start from an empty state."""
    dt, tol = DTYPES[dtype]
    hidden = 64
    spec = delta_spec(hidden, H, D, rank)
    w = random_tensors(spec, seed=H + D, std=0.25)
    g = torch.Generator().manual_seed(D)
    w["m.w0"] = torch.randn(H * D, generator=g).to(torch.bfloat16)             # decays spread over their range
    w["m.a.b"] = torch.randn(H * D, generator=g).to(torch.bfloat16)
    part, rt = load_part(spec, w, dt)
    xs = inputs(hidden, (150, 37), 3, dt)
    wf = {k: v.float() for k, v in w.items()}
    want = [plain_delta(x, H, D, wf) for x in xs]
    h = MixerHarness(part, rt, hidden, page_size=4, n_pages=8)
    got = run_in_cuts(h, xs, CUTS[cut])
    for a, b in zip(got, want):
        assert rel(a, b) < tol
    got = run_in_cuts(h, xs[::-1], CUTS[cut])
    for a, b in zip(got, want[::-1]):
        assert rel(a, b) < tol


def test_general_delta_rule_every_term_shows():
    """The plain recurrence against variants with one term changed (no removal, removal reading the new state, a decay
    without its rate, a key that is not normed in the removal): each gives something else, so the comparison of
    the engine with it means all of them; and the engine's 32-bit state after 400 tokens is the plain one."""
    hidden, H, D, rank = 64, 2, 16, 4
    spec = delta_spec(hidden, H, D, rank)
    w = random_tensors(spec, seed=5, std=0.3)
    wf = {k: v.float() for k, v in w.items()}
    x = inputs(hidden, (400,), 8, torch.float32)[0]
    r, k, v, dec, a = pz.delta_inputs(x, dict(heads=H, dim=D), wf, "m.")
    o, S = pz.delta_recurrence(r, k, v, dec, a)
    assert float(dec.min()) >= math.exp(-RATE) - 1e-6 and float(dec.max()) < 1.0

    def variant(kind):
        St = torch.zeros(H, D, D)
        out = []
        for t in range(x.shape[0]):
            u = k[t] / torch.sqrt((k[t] * k[t]).sum(-1, keepdim=True) + 1e-6)
            if kind == "raw key":
                u = k[t]
            old = St
            St = dec[t][:, :, None] * old
            if kind == "new state":
                St = St - (a[t] * u)[:, :, None] * torch.einsum("hi,hij->hj", u, St)[:, None, :]
            elif kind != "no removal":
                St = St - (a[t] * u)[:, :, None] * torch.einsum("hi,hij->hj", u, old)[:, None, :]
            St = St + k[t][:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hij,hi->hj", St, r[t]))
        return torch.stack(out)

    assert rel(variant("as stated"), o) < 1e-6
    for kind in ("no removal", "new state", "raw key"):
        assert rel(variant(kind)[2:30], o[2:30]) > 1e-2, kind        # (with raw keys the state soon overflows)
    part, rt = load_part(spec, w, torch.float32)
    hs = MixerHarness(part, rt, hidden, page_size=4, n_pages=8, max_positions=512)
    slot = hs.mgr.open_request()
    got = torch.cat([hs.step([(slot, x[:333])]), hs.step([(slot, x[333:335])]), hs.step([(slot, x[335:])])])
    assert rel(got, plain_delta(x, H, D, wf)) < 5e-5
    state = hs.mgr.layer_cache(0).states["matrix"][slot].cpu()       # [H, value, key]
    assert rel(state.transpose(1, 2), S) < 5e-5


# ------------------------------------------------------------------ whole models
def prompts_for(name, n=5, hi=150, seed=0):
    cfg = CONFIGS[name][0]
    rng = random.Random(seed)
    lens = [1, 2, hi] + [rng.randint(3, hi) for _ in range(max(0, n - 3))]
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(L)] for i, L in enumerate(lens)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("sesuzen_models")
    return {name: make_folder(tmp, name) for name in CONFIGS}


@pytest.fixture(scope="module")
def expected(folders):
    import plain_qwen2moe as reader

    out = {}
    for name in CONFIGS:
        cfg, w = reader.load_model(folders[name], torch.float32)
        want = {rid: pz.forward(cfg, w, t) for rid, t in prompts_for(name).items()}
        out[name] = (cfg, w, want, {rid: rounding_alone(cfg, w, t, want[rid]) for rid, t in prompts_for(name).items()})
    return out


def position_errors(got, want):
    return (got - want).abs().amax(dim=-1) / want.abs().max()


def rounding_alone(cfg, w, tokens, want):
    """Per position: how far the plain implementation's logits move when everything that may be computed in bfloat16
    is rounded to it.  A choice of experts that falls the other way under rounding moves a position and, through
    the states, those after it by much more than the rounding itself: the measure of an engine in bfloat16 is this
    distribution, not a bound for every position."""
    with pz.rounded_to(torch.bfloat16):
        return position_errors(pz.forward(cfg, w, tokens), want)


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


def test_residual_stream_after_every_layer_run(folders, expected):
    """Run by run in 32-bit: a layer of the loop is counted every time it runs, each time on the stream its last
    run left, with a cache of its own."""
    from ferrox_b200.engine.batch import StepEntry

    cfg, w = expected["A"][:2]
    toks = prompts_for("A")["r3"]
    want_logits, after = pz.forward(cfg, w, toks, return_layers=True)
    runs = pz.layer_runs(cfg)
    assert len(runs) > len(cfg["layers"])
    eng = engine(folders["A"], "float32")
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
    assert [i for i, _ in seen] == runs
    for n, (_, h) in enumerate(seen):
        assert rel(h, after[n]) < 2e-5, n
    assert rel(got, want_logits) < 5e-5


@pytest.mark.parametrize("name", ["A", "C"])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding_past_every_window_with_pages_given_back(folders, dtype, name):
    """A few tokens of prompt, then hundreds decoded one by one: the windowed layers give back the pages that left
    their window, except those of the kept first positions (their pools hold less than the request)."""
    import plain_qwen2moe as reader

    _, tol = DTYPES[dtype]
    cfg, w = reader.load_model(folders[name], torch.float32)
    rng = random.Random(9)
    n = 303 if name == "A" else 420
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    want = pz.forward(cfg, w, toks)
    eng = engine(folders[name], dtype, n_pages=12 if name == "A" else 6, max_slots=2)    # 96 or 384 positions a pool
    groups_smaller_than_request = [k for k, g in eng.cache.groups.items() if g.pool.n_pages * eng.cache.page_size < n]
    assert groups_smaller_than_request
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


def test_trace_replay_and_command_line_with_a_sesuzen_folder(folders, tmp_path):
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
    """A request that is preempted gives its pages and slot back and is recomputed (its state and its convolution
    tail start again from zeros); greedy decode steps are replayed graphs issued one ahead of the host."""
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
