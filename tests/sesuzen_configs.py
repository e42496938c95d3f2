"""Tiny Sesuzen configurations that differ from each other in every size, constant, in the order of layers and in
how they loop, and the helper that writes a folder of random weights for one (into a temporary folder, never
committed)."""
from __future__ import annotations

ARCH = "Sesuzen"


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def attention(heads, kv_heads, dim, vdim, scale, mlp, window=None, keep_first=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return {"type": "attention", "mixer": m, "mlp": mlp}


def delta(heads, dim, mlp, decay_rank=None):
    m = {"heads": heads, "dim": dim}
    if decay_rank:
        m["decay_rank"] = decay_rank
    return {"type": "general_delta", "mixer": m, "mlp": mlp}


# A: sizes in steps of 16 (the tensor-core attention takes them in bfloat16); values wider than keys; a window that
# crosses pages and keeps five first positions; two experts of six; a dense layer; a layer without feed-forward; three
# taps; layers 1 and 2 run twice.
SESUZEN_A = {
    "architecture": ARCH, "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
    "max_positions": 512, "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        delta(2, 16, dense(96)),
        attention(4, 2, 32, 48, 0.21, moe(6, 2, 32), window=21, keep_first=5),
        delta(4, 16, None, decay_rank=8),
        attention(2, 1, 16, 16, 0.3, moe(4, 1, 48), window=9, keep_first=9),
    ],
}

# B: sizes that are no multiple of 16 or 8 (the warp-per-row attention in both engines); as many key heads as query
# heads; one tap (no convolution state to speak of); no loop and no cap; all experts of three; one of five; a window
# of one that keeps nothing, a window that keeps more than it spans, and an attention without a mask.
SESUZEN_B = {
    "architecture": ARCH, "vocab": 97, "width": 72, "norm": {"eps": 3e-6}, "canon": {"taps": 1},
    "max_positions": 400,
    "layers": [
        attention(3, 3, 20, 12, 0.35, moe(3, 3, 24), window=1),
        delta(3, 12, moe(5, 1, 16), decay_rank=5),
        attention(6, 1, 24, 40, 0.15, dense(50), window=4, keep_first=11),
        attention(2, 2, 36, 36, 0.2, None),
        delta(1, 40, dense(24), decay_rank=3),
    ],
}

# C: larger heads at the page size of serving: keys of 128 and values of 64 on one kv head, windows beyond a page of
# 64 that keep most of the first page or a few positions, a state of 64 x 64 a head, five taps, one layer that runs
# three times.
SESUZEN_C = {
    "architecture": ARCH, "vocab": 131, "width": 128, "norm": {"eps": 1e-6}, "canon": {"taps": 5},
    "max_positions": 1024, "logit_softcap": 40.0, "loop": {"start": 0, "stop": 1, "times": 3},
    "layers": [
        attention(8, 1, 128, 64, 0.09, moe(8, 2, 96), window=70, keep_first=60),
        delta(4, 64, moe(8, 3, 64)),
        attention(4, 4, 64, 64, 0.12, dense(160), window=65, keep_first=3),
    ],
}

CONFIGS = {"A": (SESUZEN_A, 31), "B": (SESUZEN_B, 32), "C": (SESUZEN_C, 33)}
# C runs a layer three times and chooses among eight experts five times a position: with larger weights bfloat16
# rounding alone moves its logits by a tenth of their size
STD = {"A": 0.15, "B": 0.15, "C": 0.06}


def make_folder(tmp_path, name, std=None):
    from ferrox_b200 import write_random_model

    cfg, seed = CONFIGS[name]
    std = std or STD[name]
    folder = str(tmp_path / f"sesuzen_{name}")
    write_random_model(folder, cfg, seed, dtype="bfloat16", std=std, norm_init="around_one")
    return folder
