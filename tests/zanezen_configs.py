"""Tiny Zanezen configurations that differ from each other in every size, constant and in the order of layers, and the
helper that writes a folder of random weights for one (into a temporary folder, never committed)."""
from __future__ import annotations

ARCH = "Zanezen"


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, shared_ff=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale},
            "shared": None if shared_ff is None else {"ff": shared_ff}}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, diff, mlp, conv=None, rotary=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if conv:
        m["conv"] = conv
    if rotary:
        m["rot"] = rotary
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, rotary, vdim, kv_rank, scale, mlp):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "rot": rotary, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale}, "mlp": mlp}


# A: sizes in steps of 16 (the tensor-core attention takes them in bfloat16); values wider than keys; stretched
# frequencies whose ramp lies inside the pairs; two experts of six with a shared one; an attention layer first.
ZANEZEN_A = {
    "architecture": ARCH, "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "residual_mult": 0.5,
    "layers": [
        attention(4, 2, 32, 48, 0.2, 0.3, moe(6, 2, 32, 1.5, 64), conv=4, rotary=rot(16, 500.0, (4.0, 64, 8.0, 1.0)),
                  softcap=20.0),
        mlstm(2, 16, 32, 10.0, dense(96)),
        latent(4, 16, 32, rot(16, 10000.0), 16, 48, 0.17, dense(80)),
        attention(2, 2, 16, 16, 0.3, 0.6, moe(4, 1, 48, 1.0), conv=2, rotary=rot(16, 10000.0)),
        mlstm(4, 16, 16, 4.0, moe(6, 2, 32, 1.5, 64)),
    ],
}

# B: sizes that are no multiple of 16 or 8 (the warp-per-row attention in both engines); as many key heads as query
# heads; a layer without feed-forward; three experts of three; no multiplier on the residual sum and none on the
# embedding; an attention without convolution, rotation and cap; a latent layer whose rotated part is wider than what
# is rotated, with stretched frequencies; one head.
ZANEZEN_B = {
    "architecture": ARCH, "vocab": 97, "width": 72, "norm": {"eps": 3e-6}, "residual_mult": 1.0,
    "layers": [
        latent(3, 12, 6, rot(4, 77.0, (2.0, 16, 4.0, 1.0)), 20, 40, 0.3, moe(3, 3, 24, 2.5, 24)),
        attention(3, 3, 20, 12, 0.35, 0.8, None, conv=3, rotary=rot(8, 1000.0), softcap=5.0),
        mlstm(3, 12, 20, 15.0, moe(5, 2, 16, 0.7)),
        attention(6, 1, 24, 40, 0.15, 0.2, dense(50)),
        mlstm(1, 40, 8, 2.0, None),
        latent(1, 24, 8, rot(8, 1000.0), 28, 36, 0.25, dense(24)),
    ],
}

# C: larger heads at the page size of serving: keys of 64 and values of 128 on one kv head, a state of 128 x 64 a head,
# a latent of 192 with 64 rotated, five taps.
ZANEZEN_C = {
    "architecture": ARCH, "vocab": 131, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
    "residual_mult": 0.7,
    "layers": [
        mlstm(2, 128, 64, 15.0, dense(160)),
        attention(8, 1, 64, 128, 0.11, 0.5, moe(8, 3, 96, 2.0, 160), conv=5, rotary=rot(32, 20000.0, (2.0, 256, 32.0, 1.0)),
                  softcap=30.0),
        latent(8, 64, 64, rot(64, 250000.0), 64, 192, 0.1, moe(8, 2, 96, 2.0, 160)),
    ],
}

CONFIGS = {"A": (ZANEZEN_A, 41), "B": (ZANEZEN_B, 42), "C": (ZANEZEN_C, 43)}
STD = {"A": 0.15, "B": 0.15, "C": 0.07}


def make_folder(tmp_path, name, std=None):
    from ferrox_b200 import write_random_model

    cfg, seed = CONFIGS[name]
    folder = str(tmp_path / f"zanezen_{name}")
    write_random_model(folder, cfg, seed, dtype="bfloat16", std=std or STD[name], norm_init="around_one")
    return folder
