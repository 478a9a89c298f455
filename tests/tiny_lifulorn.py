"""Small Lifulorn configurations with seeded random weights for the tests.

Sizes differ from configuration to configuration in everything the design lets differ: width, vocabulary, order and kinds of the
layers, heads and kv heads (also equal, also sixteen query heads a kv head), key and value sizes that differ from each other and
are no multiple of 32 or of 8, rotated dimensions (all of a head, a part, none), both kinds of frequency scaling with constants
that put pairs on every branch (also none), windows (narrower than a page, wider than the context, none), a soft cap or none,
blended values or none, taps (also 1: no convolution state), experts and `top` (also 1, also all: the fixed configurations
have one layer each whose router really chooses, so that few positions lie near a router's close call, where a bfloat16 run may
choose otherwise), a shared expert or none, layers without feed-forward, the residual factor and the per-layer token input
(also absent).  Weights are drawn in float32 from a generator seeded by (seed, tensor name), sized so that every sublayer moves the stream visibly, and rounded to bfloat16 so that both
engines and the plain implementation hold the same numbers.  This file shares nothing with the engine package.
"""

from __future__ import annotations

import copy
import hashlib
import math
import random
from typing import Dict, Optional

import torch


def att(heads, kv_heads, dim, vdim, *, window=None, rot=None, base=10000.0, scaling=None, scale=None, v_mix=False, kind="attention",
        softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if v_mix:
        m["v_mix"] = True
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": kind, "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv=4):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(experts, top, ff, limit=1.0, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def model(width, vocab, eps, layers, *, residual_mult=None, side=None):
    out = {"architecture": "Lifulorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if residual_mult is not None:
        out["residual_mult"] = residual_mult
    if side:
        out["token_side"] = {"dim": side}
    return out


STEPPED = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}       # wavelengths of 16 rotated dimensions fall on all three branches
RAMPED = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}

# A: every kind of layer, blended values over both kinds of attention, windows that pass within the prompts, a layer without
#    feed-forward, a rotation over a part of the head and over all of it
TINY_LA = model(80, 113, 1e-5, [
    layer(att(6, 3, 40, 24, window=37, rot=16, scaling=STEPPED, scale=0.2, v_mix=True), moe(6, 2, 24, 1.5, shared=(40, 0.75))),
    layer(delta(4, 2, 24, 40, conv=3), moe(3, 3, 24, 1.5, shared=(40, 0.75))),
    layer(att(6, 3, 16, 24, window=20, rot=16, base=500.0, scaling=RAMPED, scale=0.3, v_mix=True, kind="attention_2", softcap=3.0),
          moe(5, 5, 16, 0.5, shared=(8, 2.0))),
    layer(att(2, 1, 8, 8, window=5, rot=4, base=100.0), None),
    layer(delta(3, 3, 8, 16, conv=2), None),
], residual_mult=0.7, side=12)

# B: what a model may happen to make equal or 1: one kv head per head and a single head, key and value sizes alike, no rotation,
#    no scaling, no window, a window wider than anything fed, one tap (no convolution state), one expert per token, no shared
#    expert, no factor on the stream, no token input, values blended by one layer only (nothing to blend with)
TINY_LB = model(48, 61, 1e-6, [
    layer(delta(1, 1, 20, 12, conv=1), moe(2, 1, 16, 1.0)),
    layer(att(1, 1, 36, 36, scale=0.25), moe(4, 4, 40, 3.0, shared=(16, 1.0))),
    layer(att(3, 3, 8, 20, window=400, rot=8, base=50.0, v_mix=True, kind="attention_2"), moe(3, 3, 24, 1.0)),
    layer(att(3, 3, 12, 12, window=1, rot=6, base=20.0, scaling=RAMPED, kind="attention_2", softcap=50.0), None),
])

# C: sixteen query heads on one kv head (two blocks of heads in the attention kernel) with head sizes 96 / 64, a window beyond
#    the length of a piece of keys, a state of 136 x 72 a head (rows and columns that fill no block evenly), many experts
TINY_LC = model(96, 131, 1e-5, [
    layer(att(16, 1, 96, 64, window=300, rot=32, base=50000.0, scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256},
              v_mix=True), moe(16, 4, 32, 1.0, shared=(32, 1.0))),
    layer(delta(4, 2, 136, 72, conv=4), moe(8, 8, 32, 1.0, shared=(32, 1.0))),
    layer(att(4, 1, 16, 64, window=260, rot=16, base=1000.0, scaling={"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0},
              scale=0.4, v_mix=True, kind="attention_2", softcap=8.0), moe(2, 2, 48, 2.0)),
], residual_mult=0.5, side=8)

CONFIGS_L = {"LA": TINY_LA, "LB": TINY_LB, "LC": TINY_LC}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    E, V = cfg["width"], cfg["vocab"]
    side = (cfg.get("token_side") or {}).get("dim", 0)
    out = {"embed": (V, E), "head": (V, E), "final.norm": (E,)}
    if side:
        out["side.embed"] = (V, side * len(cfg["layers"]))
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (E,)
        out[p + "ls1"] = (E,)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if l["type"] == "delta":
            K = m["conv"]
            out.update({p + "mix.q": (G * d, E), p + "mix.k": (G * d, E), p + "mix.v": (H * dv, E), p + "mix.q.conv": (G * d, K),
                        p + "mix.k.conv": (G * d, K), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, E), p + "mix.a": (H, E),
                        p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.g": (H * dv, E), p + "mix.norm": (dv,),
                        p + "mix.o": (E, H * dv)})
        else:
            out.update({p + "mix.q": (H * d, E), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, E), p + "mix.k.b": (G * d,),
                        p + "mix.v": (G * dv, E), p + "mix.v.b": (G * dv,), p + "mix.sink": (H,), p + "mix.o": (E, H * dv)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        f = l["mlp"]
        if f is not None:
            out[p + "norm2"] = (E,)
            out[p + "ls2"] = (E,)
            n, ff = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"] = (n, E)
            for e in range(n):
                out.update({f"{p}mlp.e{e}.gate": (ff, E), f"{p}mlp.e{e}.up": (ff, E), f"{p}mlp.e{e}.down": (E, ff)})
            if f.get("shared"):
                fs = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (fs, E), p + "mlp.shared.up": (fs, E), p + "mlp.shared.down": (E, fs),
                            p + "mlp.shared.sg": (1, E)})
        if side:
            out.update({p + "side.gate": (side, E), p + "side.proj": (E, side), p + "side.norm": (E,)})
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by checkpoint name."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g = torch.Generator(device="cpu").manual_seed(int.from_bytes(h[:7], "little"))
        r = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if last == "vmix":
            t = 0.35 + 0.1 * r
        elif last == "sink":
            t = 1.0 * r
        elif last in ("dt_bias", "A_log"):
            t = 0.5 * r
        elif last == "b" and len(shape) == 1:
            t = 0.2 * r                           # biases of q, k, v
        elif last == "conv":
            t = 0.5 * r
        elif len(shape) == 1:
            t = 1.0 + 0.1 * r                     # norm weights, layer scales
        elif name in ("embed", "side.embed"):
            t = 0.7 * r
        elif last == "router":
            t = 3.0 * r / math.sqrt(shape[1])     # logits spread enough for the choice to be clear
        elif name.endswith("mix.q") or name.endswith("mix.k"):
            t = 1.2 * r / math.sqrt(shape[1])
        elif name.endswith(".gate") or name.endswith(".up"):
            t = 1.5 * r / math.sqrt(shape[1])     # some products beyond the experts' limits
        else:
            t = r / math.sqrt(shape[1])           # a projection: outputs about as large as its inputs
        out[name] = t.to(torch.bfloat16)
    return out


def random_config(seed: int) -> dict:
    """A seeded configuration: two to five layers of any kind in any order with a feed-forward or none."""
    rng = random.Random(1000 + seed)
    width = rng.choice([40, 56, 64, 88, 128])
    vocab = rng.choice([53, 89, 150, 257])
    G_mix, dv_mix = rng.choice([1, 2, 3]), rng.choice([8, 12, 24, 40])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "attention_2", "delta"])
        if kind == "delta":
            G = rng.choice([1, 2, 3])
            mixer = delta(G * rng.choice([1, 2]), G, rng.choice([8, 20, 33, 64]), rng.choice([8, 24, 40, 70]), conv=rng.choice([1, 2, 4]))
        else:
            mix = rng.random() < 0.6
            G = G_mix if mix else rng.choice([1, 2, 4])
            d = rng.choice([8, 16, 24, 48, 72])
            dv = dv_mix if mix else rng.choice([8, 16, 28, 64])
            rot = rng.choice([0, d // 2 - (d // 2) % 2, d - d % 2])
            if kind == "attention":
                sc = rng.choice([None, {"factor": rng.choice([2.0, 8.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]), "original": rng.choice([16, 64, 512])}])
            else:
                sc = rng.choice([None, {"factor": rng.choice([2.0, 16.0]), "original": rng.choice([16, 64, 512]), "fast": rng.choice([4.0, 32.0]),
                                        "slow": rng.choice([0.5, 1.0])}])
            mixer = att(G * rng.choice([1, 2, 5]), G, d, dv, window=rng.choice([None, 1, 3, 17, 64, 90]), rot=rot,
                        base=rng.choice([30.0, 10000.0, 500000.0]), scaling=sc if rot else None, scale=rng.choice([None, 0.15, 0.4]),
                        v_mix=mix, kind=kind, softcap=rng.choice([None, 2.0, 30.0]) if kind == "attention_2" else None)
        n = rng.choice([2, 4, 7, 9])
        mlp = rng.choice([None, moe(n, rng.randint(1, min(n, 4)), rng.choice([8, 24, 40]), rng.choice([0.5, 1.0, 7.0]),
                                    shared=rng.choice([None, (rng.choice([8, 24]), rng.choice([0.5, 2.0]))]))])
        layers.append(layer(mixer, mlp))
    return model(width, vocab, rng.choice([1e-5, 1e-6]), layers, residual_mult=rng.choice([None, 0.5, 1.4]), side=rng.choice([None, 4, 10]))
