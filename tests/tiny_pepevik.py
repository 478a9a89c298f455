"""Small Pepevik configurations with seeded random weights for the tests.

Sizes differ from configuration to configuration in everything the design lets differ: width, vocabulary, order of the layers,
heads and kv heads (also equal, also sixteen query heads a kv head), key and value sizes that differ from each other and are
no multiple of 32 or of 8, the query factor's constants (also none), the recurrence's width, state sizes that are no multiple
of 8, taps (also 1: no convolution state), groups and norm groups (also 1), experts, groups of experts (also one group, also
one expert a group), `top` (also 1), layers without feed-forward, layers that run another layer's weights, the residual factor
and the embedding's (also absent).  Weights are drawn in float32 from a generator seeded by (seed, tensor name), sized so that
every sublayer moves the stream visibly, and rounded to bfloat16 so that both engines and the plain implementation hold the same
numbers.  This file shares nothing with the engine package.
"""

from __future__ import annotations

import copy
import hashlib
import math
from typing import Dict

import torch


def par(heads, kv_heads, dim, vdim, width, *, scale=None, temp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if temp is not None:
        left["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width}}}


def ssm(heads, vdim, state, *, groups=1, conv=1, norm_groups=1):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, count=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(mixer, mlp, weights_of=None):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model(width, vocab, eps, layers, *, max_positions=512, residual_mult=None, embedding_scale=None):
    out = {"architecture": "Pepevik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "max_positions": max_positions,
           "layers": layers}
    if residual_mult is not None:
        out["residual_mult"] = residual_mult
    if embedding_scale is not None:
        out["embedding"] = {"scale": embedding_scale}
    return out


_A_PAR = par(6, 3, 24, 40, 72, temp=(0.5, 8))
_A_SSM = ssm(4, 12, 16, groups=2, conv=3, norm_groups=2)
# A: both kinds of mixer and of feed-forward, a layer run twice more in another order, a state-space layer without feed-forward
#    with four taps and a state size that is no multiple of 8
TINY_PA = model(64, 97, 1e-5, [
    layer(_A_PAR, moe(8, 3, 24, count=4, keep=2)),
    layer(_A_SSM, dense(48)),
    layer(_A_PAR, moe(8, 3, 24, count=4, keep=2), weights_of=0),
    layer(ssm(2, 40, 24, groups=1, conv=4, norm_groups=1), None),
    layer(_A_PAR, moe(8, 3, 24, count=4, keep=2), weights_of=2),
], residual_mult=0.7, embedding_scale=3.0)

# B: what a model may happen to make equal or 1: one kv head per head and a single head, no query factor, no factor on the
#    stream or the embedding, one tap (no convolution state), one group everywhere, one expert per token, every expert a group of
#    its own, a state-space layer first
TINY_PB = model(48, 61, 1e-6, [
    layer(ssm(1, 20, 8, groups=1, conv=1, norm_groups=1), moe(5, 1, 16, count=5, keep=2)),
    layer(par(1, 1, 36, 8, 20, scale=0.3), dense(80)),
    layer(par(3, 3, 8, 20, 100, temp=(1.5, 1)), moe(6, 2, 40, count=1, keep=1)),
    layer(ssm(6, 8, 40, groups=3, conv=2, norm_groups=6), None),
], max_positions=300)

# C: sixteen query heads on one kv head (two blocks of heads in the attention kernel) with head sizes 96 / 64, many experts of
#    which four of two groups are used, a wide recurrence
TINY_PC = model(96, 131, 1e-5, [
    layer(par(16, 1, 96, 64, 200, temp=(0.25, 32)), moe(16, 4, 32, count=4, keep=2)),
    layer(ssm(8, 16, 32, groups=2, conv=4, norm_groups=4), moe(16, 4, 32, count=4, keep=2)),
    layer(par(4, 2, 16, 48, 64, temp=(0.5, 64)), dense(128)),
    layer(ssm(8, 16, 32, groups=2, conv=4, norm_groups=4), moe(16, 4, 32, count=4, keep=2), weights_of=1),
], residual_mult=0.5, embedding_scale=9.0)

CONFIGS_P = {"PA": TINY_PA, "PB": TINY_PB, "PC": TINY_PC}


def owner(cfg: dict, i: int) -> int:
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    E, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, E), "pos": (cfg["max_positions"], E), "head": (V, E)}

    def norm(name):
        out.update({name: (E,), name + ".b": (E,), name + ".alpha": ()})

    norm("final.norm")
    for i, l in enumerate(cfg["layers"]):
        if owner(cfg, i) != i:
            continue
        p, m = f"l{i}.", l["mixer"]
        norm(p + "norm1")
        if l["type"] == "parallel":
            lf, W = m["left"], m["right"]["width"]
            H, G, d, dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            out.update({p + "mix.left.q": (H * d, E), p + "mix.left.k": (G * d, E), p + "mix.left.v": (G * dv, E),
                        p + "mix.left.q.norm": (d,), p + "mix.left.k.norm": (d,), p + "mix.left.r1": (H,), p + "mix.left.r2": (H,),
                        p + "mix.left.pb": (H,), p + "mix.left.o": (E, H * dv), p + "mix.right.z": (W, E), p + "mix.right.z.b": (W,),
                        p + "mix.right.x": (W, E), p + "mix.right.x.b": (W,), p + "mix.right.g": (W, E), p + "mix.right.o": (E, W),
                        p + "mix.left.out": (E,), p + "mix.right.out": (E,)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], E), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                        p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],),
                        p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (E, inner)})
        f = l["mlp"]
        if f is None:
            continue
        norm(p + "norm2")
        if f["kind"] == "dense":
            out.update({p + "mlp.up": (f["ff"], E), p + "mlp.down": (E, f["ff"])})
        else:
            n, ff = f["router"]["experts"], f["expert"]["ff"]
            out.update({p + "mlp.router": (n, E), p + "mlp.correction": (n,)})
            for e in range(n):
                out.update({f"{p}mlp.e{e}.gate": (ff, E), f"{p}mlp.e{e}.up": (ff, E), f"{p}mlp.e{e}.down": (E, ff)})
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by checkpoint name."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g = torch.Generator(device="cpu").manual_seed(int.from_bytes(h[:7], "little"))
        r = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = 0.6 + 0.05 * r
        elif name.endswith(".r1") or name.endswith(".r2"):
            t = 0.2 + 0.5 * r.abs()               # the distance term is a penalty that grows with the logarithm of the distance
        elif last in ("pb", "correction", "dt_bias", "A_log") or name.endswith(".z.b") or name.endswith(".x.b"):
            t = 0.5 * r
        elif name.endswith("conv.b") or (last == "b" and len(shape) == 1):
            t = 0.1 * r
        elif name.endswith(".conv"):
            t = 0.5 * r
        elif len(shape) == 1:
            t = 1.0 + 0.1 * r                     # norm weights, D
        elif name == "embed":
            t = 0.5 * r
        elif name == "pos":
            t = 0.3 * r
        elif last == "router":
            t = 3.0 * r / math.sqrt(shape[1])     # scores spread enough for the choice to be clear
        elif name.endswith(".left.q") or name.endswith(".left.k"):
            t = 2.0 * r / math.sqrt(shape[1])
        else:
            t = r / math.sqrt(shape[1])           # a projection: outputs about as large as its inputs
        out[name] = t.to(torch.bfloat16)
    return out
