"""A plain, slow implementation of the Lifulorn decoder, one function per mechanism, written from the
architecture's equations and sharing no code with the engine.  It takes the content of a config.json and a
dict of tensors by checkpoint name and runs one whole sequence at a time on the CPU; there is no cache: every
function sees all tokens of the sequence, and the recurrence walks them one by one.

Notation: T tokens, width E, x the residual stream [T, E], u the normed input of a sublayer, m the model's factor
on everything that is added to the stream.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x, eps):
    """x over its root mean square along the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# -- rotary frequencies ---------------------------------------------------------------------------------------------

def plain_frequencies(dims: int, base: float):
    i = torch.arange(dims // 2, dtype=torch.float64)
    return base ** (-2.0 * i / dims)


def stepped_frequencies(dims: int, base: float, sc: dict):
    """Frequencies whose long wavelengths are slowed by `factor`, short ones kept, and the ones between blended by where
    their wavelength lies between original / low and original / high."""
    f = plain_frequencies(dims, base)
    factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.clone()
    for i in range(f.numel()):
        wl = 2.0 * math.pi / float(f[i])
        if wl < original / high:
            continue
        if wl > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / wl - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out, 1.0


def ramped_frequencies(dims: int, base: float, sc: dict):
    """Frequencies blended into slowed ones along a ramp over the pair index, between the pairs that make `fast` and `slow`
    turns within `original` tokens; cos and sin grow by 0.1 ln(factor) + 1."""
    f = plain_frequencies(dims, base)
    factor, original = float(sc["factor"]), float(sc["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, magnitude, dims: int):
    """x [T, heads, d]: the first `dims` elements of every head turn, element i against i + dims / 2."""
    if dims == 0:
        return x
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = (ang.cos() * magnitude).to(x.dtype)[:, None, :], (ang.sin() * magnitude).to(x.dtype)[:, None, :]
    half = dims // 2
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), dim=-1)


# -- mixers ---------------------------------------------------------------------------------------------------------

def sink_attention(u, w, p: str, c: dict, kind: str, v_first: Optional[torch.Tensor]):
    """Causal grouped-query softmax attention within a sliding window, with one more term exp(sink_h) in every softmax's
    denominator.  -> (output [T, E], this layer's values before any mixing with the first layer's)."""
    T = u.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (u @ w[p + ".q"].T + w[p + ".q.b"]).view(T, H, d)
    k = (u @ w[p + ".k"].T + w[p + ".k.b"]).view(T, G, d)
    v = (u @ w[p + ".v"].T + w[p + ".v.b"]).view(T, G, dv)
    rot = c.get("rot")
    if rot:
        dims, base, sc = int(rot["dims"]), float(rot["base"]), rot.get("scaling")
        if not sc:
            freq, mag = plain_frequencies(dims, base), 1.0
        elif kind == "attention":
            freq, mag = stepped_frequencies(dims, base, sc)
        else:
            freq, mag = ramped_frequencies(dims, base, sc)
        pos = torch.arange(T)
        q, k = rotate(q, pos, freq, mag, dims), rotate(k, pos, freq, mag, dims)
    own_v = v
    if c.get("v_mix") and v_first is not None:
        lam = w[p + ".vmix"]
        v = (1.0 - lam) * v + lam * v_first
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    mask = c.get("mask")
    if mask:
        seen = seen & (i - j < int(mask["size"]))
    cap = c.get("softcap") if kind == "attention_2" else None        # only the second kind caps its scores
    out = torch.zeros(T, H, dv, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * c["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, float("-inf"))
        s = torch.cat((s, w[p + ".sink"][h].expand(T, 1)), dim=1)
        a = torch.softmax(s, dim=1)[:, :T]
        out[:, h] = a @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + ".o"].T, own_v


def short_convolution(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_i taps[:, K-1-i] x_(t-i), zeros before the start, no bias."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for i in range(K):
        y[i:] += x[: T - i] * taps[:, K - 1 - i] if i else x * taps[:, K - 1]
    return y


def delta_rule(u, w, p: str, c: dict, eps: float):
    """The gated delta rule: per head a state S [dim, vdim] that decays, is corrected towards the value at the current key
    and is read by the query, token by token."""
    T = u.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(short_convolution(u @ w[p + ".q"].T, w[p + ".q.conv"])).view(T, G, d)
    k = silu(short_convolution(u @ w[p + ".k"].T, w[p + ".k.conv"])).view(T, G, d)
    v = silu(short_convolution(u @ w[p + ".v"].T, w[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(u @ w[p + ".b"].T)
    decay = torch.exp(-torch.exp(w[p + ".A_log"]) * torch.nn.functional.softplus(u @ w[p + ".a"].T + w[p + ".dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(d, dv, dtype=u.dtype)
        for t in range(T):
            S = decay[t, h] * S
            corr = beta[t, h] * (v[t, h] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], corr)
            out[t, h] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w[p + ".norm"]
    out = out.reshape(T, H * dv) * silu(u @ w[p + ".g"].T)
    return out @ w[p + ".o"].T


# -- feed-forward ---------------------------------------------------------------------------------------------------

def clamped_expert(u, w, p: str, limit: float):
    g = (u @ w[p + ".gate"].T).clamp(max=limit)
    up = (u @ w[p + ".up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (up + 1.0)) @ w[p + ".down"].T


def expert_mixture(u, w, p: str, c: dict, margins: Optional[list] = None):
    """Every token's `top` experts by router logit, weighted by the softmax over the chosen logits, plus a shared expert
    times the sigmoid of one number per token.  margins, if given, receives per token the gap between the smallest chosen
    logit and the largest one that was not chosen (how close the choice was)."""
    r = c["router"]
    z = u @ w[p + ".router"].T
    top, idx = torch.topk(z, int(r["top"]), dim=1)
    if margins is not None and int(r["top"]) < z.shape[1]:
        ordered = z.sort(dim=1, descending=True).values
        margins.append(ordered[:, int(r["top"]) - 1] - ordered[:, int(r["top"])])
    wt = torch.softmax(top, dim=1)
    out = torch.zeros_like(u)
    for e in range(int(r["experts"])):
        ye = clamped_expert(u, w, f"{p}.e{e}", float(c["expert"]["limit"]))
        out = out + ye * (wt * (idx == e)).sum(dim=1, keepdim=True)
    sh = c.get("shared")
    if sh:
        out = out + clamped_expert(u, w, p + ".shared", float(sh["limit"])) * torch.sigmoid(u @ w[p + ".shared.sg"].T)
    return out


def token_side(x, tokens, w, layer: int, side_dim: int, eps: float):
    """What a layer adds from the per-layer token table (before the model's factor): a gated slice of the token's row,
    projected to the width and RMS-normed with a plain weight."""
    ids = torch.tensor(tokens, dtype=torch.long)
    e = w["side.embed"][ids][:, layer * side_dim:(layer + 1) * side_dim]
    y = (gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e) @ w[f"l{layer}.side.proj"].T
    return rms_unit(y, eps) * w[f"l{layer}.side.norm"]


# -- the model ------------------------------------------------------------------------------------------------------

def forward_sequence(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32, layers_out: Optional[list] = None,
                     margins: Optional[list] = None):
    """-> logits [T, vocab] for every place of the sequence.  layers_out, if given, receives the stream after every layer;
    margins the routers' gaps between the last chosen and the first unchosen logit, one tensor [T] per routed layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    m = float(cfg.get("residual_mult", 1.0))
    side = cfg.get("token_side")
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        u = rms_norm(x, w[p + ".norm1"], eps)
        kind = layer["type"]
        if kind in ("attention", "attention_2"):
            a, own_v = sink_attention(u, w, p + ".mix", layer["mixer"], kind, v_first)
            if layer["mixer"].get("v_mix") and v_first is None:
                v_first = own_v
        elif kind == "delta":
            a = delta_rule(u, w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(kind)
        x = x + m * a * w[p + ".ls1"]
        if layer.get("mlp") is not None:
            u = rms_norm(x, w[p + ".norm2"], eps)
            x = x + m * expert_mixture(u, w, p + ".mlp", layer["mlp"], margins) * w[p + ".ls2"]
        if side:
            x = x + m * token_side(x, tokens, w, i, int(side["dim"]), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n):
        with torch.no_grad():
            toks.append(int(forward_sequence(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
