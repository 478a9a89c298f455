"""A plain, slow implementation of the Pepevik decoder, one function per mechanism, written from the
architecture's equations and sharing no code with the engine.  It takes the content of a config.json and a
dict of tensors by checkpoint name and runs one whole sequence at a time on the CPU; there is no cache: every
function sees all tokens of the sequence, and the recurrences walk them one by one.

Notation: T tokens, width E, x the residual stream [T, E], u the normed input of a sublayer.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def dynamic_tanh(x, w, name):
    """tanh(alpha x) * weight + bias, element by element; no statistics of the row."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms_unit(x, eps):
    """x over its root mean square along the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens: List[int], w, scale: float):
    """Token rows times a constant plus the learned vector of every place (unscaled)."""
    ids = torch.tensor(tokens, dtype=torch.long)
    return w["embed"][ids] * scale + w["pos"][: len(tokens)]


def query_temperature(T: int, coef: float, every: int, dtype):
    """1 + coef * ln(floor((p + 1) / every) + 1) for the places p = 0 .. T-1."""
    p = torch.arange(T, dtype=torch.long)
    return 1.0 + coef * torch.log(((p + 1) // every + 1).to(dtype))


def sigmoid_attention(u, w, p: str, c: dict, eps: float):
    """Causal grouped-query attention whose weights are sigmoids, each key by itself: no normalisation over keys.
    score(i, j) = q_i . k_j * scale - r1 ln(1 + r2 (i - j)) + pb, per head; q and k normed per head, q warmed up by place."""
    T = u.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (u @ w[p + ".q"].T).view(T, H, d)
    k = (u @ w[p + ".k"].T).view(T, G, d)
    v = (u @ w[p + ".v"].T).view(T, G, dv)
    q = rms_unit(q, eps) * w[p + ".q.norm"]
    k = rms_unit(k, eps) * w[p + ".k.norm"]
    qt = c.get("q_temp")
    if qt:
        q = q * query_temperature(T, qt["coef"], qt["every"], u.dtype)[:, None, None]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).clamp(min=0).to(u.dtype)
    seen = j <= i
    out = torch.zeros(T, H, dv, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * c["scale"]
        s = s - w[p + ".r1"][h] * torch.log1p(w[p + ".r2"][h] * dist) + w[p + ".pb"][h]
        a = torch.sigmoid(s) * seen
        out[:, h] = a @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + ".o"].T


def min_gru(u, w, p: str):
    """A gated recurrence whose gates see the current token only: S_t = (1 - z_t) S_{t-1} + z_t c_t from S = 0, with
    c = a + 1/2 for a >= 0 and sigmoid(a) below; the state times silu of a gate projection goes through W_o."""
    T = u.shape[0]
    z = torch.sigmoid(u @ w[p + ".z"].T + w[p + ".z.b"])
    a = u @ w[p + ".x"].T + w[p + ".x.b"]
    cand = torch.where(a >= 0, a + 0.5, torch.sigmoid(a))
    S = torch.zeros(z.shape[1], dtype=u.dtype)
    states = []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        states.append(S)
    S = torch.stack(states)
    return (S * silu(u @ w[p + ".g"].T)) @ w[p + ".o"].T


def parallel_mixer(u, w, p: str, c: dict, eps: float):
    """Half the sum of the two mixers' outputs, each RMS-normed over the width with a plain weight of its own."""
    a = sigmoid_attention(u, w, p + ".left", c["left"], eps)
    b = min_gru(u, w, p + ".right")
    return 0.5 * (rms_unit(a, eps) * w[p + ".left.out"] + rms_unit(b, eps) * w[p + ".right.out"])


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K] whose last column meets the current token, zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat((torch.zeros(K - 1, C, dtype=x.dtype), x), dim=0)
    y = bias.expand(T, C).clone()
    for j in range(K):
        y = y + taps[:, j] * padded[j:j + T]
    return y


def mamba2(u, w, p: str, c: dict, eps: float):
    """State-space mixer: per head S_t = exp(-exp(A) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; x, B, C through a
    short convolution and silu; y gated by silu(z) BEFORE a group-wise RMS norm; then W_o."""
    T = u.shape[0]
    Hn, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = Hn * P
    proj = u @ w[p + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"]))
    x = xbc[:, :inner].view(T, Hn, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + ".dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w[p + ".A_log"]) * dt)                     # [T, heads]
    y = torch.zeros(T, Hn, P, dtype=u.dtype)
    S = torch.zeros(Hn, N, P, dtype=u.dtype)
    per = Hn // G
    for t in range(T):
        Bh = B[t].repeat_interleave(per, dim=0)                              # [heads, N]
        Ch = C[t].repeat_interleave(per, dim=0)
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bh[:, :, None] * x[t][:, None, :]
        y[t] = (S * Ch[:, :, None]).sum(dim=1) + w[p + ".D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    ng = c["norm_groups"]
    y = rms_unit(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w[p + ".norm"]
    return y @ w[p + ".o"].T


def dense_ff(u, w, p: str):
    """W_down relu(W_up u)^2."""
    return torch.relu(u @ w[p + ".up"].T) ** 2 @ w[p + ".down"].T


def route(u, w, p: str, r: dict, margins: Optional[list] = None):
    """-> (chosen experts [T, top], their weights [T, top]).  Scores are sigmoids of the router's logits; the choice adds a
    correction per expert and is limited to the best groups (a group counts by the sum of its two largest choice scores; experts
    of other groups are out, whatever their sign); the weights are the chosen experts' own scores over their sum.  `margins`, if
    given, receives [T]: by how much the choice was made, the smaller of the gap between the last kept group and the first one left
    out and the gap between the last chosen expert and the first allowed one left out."""
    s = torch.sigmoid(u.float() @ w[p + ".router"].float().T)
    choice = s + w[p + ".correction"].float()
    T, E = s.shape
    gc, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // gc
    grouped = choice.view(T, gc, per)
    gscore = grouped.topk(min(2, per), dim=-1).values.sum(dim=-1)
    best = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, gc, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(T, gc, per).reshape(T, E), choice, torch.full_like(choice, -math.inf))
    idx = masked.topk(r["top"], dim=-1).indices
    if margins is not None:
        gap = torch.full((T,), math.inf)
        if keep < gc:
            g = gscore.sort(dim=-1, descending=True).values
            gap = g[:, keep - 1] - g[:, keep]
        if r["top"] < keep * per:
            c = masked.sort(dim=-1, descending=True).values
            gap = torch.minimum(gap, c[:, r["top"] - 1] - c[:, r["top"]])
        margins.append(gap)
    wts = s.gather(1, idx)
    return idx, wts / (wts.sum(dim=-1, keepdim=True) + 1e-20)


def moe_ff(u, w, p: str, m: dict, margins: Optional[list] = None):
    idx, wts = route(u, w, p, m["router"], margins)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for e, a in zip(idx[t].tolist(), wts[t]):
            q = f"{p}.e{e}"
            out[t] += a.to(u.dtype) * ((silu(u[t] @ w[q + ".gate"].T) * (u[t] @ w[q + ".up"].T)) @ w[q + ".down"].T)
    return out


def forward_sequence(config: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
                     streams: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """-> logits [T, vocab].  `streams`, if given, receives the residual stream after every run of a layer; `margins` one [T] per
    routed feed-forward run (see `route`)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    if len(tokens) > config["max_positions"]:
        raise ValueError("more tokens than the model has places")
    x = embed(tokens, w, (config.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(config["layers"]):
        o = i
        while config["layers"][o].get("weights_of") is not None:
            o = config["layers"][o]["weights_of"]
        p = f"l{o}"
        u = dynamic_tanh(x, w, p + ".norm1")
        if layer["type"] == "parallel":
            x = x + m * parallel_mixer(u, w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            x = x + m * mamba2(u, w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            u = dynamic_tanh(x, w, p + ".norm2")
            if layer["mlp"]["kind"] == "dense":
                x = x + m * dense_ff(u, w, p + ".mlp")
            else:
                x = x + m * moe_ff(u, w, p + ".mlp", layer["mlp"], margins)
        if streams is not None:
            streams.append(x.clone())
    return dynamic_tanh(x, w, "final.norm") @ w["head"].T


def greedy_generate(config: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        with torch.no_grad():
            t = int(forward_sequence(config, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
