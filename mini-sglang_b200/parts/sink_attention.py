from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorDecl
from .base import Mixer, register_mixer
from .context import KVCacheView, StepContext


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    """Causal grouped-query softmax attention over the paged cache with one more term in every softmax's denominator.

    q = Wq x (+ bq) [heads, key_dim], k = Wk x (+ bk) [kv heads, key_dim], v = Wv x (+ bv) [kv heads, value_dim]; the layer's
    position encoding turns the first elements of every q and k head (a partial rotation in halves; v is not turned);
    score(i, j) = q_i . k_j * scale, then cap * tanh(score / cap) where the part has a `softcap`; the query at i sees the keys
    j <= i with i - j < window (all earlier keys without a window); weights = exp(score) / (sum_seen exp(score) + exp(sink_h))
    with a learned number per head that has no key and no value, is neither scaled nor capped and counts once; output
    projection on the heads side by side.

    Blended values (`value_mix`): the first layer of a model that has it ("first") hands its values of the step's tokens on
    under `value_mix_key`; a later layer ("blend") caches and reads v <- (1 - lambda) v + lambda v_first with a learned number
    lambda.  Both must have the same kv heads and value size.

    Scores, soft cap, softmax and its weights, the sink and the rotation's angles are float32 in both precisions; in
    bfloat16 the rotated q and k, the (blended) v as cached and the weights as operands of the value product are rounded.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, window (None: all keys), softcap (None: none),
            bias, value_mix (None, "first", "blend"), value_mix_key, names (q, k, v, q_bias, k_bias, v_bias, sink, mix, out).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.n_q, self.n_kv = int(s["hidden_size"]), int(s["num_heads"]), int(s["num_kv_heads"])
        self.d, self.dv = int(s["key_dim"]), int(s["value_dim"])
        if self.n_q % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if max(self.d, self.dv) > ops.SINK_ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"head sizes {self.d}, {self.dv}: the attention kernel takes up to {ops.SINK_ATTENTION_MAX_HEAD_DIM}")
        self.scale = float(s["scale"])
        self.window = int(s["window"]) if s.get("window") else None
        self.softcap = float(s["softcap"]) if s.get("softcap") else 0.0
        self.bias = bool(s.get("bias", False))
        self.value_mix, self.value_mix_key = s.get("value_mix"), s.get("value_mix_key", "first_values")
        if self.value_mix not in (None, "first", "blend"):
            raise ValueError(f"value_mix {self.value_mix!r}: None, 'first' or 'blend'")
        self.position = position
        if position is not None and not hasattr(position, "step_angles"):
            raise ValueError("this mixer takes a position encoding that makes the angles of a step's positions (step_angles)")
        names = {"q": "q", "k": "k", "v": "v", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink", "mix": "vmix", "out": "o"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.Cq, self.Ck, self.Cv = self.n_q * self.d, self.n_kv * self.d, self.n_kv * self.dv
        self.w_in = self.b_in = self.w_out = self.sink = None
        self.lam = 0.0

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        t = {n["q"]: TensorDecl((self.Cq, self.E)), n["k"]: TensorDecl((self.Ck, self.E)), n["v"]: TensorDecl((self.Cv, self.E)),
             n["sink"]: TensorDecl((self.n_q,), kind="vector", std=1.0), n["out"]: TensorDecl((self.E, self.n_q * self.dv))}
        if self.bias:
            t[n["q_bias"]] = TensorDecl((self.Cq,), kind="vector", std=0.1)
            t[n["k_bias"]] = TensorDecl((self.Ck,), kind="vector", std=0.1)
            t[n["v_bias"]] = TensorDecl((self.Cv,), kind="vector", std=0.1)
        if self.value_mix is not None:
            t[n["mix"]] = TensorDecl((), kind="vector", std=0.3, optional=self.value_mix == "first")
        return t

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in = torch.cat((f(n["q"]), f(n["k"]), f(n["v"])), dim=0).contiguous()
        self.w_out = f(n["out"]).contiguous()
        if self.bias:
            self.b_in = torch.cat((f(n["q_bias"]), f(n["k_bias"]), f(n["v_bias"])), dim=0).to(self.env.dtype).contiguous()
        self.sink = f(n["sink"]).float().contiguous()
        if self.value_mix == "blend":
            self.lam = float(f(n["mix"]).float().item())

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.n_kv, self.d, self.window, q_heads=self.n_q, library="mixers_delta", even_cut=False,
                           v_head_dim=self.dv)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: KVCacheView, writes_cache: bool = True) -> torch.Tensor:
        Cq, Ck, Cv = self.Cq, self.Ck, self.Cv
        proj = ops.linear(x, self.w_in, self.b_in)
        v_own = proj[:, Cq + Ck:Cq + Ck + Cv]
        v_first = None
        if self.value_mix == "first":
            ctx.shared[self.value_mix_key] = v_own
        elif self.value_mix == "blend":
            v_first = ctx.shared.get(self.value_mix_key)
            if v_first is None or v_first.shape != v_own.shape:
                raise ValueError("blended values: no earlier layer of the step handed on values of this layer's shape")
        angles = self.position.step_angles(ctx) if self.position is not None else None
        q = ops.sink_qkv_prep(proj, n_q=self.n_q, n_kv=self.n_kv, d=self.d, dv=self.dv, angles=angles, v_first=v_first, lam=self.lam,
                              out_loc=cache.group.out_loc if writes_cache else None, k_cache=cache.k if writes_cache else None,
                              v_cache=cache.v if writes_cache else None, page_size=cache.page_size)
        out = torch.empty((ctx.T, self.n_q * self.dv), dtype=x.dtype, device=x.device)
        ops.sink_attention(q, out, cache.k, cache.v, q_start=ctx.q_start, kv_len=ctx.kv_len, block_table=cache.group.block_table,
                           n_kv=self.n_kv, page_size=cache.page_size, scale=self.scale, softcap=self.softcap, window=self.window or 0,
                           sink=self.sink, q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)
        return ops.linear(out, self.w_out)
