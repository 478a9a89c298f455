from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorDecl
from .base import Mixer, Projected, register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer, Projected):
    """Causal grouped-query attention over all earlier keys whose weights are sigmoids: no softmax, nothing is normed over the
    keys, so a key's weight does not depend on the other keys.

    q = Wq x, k = Wk x [heads resp. kv heads, key_dim], v = Wv x [kv heads, value_dim]; every head of q and of k is RMS-normed by
    itself with one weight of key_dim shared by all heads (plain weight); no rotation; the query at position i is multiplied by
    1 + temp_coef * ln(floor((i + 1) / temp_every) + 1) (temp_coef 0: no such factor); the weight of key j <= i is

        sigmoid(q_i . k_j * scale - r1_h * ln(1 + r2_h * (i - j)) + pb_h)

    with three learned numbers per head; o_i = sum_j weight * v_j; output projection on the heads side by side.  The part after
    the dot product depends on the head and the distance only; it is made once at load as a table [heads, max_positions] (in
    double precision, kept in float32), so no kernel evaluates a logarithm per score.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, norm_eps, temp_coef, temp_every, max_positions,
            names (what the checkpoint calls q, k, v, q_norm, k_norm, r1, r2, pb, out below the part's prefix).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.n_q, self.n_kv = int(s["hidden_size"]), int(s["num_heads"]), int(s["num_kv_heads"])
        self.d, self.dv = int(s["key_dim"]), int(s["value_dim"])
        if self.n_q % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if max(self.d, self.dv) > ops.SIGMOID_ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"head sizes {self.d}, {self.dv}: the sigmoid attention kernel takes up to {ops.SIGMOID_ATTENTION_MAX_HEAD_DIM}")
        self.scale, self.eps = float(s["scale"]), float(s["norm_eps"])
        self.temp_coef, self.temp_every = float(s.get("temp_coef", 0.0)), int(s.get("temp_every", 1))
        if self.temp_coef != 0.0 and self.temp_every < 1:
            raise ValueError("temp_every must be at least 1")
        self.max_positions = int(s["max_positions"])
        names = {"q": "q", "k": "k", "v": "v", "q_norm": "q_norm", "k_norm": "k_norm", "r1": "r1", "r2": "r2", "pb": "pb", "out": "out"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.Cq, self.Ck, self.Cv = self.n_q * self.d, self.n_kv * self.d, self.n_kv * self.dv
        self.w_in = self.w_out = self.q_norm = self.k_norm = self.bias = None

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["q"]: TensorDecl((self.Cq, self.E)), n["k"]: TensorDecl((self.Ck, self.E)), n["v"]: TensorDecl((self.Cv, self.E)),
                n["q_norm"]: TensorDecl((self.d,), kind="vector", init="norm"),
                n["k_norm"]: TensorDecl((self.d,), kind="vector", init="norm"),
                n["r1"]: TensorDecl((self.n_q,), kind="vector", init="norm"), n["r2"]: TensorDecl((self.n_q,), kind="vector", init="norm"),
                n["pb"]: TensorDecl((self.n_q,), kind="vector", std=0.5), n["out"]: TensorDecl((self.E, self.n_q * self.dv))}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in = torch.cat((f(n["q"]), f(n["k"]), f(n["v"])), dim=0).contiguous()
        self.w_out = f(n["out"]).contiguous()
        self.q_norm, self.k_norm = f(n["q_norm"]).float().contiguous(), f(n["k_norm"]).float().contiguous()
        r1, r2, pb = (f(n[k]).double() for k in ("r1", "r2", "pb"))
        dist = torch.arange(self.max_positions, dtype=torch.float64, device=r1.device)
        self.bias = (pb[:, None] - r1[:, None] * torch.log1p(r2[:, None] * dist[None, :])).float().contiguous()     # [heads, distances]

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.d, None, q_heads=self.n_q, library="mixers_gated", even_cut=False, v_head_dim=self.dv)

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        Cq, Ck, Cv = self.Cq, self.Ck, self.Cv
        q = ops.headnorm_kvwrite(proj[:, :Cq], proj[:, Cq:Cq + Ck], proj[:, Cq + Ck:Cq + Ck + Cv], n_q=self.n_q, n_kv=self.n_kv,
                                 q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, temp_coef=self.temp_coef,
                                 temp_every=self.temp_every, positions=ctx.positions,
                                 out_loc=cache.group.out_loc if writes_cache else None, k_cache=cache.k if writes_cache else None,
                                 v_cache=cache.v if writes_cache else None, page_size=cache.page_size)
        ops.sigmoid_attention(q, act, cache.k, cache.v, q_start=ctx.q_start, kv_len=ctx.kv_len, block_table=cache.group.block_table,
                              n_kv=self.n_kv, page_size=cache.page_size, scale=self.scale, bias=self.bias,
                              q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)
        if out_scale != 1.0:
            act.mul_(out_scale)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)
