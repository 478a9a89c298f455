from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorDecl
from .base import Mixer, register_mixer


@register_mixer("gated_delta")
class GatedDeltaRule(Mixer):
    """A linear-attention mixer whose state is corrected towards the current value (the gated delta rule).

    q = Wq x, k = Wk x [kv heads, key_dim], v = Wv x [heads, value_dim], no biases; each passes a short causal convolution
    over time per channel (taps [channels, taps], the last column is the current token's, no bias, zeros before the start;
    the last taps - 1 inputs are carried as state) and silu; q and k become unit vectors per head, u / sqrt(sum u^2 + 1e-6),
    and q is multiplied by key_dim^-1/2; head h reads q/k head h // (heads / kv heads).  Per head and token a write strength
    beta = sigmoid(Wb x) and a decay g = exp(-exp(A_log_h) softplus(Wa x + dt_bias_h)).  Per head and request a float32 state
    S [key_dim, value_dim] that starts at zero:

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    so the read-out sees the current token's write.  Every head's o is RMS-normed over value_dim with one plain weight for all
    heads, times silu(Wg x); output projection.  All input projections are one product; unit norms, beta, decay, state and the
    output norm are float32.

    params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, norm_eps, names.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.heads, self.n_kv = int(s["hidden_size"]), int(s["num_heads"]), int(s["num_kv_heads"])
        self.d, self.dv, self.taps = int(s["key_dim"]), int(s["value_dim"]), int(s.get("conv_taps", 1))
        self.eps = float(s["norm_eps"])
        if self.heads % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.d > ops.DELTA_RULE_MAX_KEY_DIM:
            raise ValueError(f"key size {self.d}: the delta-rule kernel takes up to {ops.DELTA_RULE_MAX_KEY_DIM}")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"{self.taps} taps: the convolution kernel takes 1 to {ops.CONV_MAX_TAPS}")
        names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "a": "a",
                 "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "out": "o"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.Ck, self.Cv = self.n_kv * self.d, self.heads * self.dv
        self.conv_channels = 2 * self.Ck + self.Cv
        self.w_in = self.w_out = self.conv_w = self.a_log = self.dt_bias = self.norm = None

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["q"]: TensorDecl((self.Ck, self.E)), n["k"]: TensorDecl((self.Ck, self.E)), n["v"]: TensorDecl((self.Cv, self.E)),
                n["q_conv"]: TensorDecl((self.Ck, self.taps), kind="vector", std=0.5),
                n["k_conv"]: TensorDecl((self.Ck, self.taps), kind="vector", std=0.5),
                n["v_conv"]: TensorDecl((self.Cv, self.taps), kind="vector", std=0.5),
                n["beta"]: TensorDecl((self.heads, self.E)), n["a"]: TensorDecl((self.heads, self.E)),
                n["a_log"]: TensorDecl((self.heads,), kind="vector", std=0.5), n["dt_bias"]: TensorDecl((self.heads,), kind="vector", std=0.5),
                n["gate"]: TensorDecl((self.Cv, self.E)), n["norm"]: TensorDecl((self.dv,), kind="vector", init="norm"),
                n["out"]: TensorDecl((self.E, self.Cv))}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        # packed rows [q | k | v | gate | a | beta], padded with zero rows to a multiple of 16
        w_in = torch.cat((f(n["q"]), f(n["k"]), f(n["v"]), f(n["gate"]), f(n["a"]), f(n["beta"])), dim=0)
        pad = -w_in.shape[0] % 16
        if pad:
            w_in = torch.cat((w_in, w_in.new_zeros((pad, w_in.shape[1]))), dim=0)
        self.w_in, self.w_out = w_in.contiguous(), f(n["out"]).contiguous()
        self.conv_w = torch.cat((f(n["q_conv"]), f(n["k_conv"]), f(n["v_conv"])), dim=0).float().t().contiguous()      # [taps, channels]
        self.a_log, self.dt_bias = f(n["a_log"]).float().contiguous(), f(n["dt_bias"]).float().contiguous()
        self.norm = f(n["norm"]).float().contiguous()

    def cache_need(self):
        return (StateNeed((max(self.taps - 1, 1), self.conv_channels), "compute"), StateNeed((self.heads, self.d, self.dv), "float32"))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        conv, rec = cache
        cc, Cv, H = self.conv_channels, self.Cv, self.heads
        proj = ops.linear(x, self.w_in)
        qkv = ops.causal_conv_act(proj[:, :cc], self.conv_w, None, state=conv.state if self.taps > 1 else None,
                                  token_req=ctx.token_req, q_start=ctx.q_start, slots=ctx.slots)
        o = ops.delta_rule(qkv, proj[:, cc + Cv:cc + Cv + H], proj[:, cc + Cv + H:cc + Cv + 2 * H], heads=H, kv_heads=self.n_kv,
                           key_dim=self.d, value_dim=self.dv, a_log=self.a_log, dt_bias=self.dt_bias, state=rec.state,
                           q_start=ctx.q_start, slots=ctx.slots, q_lens=None if ctx.uniform_decode else ctx.host_q_lens,
                           workspace=ctx.workspace)
        act = torch.empty((x.shape[0], Cv), dtype=x.dtype, device=x.device)
        ops.group_rms_gate(o, H, self.norm, self.eps, proj[:, cc:cc + Cv], act, ops.ACT_SILU)
        return ops.linear(act, self.w_out)
