from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorDecl
from .base import Mixer, Projected, register_mixer


@register_mixer("mingru")
class MinGRU(Mixer, Projected):
    """A gated recurrence per channel whose gates read the current token only (minGRU).

    z = sigmoid(Wz x + bz), a = Wx x + bx, both of size `width`; candidate c = a + 1/2 where a >= 0 and sigmoid(a) below;
    S_t = (1 - z_t) S_(t-1) + z_t c_t element by element, from S = 0, a float32 state per request; output Wo (S_t * silu(Wg x)).
    The three input projections are one product; gates, candidate and state are float32.

    params: hidden_size, width, names (z, z_bias, x, x_bias, gate, out).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        self.E, self.W = int(spec["hidden_size"]), int(spec["width"])
        names = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}
        names.update(spec.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.w_in = self.w_out = self.z_bias = self.x_bias = None

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["z"]: TensorDecl((self.W, self.E)), n["x"]: TensorDecl((self.W, self.E)), n["gate"]: TensorDecl((self.W, self.E)),
                n["z_bias"]: TensorDecl((self.W,), kind="vector", std=0.5), n["x_bias"]: TensorDecl((self.W,), kind="vector", std=0.5),
                n["out"]: TensorDecl((self.E, self.W))}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in = torch.cat((f(n["z"]), f(n["x"]), f(n["gate"])), dim=0).contiguous()
        self.w_out = f(n["out"]).contiguous()
        self.z_bias, self.x_bias = f(n["z_bias"]).float().contiguous(), f(n["x_bias"]).float().contiguous()

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        return StateNeed((self.W,), "float32")

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        W = self.W
        ops.mingru(proj[:, :W], proj[:, W:2 * W], proj[:, 2 * W:3 * W], self.z_bias, self.x_bias, state=cache.state,
                   q_start=ctx.q_start, slots=ctx.slots, out=act, scale=out_scale,
                   q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)


@register_mixer("state_space")
class StateSpaceMixer(Mixer):
    """A selective state-space mixer with a scalar decay per head and token (the Mamba-2 form).

    One input product, laid out [z: inner | x: inner | B: groups * N | C: groups * N | dt: heads] with inner = heads * head_dim;
    x, B and C pass a short causal convolution per channel (taps with a bias; the last taps - 1 inputs are carried as state) and
    silu; step = softplus(dt + dt_bias); per head h on group h // (heads / groups) a float32 state S [N, head_dim] per request:

        S_t = exp(-exp(A_log_h) step_t) S_(t-1) + step_t B_t x_t^T,    y_t = S_t^T C_t + D_h x_t

    y (heads side by side) times silu(z), then RMS-normed in `norm_groups` equal parts (plain weight), then the output
    projection.  Steps, decays, state, gate and norm are float32.  `out_scale` multiplies what the part returns (float32).

    params: hidden_size, num_heads, head_dim, state_size, groups, conv_taps, norm_groups, norm_eps, out_scale, names.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.heads, self.P, self.N = int(s["hidden_size"]), int(s["num_heads"]), int(s["head_dim"]), int(s["state_size"])
        self.groups, self.taps, self.norm_groups = int(s.get("groups", 1)), int(s.get("conv_taps", 1)), int(s.get("norm_groups", 1))
        self.eps, self.out_scale = float(s["norm_eps"]), float(s.get("out_scale", 1.0))
        self.inner = self.heads * self.P
        if self.heads % self.groups:
            raise ValueError("num_heads must be a multiple of groups")
        if self.inner % self.norm_groups:
            raise ValueError("the heads side by side must divide into norm_groups equal parts")
        if self.N > ops.SSM_MAX_STATE:
            raise ValueError(f"state size {self.N}: the scan kernel takes up to {ops.SSM_MAX_STATE}")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"{self.taps} taps: the convolution kernel takes 1 to {ops.CONV_MAX_TAPS}")
        self.conv_channels = self.inner + 2 * self.groups * self.N
        self.in_width = 2 * self.inner + 2 * self.groups * self.N + self.heads
        names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D", "norm": "norm",
                 "out": "o"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.w_in = self.w_out = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm = None

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["in"]: TensorDecl((self.in_width, self.E)), n["conv"]: TensorDecl((self.conv_channels, self.taps), kind="vector", std=0.5),
                n["conv_bias"]: TensorDecl((self.conv_channels,), kind="vector", std=0.1),
                n["dt_bias"]: TensorDecl((self.heads,), kind="vector", std=0.5), n["a_log"]: TensorDecl((self.heads,), kind="vector", std=0.5),
                n["skip"]: TensorDecl((self.heads,), kind="vector", init="norm"),
                n["norm"]: TensorDecl((self.inner,), kind="vector", init="norm"), n["out"]: TensorDecl((self.E, self.inner))}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in, self.w_out = f(n["in"]).contiguous(), f(n["out"]).contiguous()
        self.conv_w = f(n["conv"]).float().t().contiguous()              # [taps, channels]
        self.conv_b = f(n["conv_bias"]).float().contiguous()
        self.dt_bias, self.a_log, self.skip = (f(n[k]).float().contiguous() for k in ("dt_bias", "a_log", "skip"))
        self.norm = f(n["norm"]).float().contiguous()

    def cache_need(self):
        return (StateNeed((self.taps - 1, self.conv_channels), "compute"), StateNeed((self.heads, self.N, self.P), "float32"))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        conv, ssm = cache
        inner, cc = self.inner, self.conv_channels
        proj = ops.linear(x, self.w_in)
        xbc = ops.causal_conv_act(proj[:, inner:inner + cc], self.conv_w, self.conv_b, state=conv.state if self.taps > 1 else None,
                                  token_req=ctx.token_req, q_start=ctx.q_start, slots=ctx.slots)
        y = ops.ssm_scan(xbc, proj[:, inner + cc:inner + cc + self.heads], heads=self.heads, groups=self.groups, state_size=self.N,
                         dt_bias=self.dt_bias, a_log=self.a_log, skip=self.skip, state=ssm.state, q_start=ctx.q_start, slots=ctx.slots,
                         q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)
        act = torch.empty((x.shape[0], inner), dtype=x.dtype, device=x.device)
        ops.gate_group_norm(y, proj[:, :inner], self.norm, self.norm_groups, self.eps, act, self.out_scale)
        return ops.linear(act, self.w_out, out_dtype=torch.float32)
