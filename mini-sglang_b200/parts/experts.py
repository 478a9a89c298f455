from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of small gated feed-forwards of which every token uses `top`.

    Router: scores s = sigmoid(Wr x) with float32 sums; the choice goes by s + correction (a learned number per expert that takes
    no part in the weights); the experts form `groups` equal groups of neighbours, a group counts by the sum of its two largest
    choice scores, and only experts of the `keep_groups` best groups can be chosen; the `top` largest choice scores win; their
    weights are their s over the sum of those (+ 1e-20).  Expert: down_e (silu(gate_e x) * (up_e x)), no biases.  The output is
    the weighted sum of the chosen experts' outputs, in float32, times `out_scale`.

    A few (token, choice) pairs - and every step that a CUDA graph replays - read the chosen experts' rows straight from the
    stacked weights (two launches whatever the choice).  Many tokens are put in the order of their experts on the device; in
    bfloat16 the library's grouped matrix product then runs every expert's gate/up rows in one launch and every down product in
    another, with the experts' row ranges read on the device (rows of bfloat16, summed in float32); in float32, or where the
    sizes are no multiples of 8, the host reads the experts' counts (one small copy) and runs one gate/up product with its
    activation and one down product per expert that has tokens.  One kernel sums every token's rows with their weights.

    params: hidden_size, intermediate_size, num_experts, top, groups, keep_groups, out_scale,
            names (router, correction, expert (with {e} for the expert's number), gate, up, down).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        s = spec
        self.H, self.F, self.n_exp, self.top = int(s["hidden_size"]), int(s["intermediate_size"]), int(s["num_experts"]), int(s["top"])
        self.n_groups, self.keep = int(s.get("groups", 1)), int(s.get("keep_groups", s.get("groups", 1)))
        self.out_scale = float(s.get("out_scale", 1.0))
        if self.n_exp > ops.ROUTE_MAX_EXPERTS or self.n_groups > ops.ROUTE_MAX_GROUPS:
            raise ValueError(f"the router kernel takes up to {ops.ROUTE_MAX_EXPERTS} experts in up to {ops.ROUTE_MAX_GROUPS} groups")
        if self.n_groups < 1 or self.n_exp % self.n_groups or not 1 <= self.keep <= self.n_groups:
            raise ValueError("the experts must divide into equal groups, of which 1 .. all are kept")
        if not 1 <= self.top <= self.keep * (self.n_exp // self.n_groups):
            raise ValueError(f"top = {self.top}: the kept groups hold {self.keep * (self.n_exp // self.n_groups)} experts")
        names = {"router": "router", "correction": "correction", "expert": "e{e}", "gate": "gate", "up": "up", "down": "down"}
        names.update(s.get("names") or {})
        self.names = names
        self.router = self.correction = self.down = self.gate_up = None

    def _expert(self, e: int, what: str) -> str:
        return self.name(self.names["expert"].format(e=e) + "." + self.names[what])

    def tensors(self) -> Dict[str, TensorDecl]:
        t = {self.name(self.names["router"]): TensorDecl((self.n_exp, self.H), std=0.5),
             self.name(self.names["correction"]): TensorDecl((self.n_exp,), kind="vector", std=0.1)}
        for e in range(self.n_exp):
            t[self._expert(e, "gate")] = TensorDecl((self.F, self.H))
            t[self._expert(e, "up")] = TensorDecl((self.F, self.H))
            t[self._expert(e, "down")] = TensorDecl((self.H, self.F))
        return t

    def load(self, src) -> None:
        f = src.fetch
        self.router = f(self.name(self.names["router"])).contiguous()
        self.correction = f(self.name(self.names["correction"])).float().contiguous()
        # [E, 2, F, H]: an expert's gate and up side by side are the packed matrix of the fused product + activation
        self.gate_up = torch.stack([torch.stack((f(self._expert(e, "gate")), f(self._expert(e, "up")))) for e in range(self.n_exp)]).contiguous()
        self.down = torch.stack([f(self._expert(e, "down")) for e in range(self.n_exp)]).contiguous()

    def forward(self, x, ctx):
        idx, wts = ops.route(x, self.router, self.correction, n_groups=self.n_groups, keep=self.keep, top=self.top)
        T = x.shape[0]
        if ctx.uniform_decode or T * self.top <= ops.EXPERTS_FEW_PAIRS:
            return ops.experts_few(x, self.gate_up, self.down, idx, wts, self.out_scale)
        counts, place = ops.expert_order(idx, self.n_exp)
        rows = ops.expert_gather(x, place, self.top)
        if x.dtype == torch.bfloat16 and self.H % 8 == 0 and self.F % 8 == 0 and hasattr(torch, "_grouped_mm"):
            # the library's grouped product takes the experts' row ranges from the device: two launches, nothing read on the host
            ends = torch.cumsum(counts, 0, dtype=torch.int32)
            a = ops.swiglu(torch._grouped_mm(rows, self.gate_up.view(self.n_exp, 2 * self.F, self.H).transpose(-2, -1), offs=ends))
            y = torch._grouped_mm(a, self.down.transpose(-2, -1), offs=ends)
            return ops.expert_combine(y, place, wts, self.out_scale)
        y = torch.empty((T * self.top, self.H), dtype=torch.float32, device=x.device)
        at = 0
        for e, n in enumerate(counts.tolist()):          # the one read of device data on the host: the experts' row counts
            if n:
                a = ops.linear_swiglu(rows[at:at + n], self.gate_up[e].view(2 * self.F, self.H))
                y[at:at + n] = ops.linear(a, self.down[e], out_dtype=torch.float32)
                at += n
        return ops.expert_combine(y, place, wts, self.out_scale)


@register_feed_forward("softmax_experts")
class SoftmaxExperts(FeedForward):
    """A mixture of small clamped gated feed-forwards chosen by the largest router logits, beside a shared one.

    Router: z = Wr x with float32 sums; the `top` experts with the largest logits are chosen (the lower index wins a tie) and
    their weights are the softmax over the chosen logits only.  Expert, no biases: g = min(gate_e x, limit),
    u = clamp(up_e x, -limit, limit), down_e (g * sigmoid(1.702 g) * (u + 1)).  The output is the weighted sum of the chosen
    experts' outputs in float32.  With `shared_size` > 0 a shared expert of the same form (sizes and limit of its own) runs
    for every token and is added, times sigmoid(wsg . x), one number per token that the router kernel makes beside its logits.

    The launches are those of `routed_experts`: a few (token, choice) pairs and every CUDA-graph step stream the chosen
    experts' rows; many tokens are put in the order of their experts for one grouped product each way.

    params: hidden_size, intermediate_size, limit, num_experts, top, shared_size, shared_limit,
            names (router, expert (with {e}), gate, up, down, shared, shared_gate).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        s = spec
        self.H, self.F, self.n_exp, self.top = int(s["hidden_size"]), int(s["intermediate_size"]), int(s["num_experts"]), int(s["top"])
        self.limit = float(s["limit"])
        self.Fs, self.shared_limit = int(s.get("shared_size") or 0), float(s.get("shared_limit") or 0.0)
        if self.n_exp > ops.ROUTE_MAX_EXPERTS:
            raise ValueError(f"the router kernel takes up to {ops.ROUTE_MAX_EXPERTS} experts")
        if not 1 <= self.top <= self.n_exp:
            raise ValueError(f"top = {self.top}: the model has {self.n_exp} experts")
        names = {"router": "router", "expert": "e{e}", "gate": "gate", "up": "up", "down": "down", "shared": "shared",
                 "shared_gate": "shared.sg"}
        names.update(s.get("names") or {})
        self.names = names
        self.router = self.down = self.gate_up = self.sh_gate_up = self.sh_down = self.sh_gate = None

    def _expert(self, e: int, what: str) -> str:
        return self.name(self.names["expert"].format(e=e) + "." + self.names[what])

    def tensors(self) -> Dict[str, TensorDecl]:
        t = {self.name(self.names["router"]): TensorDecl((self.n_exp, self.H), std=0.5)}
        for e in range(self.n_exp):
            t[self._expert(e, "gate")] = TensorDecl((self.F, self.H))
            t[self._expert(e, "up")] = TensorDecl((self.F, self.H))
            t[self._expert(e, "down")] = TensorDecl((self.H, self.F))
        if self.Fs:
            sh = self.name(self.names["shared"])
            t[f"{sh}.{self.names['gate']}"] = TensorDecl((self.Fs, self.H))
            t[f"{sh}.{self.names['up']}"] = TensorDecl((self.Fs, self.H))
            t[f"{sh}.{self.names['down']}"] = TensorDecl((self.H, self.Fs))
            t[self.name(self.names["shared_gate"])] = TensorDecl((1, self.H), std=0.5)
        return t

    def load(self, src) -> None:
        f = src.fetch
        self.router = f(self.name(self.names["router"])).contiguous()
        self.gate_up = torch.stack([torch.stack((f(self._expert(e, "gate")), f(self._expert(e, "up")))) for e in range(self.n_exp)]).contiguous()
        self.down = torch.stack([f(self._expert(e, "down")) for e in range(self.n_exp)]).contiguous()
        if self.Fs:
            sh = self.name(self.names["shared"])
            self.sh_gate_up = torch.cat((f(f"{sh}.{self.names['gate']}"), f(f"{sh}.{self.names['up']}")), dim=0).contiguous()
            self.sh_down = f(f"{sh}.{self.names['down']}").contiguous()
            self.sh_gate = f(self.name(self.names["shared_gate"])).reshape(-1).contiguous()

    def forward(self, x, ctx):
        idx, wts, sgate = ops.route(x, self.router, None, n_groups=1, keep=1, top=self.top, softmax=True, gate_row=self.sh_gate)
        shared = None
        if self.Fs:
            a = ops.clamped_glu(ops.linear(x, self.sh_gate_up), self.shared_limit)
            shared = ops.linear(a, self.sh_down, out_dtype=torch.float32)
        T = x.shape[0]
        if ctx.uniform_decode or T * self.top <= ops.EXPERTS_FEW_PAIRS:
            return ops.experts_few(x, self.gate_up, self.down, idx, wts, limit=self.limit, extra=shared, extra_gate=sgate)
        counts, place = ops.expert_order(idx, self.n_exp)
        rows = ops.expert_gather(x, place, self.top)
        if x.dtype == torch.bfloat16 and self.H % 8 == 0 and self.F % 8 == 0 and hasattr(torch, "_grouped_mm"):
            ends = torch.cumsum(counts, 0, dtype=torch.int32)
            gu = torch._grouped_mm(rows, self.gate_up.view(self.n_exp, 2 * self.F, self.H).transpose(-2, -1), offs=ends)
            y = torch._grouped_mm(ops.clamped_glu(gu, self.limit), self.down.transpose(-2, -1), offs=ends)
            return ops.expert_combine(y, place, wts, extra=shared, extra_gate=sgate)
        y = torch.empty((T * self.top, self.H), dtype=torch.float32, device=x.device)
        at = 0
        for e, n in enumerate(counts.tolist()):          # the one read of device data on the host: the experts' row counts
            if n:
                a = ops.clamped_glu(ops.linear(rows[at:at + n], self.gate_up[e].view(2 * self.F, self.H)), self.limit)
                y[at:at + n] = ops.linear(a, self.down[e], out_dtype=torch.float32)
                at += n
        return ops.expert_combine(y, place, wts, extra=shared, extra_gate=sgate)
