from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, Projected, register_feed_forward


@register_feed_forward("swiglu_mlp")
class SwiGLUMLP(FeedForward):
    """down(silu(gate(x)) * up(x)), dense, no biases (mini_sglang/models/qwen3.py:100-126).
    gate_proj and up_proj are packed row-wise into one [2I, H] matrix so one product feeds the
    activation kernel (the packing of mini_sglang/layers/linear.py:126-138).
    params: hidden_size, intermediate_size."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.H, self.I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.gate_up = self.down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.name("gate_proj.weight"): TensorDecl((self.I, self.H)),
                self.name("up_proj.weight"): TensorDecl((self.I, self.H)),
                self.name("down_proj.weight"): TensorDecl((self.H, self.I))}

    def load(self, src) -> None:
        self.gate_up = torch.cat((src.fetch(self.name("gate_proj.weight")), src.fetch(self.name("up_proj.weight"))),
                                 dim=0).contiguous()
        self.down = src.fetch(self.name("down_proj.weight")).contiguous()

    def forward(self, x, ctx):
        return ops.linear(ops.linear_swiglu(x, self.gate_up), self.down)

    def fused_decode_fields(self):
        return {"kind": "swiglu_mlp", "gate_up": self.gate_up, "down": self.down, "H": self.H, "I": self.I}


ACTIVATIONS = {"silu": ops.ACT_SILU, "gelu_tanh": ops.ACT_GELU_TANH}


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward, Projected):
    """down(act(gate(x)) * up(x)), dense, no biases, with act = "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z +
    0.044715 z^3)))).  gate and up are packed row-wise into one [2I, H] matrix.  params: hidden_size, intermediate_size,
    activation, names (what the checkpoint calls gate, up and down below the part's prefix; default "gate_proj.weight" ...)."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.H, self.I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        act = spec.get("activation", "silu")
        if act not in ACTIVATIONS:
            raise ValueError(f"unknown activation {act!r}; known: " + ", ".join(sorted(ACTIVATIONS)))
        self.act = ACTIVATIONS[act]
        names = spec.get("names") or {}
        self.n_gate, self.n_up, self.n_down = (self.name(names.get(k, d)) for k, d in
                                                (("gate", "gate_proj.weight"), ("up", "up_proj.weight"), ("down", "down_proj.weight")))
        self.gate_up = self.down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.n_gate: TensorDecl((self.I, self.H)), self.n_up: TensorDecl((self.I, self.H)),
                self.n_down: TensorDecl((self.H, self.I))}

    def load(self, src) -> None:
        self.gate_up = torch.cat((src.fetch(self.n_gate), src.fetch(self.n_up)), dim=0).contiguous()
        self.down = src.fetch(self.n_down).contiguous()

    def in_weight(self):
        return self.gate_up

    def out_weight(self):
        return self.down

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        assert out_scale == 1.0
        ops.gated_act(proj[:, :self.I], proj[:, self.I:2 * self.I], act, self.act)

    def forward(self, x, ctx):
        if self.act == ops.ACT_SILU:        # product and activation in one kernel where the engine has it (few rows; many rows in bfloat16)
            return ops.linear(ops.linear_swiglu(x, self.gate_up), self.down)
        return self.forward_projected(x, ctx)


UNARY_ACTIVATIONS = {"silu": ops.ACT_SILU, "gelu_tanh": ops.ACT_GELU_TANH, "relu2": ops.ACT_RELU2, "relu": ops.ACT_RELU}


@register_feed_forward("plain_mlp")
class PlainMLP(FeedForward):
    """down(act(up(x))), dense, no gate, no biases; act = "relu2" (the square of relu), "relu", "silu" or "gelu_tanh".  The result
    is float32, times `out_scale` (applied to the activation, before the second product).
    params: hidden_size, intermediate_size, activation, out_scale, names (up, down)."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.H, self.I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        act = spec.get("activation", "relu2")
        if act not in UNARY_ACTIVATIONS:
            raise ValueError(f"unknown activation {act!r}; known: " + ", ".join(sorted(UNARY_ACTIVATIONS)))
        self.act, self.out_scale = UNARY_ACTIVATIONS[act], float(spec.get("out_scale", 1.0))
        names = spec.get("names") or {}
        self.n_up, self.n_down = self.name(names.get("up", "up_proj.weight")), self.name(names.get("down", "down_proj.weight"))
        self.up = self.down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.n_up: TensorDecl((self.I, self.H)), self.n_down: TensorDecl((self.H, self.I))}

    def load(self, src) -> None:
        self.up, self.down = src.fetch(self.n_up).contiguous(), src.fetch(self.n_down).contiguous()

    def forward(self, x, ctx):
        u = ops.linear(x, self.up)
        return ops.linear(ops.unary_act(u, self.act, self.out_scale, out=u), self.down, out_dtype=torch.float32)
