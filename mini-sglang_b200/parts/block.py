from __future__ import annotations

from typing import Dict

from ..weights.loader import TensorDecl
import torch

from .. import ops
from ..config.spec import PartSpec
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv, Part, Projected, build_part,
                   register_block)


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    """res += delta_in; y = norm_in(res); a = mixer(y); res += a; y = norm_post(res); delta_out = ffn(y)

    The block returns its feed-forward output un-added together with the stream, so the next
    norm (the next block's, or the model's final norm) fuses the sum, as the reference does
    (mini_sglang/models/qwen3.py:162-178).  Roles: norms "input" and "post_mixer", "mixer", "feed_forward";
    what the checkpoint calls each of them below the layer's prefix comes from the layer description
    (`LayerSpec.names`).  Position encodings with equal parameters are one object shared by all layers."""

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        at = layer_spec.part_prefix
        self.position = None
        if layer_spec.position is not None:
            self.position = env.shared(layer_spec.position, lambda: build_part(
                POSITION_ENCODINGS, "position encoding", layer_spec.position, layer_spec.prefix, env))
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=self.position)
        self.norm_post = self.ffn = None
        if layer_spec.feed_forward is not None:      # a layer without a feed-forward hands its mixer's output on un-added
            self.norm_post = build_part(NORMS, "norm", layer_spec.norms["post_mixer"], at("post_mixer"), env)
            self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)

    def parts(self):
        return [p for p in (self.position, self.norm_in, self.mixer, self.norm_post, self.ffn) if p is not None]

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, src) -> None:
        for part in self.parts():
            part.load(src)

    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        # residual: float32 stream, updated in place; delta: the previous block's output or None
        y = self.norm_in.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
        a = self.mixer.forward(y, ctx, cache, writes_cache)
        if self.ffn is None:
            return a, residual
        y = self.norm_post.forward(x=a, residual=residual, residual_out=residual)
        return self.ffn.forward(y, ctx), residual

    def fused_decode_fields(self):
        """This arrangement is the one the whole-step decode kernel walks (norm, mixer, residual sum, norm, feed-forward,
        residual sum); it takes part if all four parts do."""
        if self.ffn is None:
            return None
        parts = {"norm_in": self.norm_in.fused_decode_fields(), "mixer": self.mixer.fused_decode_fields(),
                 "norm_post": self.norm_post.fused_decode_fields(), "ffn": self.ffn.fused_decode_fields()}
        if any(v is None for v in parts.values()):
            return None
        return {"kind": "prenorm_residual", **parts}


@register_block("parallel_shared_norm")
class ParallelSharedNormBlock(Block):
    """res += delta_in; y = norm(res); delta_out = mixer(y) + ffn(y): one norm, whose output the mixer and the feed-forward
    read side by side; the layer may have no feed-forward.  The sum comes back un-added in float32, so that the next norm
    fuses it into the float32 stream.

    Where the mixer and the feed-forward are given by their projections (`Projected`), the layer is two matrix products:
    every input projection of both stacked row-wise into one, every output projection stacked along its inner dimension into
    the other, whose float32 result is the sum of the sublayers.  The stacked matrices are padded with zeros to the row
    and inner sizes that the weight-streaming kernel for a few tokens takes.  Role of the norm: "input"."""

    ROWS_TO, INNER_TO = 16, 32

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        at = layer_spec.part_prefix
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=None)
        self.ffn = None
        if layer_spec.feed_forward is not None:
            self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)
        self.stacked = isinstance(self.mixer, Projected) and (self.ffn is None or isinstance(self.ffn, Projected))
        self.w_in = self.w_out = None

    def parts(self):
        return [p for p in (self.norm_in, self.mixer, self.ffn) if p is not None]

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, src) -> None:
        for part in self.parts():
            part.load(src)
        if not self.stacked:
            return
        subs = [p for p in (self.mixer, self.ffn) if p is not None]
        self.in_widths = [p.in_weight().shape[0] for p in subs]
        self.mid_widths = [p.out_weight().shape[1] for p in subs]
        w_in = torch.cat([p.in_weight() for p in subs], dim=0)
        w_out = torch.cat([p.out_weight() for p in subs], dim=1)
        pad_rows = -w_in.shape[0] % self.ROWS_TO
        pad_inner = -w_out.shape[1] % self.INNER_TO
        if pad_rows:
            w_in = torch.cat((w_in, w_in.new_zeros((pad_rows, w_in.shape[1]))), dim=0)
        if pad_inner:
            w_out = torch.cat((w_out, w_out.new_zeros((w_out.shape[0], pad_inner))), dim=1)
        self.w_in, self.w_out, self.pad_inner = w_in.contiguous(), w_out.contiguous(), pad_inner

    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        y = self.norm_in.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
        if not self.stacked:
            out = self.mixer.forward(y, ctx, cache, writes_cache).float()
            if self.ffn is not None:
                out = out + self.ffn.forward(y, ctx).float()
            return out, residual
        proj = ops.linear(y, self.w_in)
        act = torch.empty((y.shape[0], self.w_out.shape[1]), dtype=y.dtype, device=y.device)
        if self.pad_inner:
            act[:, act.shape[1] - self.pad_inner:].zero_()
        a, m = self.in_widths[0], self.mid_widths[0]
        self.mixer.middle(proj[:, :a], act[:, :m], ctx, cache, writes_cache)
        if self.ffn is not None:
            self.ffn.middle(proj[:, a:a + self.in_widths[1]], act[:, m:m + self.mid_widths[1]], ctx)
        return ops.linear(act, self.w_out, out_dtype=torch.float32), residual


@register_block("sandwich_residual")
class SandwichResidualBlock(Block):
    """A norm before and after every sublayer:

        res += m * norm_mixer_out(mixer(norm_in(res)));   res += m * norm_ffn_out(ffn(norm_ffn_in(res)))

    with one factor m for both sums (`block_params["residual_scale"]`, default 1); the layer may have no feed-forward.  The
    sums are float32.  Each sublayer's output norm, the sum and the following sublayer's input norm are one kernel
    (`ops.postnorm_residual`); the block hands the stream on with nothing left un-added.  Roles of the norms: "input",
    "mixer_out", "ffn_in", "ffn_out" (all `rmsnorm`)."""

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        at = layer_spec.part_prefix
        self.scale = float(layer_spec.block_params.get("residual_scale", 1.0))
        self.position = None
        if layer_spec.position is not None:
            self.position = env.shared(layer_spec.position, lambda: build_part(
                POSITION_ENCODINGS, "position encoding", layer_spec.position, layer_spec.prefix, env))
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
        self.norm_mixer_out = build_part(NORMS, "norm", layer_spec.norms["mixer_out"], at("mixer_out"), env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=self.position)
        self.ffn = self.norm_ffn_in = self.norm_ffn_out = None
        if layer_spec.feed_forward is not None:
            self.norm_ffn_in = build_part(NORMS, "norm", layer_spec.norms["ffn_in"], at("ffn_in"), env)
            self.norm_ffn_out = build_part(NORMS, "norm", layer_spec.norms["ffn_out"], at("ffn_out"), env)
            self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)
        for n in (self.norm_mixer_out, self.norm_ffn_in, self.norm_ffn_out):
            if n is not None and not hasattr(n, "eps"):
                raise ValueError("the sandwich block fuses RMS norms; another kind of norm is not taken here")
        self._w = {}

    def parts(self):
        return [p for p in (self.position, self.norm_in, self.mixer, self.norm_mixer_out, self.norm_ffn_in, self.ffn,
                            self.norm_ffn_out) if p is not None]

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, src) -> None:
        for part in self.parts():
            part.load(src)
        # the fused kernel reads float32 weights (exact: the checkpoint's values widened)
        self._w = {k: n.weight.float().contiguous() for k, n in (("mixer_out", self.norm_mixer_out), ("ffn_in", self.norm_ffn_in),
                                                                  ("ffn_out", self.norm_ffn_out)) if n is not None}

    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        y = self.norm_in.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
        a = self.mixer.forward(y, ctx, cache, writes_cache)
        if self.ffn is None:
            ops.postnorm_residual(a, self._w["mixer_out"], self.norm_mixer_out.eps, self.scale, residual, out_dtype=self.env.dtype)
            return None, residual
        y = ops.postnorm_residual(a, self._w["mixer_out"], self.norm_mixer_out.eps, self.scale, residual,
                                  next_weight=self._w["ffn_in"], next_eps=self.norm_ffn_in.eps, out_dtype=self.env.dtype)
        f = self.ffn.forward(y, ctx)
        ops.postnorm_residual(f, self._w["ffn_out"], self.norm_ffn_out.eps, self.scale, residual, out_dtype=self.env.dtype)
        return None, residual


class TokenSideTable(Part):
    """A table with one row per token of the vocabulary whose columns are shared out among the layers (layer i reads its own
    slice of a token's row).  One object holds it for all layers.  params: table (tensor name), vocab_size, columns."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.tensor_name, self.V, self.C = spec["table"], int(spec["vocab_size"]), int(spec["columns"])
        self.table = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor_name: TensorDecl((self.V, self.C))}

    def load(self, src) -> None:
        if self.table is None:
            self.table = src.fetch(self.tensor_name).contiguous()


@register_block("scaled_side_residual")
class ScaledSideResidualBlock(Block):
    """Pre-norm sublayers whose outputs are scaled element by element before they join the float32 stream, and a per-layer
    token input after them:

        res += m * s1 * mixer(norm_in(res));   res += m * s2 * ffn(norm_post(res))
        y = Wp (gelu_tanh(Wg res) * E[token][offset : offset + dim]);   res += m * rms(y) * wn

    with one factor m (`residual_scale`) and learned vectors s1, s2 of the width (`mixer_scale_name`, `ffn_scale_name`; full
    tensor names).  The layer may have no feed-forward.  `side` (or None) describes the token input: E is a table of
    `columns` columns per token shared by all layers (`table`), this layer reads `dim` of them from `offset`; Wg [dim, H],
    Wp [H, dim] and the plain RMS-norm weight wn are the layer's own (`gate`, `proj`, `norm`).  The sums, the products
    m * s and both norms are float32; a scaled sum and the norm that follows it are one kernel, and so are the side input's
    norm and its sum.  The block hands the stream on with nothing left un-added.  Roles of the norms: "input", "post_mixer"
    (`rmsnorm`).  block_params: residual_scale, mixer_scale_name, ffn_scale_name, hidden_size, norm_eps, side."""

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        at = layer_spec.part_prefix
        bp = layer_spec.block_params
        self.m, self.H, self.eps = float(bp.get("residual_scale", 1.0)), int(bp["hidden_size"]), float(bp["norm_eps"])
        self.position = None
        if layer_spec.position is not None:
            self.position = env.shared(layer_spec.position, lambda: build_part(
                POSITION_ENCODINGS, "position encoding", layer_spec.position, layer_spec.prefix, env))
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=self.position)
        self.norm_post = self.ffn = None
        if layer_spec.feed_forward is not None:
            self.norm_post = build_part(NORMS, "norm", layer_spec.norms["post_mixer"], at("post_mixer"), env)
            self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)
            if not hasattr(self.norm_post, "eps"):
                raise ValueError("this block fuses an RMS norm behind the mixer's sum; another kind of norm is not taken here")
        self.n_s1, self.n_s2 = bp["mixer_scale_name"], bp.get("ffn_scale_name")
        self.side = dict(bp["side"]) if bp.get("side") else None
        self.side_table = None
        if self.side is not None:
            tspec = PartSpec("token_side_table", {k: self.side[k] for k in ("table", "vocab_size", "columns")})
            self.side_table = env.shared(tspec, lambda: TokenSideTable(tspec, "", env))
        self.s1 = self.s2 = self.w_post = self.side_gate = self.side_proj = self.side_norm = None

    def parts(self):
        return [p for p in (self.position, self.norm_in, self.mixer, self.norm_post, self.ffn, self.side_table) if p is not None]

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in self.parts():
            out.update(part.tensors())
        out[self.n_s1] = TensorDecl((self.H,), kind="vector", init="norm")
        if self.ffn is not None:
            out[self.n_s2] = TensorDecl((self.H,), kind="vector", init="norm")
        if self.side is not None:
            d = int(self.side["dim"])
            out[self.side["gate"]] = TensorDecl((d, self.H))
            out[self.side["proj"]] = TensorDecl((self.H, d))
            out[self.side["norm"]] = TensorDecl((self.H,), kind="vector", init="norm")
        return out

    def load(self, src) -> None:
        for part in self.parts():
            part.load(src)
        # m * s in float32: the factor of what a sublayer adds to the stream
        self.s1 = (src.fetch(self.n_s1).float() * self.m).contiguous()
        if self.ffn is not None:
            self.s2 = (src.fetch(self.n_s2).float() * self.m).contiguous()
            self.w_post = self.norm_post.weight.float().contiguous()
        if self.side is not None:
            self.side_gate, self.side_proj = src.fetch(self.side["gate"]).contiguous(), src.fetch(self.side["proj"]).contiguous()
            self.side_norm = src.fetch(self.side["norm"]).float().contiguous()

    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        y = self.norm_in.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
        a = self.mixer.forward(y, ctx, cache, writes_cache)
        dt = self.env.dtype
        if self.ffn is not None:
            y = ops.scaled_add_norm(a, self.s1, residual, weight=self.w_post, eps=self.norm_post.eps, out_dtype=dt)
            f = self.ffn.forward(y, ctx)
            x = ops.scaled_add_norm(f, self.s2, residual, out_dtype=dt if self.side is not None else None)
        else:
            x = ops.scaled_add_norm(a, self.s1, residual, out_dtype=dt if self.side is not None else None)
        if self.side is not None:
            gate = ops.linear(x, self.side_gate)
            g = ops.side_gate_mul(gate, self.side_table.table, ctx.input_ids, int(self.side["offset"]))
            yv = ops.linear(g, self.side_proj, out_dtype=torch.float32)
            ops.postnorm_residual(yv, self.side_norm, self.eps, self.m, residual, out_dtype=dt)
        return None, residual
