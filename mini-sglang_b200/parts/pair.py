from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorDecl
from .base import MIXERS, Mixer, Projected, build_part, register_mixer


@register_mixer("weighted_pair")
class WeightedPair(Mixer, Projected):
    """Two mixers side by side on the same input: first_scale * first(x) + second_scale * second(x).

    Both are `Projected` parts, so their input projections are one product and their output projections another: the
    scales go onto what enters the output product.  What each keeps between steps is kept side by side too: the pair
    declares the needs of the first followed by those of the second.

    params: hidden_size, first, second (PartSpecs of registered mixers), first_scale, second_scale, first_name, second_name
            (what the checkpoint calls them below the pair's prefix).
    """

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        self.subs = []
        for which in ("first", "second"):
            part = build_part(MIXERS, "mixer", spec[which], self.name(spec.get(which + "_name", which)), env, position=position)
            if not isinstance(part, Projected):
                raise ValueError(f"a weighted pair takes mixers that are given by their projections; {spec[which].kind!r} is not")
            self.subs.append(part)
        self.scales = [float(spec.get("first_scale", 1.0)), float(spec.get("second_scale", 1.0))]
        self.graph_safe = all(p.graph_safe for p in self.subs)
        self.w_in = self.w_out = None
        self._needs = []
        for p in self.subs:
            need = p.cache_need()
            self._needs.append(() if need is None else (need if isinstance(need, tuple) else (need,)))

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for p in self.subs:
            out.update(p.tensors())
        return out

    def load(self, src) -> None:
        for p in self.subs:
            p.load(src)
        self.w_in = torch.cat([p.in_weight() for p in self.subs], dim=0).contiguous()
        self.w_out = torch.cat([p.out_weight() for p in self.subs], dim=1).contiguous()
        self.in_widths = [p.in_weight().shape[0] for p in self.subs]
        self.mid_widths = [p.out_weight().shape[1] for p in self.subs]

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        needs = tuple(n for ns in self._needs for n in ns)
        return needs if needs else None

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        caches = tuple(cache) if isinstance(cache, tuple) else ((cache,) if cache is not None else ())
        a = m = c = 0
        for p, scale, ns, wi, wm in zip(self.subs, self.scales, self._needs, self.in_widths, self.mid_widths):
            mine = caches[c:c + len(ns)]
            sub_cache = None if not ns else (mine if isinstance(p.cache_need(), tuple) else mine[0])
            p.middle(proj[:, a:a + wi], act[:, m:m + wm], ctx, sub_cache, writes_cache, out_scale * scale)
            a, m, c = a + wi, m + wm, c + len(ns)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)


@register_mixer("normed_pair")
class NormedPair(Mixer):
    """Two mixers side by side on the same input whose outputs are each RMS-normed over the model width (plain weights of their
    own) before they are joined: out_scale * weight * (norm_a(first(x)) + norm_b(second(x))), in float32.

    Both are `Projected` parts: their input projections are one product; each has its own output product (the norms sit behind
    them), written in float32, and one kernel norms and joins the two.  What each keeps between steps is kept side by side: the
    pair declares the needs of the first followed by those of the second.

    params: hidden_size, first, second (PartSpecs of registered mixers), first_name, second_name (what the checkpoint calls them
            below the pair's prefix), first_norm_name, second_norm_name (the norms' weights, below the pair's prefix), norm_eps,
            weight (of each half in the sum; default 1/2), out_scale.
    """

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        self.E = int(spec["hidden_size"])
        self.subs = []
        for which in ("first", "second"):
            part = build_part(MIXERS, "mixer", spec[which], self.name(spec.get(which + "_name", which)), env, position=position)
            if not isinstance(part, Projected):
                raise ValueError(f"a normed pair takes mixers that are given by their projections; {spec[which].kind!r} is not")
            self.subs.append(part)
        self.norm_names = [self.name(spec.get("first_norm_name", "first.out")), self.name(spec.get("second_norm_name", "second.out"))]
        self.eps = float(spec["norm_eps"])
        self.join_scale = float(spec.get("weight", 0.5)) * float(spec.get("out_scale", 1.0))
        self.graph_safe = all(p.graph_safe for p in self.subs)
        self.w_in = self.norm_w = None
        self._needs = []
        for p in self.subs:
            need = p.cache_need()
            self._needs.append(() if need is None else (need if isinstance(need, tuple) else (need,)))

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for p in self.subs:
            out.update(p.tensors())
        for n in self.norm_names:
            out[n] = TensorDecl((self.E,), kind="vector", init="norm")
        return out

    def load(self, src) -> None:
        for p in self.subs:
            p.load(src)
        self.w_in = torch.cat([p.in_weight() for p in self.subs], dim=0).contiguous()
        self.in_widths = [p.in_weight().shape[0] for p in self.subs]
        self.norm_w = [src.fetch(n).float().contiguous() for n in self.norm_names]

    def cache_need(self):
        needs = tuple(n for ns in self._needs for n in ns)
        return needs if needs else None

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        from .. import ops
        caches = tuple(cache) if isinstance(cache, tuple) else ((cache,) if cache is not None else ())
        proj = ops.linear(x, self.w_in)
        outs, a, c = [], 0, 0
        for p, ns, wi in zip(self.subs, self._needs, self.in_widths):
            mine = caches[c:c + len(ns)]
            sub_cache = None if not ns else (mine if isinstance(p.cache_need(), tuple) else mine[0])
            w_out = p.out_weight()
            act = torch.empty((x.shape[0], w_out.shape[1]), dtype=x.dtype, device=x.device)
            p.middle(proj[:, a:a + wi], act, ctx, sub_cache, writes_cache)
            outs.append(ops.linear(act, w_out, out_dtype=torch.float32))
            a, c = a + wi, c + len(ns)
        return ops.pair_norm(outs[0], outs[1], self.norm_w[0], self.norm_w[1], self.eps, self.join_scale)
