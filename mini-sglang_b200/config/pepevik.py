"""Pepevik: typed configuration and model description.

A decoder whose layers are listed one by one in config.json (`layers`): every entry names the kind of its mixer (`type`), the
mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  An entry with `weights_of: j` is another
run of layer j's weights with a cache and state of its own.  The embedding is scaled by a constant and gets a learned vector per
place.  A layer is pre-norm with Dynamic-Tanh norms, and what a sublayer adds to the float32 stream is multiplied by one
constant of the model (`residual_mult`).  Mixers:

  parallel   a sigmoid attention (no softmax; per-head q/k norm, a query factor that grows with the place, a logarithmic
             distance penalty and a bias per head) beside a minGRU recurrence, each output RMS-normed over the width, half
             their sum
  mamba2     a state-space mixer with a scalar decay per head and token, a short convolution on x, B and C, and a gate before
             a group-wise RMS norm

Feed-forwards: `dense` (down(relu(up x)^2)) and `moe` (sigmoid-scored experts chosen within the best groups, with a correction
that only steers the choice).  The head is a matrix of its own.  Everything that differs between models of the design is read
here; nothing else in the engine knows the design's name.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no {key!r}")
    return d[key]


@dataclasses.dataclass
class PepevikLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]
    weights_of: Optional[int]


@dataclasses.dataclass
class PepevikConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    max_positions: int
    layers: List[PepevikLayer]
    eos_token_ids: List[int] = dataclasses.field(default_factory=list)
    raw: Dict[str, Any] = dataclasses.field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PepevikConfig":
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layer {i}"
            wo = entry.get("weights_of")
            layers.append(PepevikLayer(type=str(_need(entry, "type", where)), mixer=dict(_need(entry, "mixer", where)),
                                       mlp=dict(entry["mlp"]) if entry.get("mlp") is not None else None,
                                       weights_of=int(wo) if wo is not None else None))
        eos = raw.get("eos_token_id", [])
        eos = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        emb = raw.get("embedding") or {}
        cfg = cls(width=int(_need(raw, "width", "the model")), vocab=int(_need(raw, "vocab", "the model")),
                  norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                  residual_mult=float(raw.get("residual_mult", 1.0)), embedding_scale=float(emb.get("scale", 1.0)),
                  max_positions=int(_need(raw, "max_positions", "the model")), layers=layers, eos_token_ids=eos, raw=dict(raw))
        cfg.check()
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it is another run of an earlier layer's weights)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: the weights_of entries from layer {i} on form a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or self.max_positions <= 0 or not self.layers:
            raise ConfigError("width, vocab, max_positions and the number of layers must be positive")
        for i, l in enumerate(self.layers):
            if l.weights_of is not None and not 0 <= l.weights_of < len(self.layers):
                raise ConfigError(f"config.json: layer {i} names weights_of {l.weights_of}, the model has {len(self.layers)} layers")
            self.owner(i)
            if l.type not in _MIXERS:
                raise ConfigError(f"config.json: layer {i} has type {l.type!r}; known: " + ", ".join(sorted(_MIXERS)))
            if l.mlp is not None and l.mlp.get("kind") not in _FEED_FORWARDS:
                raise ConfigError(f"config.json: layer {i} has a feed-forward of kind {l.mlp.get('kind')!r}; known: "
                                  + ", ".join(sorted(_FEED_FORWARDS)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def _parallel(cfg: PepevikConfig, m: Dict[str, Any], where: str) -> PartSpec:
    """Half the sum of a sigmoid attention ("left") and a minGRU ("right"), each RMS-normed over the width."""
    lf, rt = _need(m, "left", where), _need(m, "right", where)
    heads = int(_need(lf, "heads", where + ".left"))
    dim = int(_need(lf, "dim", where + ".left"))
    temp = lf.get("q_temp") or {}
    left = PartSpec("sigmoid_attention", {
        "hidden_size": cfg.width, "num_heads": heads, "num_kv_heads": int(lf.get("kv_heads") or heads), "key_dim": dim,
        "value_dim": int(lf.get("vdim") or dim), "scale": float(_need(lf, "scale", where + ".left")), "norm_eps": cfg.norm_eps,
        "temp_coef": float(temp.get("coef", 0.0)), "temp_every": int(temp.get("every", 1)), "max_positions": cfg.max_positions,
        "names": {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1", "r2": "r2", "pb": "pb", "out": "o"}})
    right = PartSpec("mingru", {"hidden_size": cfg.width, "width": int(_need(rt, "width", where + ".right")),
                                "names": {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}})
    return PartSpec("normed_pair", {"hidden_size": cfg.width, "first": left, "second": right, "first_name": "left",
                                    "second_name": "right", "first_norm_name": "left.out", "second_norm_name": "right.out",
                                    "norm_eps": cfg.norm_eps, "weight": 0.5, "out_scale": cfg.residual_mult})


def _mamba2(cfg: PepevikConfig, m: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("state_space", {
        "hidden_size": cfg.width, "num_heads": int(_need(m, "heads", where)), "head_dim": int(_need(m, "vdim", where)),
        "state_size": int(_need(m, "state", where)), "groups": int(m.get("groups") or 1), "conv_taps": int(m.get("conv") or 1),
        "norm_groups": int(m.get("norm_groups") or 1), "norm_eps": cfg.norm_eps, "out_scale": cfg.residual_mult,
        "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
                  "norm": "norm", "out": "o"}})


def _dense(cfg: PepevikConfig, f: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("plain_mlp", {"hidden_size": cfg.width, "intermediate_size": int(_need(f, "ff", where)), "activation": "relu2",
                                  "out_scale": cfg.residual_mult, "names": {"up": "up", "down": "down"}})


def _moe(cfg: PepevikConfig, f: Dict[str, Any], where: str) -> PartSpec:
    r = _need(f, "router", where)
    n = int(_need(r, "experts", where + ".router"))
    g = r.get("groups") or {}
    count = int(g.get("count") or 1)
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "intermediate_size": int(_need(_need(f, "expert", where), "ff", where + ".expert")),
        "num_experts": n, "top": int(_need(r, "top", where + ".router")), "groups": count, "keep_groups": int(g.get("keep") or count),
        "out_scale": cfg.residual_mult,
        "names": {"router": "router", "correction": "correction", "expert": "e{e}", "gate": "gate", "up": "up", "down": "down"}})


_MIXERS = {"parallel": _parallel, "mamba2": _mamba2}
_FEED_FORWARDS = {"dense": _dense, "moe": _moe}
PEPEVIK_LAYER_NAMES = {"mixer": "mix", "feed_forward": "mlp"}


def build_pepevik_spec(cfg: PepevikConfig) -> ModelSpec:
    """scaled embedding + places -> runs of (norm, mixer, scaled sum; norm, feed-forward, scaled sum) -> norm -> head.  Layers that
    own tensors become the model's layers; every entry of config.json's list is one run, in order, with a cache id of its own.
    The mixers and feed-forwards multiply what they return by `residual_mult` themselves (in float32), so the block adds it as
    it is."""
    owners = sorted({cfg.owner(i) for i in range(len(cfg.layers))})
    index = {o: k for k, o in enumerate(owners)}

    def norm(name: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"size": cfg.width, "name": name})

    layers = []
    for o in owners:
        l = cfg.layers[o]
        norms = {"input": norm(f"l{o}.norm1")}
        ffn = None
        if l.mlp is not None:
            ffn = _FEED_FORWARDS[l.mlp["kind"]](cfg, l.mlp, f"layer {o}.mlp")
            norms["post_mixer"] = norm(f"l{o}.norm2")
        layers.append(LayerSpec(prefix=f"l{o}", mixer=_MIXERS[l.type](cfg, l.mixer, f"layer {o}.mixer"), feed_forward=ffn, norms=norms,
                                position=None, block="prenorm_residual", names=PEPEVIK_LAYER_NAMES))
    return ModelSpec(
        architecture="Pepevik", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_position_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed",
                                                        "position_name": "pos", "max_positions": cfg.max_positions,
                                                        "scale": cfg.embedding_scale}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, "name": "head"}),
        layers=layers, schedule=[Run(layer=index[cfg.owner(i)], cache=i) for i in range(len(cfg.layers))],
        max_context_len=cfg.max_positions, eos_token_ids=list(cfg.eos_token_ids), checkpoint_dtype="bfloat16")


register_architecture("Pepevik", PepevikConfig, build_pepevik_spec)
