"""Lifulorn: typed configuration and model description.

A decoder whose layers are listed one by one in config.json (`layers`): every entry names the kind of its mixer (`type`), the
mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  A layer is pre-norm with RMS norms; what a
sublayer adds to the float32 stream is multiplied by one constant of the model (`residual_mult`) and, element by element, by a
learned vector of the layer (`ls1` for the mixer, `ls2` for the feed-forward).  After the feed-forward every layer adds an
RMS-normed projection of its own slice of a per-token table, gated by the stream (`token_side`).  Mixers:

  attention    grouped-query softmax attention with biases on q, k, v, a partial rotation in halves whose long wavelengths
               are slowed in steps (factor, low, high, original), a sliding window, one learned term per head in every
               softmax's denominator, and values blended with those of the first such layer
  attention_2  the same with frequencies slowed along a ramp (factor, original, fast, slow; cos and sin grow with the
               factor) and scores capped by a tanh
  delta        the gated delta rule: short convolutions on q, k, v, unit-length q and k, a decay and a write strength per
               head and token, a float32 state per head that is corrected towards the value at the current key

Feed-forward: `moe`, small clamped gated experts chosen by the largest router logits and weighted by the softmax over the
chosen logits, beside a shared expert times a sigmoid gate.  Everything that differs between models of the design is read
here; nothing else in the engine knows the design's name.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run

NO_POSITION_LIMIT = 1 << 20      # the design has no table of places; the context is bounded by the cache alone


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no {key!r}")
    return d[key]


@dataclasses.dataclass
class LifulornLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass
class LifulornConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    side_dim: int                     # 0: no per-layer token input
    layers: List[LifulornLayer]
    max_positions: int = NO_POSITION_LIMIT
    eos_token_ids: List[int] = dataclasses.field(default_factory=list)
    raw: Dict[str, Any] = dataclasses.field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LifulornConfig":
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layer {i}"
            layers.append(LifulornLayer(type=str(_need(entry, "type", where)), mixer=dict(_need(entry, "mixer", where)),
                                        mlp=dict(entry["mlp"]) if entry.get("mlp") is not None else None))
        eos = raw.get("eos_token_id", [])
        eos = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        side = raw.get("token_side") or {}
        cfg = cls(width=int(_need(raw, "width", "the model")), vocab=int(_need(raw, "vocab", "the model")),
                  norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                  residual_mult=float(raw.get("residual_mult", 1.0)), side_dim=int(side.get("dim") or 0), layers=layers,
                  max_positions=int(raw.get("max_positions") or NO_POSITION_LIMIT), eos_token_ids=eos, raw=dict(raw))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or not self.layers:
            raise ConfigError("width, vocab and the number of layers must be positive")
        if self.side_dim < 0:
            raise ConfigError("token_side.dim must not be negative")
        for i, l in enumerate(self.layers):
            if l.type not in _MIXERS:
                raise ConfigError(f"config.json: layer {i} has type {l.type!r}; known: " + ", ".join(sorted(_MIXERS)))
            if l.mlp is not None and l.mlp.get("kind", "moe") not in _FEED_FORWARDS:
                raise ConfigError(f"config.json: layer {i} has a feed-forward of kind {l.mlp.get('kind')!r}; known: "
                                  + ", ".join(sorted(_FEED_FORWARDS)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def _rotation(m: Dict[str, Any], kind: str, where: str) -> Optional[PartSpec]:
    rot = m.get("rot")
    if not rot or not int(rot.get("dims") or 0):
        return None
    dims = int(rot["dims"])
    if dims % 2 or dims > int(m["dim"]):
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most the key size")
    sc = rot.get("scaling")
    return PartSpec("rope_stepped" if kind == "attention" else "rope_yarn",
                    {"rotary_dim": dims, "theta": float(_need(rot, "base", where + ".rot")), "scaling": dict(sc) if sc else None,
                     "max_positions": 0})


def _attention(kind: str):
    def build(cfg: LifulornConfig, m: Dict[str, Any], where: str, v_role: Optional[str]) -> PartSpec:
        heads = int(_need(m, "heads", where))
        dim = int(_need(m, "dim", where))
        mask = m.get("mask") or {}
        return PartSpec("sink_attention", {
            "hidden_size": cfg.width, "num_heads": heads, "num_kv_heads": int(m.get("kv_heads") or heads), "key_dim": dim,
            "value_dim": int(m.get("vdim") or dim), "scale": float(_need(m, "scale", where)),
            "window": int(mask["size"]) if mask.get("size") else None,
            "softcap": float(m["softcap"]) if kind == "attention_2" and m.get("softcap") else None,
            "value_mix": v_role, "value_mix_key": "first_values", "bias": True,
            "names": {"q": "q", "k": "k", "v": "v", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink", "mix": "vmix",
                      "out": "o"}})
    return build


def _delta(cfg: LifulornConfig, m: Dict[str, Any], where: str, v_role: Optional[str]) -> PartSpec:
    heads = int(_need(m, "heads", where))
    return PartSpec("gated_delta", {
        "hidden_size": cfg.width, "num_heads": heads, "num_kv_heads": int(m.get("kv_heads") or heads),
        "key_dim": int(_need(m, "dim", where)), "value_dim": int(_need(m, "vdim", where)), "conv_taps": int(m.get("conv") or 1),
        "norm_eps": cfg.norm_eps,
        "names": {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "a": "a",
                  "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "out": "o"}})


def _moe(cfg: LifulornConfig, f: Dict[str, Any], where: str) -> PartSpec:
    r = _need(f, "router", where)
    ex = _need(f, "expert", where)
    sh = f.get("shared")
    return PartSpec("softmax_experts", {
        "hidden_size": cfg.width, "intermediate_size": int(_need(ex, "ff", where + ".expert")),
        "limit": float(_need(ex, "limit", where + ".expert")), "num_experts": int(_need(r, "experts", where + ".router")),
        "top": int(_need(r, "top", where + ".router")),
        "shared_size": int(_need(sh, "ff", where + ".shared")) if sh else 0,
        "shared_limit": float(_need(sh, "limit", where + ".shared")) if sh else 0.0,
        "names": {"router": "router", "expert": "e{e}", "gate": "gate", "up": "up", "down": "down", "shared": "shared",
                  "shared_gate": "shared.sg"}})


_MIXERS = {"attention": _attention("attention"), "attention_2": _attention("attention_2"), "delta": _delta}
_FEED_FORWARDS = {"moe": _moe}
LIFULORN_LAYER_NAMES = {"mixer": "mix", "feed_forward": "mlp"}


def build_lifulorn_spec(cfg: LifulornConfig) -> ModelSpec:
    """embedding -> layers of (norm, mixer, scaled sum; norm, feed-forward, scaled sum; per-layer token input) -> norm -> head.
    One `LayerSpec` and one `Run` per listed layer.  The first layer whose mixer asks for blended values keeps its own and
    hands them on ("first"); the later ones blend theirs with those ("blend")."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name})

    layers = []
    seen_first = False
    for i, l in enumerate(cfg.layers):
        v_role = None
        if l.type in ("attention", "attention_2") and l.mixer.get("v_mix"):
            v_role = "blend" if seen_first else "first"
            seen_first = True
        norms = {"input": norm(f"l{i}.norm1")}
        ffn = None
        if l.mlp is not None:
            ffn = _FEED_FORWARDS[l.mlp.get("kind", "moe")](cfg, l.mlp, f"layer {i}.mlp")
            norms["post_mixer"] = norm(f"l{i}.norm2")
        position = _rotation(l.mixer, l.type, f"layer {i}.mixer") if l.type in ("attention", "attention_2") else None
        block_params = {"residual_scale": cfg.residual_mult, "mixer_scale_name": f"l{i}.ls1", "ffn_scale_name": f"l{i}.ls2",
                        "hidden_size": cfg.width, "norm_eps": cfg.norm_eps}
        if cfg.side_dim:
            block_params["side"] = {"table": "side.embed", "vocab_size": cfg.vocab, "columns": len(cfg.layers) * cfg.side_dim,
                                    "offset": i * cfg.side_dim, "dim": cfg.side_dim, "gate": f"l{i}.side.gate",
                                    "proj": f"l{i}.side.proj", "norm": f"l{i}.side.norm"}
        layers.append(LayerSpec(prefix=f"l{i}", mixer=_MIXERS[l.type](cfg, l.mixer, f"layer {i}.mixer", v_role), feed_forward=ffn,
                                norms=norms, position=position, block="scaled_side_residual", names=LIFULORN_LAYER_NAMES,
                                block_params=block_params))
    return ModelSpec(
        architecture="Lifulorn", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, "name": "head"}),
        layers=layers, schedule=[Run(layer=i, cache=i) for i in range(len(cfg.layers))],
        max_context_len=cfg.max_positions, eos_token_ids=list(cfg.eos_token_ids), checkpoint_dtype="bfloat16")


register_architecture("Lifulorn", LifulornConfig, build_lifulorn_spec)
