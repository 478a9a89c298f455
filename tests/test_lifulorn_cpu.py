"""Lifulorn without a GPU: the configuration reader and the model description against the tiny configurations, the engine's
frequency tables against the plain ones, the plain implementation's mechanisms against closed forms and hand-made cases, and
what the model-level bound of the GPU tests can tell apart."""

import copy
import math

import pytest
import torch

import plain_lifulorn as pl
from tiny_models import random_tokens
from tiny_lifulorn import CONFIGS_L, RAMPED, STEPPED, make_weights, random_config, tensor_shapes

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(CONFIGS_L) + [f"random{s}" for s in range(8)])
def test_description_declares_the_checkpoints_tensors(name):
    from mini_sglang_b200.config import architecture_of
    from mini_sglang_b200.parts.model import expected_tensors
    raw = CONFIGS_L[name] if name in CONFIGS_L else random_config(int(name[6:]))
    arch = architecture_of(raw)
    assert arch.name == "Lifulorn"
    spec = arch.build_spec(arch.config_cls.from_dict(raw))
    spec.validate()
    want = tensor_shapes(raw)
    got = {k: d for k, d in expected_tensors(spec).items() if not d.optional or k in want}
    assert set(got) == set(want)
    for k, decl in got.items():
        assert tuple(decl.shape) == tuple(want[k]), (k, decl.shape, want[k])
    assert [r.cache for r in spec.schedule] == list(range(len(raw["layers"])))
    roles = [l.mixer.get("value_mix") for l in spec.layers if l.mixer.kind == "sink_attention"]
    asked = [bool(e["mixer"].get("v_mix")) for e in raw["layers"] if e["type"] != "delta"]
    assert [r is not None for r in roles] == asked
    assert [r for r in roles if r] == (["first"] + ["blend"] * (sum(asked) - 1) if any(asked) else [])
    for l, entry in zip(spec.layers, raw["layers"]):
        assert (l.feed_forward is None) == (entry["mlp"] is None)
        assert l.mixer.kind == {"attention": "sink_attention", "attention_2": "sink_attention", "delta": "gated_delta"}[entry["type"]]
        if entry["type"] != "delta":
            assert l.mixer["window"] == (entry["mixer"].get("mask") or {}).get("size")
            assert (l.mixer["softcap"] is not None) == (entry["type"] == "attention_2" and entry["mixer"].get("softcap") is not None)


def test_configuration_refusals():
    from mini_sglang_b200.config import ConfigError, architecture_of
    raw = CONFIGS_L["LA"]
    arch = architecture_of(raw)
    for change in (lambda c: c["layers"][0].__setitem__("type", "something"),
                   lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"),
                   lambda c: c["layers"][0]["mixer"].pop("heads"),
                   lambda c: c["layers"][0]["mixer"].pop("scale"),
                   lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 15),
                   lambda c: c["layers"][1]["mixer"].pop("vdim"),
                   lambda c: c["layers"][0]["mlp"]["router"].pop("top"),
                   lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"),
                   lambda c: c.pop("norm"),
                   lambda c: c.pop("width")):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError):
            arch.build_spec(arch.config_cls.from_dict(bad))


@pytest.mark.parametrize("dims,base,sc", [(16, 10000.0, STEPPED), (32, 50000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}),
                                          (8, 30.0, None), (64, 500000.0, {"factor": 2.0, "low": 2.0, "high": 2.0, "original": 100})])
def test_stepped_frequencies_of_the_engine_equal_the_plain_ones(dims, base, sc):
    from mini_sglang_b200.parts.rope import stepped_frequencies
    got = stepped_frequencies(dims, base, sc)
    want = pl.stepped_frequencies(dims, base, sc)[0] if sc else pl.plain_frequencies(dims, base)
    torch.testing.assert_close(got, want, rtol=1e-14, atol=0)
    if sc is STEPPED:        # all three branches are taken
        plain = pl.plain_frequencies(dims, base)
        ratio = (got / plain).tolist()
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-15 and any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)


@pytest.mark.parametrize("dims,base,sc", [(16, 500.0, RAMPED), (6, 20.0, RAMPED), (32, 250000.0, {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0})])
def test_ramped_frequencies_of_the_engine_equal_the_plain_ones(dims, base, sc):
    from mini_sglang_b200.parts.rope import yarn_frequencies
    got, mag = yarn_frequencies(dims, base, sc)
    want, wmag = pl.ramped_frequencies(dims, base, sc)
    torch.testing.assert_close(got, want, rtol=1e-14, atol=0)
    assert mag == wmag == 0.1 * math.log(sc["factor"]) + 1.0


def test_rotation_turns_pairs_in_halves_and_leaves_the_rest():
    x = torch.arange(1, 13, dtype=F64).view(1, 1, 12).repeat(3, 1, 1)
    f = torch.tensor([0.5, 0.25], dtype=F64)
    y = pl.rotate(x, torch.tensor([0, 2, 7]), f, 1.0, 4)
    assert torch.equal(y[0], x[0])                                   # position 0: nothing turns
    assert torch.equal(y[:, :, 4:], x[:, :, 4:])                     # the rest of the head passes
    a = 7 * 0.25
    assert abs(float(y[2, 0, 1]) - (2 * math.cos(a) - 4 * math.sin(a))) < 1e-12      # element 1 pairs with element 3
    assert abs(float(y[2, 0, 3]) - (4 * math.cos(a) + 2 * math.sin(a))) < 1e-12
    torch.testing.assert_close(pl.rotate(x, torch.tensor([0, 2, 7]), f, 1.5, 4)[1, 0, :4], 1.5 * y[1, 0, :4])


def _attention_case(window=None, softcap=None, sink=0.0, T=9):
    torch.manual_seed(0)
    c = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.5}
    if window:
        c["mask"] = {"size": window}
    if softcap:
        c["softcap"] = softcap
    w = {"m.q": torch.randn(8, 5, dtype=F64), "m.k": torch.randn(4, 5, dtype=F64), "m.v": torch.randn(3, 5, dtype=F64),
         "m.q.b": torch.randn(8, dtype=F64), "m.k.b": torch.randn(4, dtype=F64), "m.v.b": torch.randn(3, dtype=F64),
         "m.sink": torch.tensor([sink, sink - 1.0], dtype=F64), "m.o": torch.eye(6, dtype=F64)}
    return c, w, torch.randn(T, 5, dtype=F64)


def test_sink_attention_closed_forms():
    c, w, u = _attention_case(sink=-80.0)
    full, _ = pl.sink_attention(u, w, "m", c, "attention", None)
    # a sink far below every score changes nothing; the first token then returns its own value
    v = u @ w["m.v"].T + w["m.v.b"]
    torch.testing.assert_close(full[0, :3], v[0])
    # a sink far above every score takes all the weight
    c2, w2, _ = _attention_case(sink=80.0)
    zero, _ = pl.sink_attention(u, w2, "m", c2, "attention", None)
    assert zero.abs().max() < 1e-20
    # a window of one token: every token returns its own value, weighted against the sink
    c3, w3, _ = _attention_case(window=1, sink=0.3)
    one, _ = pl.sink_attention(u, w3, "m", c3, "attention", None)
    q = (u @ w3["m.q"].T + w3["m.q.b"]).view(-1, 2, 4)
    k = u @ w3["m.k"].T + w3["m.k.b"]
    s = (q[:, 0] * k).sum(-1) * 0.5
    torch.testing.assert_close(one[:, :3], v * (torch.exp(s) / (torch.exp(s) + math.exp(0.3)))[:, None])
    # the soft cap bounds the scores: with a tiny cap all seen keys weigh alike
    c4, w4, _ = _attention_case(softcap=1e-9, sink=-80.0)
    flat, _ = pl.sink_attention(u, w4, "m", c4, "attention_2", None)
    torch.testing.assert_close(flat[:, :3], torch.cumsum(v, 0) / torch.arange(1, 10, dtype=F64)[:, None])
    same, _ = pl.sink_attention(u, w4, "m", c4, "attention", None)          # the first kind has no cap
    assert (same - flat).abs().max() > 1e-3


def test_blended_values():
    c, w, u = _attention_case(sink=-80.0)
    c["v_mix"] = True
    w["m.vmix"] = torch.tensor(0.25, dtype=F64)
    _, own = pl.sink_attention(u, w, "m", c, "attention", None)
    first = torch.randn_like(own)
    out, own2 = pl.sink_attention(u[:1], w, "m", c, "attention", first[:1])
    torch.testing.assert_close(out[0, :3], 0.75 * own[0, 0] + 0.25 * first[0, 0])
    torch.testing.assert_close(own2, own[:1])


def test_short_convolution_and_delta_rule_closed_forms():
    x = torch.arange(1, 11, dtype=F64).view(5, 2)
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]], dtype=F64)
    y = pl.short_convolution(x, taps)
    assert y[:, 1].tolist() == (2 * x[:, 1]).tolist()
    assert y[:, 0].tolist() == [100.0, 310.0, 531.0, 753.0, 975.0]
    # one head, no convolution; beta = 1 and no decay: writing a key twice leaves the state as it is, and reading with the
    # same key returns the value
    torch.manual_seed(1)
    E, d, dv = 6, 4, 3
    w = {"m.q": torch.randn(d, E, dtype=F64), "m.k": torch.randn(d, E, dtype=F64), "m.v": torch.randn(dv, E, dtype=F64),
         "m.q.conv": torch.ones(d, 1, dtype=F64), "m.k.conv": torch.ones(d, 1, dtype=F64), "m.v.conv": torch.ones(dv, 1, dtype=F64),
         "m.b": torch.zeros(1, E, dtype=F64), "m.a": torch.zeros(1, E, dtype=F64), "m.A_log": torch.tensor([0.0], dtype=F64),
         "m.dt_bias": torch.tensor([-200.0], dtype=F64), "m.g": torch.randn(dv, E, dtype=F64), "m.norm": torch.ones(dv, dtype=F64),
         "m.o": torch.eye(dv, dtype=F64)}
    w["m.q"] = w["m.k"].clone()
    c = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "conv": 1}
    u = torch.randn(1, E, dtype=F64).repeat(3, 1)
    w["m.b"] = torch.zeros(1, E, dtype=F64)
    out = pl.delta_rule(u, w, "m", c, 0.0)
    # beta = sigmoid(0) = 1/2: after t writes of the same (k, v) the state holds (1 - 2^-t) v along k; the output is normed
    # over vdim, so every token returns the same direction
    torch.testing.assert_close(out[0], out[1])
    torch.testing.assert_close(out[0], out[2])
    v = pl.silu(u[0] @ w["m.v"].T)
    want = v / torch.sqrt((v * v).mean()) * pl.silu(u[0] @ w["m.g"].T)
    torch.testing.assert_close(out[0], want)


def test_experts_closed_forms():
    torch.manual_seed(2)
    E = 5
    w = {"f.router": torch.tensor([[9.0, 0, 0, 0, 0], [0, 9.0, 0, 0, 0], [0, 0, 9.0, 0, 0]], dtype=F64)}
    for e in range(3):
        w[f"f.e{e}.gate"], w[f"f.e{e}.up"], w[f"f.e{e}.down"] = (torch.randn(4, E, dtype=F64), torch.randn(4, E, dtype=F64),
                                                                  torch.randn(E, 4, dtype=F64))
    c = {"expert": {"ff": 4, "limit": 0.7}, "router": {"experts": 3, "top": 2}}
    u = torch.tensor([[1.0, 0.5, -1.0, 0.3, 0.2]], dtype=F64)
    out = pl.expert_mixture(u, w, "f", c)
    a, b = math.exp(9.0), math.exp(4.5)
    want = (a * pl.clamped_expert(u, w, "f.e0", 0.7) + b * pl.clamped_expert(u, w, "f.e1", 0.7)) / (a + b)
    torch.testing.assert_close(out, want)
    g = torch.tensor([[5.0, -5.0]], dtype=F64)
    wl = {"x.gate": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64), "x.up": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64),
          "x.down": torch.eye(2, dtype=F64)}
    y = pl.clamped_expert(g, wl, "x", 2.0)[0]
    assert abs(float(y[0]) - 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0) < 1e-12          # gate and up cut at the limit
    assert abs(float(y[1]) - (-5.0) / (1 + math.exp(1.702 * 5.0)) * (-1.0)) < 1e-12     # the gate has no lower bound, up has


def _rel(a, b):
    return ((a - b).pow(2).mean(dim=1).sqrt() / b.pow(2).mean(dim=1).sqrt())


@pytest.mark.parametrize("name", ["LA", "LC"])
def test_the_model_level_bound_tells_faults_apart(name):
    """The GPU tests hold bfloat16 rows to 4 % of a row's rms (float32 rows to 0.02 %).  Faults of the mechanisms move rows by more: a window
    one token wider, the sink left out, values not blended, the scaling of the frequencies left out, the cap left out, a tap
    lost, the residual factor or the layers' scales forgotten."""
    cfg = CONFIGS_L[name]
    w = {k: v.double() for k, v in make_weights(cfg, 3).items()}
    toks = random_tokens(72 if name == "LA" else 330, cfg["vocab"], 5)
    with torch.no_grad():
        ref = pl.forward_sequence(cfg, w, toks, dtype=F64)

        def moved(change_cfg=None, change_w=None):
            c2, w2 = copy.deepcopy(cfg), dict(w)
            if change_cfg:
                change_cfg(c2)
            if change_w:
                change_w(w2)
            return float(_rel(pl.forward_sequence(c2, w2, toks, dtype=F64), ref).max())

        att_layers = [i for i, l in enumerate(cfg["layers"]) if l["type"] != "delta"]
        first = att_layers[0]
        last = [i for i in att_layers if cfg["layers"][i]["mixer"].get("v_mix")][-1]          # blends its values and caps its scores
        assert cfg["layers"][last]["mixer"].get("softcap")
        faults = {
            "window + 1": moved(lambda c: c["layers"][first]["mixer"]["mask"].__setitem__("size", c["layers"][first]["mixer"]["mask"]["size"] + 1)),
            "no sink": moved(None, lambda d: d.__setitem__(f"l{first}.mix.sink", d[f"l{first}.mix.sink"] - 60.0)),
            "no blending": moved(lambda c: c["layers"][last]["mixer"].pop("v_mix")),
            "no scaling": moved(lambda c: c["layers"][first]["mixer"]["rot"].pop("scaling")),
            "no cap": moved(lambda c: c["layers"][last]["mixer"].pop("softcap")),
            "no factor": moved(lambda c: c.__setitem__("residual_mult", 1.0)),
            "no layer scale": moved(None, lambda d: d.__setitem__("l1.ls1", torch.ones_like(d["l1.ls1"]))),
            "no token input": moved(lambda c: c.pop("token_side")),
            "a tap lost": moved(None, lambda d: d.__setitem__("l1.mix.k.conv", d["l1.mix.k.conv"] * torch.tensor([0.0] + [1.0] * (d["l1.mix.k.conv"].shape[1] - 1), dtype=F64))),
        }
    for what, by in faults.items():
        assert by > 0.045, f"{what} moves the rows by {by:.2%} only"
