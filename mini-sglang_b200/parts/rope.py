from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope_neox")
class RotaryNeox(PositionEncoding):
    """Rotary position encoding, NeoX style: inv_freq_i = theta^(-2i/rot), angle = pos * inv_freq_i
    in float32, the two halves of the first `rotary_dim` elements rotated against each other.
    Table [max_positions, rotary_dim] = cos | sin in float32, as
    mini_sglang/layers/rotary_embedding.py:59-67 builds it; no scaling of any kind.
    params: head_dim, rotary_dim, theta, max_positions."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self._table: Optional[torch.Tensor] = None
    def load(self, src) -> None:
        self.rotary_table()      # made with the weights, so that the memory left for the cache is measured after it

    def rotary_table(self) -> torch.Tensor:
        if self._table is None:
            # built on the host in float32, operation by operation as the reference does, so the
            # table does not depend on the device's pow/sin/cos roundings; then moved to the device
            idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
            inv_freq = 1.0 / (self.theta ** (idx / self.rotary_dim))
            t = torch.arange(self.max_positions, dtype=torch.float32)
            freqs = t[:, None] * inv_freq[None, :]
            self._table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(self.env.device)
        return self._table

    def fused_decode_fields(self):
        return {"kind": "rotary_table", "table": self.rotary_table(), "rot": self.rotary_dim, "max_pos": self.max_positions}


@register_position_encoding("rope_yarn")
class RotaryYarn(PositionEncoding):
    """Rotary position encoding in halves (element i against i + rotary_dim / 2) with YaRN's frequency scaling.

    Pair i of n = rotary_dim / 2 turns with frequency f_i = theta^(-i / n).  `scaling` = {factor, original, fast, slow} slows the
    pairs whose wavelength is long against a context of `original` tokens: a pair that makes t turns within `original` tokens
    has the (real-valued) index p(t) = n log_theta(original / (2 pi t)); between lo = max(floor(p(fast)), 0) and
    hi = min(ceil(p(slow)), rotary_dim - 1) a ramp r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) blends the plain frequency
    into the slowed one, f_i (1 - r_i) + (f_i / factor) r_i.  cos and sin are multiplied by `magnitude` = 1 + 0.1 ln(factor).
    Without `scaling`: plain frequencies, magnitude 1.

    The frequencies are made on the host in double precision and kept as float32 (`inv_freq`); kernels that make their angles
    themselves (position * frequency in float32) read them and have no position limit; `rotary_table()` gives the same angles
    as a table of `max_positions` rows for kernels that look them up.
    params: rotary_dim, theta, scaling (or None), max_positions."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.scaling = dict(spec["scaling"]) if spec.get("scaling") else None
        self.max_positions = int(spec.get("max_positions", 0))
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError("rotary_dim must be even")
        freq, self.magnitude = yarn_frequencies(self.rotary_dim, self.theta, self.scaling)
        self._freq_host = freq.to(torch.float32)
        self.inv_freq: Optional[torch.Tensor] = None
        self._table: Optional[torch.Tensor] = None
        self._freq_host64 = freq.to(torch.float64)
        self.inv_freq64: Optional[torch.Tensor] = None

    def load(self, src) -> None:
        self.inv_freq = self._freq_host.to(self.env.device).contiguous()
        self.inv_freq64 = self._freq_host64.to(self.env.device).contiguous()

    def rotary_table(self) -> torch.Tensor:
        if self._table is None:
            t = torch.arange(self.max_positions, dtype=torch.float32)
            ang = t[:, None] * self._freq_host[None, :]
            self._table = (torch.cat((ang.cos(), ang.sin()), dim=-1) * self.magnitude).contiguous().to(self.env.device)
        return self._table

    def step_angles(self, ctx) -> torch.Tensor:
        """float32 [T, rotary_dim] = cos | sin (times `magnitude`) of the step's own positions, made once a step for all
        layers that share this encoding: position times frequency and the circular functions in double precision, so that
        the angle of a far position is as exact as that of a near one and no table bounds the context."""
        return step_angles_of(self, ctx)


def step_angles_of(enc, ctx) -> torch.Tensor:
    from .. import ops
    key = ("rotary_angles", id(enc))
    table = ctx.shared.get(key)
    if table is None:
        table = ctx.shared[key] = ops.rotary_angles(ctx.positions, enc.inv_freq64, enc.magnitude, ctx.T)
    return table


@register_position_encoding("rope_stepped")
class RotarySteppedWavelengths(PositionEncoding):
    """Rotary position encoding in halves whose frequencies are slowed by the wavelength's place against a context of
    `original` tokens (the rule Llama 3.1 uses).

    Pair i of n = rotary_dim / 2 turns with f_i = theta^(-i / n), wavelength l_i = 2 pi / f_i.  `scaling` = {factor, low, high,
    original}: f_i stays where l_i < original / high, becomes f_i / factor where l_i > original / low, and in between, with
    s = (original / l_i - low) / (high - low), becomes (1 - s) f_i / factor + s f_i.  No change of magnitude.  Without
    `scaling`: plain frequencies.  Frequencies are made on the host in double precision; `step_angles(ctx)` gives cos | sin of
    the step's positions (no table, no position limit), `rotary_table()` a table of `max_positions` rows for kernels that
    look angles up.  params: rotary_dim, theta, scaling (or None), max_positions."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.scaling = dict(spec["scaling"]) if spec.get("scaling") else None
        self.max_positions = int(spec.get("max_positions", 0))
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError("rotary_dim must be even")
        self._freq_host64 = stepped_frequencies(self.rotary_dim, self.theta, self.scaling)
        self.magnitude = 1.0
        self.inv_freq = self.inv_freq64 = None
        self._table: Optional[torch.Tensor] = None
    def load(self, src) -> None:
        self.inv_freq = self._freq_host64.to(torch.float32).to(self.env.device).contiguous()
        self.inv_freq64 = self._freq_host64.to(self.env.device).contiguous()

    def rotary_table(self) -> torch.Tensor:
        if self._table is None:
            t = torch.arange(self.max_positions, dtype=torch.float64)
            ang = t[:, None] * self._freq_host64[None, :]
            self._table = torch.cat((ang.cos(), ang.sin()), dim=-1).to(torch.float32).contiguous().to(self.env.device)
        return self._table

    def step_angles(self, ctx) -> torch.Tensor:
        return step_angles_of(self, ctx)


def stepped_frequencies(rotary_dim: int, theta: float, scaling) -> torch.Tensor:
    """-> float64 frequencies [rotary_dim / 2] of `RotarySteppedWavelengths`."""
    import math
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / rotary_dim) if rotary_dim else i
    if not scaling:
        return f
    factor, original = float(scaling["factor"]), float(scaling["original"])
    low, high = float(scaling["low"]), float(scaling["high"])
    wavelength = 2.0 * math.pi / f
    blend = ((original / wavelength - low) / (high - low)) if high != low else torch.ones_like(f)
    mid = (1.0 - blend) * f / factor + blend * f
    return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mid))


def yarn_frequencies(rotary_dim: int, theta: float, scaling):
    """-> (float64 frequencies [rotary_dim / 2], magnitude) of `RotaryYarn`."""
    import math
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / rotary_dim) if rotary_dim else i
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), rotary_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0
