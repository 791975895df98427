"""Rotary position encoding as a part: the cos / sin tables of one `RopeTableSpec`.

cos[p, i] = (float) cos(p * f_i), f_i = theta^(-2i / rotary_dim), the angle formed in
double precision and rounded once (src/main/java/org/robomiri/jllm/model/Rope.java:24-38,
122-127); `linear` divides every frequency by the factor (:138-142); `yarn` blends plain and
divided frequencies over a ramp and scales cos and sin by an amplitude (:75-85,170-208).
The table is made once for the engine's context and lives on the device in float32; the
rotation itself is fused into the mixer's kernel, which takes the table, `rotary_dim` and
the pairing as parameters.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


def inverse_frequencies(spec, max_positions: int) -> torch.Tensor:
    d, theta, sc = spec.rotary_dim, spec.theta, spec.scaling
    half = d // 2
    f = [1.0 / math.pow(theta, (2.0 * i) / d) for i in range(half)]
    if sc.kind == "linear":
        f = [v / sc.factor for v in f]
    elif sc.kind == "yarn":
        orig = sc.original_max_positions or max_positions

        def correction_dim(rotations: float) -> float:
            return d * math.log(orig / (rotations * 2 * math.pi)) / (2 * math.log(theta))

        low, high = correction_dim(sc.beta_fast), correction_dim(sc.beta_slow)
        low = max(math.floor(low) if sc.truncate else low, 0)
        high = min(math.ceil(high) if sc.truncate else high, d - 1)
        if low == high:
            high += 0.001
        for i in range(half):
            plain = 1.0 / math.pow(theta, (2.0 * i) / d)
            ramp = min(max((i - low) / (high - low), 0), 1)
            f[i] = plain / sc.factor * ramp + plain * (1 - ramp)
    elif sc.kind != "none":
        raise ValueError(f"rope scaling {sc.kind!r} is not built")
    return torch.tensor(f, dtype=torch.float64)


def amplitude(sc) -> float:
    if sc.kind != "yarn":
        return 1.0
    if sc.attention_factor > 0:
        return sc.attention_factor

    def mscale(scale: float, m: float) -> float:
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    return mscale(sc.factor, sc.mscale) / mscale(sc.factor, sc.mscale_all_dim)


class RotaryTable(PositionEncoding):
    def __init__(self, spec, max_positions: int, device):
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        self.pairing = spec.pairing
        f = inverse_frequencies(spec, max_positions)
        angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * f[None, :]
        amp = amplitude(spec.scaling)
        self.cos = (torch.cos(angle) * amp).to(torch.float32).contiguous().to(device)
        self.sin = (torch.sin(angle) * amp).to(torch.float32).contiguous().to(device)
        self.max_positions = max_positions


register_position_encoding("rotary", RotaryTable, replace=True)
