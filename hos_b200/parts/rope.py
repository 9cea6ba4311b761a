"""Rotary position encoding: for pair i of a head, angle = position / theta^(2i/rotary_dim);
the pair is rotated by it (src/forward.rs:203-222).  `style` chooses the pairing:
"rotate_half" pairs (i, i + rotary_dim/2) (the reference's `neox`, used by Gemma,
src/model.rs:80-82), "interleaved" pairs (2i, 2i+1).  Dimensions beyond
rotary_dim pass unchanged.  The inverse frequencies are computed once, in 32-bit;
the kernel multiplies them by the position and takes sincosf, all in 32-bit.

With `scaling` (factor, original, fast, slow: the ramp between scaled and unscaled frequencies that
extends a trained context) pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i), where, with
turns(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turns(fast)), 0),
hi = min(ceil(turns(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
cosine and sine are then multiplied by `magnitude` = 0.1 ln(factor) + 1.  `table: "float64"` takes the
frequencies in 64-bit before they are rounded to 32-bit.

A position encoding is used by a mixer: the mixer asks it for `kernel_args()` and
hands them to the fused rotate-and-store kernel."""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import SpecError
from ..registry import register_part
from .base import Part


_shared = {}


def _ramped(freqs, dims: int, theta: float, sc) -> list:
    """The frequencies under the long-context ramp (see the module's text)."""
    def turns(t: float) -> float:
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo = max(math.floor(turns(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns(float(sc["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / float(sc["factor"]) * ramp + f * (1.0 - ramp))
    return out


class Rotary(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        style = spec.params.get("style", "rotate_half")
        if style not in ops.ROPE_STYLES:
            raise SpecError(f"arch spec error: unknown rotary pairing {style!r}")
        if self.rotary_dim % 2 != 0 or self.rotary_dim <= 0:
            raise SpecError(f"arch spec error: rotary_dim {self.rotary_dim} must be positive and even")
        self.style = ops.ROPE_STYLES[style]
        scaling = spec.params.get("scaling")
        self.magnitude = 1.0            # a factor on cosine and sine (kernels that know no scaling take it as 1)
        if scaling:
            for k in ("factor", "original", "fast", "slow"):
                if k not in scaling:
                    raise SpecError(f"arch spec error: rotary scaling needs {k!r}")
            self.magnitude = 0.1 * math.log(float(scaling["factor"])) + 1.0
        in64 = bool(scaling) or spec.params.get("table") == "float64"
        key = (str(rt.device), self.theta, self.rotary_dim, in64,
               tuple(sorted((k, float(v)) for k, v in scaling.items())) if scaling else None)
        if key not in _shared:          # layers with the same frequencies share one tensor (and what is derived from it)
            half = self.rotary_dim // 2
            if in64:
                freqs = [self.theta ** (-2.0 * i / self.rotary_dim) for i in range(half)]
                if scaling:
                    freqs = _ramped(freqs, self.rotary_dim, self.theta, scaling)
                _shared[key] = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device).contiguous()
            else:
                i = torch.arange(half, dtype=torch.float32)
                exponent = 2.0 * i / float(self.rotary_dim)
                _shared[key] = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)) \
                    .to(rt.device).contiguous()
        self.inv_freq = _shared[key]

    def kernel_args(self):
        """(inverse frequencies [rotary_dim/2] float32 on the device, rotary_dim, style code)."""
        return self.inv_freq, self.rotary_dim, self.style


class NoPosition(Part):
    """No position encoding: q and k are used as projected."""
    graph_safe = True


    def kernel_args(self):
        return None, 0, 0


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
