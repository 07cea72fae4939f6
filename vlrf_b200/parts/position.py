"""Position encodings.

A position encoding acts at one of two places and says which through `where`:
  "embedding"  it is added to the token embedding (learned absolute positions do this)
  "qk"         it transforms queries and keys inside a mixer (rotary encodings would do this)
The step gives every token its position, so an encoding never counts tokens itself.
"""
from __future__ import annotations

import torch

from .registry import register_part


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions:
    """x[t] += table[position[t]] (reference: include/model/transformer.hpp:350-361).  The table's
    row count bounds the length of a sequence."""

    where = "embedding"

    def __init__(self, table: torch.Tensor):
        if table.dim() != 2:
            raise ValueError("LearnedAbsolutePositions: the table is [positions, width]")
        self.table = table
        self.max_positions = table.shape[0]


@register_part("position", "rotary")
class RotaryPositions:
    """Rotation of queries and keys by position.  Of a vector's first `dims` entries, entry i is paired with entry
    i + dims/2 (`pairing` "half") or entry 2i with entry 2i + 1 (`pairing` "interleaved"); at position p the pair
    (u, v) becomes (u cos a − v sin a, v cos a + u sin a) with a = p · f_i and
    f_i = base^(−2i/dims); entries beyond `dims` pass unchanged.  `scaling_factor` divides every frequency (linear
    scaling: positions count `scaling_factor` times slower).  `yarn` = (factor, original, fast, slow) slows only the
    slow pairs instead: with n(t) = dims · ln(original / (2π t)) / (2 ln base) the (real-valued) index of the pair that
    turns t times over `original` positions, lo = max(⌊n(fast)⌋, 0), hi = min(⌈n(slow)⌉, dims − 1) and
    r_i = clamp((i − lo) / max(hi − lo, 0.001), 0, 1), the frequency is f_i / factor · r_i + f_i · (1 − r_i), and every
    cosine and sine is multiplied by `magnitude` = 0.1 · ln(factor) + 1.  The part holds the table f (float32, made
    in 64-bit); the mixer that is given the part applies it inside its own kernels, with angles in float32."""

    where = "qk"

    def __init__(self, base: float, dims: int, device, scaling_factor: float = 1.0, pairing: str = "half", yarn=None):
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"RotaryPositions: pairing '{pairing}' is neither 'half' nor 'interleaved'")
        self.pairing, self.interleaved = pairing, pairing == "interleaved"
        if dims <= 0 or dims % 2 != 0 or not base > 0.0:
            raise ValueError(f"RotaryPositions: {dims} dimensions cannot be rotated in pairs, or base {base} is not positive")
        if not scaling_factor > 0.0:
            raise ValueError(f"RotaryPositions: a scaling factor of {scaling_factor} is not positive")
        self.base, self.dims, self.scaling_factor = float(base), int(dims), float(scaling_factor)
        half = dims // 2
        f = [self.base ** (-2.0 * i / dims) / self.scaling_factor for i in range(half)]
        self.magnitude, self.yarn = 1.0, None
        if yarn is not None:
            import math
            factor, original, fast, slow = (float(v) for v in yarn)
            if not (factor > 0.0 and original > 0.0 and fast > 0.0 and slow > 0.0) or self.base == 1.0:
                raise ValueError(f"RotaryPositions: a scaling of {yarn} has a number that is not positive")
            self.yarn = (factor, original, fast, slow)

            def index_of(turns):
                return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo, hi = max(math.floor(index_of(fast)), 0), min(math.ceil(index_of(slow)), dims - 1)
            ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)]
            f = [fi / factor * r + fi * (1.0 - r) for fi, r in zip(f, ramp)]
            self.magnitude = 0.1 * math.log(factor) + 1.0
        f = torch.tensor(f, dtype=torch.float64)
        self.inv_freq = f.to(torch.float32).to(device).contiguous()
