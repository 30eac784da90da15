"""Frequencies of rotary positions in the rotate-half layout: coordinate i < dims / 2 pairs
with i + dims / 2 and the pair at position p turns by p * base^(-2 i / dims).  The mixers'
kernels compute the angles in 32-bit from this table and the tokens' positions."""
from __future__ import annotations

import torch


def rotary_frequencies(base: float, dims: int, device, divide_by: float = 1.0,
                       with_lo: bool = False):
    """float32 [max(1, dims / 2)] (a table of one zero when nothing is rotated); ``divide_by``:
    linear scaling of the positions, every frequency divided by it.  ``with_lo``: (hi, lo)
    tables, see :func:`split_frequencies`."""
    if dims < 0 or dims % 2:
        raise ValueError(f"rotary positions need an even number of coordinates, got {dims}")
    half = dims // 2
    freq = [float(base) ** (-2.0 * i / dims) / float(divide_by) for i in range(half)] or [0.0]
    if with_lo:
        return split_frequencies(freq, device)
    return torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)


def split_frequencies(freq64, device):
    """(hi, lo) float32 tables of frequencies given in 64-bit: hi is the rounded frequency, lo
    what the rounding left out.  The kernels that take ``freq_lo`` add the two in 64-bit, so the
    angle position x frequency keeps the frequency's full precision."""
    f64 = torch.as_tensor(freq64, dtype=torch.float64)
    hi = f64.to(torch.float32)
    lo = (f64 - hi.to(torch.float64)).to(torch.float32)
    return hi.to(device), lo.to(device)


def yarn_frequencies(base: float, dims: int, factor: float, original: float, fast: float,
                     slow: float, device, with_lo: bool = False):
    """(frequencies float32 [dims / 2], magnitude) of YaRN-scaled rotary positions.  With
    d(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi =
    min(ceil(d(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    frequency i is f_i / factor * ramp_i + f_i * (1 - ramp_i) (fast-turning pairs keep their
    frequency, slow ones are interpolated), and cos and sin are both multiplied by the
    magnitude 0.1 * ln(factor) + 1.  ``with_lo``: the frequencies as (hi, lo) tables, see
    :func:`split_frequencies`."""
    import math
    if dims <= 0 or dims % 2:
        raise ValueError(f"rotary positions need an even number of coordinates, got {dims}")

    def d_of(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d_of(fast)), 0)
    hi = min(math.ceil(d_of(slow)), dims - 1)
    freq = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        freq.append(f / factor * ramp + f * (1.0 - ramp))
    table = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)
    if with_lo:
        return split_frequencies(freq, device), 0.1 * math.log(factor) + 1.0
    return table, 0.1 * math.log(factor) + 1.0
