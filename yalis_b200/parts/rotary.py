"""Rotary position encoding with the optional llama3 frequency smoothing or YaRN interpolation.

The inverse frequencies are computed once on the host in float32 exactly as the
reference builds its table (yalis/external/model.py:786-807); the angle
``position * inv_freq`` and its sine and cosine are computed in float32 inside
the kernel for the positions of the step, so no table bounds the context.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import rope_kv_write
from .base import PagedKVCache, PositionEncoding, register_part


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict], exact_powers: bool = False) -> torch.Tensor:
    """theta_i = base^(-2i/hs); with ``scaling``: s = clamp((orig/wavelen - low)/(high - low), 0, 1),
    theta_i <- (1 - s) * theta_i / factor + s * theta_i.  float32 [head_dim / 2] on the CPU.
    ``exact_powers``: the powers are taken in float64 and rounded once (the default takes them in float32, as
    the reference's table does)."""
    if exact_powers:
        inv = torch.tensor([float(theta) ** (-2.0 * i / head_dim) for i in range(head_dim // 2)], dtype=torch.float64).float()
    else:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    if scaling is not None:
        wavelen = 2 * torch.pi / inv
        ratio = scaling["original_max_position_embeddings"] / wavelen
        smooth = (ratio - scaling["low_freq_factor"]) / (scaling["high_freq_factor"] - scaling["low_freq_factor"])
        smooth = torch.clamp(smooth, min=0.0, max=1.0)
        inv = (1 - smooth) * (inv / scaling["factor"]) + smooth * inv
    return inv.to(torch.float32)


def yarn_frequencies(dims: int, theta: float, factor: float, original: float, fast: float, slow: float):
    """YaRN: the pairs that turn often within ``original`` positions keep their frequency, those that turn
    seldom are slowed by ``factor``, with a linear ramp between.  With n(t) = dims ln(original / (2 pi t)) /
    (2 ln theta) the pair index at which a pair makes t turns, lo = max(floor(n(fast)), 0),
    hi = min(ceil(n(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):

        f_i = theta^(-2i / dims) * ((1 - r_i) + r_i / factor),    magnitude = 0.1 ln(factor) + 1

    (cosine and sine are both multiplied by the magnitude).  Returns (float32 [dims / 2] on the CPU, magnitude);
    the arithmetic is float64, rounded once."""
    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = float(theta) ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64).float(), 0.1 * math.log(factor) + 1.0


class RotaryEncoding(PositionEncoding):
    """Parameters: ``head_dim`` (the sizes that turn), ``theta``, ``scaling`` (None, the four llama3 numbers, or
    ``{"kind": "yarn", "factor", "original", "fast", "slow"}``, see ``yarn_frequencies``), ``exact_powers`` (see
    ``inverse_frequencies``), ``layout`` (``half``, the default: size i is paired with i + head_dim / 2;
    ``interleaved``: size 2i with 2i + 1).  ``magnitude`` multiplies cosine and sine (1 unless YaRN says
    otherwise).  The kernels of ``encode_and_store`` turn the half layout only; mixers that prepare their heads
    themselves read ``inv_freq``, ``interleaved`` and ``magnitude``."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        layout = spec.params.get("layout", "half")
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout {layout!r} is not one of half, interleaved")
        self.interleaved = layout == "interleaved"
        self.magnitude = 1.0
        scaling = spec.params.get("scaling")
        if scaling is not None and scaling.get("kind") == "yarn":
            self.inv_freq_host, self.magnitude = yarn_frequencies(
                self.head_dim, float(spec.params["theta"]), float(scaling["factor"]), float(scaling["original"]),
                float(scaling["fast"]), float(scaling["slow"]))
        else:
            self.inv_freq_host = inverse_frequencies(self.head_dim, float(spec.params["theta"]), scaling,
                                                     bool(spec.params.get("exact_powers", False)))
        self.inv_freq: Optional[torch.Tensor] = None

    def load(self, tensors) -> None:
        pass

    def to(self, device) -> None:
        self.inv_freq = self.inv_freq_host.to(device)

    def _half_only(self) -> None:
        if self.interleaved or self.magnitude != 1.0:
            raise ValueError("this mixer's kernels turn the half layout with magnitude 1 only")

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        self._half_only()
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        if self.inv_freq is None or self.inv_freq.device != qkv.device:
            self.to(qkv.device)
        store = cache.writable
        return rope_kv_write(qkv, ctx.positions, ctx.req_of_token, self.inv_freq, cache.k if store else None,
                             cache.v if store else None, ctx.block_tables[cache.group], num_heads, num_kv_heads,
                             head_dim, out_dtype=dtype, bad_flag=ctx.error_flag)

    def rotary_frequencies(self, head_dim: int, device):
        self._half_only()
        return self.frequencies(head_dim, device)

    def frequencies(self, head_dim: int, device):
        """The float32 frequencies on ``device``, whatever the layout."""
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        if self.inv_freq is None or self.inv_freq.device != torch.device(device):
            self.to(device)
        return self.inv_freq

    def capture_key(self, host):
        return None


class NoPositionEncoding(PositionEncoding):
    """Stores K and V unrotated (a mixer that wants positions handled elsewhere)."""

    def rotary_frequencies(self, head_dim: int, device):
        return None

    def capture_key(self, host):
        return None

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        store = cache.writable
        return rope_kv_write(qkv, ctx.positions, ctx.req_of_token, None, cache.k if store else None,
                             cache.v if store else None, ctx.block_tables[cache.group], num_heads, num_kv_heads,
                             head_dim, out_dtype=dtype, bad_flag=ctx.error_flag)


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
