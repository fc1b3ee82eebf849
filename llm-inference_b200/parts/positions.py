"""Position encodings."""

from __future__ import annotations

import math

import numpy as np
import torch

from . import ops
from .base import Part, register_part
from .context import CacheView, StepContext


class RotaryEncoding(Part):
    """Rotary position encoding over the first ``rotary_dims`` dims of each head, pairing
    dim i with i + rotary_dims / 2; inverse frequencies ``theta ** (-2 i / rotary_dims)`` are
    tabulated once in 32-bit and the kernel multiplies them by the position
    (python/instinct/backends/portable.py:115-132)."""

    def __init__(self, *, head_dim: int, theta: float, rotary_dims: int | None = None, interleaved: bool = False,
                 scaling: dict | None = None) -> None:
        self.head_dim = head_dim
        # scaling = {factor, low, high, original}: frequencies whose wavelength 2 pi / f exceeds original / low are
        # divided by factor, those shorter than original / high are kept, and between the two the frequency is
        # (1 - s) f / factor + s f with s = (original / wavelength - low) / (high - low). The table is then worked
        # out in 64-bit and rounded once.
        # scaling = {factor, original, fast, slow} is another rule, a ramp over the index of the frequency instead of its
        # wavelength: with t(n) = rotary_dims * ln(original / (2 pi n)) / (2 ln theta), lo = max(floor(t(fast)), 0) and
        # hi = min(ceil(t(slow)), rotary_dims - 1), frequency i is f / factor * r + f * (1 - r) with
        # r = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), and sine and cosine are both multiplied by the
        # ``magnitude`` 0.1 * ln(factor) + 1.
        self.ramp = None
        if scaling and "fast" in scaling:
            self.ramp = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            scaling = None
        self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")} if scaling else None
        # interleaved: dim 2i pairs with dim 2i + 1 instead of i with i + rotary_dims / 2. The
        # frequencies are the same; the mixer that owns the part calls the kernel of its layout.
        self.interleaved = bool(interleaved)
        self.rotary_dims = head_dim if rotary_dims is None else rotary_dims
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= head_dim:
            raise ValueError(f"rotary_dims={self.rotary_dims} must be even and at most head_dim={head_dim}")
        self.theta = float(theta)
        self.magnitude = 0.1 * math.log(self.ramp["factor"]) + 1.0 if self.ramp else 1.0
        self.inv_freq: torch.Tensor | None = None

    def table(self) -> np.ndarray:
        half = self.rotary_dims // 2
        if self.ramp is not None:
            c, dims = self.ramp, self.rotary_dims
            index = np.arange(half, dtype=np.float64)
            f = np.power(np.float64(self.theta), -2.0 * index / max(dims, 1))

            def turning_point(turns: float) -> float:
                return dims * math.log(c["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turning_point(c["fast"])), 0)
            hi = min(math.ceil(turning_point(c["slow"])), dims - 1)
            r = np.clip((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            return (f / c["factor"] * r + f * (1.0 - r)).astype(np.float32)
        if self.scaling is not None:
            f = np.power(np.float64(self.theta), -2.0 * np.arange(half, dtype=np.float64) / max(self.rotary_dims, 1))
            c = self.scaling
            wavelength = 2.0 * np.pi / f
            s = (c["original"] / wavelength - c["low"]) / (c["high"] - c["low"])
            blended = (1.0 - s) * f / c["factor"] + s * f
            f = np.where(wavelength < c["original"] / c["high"], f, np.where(wavelength > c["original"] / c["low"], f / c["factor"], blended))
            return f.astype(np.float32)
        exponent = -(np.arange(half, dtype=np.float32) * np.float32(2.0) / np.float32(self.rotary_dims))
        return np.power(np.float32(self.theta), exponent, dtype=np.float32)

    def load(self, tensors, dtype, device) -> None:
        self.inv_freq = torch.from_numpy(self.table()).to(device)

    def apply(
        self,
        ctx: StepContext,
        cache: CacheView,
        qkv: torch.Tensor,
        bias: torch.Tensor | None,
        q_out: torch.Tensor,
        q_heads: int,
        kv_heads: int,
        head_dim: int,
    ) -> torch.Tensor:
        """The position part's one duty towards an attention mixer: take the step's projected
        rows ``qkv`` (``[tokens, (q_heads + 2 kv_heads) * head_dim]``, bias not yet added), add
        the bias, encode each token's position into its queries and keys, store keys and values
        in the token's page of ``cache`` (unless ``cache.writes`` is false) and the queries
        densely in ``q_out``. Here all of it is one kernel."""
        if self.interleaved:
            raise ValueError("the fused q/k/v kernel pairs dim i with i + rotary_dims / 2; this part is interleaved")
        return ops.rope_kv_write(ctx, cache, qkv, bias, self.inv_freq, q_out, q_heads, kv_heads, head_dim)


    def apply_latent(self, ctx: StepContext, cache: CacheView, proj: torch.Tensor, q_offset: int, kv_offset: int, heads: int,
                     dim: int, rank: int, norm_weight: torch.Tensor, eps: float, q_rot: torch.Tensor, q_proj: torch.Tensor | None = None) -> None:
        """The same duty towards a mixer that caches one latent row per token: ``proj`` holds, per
        token, ``heads`` queries ``[dim plain | head_dim rotated]`` from column ``q_offset`` and
        ``[rank latent | head_dim rotated key part]`` from ``kv_offset``. One kernel rotates the query
        parts into ``q_rot``, RMS-norms the latent (``norm_weight``, ``eps``), rotates the key part
        and writes both to the token's cache row. Here ``head_dim`` is the size of the rotated part.
        ``q_proj``: the matrix whose rows hold the queries when they do not come out of the same product as the latent.
        Both layouts of pairs are served (``interleaved`` or halves), and the ``magnitude`` of a ramp scaling."""
        ops.latent_kv_write(ctx, cache, proj, q_offset, kv_offset, heads, dim, self.head_dim, rank, norm_weight, eps, self.inv_freq, q_rot,
                            q_proj=q_proj, halves=not self.interleaved, magnitude=self.magnitude)

    def apply_after_norm(self, ctx: StepContext, cache: CacheView, proj: torch.Tensor, bias, q_weight, k_weight, eps: float,
                         values_from_keys: bool, q_out: torch.Tensor, q_heads: int, kv_heads: int, dim: int, vdim: int, row_dim: int) -> None:
        """The same duty towards a mixer that norms all of q (and all of k) as one vector before the rotation: one kernel
        does bias, both norms, the rotation in halves and the writes (queries to ``q_out``, keys and values to the token's
        page, rows padded to ``row_dim``; with ``values_from_keys`` the values are the keys as projected)."""
        if self.interleaved:
            raise ValueError("the norm-and-rotate kernel pairs dim i with i + rotary_dims / 2; this part is interleaved")
        ops.qk_norm_rope_write(ctx, cache, proj, bias, q_weight, k_weight, eps, self.inv_freq if self.rotary_dims else None, self.magnitude,
                               values_from_keys, q_out, q_heads, kv_heads, dim, vdim, row_dim)


    def apply_after_conv_norm(self, ctx: StepContext, cache: CacheView, conv_state: torch.Tensor, proj: torch.Tensor, bias, taps: torch.Tensor,
                              q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, q_out: torch.Tensor, q_heads: int, kv_heads: int,
                              dim: int, vdim: int, row_dim: int) -> None:
        """The same duty towards a mixer whose projections pass a short convolution over time and a norm over all
        heads at once before they are rotated: one kernel does bias, convolution, both norms, the rotation and the
        writes (queries to ``q_out``, keys and values to the token's page, rows padded to ``row_dim``)."""
        if not self.interleaved:
            raise ValueError("the convolution kernel rotates interleaved pairs")
        ops.conv_norm_rope_write(ctx, cache, conv_state, proj, bias, taps, q_weight, k_weight, eps, self.inv_freq, self.rotary_dims, q_out,
                                 q_heads, kv_heads, dim, vdim, row_dim)


register_part("position", "rotary", RotaryEncoding)
