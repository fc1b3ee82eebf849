"""Position encodings."""

from __future__ import annotations

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
        self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")} if scaling else None
        # interleaved: dim 2i pairs with dim 2i + 1 instead of i with i + rotary_dims / 2. The
        # frequencies are the same; the mixer that owns the part calls the kernel of its layout.
        self.interleaved = bool(interleaved)
        self.rotary_dims = head_dim if rotary_dims is None else rotary_dims
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= head_dim:
            raise ValueError(f"rotary_dims={self.rotary_dims} must be even and at most head_dim={head_dim}")
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def table(self) -> np.ndarray:
        half = self.rotary_dims // 2
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
                     dim: int, rank: int, norm_weight: torch.Tensor, eps: float, q_rot: torch.Tensor) -> None:
        """The same duty towards a mixer that caches one latent row per token: ``proj`` holds, per
        token, ``heads`` queries ``[dim plain | head_dim rotated]`` from column ``q_offset`` and
        ``[rank latent | head_dim rotated key part]`` from ``kv_offset``. One kernel rotates the query
        parts into ``q_rot``, RMS-norms the latent (``norm_weight``, ``eps``), rotates the key part
        and writes both to the token's cache row. Here ``head_dim`` is the size of the rotated part."""
        if not self.interleaved:
            raise ValueError("the latent kernel rotates interleaved pairs")
        ops.latent_kv_write(ctx, cache, proj, q_offset, kv_offset, heads, dim, self.head_dim, rank, norm_weight, eps, self.inv_freq, q_rot)


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
