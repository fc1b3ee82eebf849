"""A recurrent mixer: minGRU, a gated recurrence whose gates read only the current token."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, StateSpec, register_part
from .context import CacheView, StepContext


class MinGRU(Part):
    """``z = sigmoid(W_z h + b_z)`` and ``u = W_x h + b_x`` (``width`` numbers each); the candidate is ``u + 1/2``
    where ``u >= 0`` and ``sigmoid(u)`` where ``u < 0``. Element by element a state ``S`` (32-bit, zero at a
    request's start) follows ``S <- (1 - z) S + z * candidate``; the output is ``W_o (S * silu(W_g h))``.

    Per-request state: ``S``. The three projections are one matrix ``[z | x | g]``; gates, candidates and the
    state are 32-bit. Because neither gate nor candidate depends on the state, the tokens' updates are affine
    maps that compose, and long prompt portions run in pieces at the same time (csrc/kernels/mingru.cu).
    Tensor names: ``prefix + z | z.b | x | x.b | g | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, width: int, out_name: str = "branch") -> None:
        self.prefix, self.hidden_size, self.width, self.out_name = prefix, hidden_size, int(width), out_name
        self.w_in = self.bias = self.w_o = None

    def cache_spec(self) -> StateSpec:
        return StateSpec(((self.width,),), (torch.float32,))

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, w = self.prefix, self.hidden_size, self.width
        return [
            TensorSpec(p + "z", (w, d)), TensorSpec(p + "z.b", (w,)), TensorSpec(p + "x", (w, d)), TensorSpec(p + "x.b", (w,)),
            TensorSpec(p + "g", (w, d)), TensorSpec(p + "o", (d, w)),
        ]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        self.w_in = torch.cat([tensors[p + n].to(device=device, dtype=dtype) for n in ("z", "x", "g")]).contiguous()
        self.bias = torch.cat([tensors[p + n].to(device=device, dtype=torch.float32) for n in ("z.b", "x.b")]).contiguous()
        self.w_o = tensors[p + "o"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t = ctx.num_tokens
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("mingru_proj", (t, 3 * self.width)))
        y = ops.mingru(ctx, proj, self.bias, cache.state[0], ctx.buffer("mingru_y", (t, self.width)))
        return ops.linear(ctx, y, self.w_o, ctx.buffer(self.out_name, (t, self.hidden_size)))


register_part("mixer", "mingru", MinGRU)
