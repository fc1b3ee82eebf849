"""Normalisation parts."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, register_part
from .context import StepContext


class RMSNorm(Part):
    """``y = v * rsqrt(mean(v^2) + eps) * weight`` with ``v = x + delta``, all in 32-bit
    (python/instinct/backends/portable.py:144-149). The add into the residual stream is
    part of the same kernel.

    In short bfloat16 steps the norm can disappear into the matrix products around it: the
    product before it adds its own output into the stream and hands over
    :class:`ops.FoldedRows` instead of a branch output; if the consumer says it takes that
    form (``folded_ok``) the norm passes it on and launches nothing."""

    foldable = True  # y = x * rsqrt(mean(x^2) + eps) * weight, nothing else: what the products' epilogues assume

    def __init__(self, *, name: str, hidden_size: int, eps: float) -> None:
        self.name, self.hidden_size, self.eps = name, hidden_size, float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + ".weight", (self.hidden_size,), init="one_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name + ".weight"].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def forward(
        self,
        ctx: StepContext,
        x: torch.Tensor,
        delta: torch.Tensor | None,
        rows: torch.Tensor | None = None,
        out_name: str = "normed",
        folded_ok: bool = False,
    ) -> torch.Tensor:
        if isinstance(delta, ops.FoldedRows):
            # The stream is already up to date. Pass the folded form on if it was made for this
            # norm and the consumer takes it; otherwise normalise the stream here.
            if folded_ok and rows is None and delta.norm is self:
                return delta
            delta = None
        count = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (count, self.hidden_size), per_token=rows is None)
        return ops.rmsnorm(ctx, x, delta, self.weight, self.eps, out, rows)


class GroupedRMSNorm(Part):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive parts, each divided by
    its own ``sqrt(mean(part^2) + eps)``, and the whole is multiplied by the weight; all 32-bit.

    Two uses. As the norm of the stream itself (``forward``, the interface of every norm part; the
    model's last norm). And as the norm of a branch's *output* in a layer that adds
    ``mult * scale * norm(branch(x))`` to its stream (``add_branch``); the same kernel can then also
    form the weighted average over depth that such a layer hands on (parts/block.py)."""

    foldable = False

    def __init__(self, *, name: str, hidden_size: int, groups: int, eps: float, around_zero: bool = False) -> None:
        if groups <= 0 or hidden_size % groups:
            raise ValueError(f"{hidden_size} columns do not cut into {groups} equal groups")
        self.name, self.hidden_size, self.groups, self.eps = name, hidden_size, int(groups), float(eps)
        # around_zero: the checkpoint stores the weight as an offset from one (the factor is 1 + w); one is
        # added once, in 32-bit, when the weights are loaded.
        self.around_zero = bool(around_zero)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.hidden_size,), init="normal" if self.around_zero else "one_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(device=device, dtype=torch.float32).contiguous()
        if self.around_zero:
            self.weight += 1.0

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, rows: torch.Tensor | None = None, out_name: str = "normed",
                folded_ok: bool = False) -> torch.Tensor:
        if delta is not None:
            raise ValueError("a grouped norm reads a stream that is up to date; it takes no pending branch output")
        count = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (count, self.hidden_size), per_token=rows is None)
        return ops.grouped_rmsnorm(ctx, x, self.weight, self.groups, self.eps, out, rows)

    def add_branch(self, ctx: StepContext, x_in: torch.Tensor, branch: torch.Tensor, scale: torch.Tensor | None, mult: float,
                   x_out: torch.Tensor, **more) -> None:
        if isinstance(branch, ops.BranchPair):
            # two mixers side by side: their combination and this norm are one kernel
            if self.groups != 1 or scale is not None or mult != 1.0 or any(v is not None for k, v in more.items() if k != "cast"):
                raise ValueError("a pair of branch outputs is added by a plain RMS norm without scale, multiplier or depth average")
            ops.pair_norm_add(ctx, x_in, branch, self.weight, self.eps, x_out, cast=more.get("cast"))
            return
        ops.branch_norm_add(ctx, x_in, branch, self.weight, scale, mult, self.groups, self.eps, x_out, **more)


class LayerNorm(Part):
    """``y = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * weight`` with ``v = x + delta``, a weight and no bias,
    all in 32-bit; the add into the residual stream is part of the same kernel. ``delta`` may be one branch output or
    an :class:`ops.BranchSum` (two sublayers that read the same normed rows). The tensor is ``name`` itself."""

    foldable = False

    def __init__(self, *, name: str, hidden_size: int, eps: float) -> None:
        self.name, self.hidden_size, self.eps = name, hidden_size, float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.hidden_size,), init="one_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, rows: torch.Tensor | None = None, out_name: str = "normed",
                folded_ok: bool = False) -> torch.Tensor:
        if isinstance(delta, ops.FoldedRows):
            delta = None  # the stream is already up to date
        count = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (count, self.hidden_size), per_token=rows is None)
        return ops.layernorm(ctx, x, delta, self.weight, self.eps, out, rows)


register_part("norm", "layernorm", LayerNorm)
register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "grouped_rmsnorm", GroupedRMSNorm)
