"""A mixer that is two mixers side by side."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import CacheSpecs, Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class ParallelMixers(Part):
    """Two mixers read the same input; the result is ``(w_a * a / rms(a) + w_b * b / rms(b)) / 2`` with ``a`` and ``b``
    their outputs, each divided by its root mean square over the model width (``eps`` inside the root) and
    multiplied by a weight per column (tensors ``names[0]``, ``names[1]``).

    Each member keeps its own cache entry (:class:`CacheSpecs`). What the part returns is :class:`ops.BranchPair`,
    the two outputs not yet combined: the norm that adds the layer's result to the stream combines them in the
    same kernel, in 32-bit."""

    def __init__(self, *, first: PartSpec, second: PartSpec, names: tuple[str, str], hidden_size: int, eps: float) -> None:
        self.members = (build_part("mixer", first), build_part("mixer", second))
        self.names, self.hidden_size, self.eps = tuple(names), hidden_size, float(eps)
        self.graph_safe = all(m.graph_safe for m in self.members)
        # Members that say where their output goes write to buffers of their own; another member's output is copied.
        for member, name in zip(self.members, ("branch_first", "branch_second")):
            if hasattr(member, "out_name"):
                member.out_name = name
        self.weights: list[torch.Tensor] = []

    def cache_spec(self) -> CacheSpecs:
        return CacheSpecs(tuple(m.cache_spec() for m in self.members))

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [spec for m in self.members for spec in m.tensor_specs()]
        return specs + [TensorSpec(name, (self.hidden_size,), init="one_plus_normal") for name in self.names]

    def load(self, tensors, dtype, device) -> None:
        for m in self.members:
            m.load(tensors, dtype, device)
        self.weights = [tensors[name].to(device=device, dtype=torch.float32).contiguous() for name in self.names]

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.members)

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> ops.BranchPair:
        outs = []
        for index, member in enumerate(self.members):
            view = cache.members[index] if cache is not None else None
            out = member.forward(ctx, view, h)
            if not hasattr(member, "out_name"):
                keep = ctx.buffer(("branch_first", "branch_second")[index], tuple(out.shape), out.dtype)
                keep.copy_(out)
                out = keep
            outs.append(out)
        return ops.BranchPair(outs[0], outs[1], self.weights[0], self.weights[1], self.eps)


register_part("mixer", "parallel_mixers", ParallelMixers)
