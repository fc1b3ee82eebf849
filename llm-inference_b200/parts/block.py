"""How one layer arranges its parts."""

from __future__ import annotations

import torch

from . import ops
from .base import Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class PreNormResidualBlock(Part):
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))``
    (python/instinct/backends/dense.py:89,104,122-129).

    The block receives the previous branch output still to be added (``delta``) so that each
    add runs inside the norm kernel that follows it, and returns its own last branch output
    the same way.

    Where the parts allow it (``takes_sink`` / ``takes_folded`` on the mixer and the
    feed-forward, ``foldable`` on the norms) and the step is short, a branch adds its output
    into the stream in its last product's epilogue and what travels on is
    :class:`ops.FoldedRows`: the norm that follows launches nothing. ``next_norm`` is the norm
    that will read this block's output (the next block's first norm, or the model's last)."""

    takes_next_norm = True

    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec) -> None:
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.feed_forward_norm = build_part("norm", feed_forward_norm)
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        self.graph_safe = all(p.graph_safe for p in self.parts)

    def tensor_specs(self):
        return [spec for part in self.parts for spec in part.tensor_specs()]

    def load(self, tensors, dtype, device) -> None:
        for part in self.parts:
            part.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self.parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta, next_norm: Part | None = None):
        mixer, ff = self.mixer, self.feed_forward
        h = self._norm(self.mixer_norm, ctx, x, delta, getattr(mixer, "takes_folded", False))
        # The mixer's and the feed-forward's outputs share one scratch buffer: the second norm
        # has consumed the former before the feed-forward's last product writes the latter.
        if getattr(mixer, "takes_sink", False) and getattr(self.feed_forward_norm, "foldable", False):
            a = mixer.forward(ctx, cache, h, sink=ops.ResidualSink(x, self.feed_forward_norm))
        else:
            a = mixer.forward(ctx, cache, h)
        h = self._norm(self.feed_forward_norm, ctx, x, a, getattr(ff, "takes_folded", False))
        if next_norm is not None and getattr(ff, "takes_sink", False) and getattr(next_norm, "foldable", False):
            return ff.forward(ctx, h, sink=ops.ResidualSink(x, next_norm))
        return ff.forward(ctx, h)

    @staticmethod
    def _norm(norm: Part, ctx: StepContext, x: torch.Tensor, delta, folded_ok: bool):
        if isinstance(delta, ops.FoldedRows):
            if getattr(norm, "foldable", False):
                return norm.forward(ctx, x, delta, folded_ok=folded_ok)
            return norm.forward(ctx, x, None)  # a norm that knows nothing of the folded form: the stream is current
        return norm.forward(ctx, x, delta)


class PostNormResidualBlock(Part):
    """``x += mult * scale1 * norm1(mixer(x)); x += mult * scale2 * norm2(feed_forward(x))``: the
    branches read the stream itself and the norms act on what they return. ``scale1`` / ``scale2``
    are learned per-column factors (None: ones), ``feed_forward`` may be None.

    With ``depth_mix`` = ``{"tensor": name, "index": i, "layers": L}`` the layer hands on, instead of
    its result, a weighted average over depth: with X_0 the embedding's output and X_(j+1) the
    result of layer j (before any averaging), layer ``i`` passes ``sum_{j <= i+1} w[j] X_j`` to what
    follows, ``w`` being the ``i + 2`` numbers of the named tensor. The X_j of a step live in one
    workspace buffer ``[L + 1, tokens, hidden]``; layer 0 also files the stream it receives as X_0.

    Every add, norm and average is one kernel per branch (``GroupedRMSNorm.add_branch``), which also
    writes the stream rounded to the compute dtype (buffer ``stream_cast``), the operand of the next
    matrix product; in 32-bit the stream is its own operand. The block never leaves a pending
    branch output: it returns None."""

    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec | None, mixer_norm: PartSpec, feed_forward_norm: PartSpec | None,
                 hidden_size: int, mult: float = 1.0, mixer_scale: str | None = None, feed_forward_scale: str | None = None,
                 depth_mix: dict | None = None, unused: tuple[str, ...] = ()) -> None:
        self.hidden_size, self.mult = hidden_size, float(mult)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = build_part("norm", feed_forward_norm) if feed_forward is not None else None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.scale_names = (mixer_scale, feed_forward_scale if feed_forward is not None else None)
        # A checkpoint may carry the second branch's scale although the layer has no feed-forward; it is read past.
        # (``unused`` names further per-column tensors of that kind.)
        self.unused_names = ([feed_forward_scale] if feed_forward is None and feed_forward_scale else []) + [n for n in unused if n != feed_forward_scale]
        self.scales: list[torch.Tensor | None] = [None, None]
        self.depth_mix = dict(depth_mix) if depth_mix else None
        self.mix: torch.Tensor | None = None

    def tensor_specs(self):
        from ..weights.loader import TensorSpec

        specs = [spec for part in self.parts for spec in part.tensor_specs()]
        specs += [TensorSpec(name, (self.hidden_size,), init="one_plus_normal") for name in self.scale_names if name]
        specs += [TensorSpec(name, (self.hidden_size,), init="one_plus_normal", optional=True) for name in self.unused_names]
        if self.depth_mix:
            specs.append(TensorSpec(self.depth_mix["tensor"], (self.depth_mix["index"] + 2,), init="half_plus_normal"))
        return specs

    def load(self, tensors, dtype, device) -> None:
        for part in self.parts:
            part.load(tensors, dtype, device)
        self.scales = [tensors[name].to(device=device, dtype=torch.float32).contiguous() if name else None for name in self.scale_names]
        if self.depth_mix:
            self.mix = tensors[self.depth_mix["tensor"]].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self.parts) + sum(4 * s.numel() for s in self.scales if s is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta):
        if delta is not None:
            raise ValueError("a post-norm block reads a stream that is up to date")
        tokens = ctx.num_tokens
        rounded = ctx.dtype != torch.float32
        cast = ctx.buffer("stream_cast", (tokens, self.hidden_size)) if rounded else None
        history = result = None
        mix = {}
        if self.depth_mix:
            index = self.depth_mix["index"]
            history = ctx.buffer("depth_history", (self.depth_mix["layers"] + 1, tokens, self.hidden_size), torch.float32, per_token=False)
            result = history[index + 1]
            mix = dict(history=history, mix=self.mix, mixed=x)
        else:
            result = x
        keep = history[0] if history is not None and self.depth_mix["index"] == 0 else None
        branch = self.mixer.forward(ctx, cache, cast if rounded else x)
        if self.feed_forward is None:
            self.mixer_norm.add_branch(ctx, x, branch, self.scales[0], self.mult, result, copy_in=keep, cast=cast, **mix)
            return None
        self.mixer_norm.add_branch(ctx, x, branch, self.scales[0], self.mult, result, copy_in=keep, cast=cast)
        branch = self.feed_forward.forward(ctx, cast if rounded else result)
        self.feed_forward_norm.add_branch(ctx, result, branch, self.scales[1], self.mult, result, cast=cast, **mix)
        return None


class ParallelResidualBlock(Part):
    """``h = norm(x); x += mixer(h) + feed_forward(h)``: one norm, and both sublayers read its output
    (``feed_forward`` may be None). The two outputs travel on together as :class:`ops.BranchSum` and the norm kernel
    that runs next (the following layer's, or the model's last) adds them into the stream in 32-bit, as the pre-norm
    block passes its pending branch output on. The feed-forward is built to write another buffer than the mixer."""

    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec | None, norm: PartSpec) -> None:
        self.mixer_norm = build_part("norm", norm)
        self.mixer = build_part("mixer", mixer)
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self.parts)

    def tensor_specs(self):
        return [spec for part in self.parts for spec in part.tensor_specs()]

    def load(self, tensors, dtype, device) -> None:
        for part in self.parts:
            part.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self.parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta):
        h = self.mixer_norm.forward(ctx, x, delta)
        a = self.mixer.forward(ctx, cache, h)
        if self.feed_forward is None:
            return a
        b = self.feed_forward.forward(ctx, h)
        if a.data_ptr() == b.data_ptr():
            raise ValueError("the mixer and the feed-forward of a parallel block must write different buffers")
        return ops.BranchSum(a, b)


register_part("block", "parallel_residual", ParallelResidualBlock)
register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "post_norm_residual", PostNormResidualBlock)
