"""Token embedding and the output head."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, StateSpec, register_part
from .context import StepContext


class TokenEmbedding(Part):
    """``x[t] = table[token[t]] * scale`` widened to the 32-bit residual stream
    (python/instinct/backends/dense.py:82; ``scale`` is 1 there). ``suffix`` is what follows
    ``name`` in the checkpoint's tensor name. With ``cast`` the step also gets the stream rounded
    to the compute dtype (buffer ``stream_cast``), which layers whose branches read the stream
    itself, without a norm in front, hand to their matrix products."""

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int, scale: float = 1.0, suffix: str = ".weight",
                 cast: bool = False) -> None:
        self.name, self.vocab_size, self.hidden_size = name, vocab_size, hidden_size
        self.scale, self.suffix, self.cast = float(scale), suffix, bool(cast)
        self.table: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + self.suffix, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name + self.suffix].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return 0  # a step reads only its tokens' rows

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.hidden_size), torch.float32)
        if self.scale == 1.0 and not self.cast:
            return ops.embedding_gather(ctx, self.table, x)
        rounded = self.cast and self.table.dtype != torch.float32  # in 32-bit the stream is its own copy
        cast = ctx.buffer("stream_cast", (ctx.num_tokens, self.hidden_size), self.table.dtype) if rounded else None
        return ops.embedding_scaled(ctx, self.table, self.scale, x, cast)


class NormedEmbedding(Part):
    """``x[t] = layer norm of table[token[t]]`` (mean taken off, a weight ``norm_name`` and no bias), in 32-bit, as the
    residual stream of the new tokens: gather and norm are one kernel."""

    def __init__(self, *, name: str, norm_name: str, vocab_size: int, hidden_size: int, eps: float) -> None:
        self.name, self.norm_name, self.vocab_size, self.hidden_size, self.eps = name, norm_name, vocab_size, hidden_size, float(eps)
        self.table: torch.Tensor | None = None
        self.norm_weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size)), TensorSpec(self.norm_name, (self.hidden_size,), init="one_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name].to(device=device, dtype=dtype).contiguous()
        self.norm_weight = tensors[self.norm_name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return 0  # a step reads only its tokens' rows

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.hidden_size), torch.float32)
        return ops.embedding_layernorm(ctx, self.table, self.norm_weight, self.eps, x)


class SinusoidEmbedding(Part):
    """``x[t] = table[token[t]] * scale + e(p)`` with ``e(p)[2i] = sin(p f_i)``, ``e(p)[2i + 1] = cos(p f_i)``,
    ``f_i = base^(-2i / hidden)`` and ``p`` the token's position in its request; the sum is 32-bit and fills
    every one of the token's ``streams`` residual streams (the stream buffer is ``[tokens, streams * hidden]``)."""

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int, scale: float = 1.0, streams: int = 1, base: float = 10000.0) -> None:
        if hidden_size % 2:
            raise ValueError("sine and cosine columns alternate: the width must be even")
        self.name, self.vocab_size, self.hidden_size = name, vocab_size, hidden_size
        self.scale, self.streams, self.base = float(scale), int(streams), float(base)
        self.table: torch.Tensor | None = None
        self.inv_freq: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def frequencies(self) -> torch.Tensor:
        """``f_i`` worked out in 64-bit and rounded once to float32."""
        i = torch.arange(self.hidden_size // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.hidden_size).to(torch.float32)

    def load(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name].to(device=device, dtype=dtype).contiguous()
        self.inv_freq = self.frequencies().to(device)

    def weight_bytes(self) -> int:
        return 0  # a step reads only its tokens' rows

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.buffer("residual_streams", (ctx.num_tokens, self.streams * self.hidden_size), torch.float32)
        return ops.embedding_sinusoid(ctx, self.table, self.inv_freq, self.scale, self.streams, x)


class BigramEmbedding(Part):
    """``x[t] = table[token[t]] + pairs[r(t)]`` in 32-bit, where ``r(t) = (previous * mul_prev + token * mul_cur) mod
    buckets`` hashes the token together with the one in front of it in its request; a request's first token
    takes the pair table's last row (number ``buckets``). The token in front of a step's first one is
    per-request state (one int32 per slot). With ``cast`` the step also gets the stream rounded to the compute
    dtype (buffer ``stream_cast``)."""

    def __init__(self, *, name: str, pairs_name: str, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int,
                 cast: bool = False) -> None:
        self.name, self.pairs_name, self.vocab_size, self.hidden_size = name, pairs_name, vocab_size, hidden_size
        self.buckets, self.mul_prev, self.mul_cur, self.cast = int(buckets), int(mul_prev), int(mul_cur), bool(cast)
        self.table: torch.Tensor | None = None
        self.pairs: torch.Tensor | None = None

    def cache_spec(self) -> StateSpec:
        return StateSpec(((1,),), (torch.int32,))

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size)), TensorSpec(self.pairs_name, (self.buckets + 1, self.hidden_size))]

    def load(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name].to(device=device, dtype=dtype).contiguous()
        self.pairs = tensors[self.pairs_name].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return 0  # a step reads only its tokens' rows

    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.hidden_size), torch.float32)
        rounded = self.cast and self.table.dtype != torch.float32  # in 32-bit the stream is its own copy
        cast = ctx.buffer("stream_cast", (ctx.num_tokens, self.hidden_size), self.table.dtype) if rounded else None
        return ops.embedding_bigram(ctx, self.table, self.pairs, cache.state[0], self.buckets, self.mul_prev, self.mul_cur, x, cast)


class OutputHead(Part):
    """``logits = h W^T`` in 32-bit. With ``tied_to`` the matrix is the embedding table and
    the checkpoint need not hold a tensor of its own (python/instinct/export.py:38-41)."""

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int, tied_to: str | None = None, suffix: str = ".weight",
                 softcap: float | None = None, scale: float | None = None) -> None:
        self.name, self.vocab_size, self.hidden_size, self.tied_to = name, vocab_size, hidden_size, tied_to
        self.suffix = suffix
        self.scale = float(scale) if scale is not None and float(scale) != 1.0 else None  # logits <- logits * scale (before any cap)
        self.softcap = float(softcap) if softcap else None  # logits <- softcap * tanh(logits / softcap)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + self.suffix, (self.vocab_size, self.hidden_size), optional=self.tied_to is not None)]

    def load(self, tensors, dtype, device) -> None:
        own = tensors.get(self.name + self.suffix)
        if own is None:
            own = tensors[self.tied_to + self.suffix]
        self.weight = own.to(device=device, dtype=dtype).contiguous()

    def share(self, embedding: TokenEmbedding) -> None:
        """Use the embedding's device tensor when both hold the same values."""
        if self.tied_to is not None and self.weight is not None and embedding.table is not None:
            if self.weight.shape == embedding.table.shape and torch.equal(self.weight, embedding.table):
                self.weight = embedding.table

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(ctx, h, self.weight, ctx.buffer("logits", (h.shape[0], self.vocab_size), torch.float32, per_token=False))
        if self.scale is not None:
            ops.scale_values(ctx, logits, self.scale)
        return ops.softcap(ctx, logits, self.softcap) if self.softcap else logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "normed_embedding", NormedEmbedding)
register_part("embedding", "sinusoid_embedding", SinusoidEmbedding)
register_part("embedding", "bigram_embedding", BigramEmbedding)
register_part("head", "linear_head", OutputHead)
