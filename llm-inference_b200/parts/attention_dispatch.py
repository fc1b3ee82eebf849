"""Chooses the attention kernel for a step.

In bfloat16, with a head size and page size the tensor-core kernels take, the step's
single-token requests (which lead the batch) go to a split-key decode kernel (mma.sync; keys
and values by TMA when head_dim is 128 and pages hold 64 rows or more, by cp.async otherwise) and
the prompt portions to the tcgen05 / TMEM kernel (head_dim 128, pages of at least 16 rows) or
else to the mma.sync prefill form. Everything else - float32, other head sizes, pages whose
size is no power of two - runs the plain kernel, which takes every shape.
``options["attention"]``: ``"auto"``, ``"plain"``, ``"flash"`` (mma.sync only) or
``"tcgen05"`` (refuse shapes the tcgen05 kernel does not take).
"""

from __future__ import annotations

import torch

from . import ops
from .context import CacheView, StepContext


def attend(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    value_head: int = -1,
    shape: ops.ScoreShape = ops.NO_SHAPE,
) -> None:
    """``shape``: a soft cap, a bias by distance and a chunk of visible keys (``ops.ScoreShape``); the plain kernel, the
    mma.sync kernels and the tcgen05 prefill kernel take it. So shaped prompt portions run on tcgen05 where its sizes hold
    (heads of 128) and the mma.sync prefill form otherwise, and decoded tokens with any shaping the cp.async split-key kernel.

    ``value_head`` >= 0: every query head's weights are applied to the values of that one kv head
    instead of its own (a mixer that mixes weights over heads asks for one such pass per kv head); the
    mma.sync kernels take it (values by cp.async from the other head's rows of the same page) and so does the
    tcgen05 prefill kernel (the value boxes' row coordinate names the other head); the TMA decode kernel does not."""
    choice = ctx.options.get("attention", "auto")
    tuned = (
        choice != "plain"
        and q.dtype == torch.bfloat16
        and ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, cache.page_size, decode=False)
    )
    if not tuned:
        if choice in ("flash", "tcgen05"):
            raise ops.KernelError("the tensor-core attention kernels do not take this shape or dtype")
        ops.paged_attention_plain(ctx, cache, q, out, q_heads, kv_heads, head_dim, scale, value_head=value_head, shape=shape)
        return
    decode_seqs = ctx.num_decode_seqs
    if decode_seqs and not ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, cache.page_size, decode=True):
        decode_seqs = 0  # more than 16 query heads per kv head: the prefill form handles one-token runs too
    if decode_seqs:
        reach = ctx.max_kv_len if not cache.window else min(ctx.max_kv_len, cache.window + 64)
        if shape.chunk:
            reach = min(reach, shape.chunk)  # a decoded token sees its own chunk at most
        tma = value_head < 0 and not shape and ops.decode_uses_tma(ctx, decode_seqs, q_heads, kv_heads, head_dim, cache.page_size)
        splits = int(ctx.options.get("decode_splits", 0)) or ops.decode_splits(decode_seqs, kv_heads, reach, tma, ops.sm_count(ctx))
        ops.paged_flash_attention(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=0, num_seqs=decode_seqs, decode=True, max_q_len=1, splits=splits, value_head=value_head, shape=shape,
        )
    if ctx.num_seqs > decode_seqs and (shape.bias is None or shape.bias_peak is not None) and choice in ("auto", "tcgen05") and ops.prefill_tcgen05_supported(
        ctx, q_heads, kv_heads, head_dim, cache.page_size, ctx.max_kv_len
    ):
        ops.paged_prefill_attention_tcgen05(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=decode_seqs, num_seqs=ctx.num_seqs - decode_seqs, max_q_len=ctx.max_q_len, value_head=value_head, shape=shape,
        )
    elif ctx.num_seqs > decode_seqs:
        if choice == "tcgen05":
            raise ops.KernelError("the tcgen05 attention kernel does not take this shape")
        ops.paged_flash_attention(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=decode_seqs, num_seqs=ctx.num_seqs - decode_seqs, decode=False, max_q_len=ctx.max_q_len, value_head=value_head,
            shape=shape,
        )


def attend_value_planes(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    planes: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
) -> None:
    """``planes[c]`` = every query head's weights applied to the values of kv head ``c``, for every ``c``. A step of
    decoded tokens only runs all passes as one launch of the split-key kernel (its grid counts pairs of value head and
    kv head): such steps are bound by launches and by the latency of one pass, not by the keys read. Other steps run
    one pass per kv head through ``attend``."""
    choice = ctx.options.get("attention", "auto")
    decode_only = ctx.num_decode_seqs == ctx.num_seqs and ctx.num_seqs == ctx.num_tokens
    if (
        decode_only
        and kv_heads > 1
        and choice != "plain"
        and q.dtype == torch.bfloat16
        and ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, cache.page_size, decode=True)
        and ctx.options.get("value_planes", "auto") != "passes"
    ):
        reach = ctx.max_kv_len if not cache.window else min(ctx.max_kv_len, cache.window + 64)
        splits = int(ctx.options.get("decode_splits", 0)) or ops.decode_splits(ctx.num_seqs, kv_heads * kv_heads, reach, False, ops.sm_count(ctx))
        ops.paged_flash_attention(
            ctx, cache, q, planes, q_heads, kv_heads, head_dim, scale,
            first_seq=0, num_seqs=ctx.num_seqs, decode=True, max_q_len=1, splits=splits, value_head=ops.EVERY_VALUE_HEAD,
        )
        return
    for c in range(kv_heads):
        attend(ctx, cache, q, planes[c], q_heads, kv_heads, head_dim, scale, value_head=c)


def attend_latent(
    ctx: StepContext,
    cache: CacheView,
    q_lat: torch.Tensor,
    q_rot: torch.Tensor,
    sink: torch.Tensor | None,
    gate: torch.Tensor | None,
    out: torch.Tensor,
    heads: int,
    rank: int,
    rot_dim: int,
    scale: float,
) -> None:
    """Attention over cached latents (parts/latent_attention.py). bfloat16 with a shape the
    tensor-core kernel takes: the step's single-token requests (which lead the batch) in one
    launch whose blocks cut every request's keys into pieces, merged by a second kernel; the
    prompt portions in another, one block per 64 (token, head) rows. float32 and every other
    shape: the plain kernel. ``options["attention"]``: ``"plain"`` forces the plain kernel,
    ``"flash"`` refuses what the tensor-core kernel does not take; ``options["latent_pieces"]``
    forces the number of pieces."""
    choice = ctx.options.get("attention", "auto")
    tuned = (
        choice != "plain" and q_lat.dtype == torch.bfloat16 and not cache.window
        and ops.latent_attention_mma_supported(ctx, heads, rank, rot_dim, cache.page_size)
    )
    if not tuned:
        if choice == "flash":
            raise ops.KernelError("the tensor-core latent attention kernel does not take this shape or dtype")
        ops.latent_attention_plain(ctx, cache, q_lat, q_rot, sink, gate, out, heads, rank, rot_dim, scale)
        return
    decode_seqs = ctx.num_decode_seqs
    if decode_seqs:
        pieces = int(ctx.options.get("latent_pieces", 0)) or ops.latent_attention_pieces(decode_seqs, heads, ctx.max_kv_len, ops.sm_count(ctx))
        ops.latent_attention_mma(ctx, cache, q_lat, q_rot, sink, gate, out, heads, rank, rot_dim, scale,
                                 first_seq=0, num_seqs=decode_seqs, max_q_len=1, pieces=pieces)
    if ctx.num_seqs > decode_seqs:
        ops.latent_attention_mma(ctx, cache, q_lat, q_rot, sink, gate, out, heads, rank, rot_dim, scale,
                                 first_seq=decode_seqs, num_seqs=ctx.num_seqs - decode_seqs, max_q_len=ctx.max_q_len)
