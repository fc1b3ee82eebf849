"""Tensor-level calls into the kernel library (and the library matrix product).

Each function checks shapes and strides, then launches on the current CUDA stream. Matrix
products in bfloat16 go to the vendor library through ``torch.mm``, as the reference sends
its linear layers to cuBLASLt (cuda/execution_context.cu:95-110); in float32 they use this
engine's own FMA kernel so that nothing runs in a reduced-precision matrix mode.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_int64
from dataclasses import dataclass
from typing import Any

import torch

from ..csrc.library import KernelError, dtype_code, ptr
from .context import CacheView, StepContext


@dataclass
class FoldedRows:
    """A normalised residual stream that nobody has materialised: ``xn`` is the stream times the
    norm's scale (bfloat16) and ``ss`` holds ``parts`` rows of partial sums of squares from which
    a consuming matrix product takes each token's 1 / rms and applies it to its outputs (the
    factor commutes with the product). ``x`` is the stream itself, already up to date, and
    ``norm`` the norm part whose scale went into ``xn``; whoever cannot take the folded form
    runs that norm on ``x`` instead (``materialise``)."""

    xn: torch.Tensor
    ss: torch.Tensor
    parts: int
    x: torch.Tensor
    norm: Any

    def materialise(self, ctx: StepContext) -> torch.Tensor:
        return self.norm.forward(ctx, self.x, None)


@dataclass
class ResidualSink:
    """What a mixer or feed-forward needs to add its output into the residual stream by itself: the
    stream and the norm part that follows (its scale is folded into the next operand)."""

    x: torch.Tensor
    norm: Any


def fold_enabled(ctx: StepContext) -> bool:
    """With ``options["fold_norms"]`` norms are folded into the products around them in bfloat16
    steps of up to 16 tokens, where the engine's own weight-streaming products run. Off by
    default: measured on one B200 in alternation (Qwen2.5-1.5B sizes, 8 requests of 2,048 keys)
    the step has 200 launches instead of 255 and takes 1.293 ms instead of 1.284 ms; with the
    folded products' extra work (partial sums of squares, 1 / rms) left out altogether it takes
    1.263 ms, so 1.6 % is all there is to gain: the norm kernels are hidden behind the products
    that follow them, which fetch their weights while the norm runs."""
    return (
        ctx.dtype == torch.bfloat16 and 0 < ctx.num_tokens <= 16 and bool(ctx.options.get("fold_norms", False))
        and ctx.options.get("gemm", "auto") != "library"
    )


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


_MM_OUT_DTYPE: bool | None = None


def _mm_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """bf16 x bf16 -> fp32 through the library, accumulating and storing in 32-bit."""
    global _MM_OUT_DTYPE
    if _MM_OUT_DTYPE is None:
        try:
            a = torch.zeros(8, 16, dtype=torch.bfloat16, device=x.device)
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _MM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    if _MM_OUT_DTYPE:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        out.copy_(torch.mm(x, weight.t()))


def linear(
    ctx: StepContext,
    x: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    bias: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out = x @ weight.T (+ bias)``; ``weight`` is ``[out_features, in_features]``. ``x`` may be
    :class:`FoldedRows` (bias-free products only): the product then applies the norm's 1 / rms."""
    if isinstance(x, FoldedRows):
        folded = x
        m, k = folded.xn.shape
        kernel = None
        if bias is None and fold_enabled(ctx) and weight.shape[1] == k and tuple(out.shape) == (m, weight.shape[0]):
            epilogue = 1 if out.dtype == torch.float32 else 0
            kernel = _small_gemm_kernel(ctx, m, weight.shape[0], k, epilogue)
        if kernel is None:
            return linear(ctx, folded.materialise(ctx), weight, out, bias)
        _small_gemm(ctx, kernel, folded.xn, weight, out, epilogue, scale=folded)
        return out
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or tuple(out.shape) != (m, n):  # the message is built only when needed: this runs per product
        _need(weight.shape[1] == k, f"linear: x is [{m},{k}] but weight is {list(weight.shape)}")
        _need(False, f"linear: out is {list(out.shape)}, expected [{m},{n}]")
    _need(x.is_contiguous() and weight.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
    if m == 0:
        return out
    if x.dtype == torch.float32:
        _need(weight.dtype == torch.float32 and out.dtype == torch.float32, "linear: float32 path needs float32 operands")
        _need(bias is None or bias.dtype == torch.float32, "linear: bias must be float32")
        ctx.lib.call(
            "b200_gemm_f32", ptr(x), ptr(weight), ptr(bias), ptr(out), c_int(m), c_int(n), c_int(k),
            c_int(k), c_int(k), c_int(n), ctx.stream,
        )
        return out
    _need(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16, "linear: bfloat16 path needs bfloat16 operands")
    if bias is None:
        epilogue = 1 if out.dtype == torch.float32 else 0
        kernel = _small_gemm_kernel(ctx, m, n, k, epilogue)
        if kernel is not None:
            _small_gemm(ctx, kernel, x, weight, out, epilogue)
            return out
    if out.dtype == torch.float32:
        _need(bias is None, "linear: no bias on the 32-bit output path")
        _mm_f32_out(x, weight, out)
    elif bias is not None:
        torch.addmm(bias, x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out=out)
    return out


def _small_gemm_kernel(ctx: StepContext, m: int, n: int, k: int, epilogue: int) -> str | None:
    """Which of this engine's own weight-streaming products takes the shape, if any.

    ``options["gemm"]``: ``"auto"`` (tcgen05 kernel, else the mma.sync one), ``"tcgen05"``,
    ``"skinny"``, or ``"library"`` (always the vendor library)."""
    choice = ctx.options.get("gemm", "auto")
    if choice == "library":
        return None
    key = (m, n, k, epilogue, choice)
    if key not in _GEMM_CHOICES:
        if len(_GEMM_CHOICES) > 4096:
            _GEMM_CHOICES.clear()
        _GEMM_CHOICES[key] = _choose_small_gemm(ctx, m, n, k, epilogue, choice)
    return _GEMM_CHOICES[key]


_GEMM_CHOICES: dict[tuple, str | None] = {}  # the rule below is a pure function of its key


def _choose_small_gemm(ctx: StepContext, m: int, n: int, k: int, epilogue: int, choice: str) -> str | None:
    stream = bool(ctx.lib.lib.b200_stream_gemm_supported(m, n, k, epilogue))
    skinny = bool(ctx.lib.lib.b200_skinny_gemm_supported(m, n, k, epilogue))
    if choice == "tcgen05":
        return "stream" if stream else None
    if choice == "skinny":
        return "skinny" if skinny else None
    # auto, from measurements on a B200 (graph-timed, weights from HBM, 1.5B shape): for up to
    # 16 rows the mma.sync kernel wins on small matrices, whose time is all launch and ramp
    # (3.0 vs 5.1 us for the 6 MB q/k/v product), and the tcgen05 kernel on large ones (down
    # 11.4 vs 14.1 us, output head 74 vs 107 us; vendor library 16.8 and 78 us). With more
    # rows the vendor library's tiles are faster on products with a short inner dimension
    # (64 rows, q/k/v: 4.6 vs 7.7 us; output head 84 vs 89 us), and it keeps those; products with
    # a long one (down: K = 8960 or 18944), which the tcgen05 kernel splits over a cluster,
    # stay here up to 64 rows (32 rows 10.2 vs 13.1 us, 64 rows 11.8 vs 13.2 us; at 128 rows
    # 15.5 vs 13.3 us the library wins again).
    # Inside a decode step the comparison shifts towards the engine's own kernels, which overlap
    # their neighbours (programmatic dependent launch) where the library's do not: with all
    # products on the tcgen05 kernel a step of 32 requests takes 1.85 ms against 1.90 ms, one of
    # 64 requests 2.57 ms against 2.25 ms. So up to 32 rows everything stays here.
    # At the 7B and 14B shapes the same rule holds: steps of 32 requests 3.76 against 4.07 ms
    # (7B) and 8.06 against 8.30 ms (14B) with the library for every product above 16 rows;
    # at 64 rows only the down products (K of 8960 and more) are worth keeping (14B: 11.66 ms
    # against 11.93 ms with q/k/v and o, K = 5120, kept too).
    if m > 16:
        return "stream" if stream and (m <= 32 or (m <= 64 and k >= 8192)) else None
    weight_bytes = 2 * n * k
    if skinny and weight_bytes < (16 << 20):
        return "skinny"
    return "stream" if stream else ("skinny" if skinny else None)


def linear_swiglu(ctx: StepContext, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """``out = silu(gate) * up`` of ``x @ weight.T`` with interleaved gate/up rows, in one
    kernel. Returns False (doing nothing) when no fused kernel takes the shape."""
    folded = x if isinstance(x, FoldedRows) else None
    if folded is not None:
        x = folded.xn
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype != torch.bfloat16 or m == 0:
        return False
    kernel = _small_gemm_kernel(ctx, m, n, k, 2)
    if kernel is None or (folded is not None and not fold_enabled(ctx)):
        return False
    _need(tuple(out.shape) == (m, n // 2) and out.is_contiguous() and x.is_contiguous(), "linear_swiglu: bad operands")
    _small_gemm(ctx, kernel, x, weight, out, 2, scale=folded)
    return True


def linear_into_residual(ctx: StepContext, a: torch.Tensor, weight: torch.Tensor, sink: ResidualSink) -> FoldedRows | None:
    """``sink.x += a @ weight.T`` inside the product's epilogue, which also writes the stream times
    the scale of the norm that follows and its partial sums of squares: returns them as
    :class:`FoldedRows`, or None (doing nothing) when the step, the norm or the shape does not
    allow it and the caller has to produce the branch output as a tensor."""
    m, k = a.shape
    n = weight.shape[0]
    norm = sink.norm
    weight_of_norm = getattr(norm, "weight", None)
    if not fold_enabled(ctx) or not getattr(norm, "foldable", False) or weight_of_norm is None:
        return None
    if a.dtype != torch.bfloat16 or tuple(sink.x.shape) != (m, n) or sink.x.dtype != torch.float32:
        return None
    kernel = _small_gemm_kernel(ctx, m, n, k, 0)
    if kernel is None:
        return None
    parts = int(getattr(ctx.lib.lib, f"b200_{kernel}_gemm_fold_parts")(*((m, n, k) if kernel == "stream" else (n, k))))
    xn = ctx.buffer("fold_xn", (m, n), torch.bfloat16)
    ss = ctx.buffer(f"fold_ss_{n}_{k}", (parts, 16), torch.float32, per_token=False)
    _small_gemm(ctx, kernel, a, weight, None, 0, sink=(sink.x, weight_of_norm, xn, ss))
    return FoldedRows(xn=xn, ss=ss, parts=parts, x=sink.x, norm=norm)


_SKINNY_SCRATCH: dict[tuple[int, int, int], tuple[int, int]] = {}  # (m, n, k) -> (floats, counters)


def _small_gemm(
    ctx: StepContext, kernel: str, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None, epilogue: int,
    scale: FoldedRows | None = None, sink: tuple | None = None,
) -> None:
    """Launch a weight-streaming product. The mma.sync kernel keeps the partial sums of blocks
    that share rows of the weight matrix, and their arrival counters, in the step's workspace;
    the tcgen05 kernel reduces inside its clusters and needs none. ``scale``: the operand is a
    folded norm's ``xn`` and the outputs take the tokens' 1 / rms; ``sink``: (stream, next norm's
    scale, xn, ss) for the residual epilogue (see NormFold in csrc/kernels/common.cuh)."""
    from ctypes import byref

    m, k = x.shape
    n = weight.shape[0]
    head = [ptr(weight), ptr(x), ptr(out), c_int(m), c_int(n), c_int(k), c_int(epilogue)]
    folding = scale is not None or sink is not None
    if folding:
        width = k if scale is not None else 0
        eps = float(scale.norm.eps) if scale is not None else 0.0
        fold = [
            ptr(scale.ss if scale is not None else None), c_int(scale.parts if scale is not None else 0), c_int(width),
            c_float(eps),
        ] + ([ptr(t) for t in sink] if sink is not None else [ptr(None)] * 4)
    else:
        fold = []
    suffix = "_fold" if folding else ""
    if kernel == "stream":
        ctx.lib.call("b200_stream_gemm" + suffix, *head, ptr(ctx.err), *fold, ctx.stream)
        return
    need = _SKINNY_SCRATCH.get((m, n, k))
    if need is None:
        floats, counters = c_int64(0), c_int(0)
        ctx.lib.lib.b200_skinny_gemm_scratch(m, n, k, byref(floats), byref(counters))
        need = _SKINNY_SCRATCH[(m, n, k)] = (floats.value, counters.value)
    floats, counters = need
    scratch = counter_buf = None
    if floats:
        scratch = ctx.buffer("gemm_partials", (floats,), torch.float32, per_token=False)
        counter_buf = ctx.workspace.zeros("gemm_counters", max(counters, 4096), torch.int32)
    ctx.lib.call(
        "b200_skinny_gemm" + suffix, *head, ptr(scratch), c_int64(floats), ptr(counter_buf),
        c_int(counter_buf.numel() if counter_buf is not None else 0), *fold, ctx.stream,
    )


def embedding_gather(ctx: StepContext, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, hidden) and out.dtype == torch.float32, "embedding: bad output")
    ctx.lib.call(
        "b200_embedding_gather", ptr(table), c_int(dtype_code(table.dtype)), ptr(ctx.token_ids), ptr(out),
        c_int(ctx.num_tokens), c_int(hidden), c_int(vocab), ptr(ctx.err), ctx.stream,
    )
    return out


def rmsnorm(
    ctx: StepContext,
    x: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: torch.Tensor | None = None,
) -> torch.Tensor:
    hidden = x.shape[1]
    num_rows = x.shape[0] if rows is None else rows.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (hidden,), "rmsnorm: weight must be float32 [hidden]")
    _need(tuple(out.shape) == (num_rows, hidden) and out.is_contiguous(), "rmsnorm: bad output shape")
    _need(delta is None or (delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous()), "rmsnorm: bad delta")
    ctx.lib.call(
        "b200_rmsnorm", ptr(x), ptr(delta), ptr(weight), ptr(out), ptr(rows), c_int(num_rows), c_int(hidden),
        c_float(eps), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def silu_mul(ctx: StepContext, gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    tokens, twice = gate_up.shape
    inter = twice // 2
    _need(twice == 2 * inter and tuple(out.shape) == (tokens, inter), "silu_mul: bad shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype, "silu_mul: bad operands")
    ctx.lib.call(
        "b200_silu_mul", ptr(gate_up), ptr(out), c_int(tokens), c_int(inter), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def rope_kv_write(
    ctx: StepContext,
    cache: CacheView,
    qkv: torch.Tensor,
    bias: torch.Tensor | None,
    inv_freq: torch.Tensor,
    q_out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
) -> torch.Tensor:
    tokens = qkv.shape[0]
    width = (q_heads + 2 * kv_heads) * head_dim
    rot = 2 * inv_freq.numel()
    _need(tuple(qkv.shape) == (tokens, width) and qkv.is_contiguous(), "rope_kv_write: bad qkv")
    _need(tuple(q_out.shape) == (tokens, q_heads * head_dim) and q_out.is_contiguous(), "rope_kv_write: bad q_out")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "rope_kv_write: bias must be float32 [width]")
    _need(inv_freq.dtype == torch.float32, "rope_kv_write: inverse frequencies must be float32")
    _need(cache.keys.dtype == qkv.dtype and cache.values.dtype == qkv.dtype, "rope_kv_write: cache dtype differs")
    ctx.lib.call(
        "b200_rope_kv_write", ptr(qkv), ptr(bias), ptr(inv_freq), ptr(ctx.positions), ptr(ctx.token_seq),
        ptr(getattr(ctx, "seq_kv_len", None)), ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages),
        ptr(cache.keys), ptr(cache.values), ptr(q_out), c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(rot),
        c_int(cache.page_size), c_int(1 if cache.writes else 0), c_int(dtype_code(qkv.dtype)), ptr(ctx.err), ctx.stream,
    )
    return q_out


@dataclass(frozen=True)
class ScoreShape:
    """What an attention kernel does to a scaled score before the softmax, beyond masking the future: ``softcap``
    (``s <- softcap * tanh(s / softcap)``), ``bias`` (float32 ``[q_heads, reach + 1]`` on the device: the row of the
    query head at ``min(position - key, reach)`` is added after the cap) and ``chunk`` (a query sees only keys from
    ``floor(position / chunk) * chunk`` on). The plain kernel, the ``mma.sync`` kernels and the tcgen05 prefill
    kernel take it (the last wants ``bias_peak`` beside a bias)."""

    softcap: float = 0.0
    bias: torch.Tensor | None = None
    chunk: int = 0
    bias_peak: torch.Tensor | None = None  # float32 [q_heads]: each row's largest entry (the tcgen05 kernel bounds exponents with it)

    def __bool__(self) -> bool:
        return bool(self.softcap > 0.0 or self.bias is not None or self.chunk > 0)

    def arguments(self, q_heads: int) -> list:
        if self.bias is not None:
            _need(self.bias.dtype == torch.float32 and self.bias.dim() == 2 and self.bias.shape[0] == q_heads and self.bias.is_contiguous(),
                  "attention: the bias by distance is float32 [q_heads, reach + 1]")
        reach = self.bias.shape[1] - 1 if self.bias is not None else 0
        return [c_float(self.softcap), ptr(self.bias), c_int(reach), c_int(self.chunk)]


NO_SHAPE = ScoreShape()


def paged_attention_plain(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_token: int = 0,
    num_tokens: int | None = None,
    value_head: int = -1,
    shape: ScoreShape = NO_SHAPE,
) -> torch.Tensor:
    """Attention of rows ``first_token .. first_token + num_tokens`` of the step over the cache. With
    ``value_head`` >= 0 every query head's weights are applied to the values of that kv head."""
    tokens = ctx.num_tokens - first_token if num_tokens is None else num_tokens
    if tokens <= 0:
        return out
    _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype, "attention: bad operands")
    _need(cache.keys.dtype == q.dtype, "attention: cache dtype differs from the queries'")
    row_bytes = q_heads * head_dim * q.element_size()
    ctx.lib.call(
        "b200_paged_attention_plain",
        ptr(q) if first_token == 0 else _offset(q, first_token * row_bytes),
        ptr(cache.keys), ptr(cache.values),
        _offset(ctx.positions, first_token * 4), _offset(ctx.token_seq, first_token * 4),
        ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages),
        ptr(out) if first_token == 0 else _offset(out, first_token * row_bytes),
        c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size),
        c_int(cache.window), c_float(scale), c_int(value_head), *shape.arguments(q_heads), c_int(dtype_code(q.dtype)), ptr(ctx.err),
        ctx.stream,
    )
    return out


NUM_SMS = 148  # a B200; only what `decode_splits` assumes when no device is asked (tests on the CPU)
DECODE_STAGES = 3  # pieces in flight per warp of the TMA decode kernel
MAX_DECODE_SPLITS = 64  # what the merge kernel takes in one round trip


def flash_attention_supported(ctx: StepContext, q_heads: int, kv_heads: int, head_dim: int, page_size: int, decode: bool) -> bool:
    return bool(ctx.lib.lib.b200_flash_attention_supported(q_heads, kv_heads, head_dim, page_size, 1 if decode else 0))


def decode_uses_tma(ctx: StepContext, num_seqs: int, q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether a decode step's attention runs the kernel whose warps load by TMA: whenever
    the shape suits it (head_dim 128, pages of 64 rows or more), unless
    ``options["decode_loader"]`` says ``"cp_async"``."""
    loader = ctx.options.get("decode_loader", "auto")
    if loader == "cp_async" or not ctx.lib.lib.b200_decode_attention_tma_supported(q_heads, kv_heads, head_dim, page_size):
        _need(loader != "tma", "the TMA decode kernel does not take this shape")
        return False
    return True


def sm_count(ctx: StepContext) -> int:
    """SMs of the device the step runs on (the library asks the device once)."""
    return int(ctx.lib.lib.b200_sm_count())


EVERY_VALUE_HEAD = -2  # `value_head` of paged_flash_attention: the passes of all kv heads in one launch


def decode_splits(num_seqs: int, kv_heads: int, max_kv_len: int, tma: bool = False, num_sms: int = NUM_SMS) -> int:
    """How many blocks cut each request's keys in a decode step: at least one 64-key tile
    each, and few enough that the merge of their partial results stays cheap. The cp.async
    kernel (three blocks per SM) wants about two waves of blocks. The TMA kernel (rings three
    deep, two blocks per SM) wants all its blocks resident at once: measured on a B200 at
    2,048 keys, 64 requests x 2 kv heads take 26 us in 2 splits and 35 us in 6, and 64 x 8
    take 82 us unsplit. Normally at most 16 splits (14 or fewer for 10 to 24 pairs of up to 4,096 keys, see below). Very few pairs with many keys go up to 64
    while every split keeps four tiles: one request of the 1.5B shape with 30,000 keys is 32
    blocks for 148 SMs in 16 splits (1.94 ms per step) and 128 blocks in 64 (1.35 ms); 8,192
    keys: 1.36 -> 1.15 ms. With 8 such requests 18 splits were no faster than 16 (2.26 vs
    2.17 ms): the wider merge costs what the two extra splits gain."""
    tiles = max(1, (max_kv_len + 63) // 64)
    pairs = max(1, num_seqs * kv_heads)
    want = (2 if tma else 6) * num_sms // pairs  # rounded down: one block too many would start another wave
    if want >= 32:
        most = max(16, min(MAX_DECODE_SPLITS, tiles // 4))
    elif tma and want >= 12 and tiles <= 64:
        # 10 to 24 pairs of up to 4,096 keys: the blocks share their SMs with the kernels around them in the chain, and
        # about 1.5 blocks per SM leave those room to move in early. Measured at 2,100-2,300 keys,
        # 1.5B shape, ms per step with 16 (or the 2-per-SM count) -> with this rule: batch 5 1.125 ->
        # 1.115, 6 1.131 -> 1.121, 7 1.137 -> 1.131, 8 1.153 -> 1.132 (1,200 keys 1.112 -> 1.090,
        # 3,800 keys 1.217 -> 1.199), 9 1.273 -> 1.268, 10 1.282 -> 1.264, 12 unchanged; 7B shape,
        # batch 4: 2.722 -> 2.686. With more pairs (batch 16: 9 splits, 32: 4, 64: 2) two per SM
        # stay the best, with fewer (batch 4: 16 or 20 splits) the blocks do not fill the SMs; with
        # more keys the attention wants the SMs for itself (batch 8, 8,192 keys: 1.353 ms with 16
        # splits, 1.378 with 13; 30,000 keys: 2.097 and 2.136).
        most = min(14, (3 * num_sms // 2) // pairs)
    else:
        most = 16
    return max(1, min(tiles, most, want))


def paged_flash_attention(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_seq: int,
    num_seqs: int,
    decode: bool,
    max_q_len: int,
    splits: int = 1,
    value_head: int = -1,
    shape: ScoreShape = NO_SHAPE,
) -> torch.Tensor:
    """Tensor-core attention for requests ``first_seq .. first_seq + num_seqs`` of the step. With ``value_head`` >= 0
    every query head's weights are applied to the values of that kv head (the cp.async kernel only). With
    ``EVERY_VALUE_HEAD`` (a step of decoded tokens only) one launch runs that pass for every kv head and ``out`` is
    ``[kv_heads, tokens, q_heads * head_dim]``."""
    if num_seqs <= 0:
        return out
    planes = 1
    if value_head == EVERY_VALUE_HEAD:
        _need(decode and num_seqs == ctx.num_tokens, "flash attention: every value head in one launch is for steps of decoded tokens only")
        _need(out.shape[0] == kv_heads and out.shape[1] == num_seqs, "flash attention: one plane of results per value head")
        planes = kv_heads
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.keys.dtype == torch.bfloat16, "flash attention is bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous(), "flash attention: operands must be contiguous")
    _need(not decode or first_seq == 0, "flash attention: decoded tokens must lead the batch")
    scratch = None
    # The cp.async kernel merges its splits on chip by a thread-block cluster when there are
    # very few (request, kv head) pairs, otherwise through scratch by a second small kernel:
    # measured on a B200, the cluster form wins at batch 1 (1.48 vs 1.66 ms per step of the
    # 1.5B shape) and loses from batch 8 on (1.72 vs 1.65 ms), where clusters of 16 blocks are
    # slow to place. The TMA kernel always goes through scratch unless told otherwise: at
    # batch 1 both forms take 1.10 ms per step (the cp.async kernel 1.15), at batch 2 scratch
    # 1.10 and the cluster 1.12, from batch 4 on the cluster loses.
    use_tma = decode and value_head == -1 and not shape and decode_uses_tma(ctx, num_seqs, q_heads, kv_heads, head_dim, cache.page_size)
    merge = ctx.options.get("attention_merge", "auto")
    if merge == "auto":
        merge = "cluster" if num_seqs * kv_heads * planes <= 4 and not use_tma else "scratch"
    if decode and splits > 1 and (splits > 16 or merge == "scratch"):
        scratch = ctx.buffer("attention_partials", (planes * num_seqs * q_heads * splits * (head_dim + 2),), torch.float32, per_token=False)
    # Keys and values by TMA into per-warp rings where the shape allows; "cp_async" keeps the
    # block-wide cp.async tiles.
    if use_tma:
        ctx.lib.call(
            "b200_paged_decode_attention_tma", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
            ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(num_seqs), c_int(cache.max_pages),
            c_int(cache.num_pages), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size),
            c_int(cache.window), c_float(scale), c_int(splits), c_int(int(ctx.options.get("decode_stages", DECODE_STAGES))),
            ptr(scratch), ptr(ctx.err), ctx.stream,
        )
        if scratch is not None:
            ctx.lib.calls += 1  # the merge kernel is a launch of its own
        return out
    ctx.lib.call(
        "b200_paged_flash_attention", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
        ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(first_seq), c_int(num_seqs),
        c_int(num_seqs if decode else ctx.num_tokens), c_int(max_q_len), c_int(cache.max_pages), c_int(cache.num_pages),
        c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size), c_int(cache.window), c_float(scale),
        c_int(1 if decode else 0), c_int(splits), c_int(value_head), *shape.arguments(q_heads), ptr(scratch), ptr(ctx.err), ctx.stream,
    )
    if scratch is not None:
        ctx.lib.calls += 1  # the merge kernel is a launch of its own
    return out


def prefill_tcgen05_supported(ctx: StepContext, q_heads: int, kv_heads: int, head_dim: int, page_size: int, max_kv_len: int) -> bool:
    return bool(ctx.lib.lib.b200_flash_prefill_tcgen05_supported(q_heads, kv_heads, head_dim, page_size, max_kv_len))


def paged_prefill_attention_tcgen05(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_seq: int,
    num_seqs: int,
    max_q_len: int,
    value_head: int = -1,
    shape: ScoreShape = NO_SHAPE,
) -> torch.Tensor:
    """Prompt-portion attention on tcgen05 / TMEM for requests ``first_seq ..`` of the step. ``value_head`` >= 0:
    every query head's weights are applied to the values of that kv head. ``shape``: a soft cap, a bias by distance
    (with its rows' maxima) and chunks of visible keys."""
    _need(shape.bias is None or (shape.bias_peak is not None and shape.bias_peak.dtype == torch.float32 and shape.bias_peak.numel() == q_heads),
          "tcgen05 attention: a bias by distance comes with its rows' maxima, float32 [q_heads]")
    reach = shape.arguments(q_heads)[2]
    if num_seqs <= 0:
        return out
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.keys.dtype == torch.bfloat16, "tcgen05 attention is bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and cache.keys.is_contiguous() and cache.values.is_contiguous(), "tcgen05 attention: operands must be contiguous")
    ctx.lib.call(
        "b200_flash_prefill_tcgen05", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
        ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(first_seq), c_int(num_seqs), c_int(max_q_len),
        c_int(ctx.max_kv_len), c_int(cache.max_pages), c_int(cache.num_pages), c_int(q_heads), c_int(kv_heads),
        c_int(head_dim), c_int(cache.page_size), c_int(cache.window), c_float(scale), c_int(value_head), c_float(shape.softcap), ptr(shape.bias), ptr(shape.bias_peak), reach,
        c_int(shape.chunk), ptr(ctx.err), ctx.stream,
    )
    return out


def _offset(tensor: torch.Tensor, nbytes: int) -> int:
    return tensor.data_ptr() + nbytes


def argmax_rows(lib, logits: torch.Tensor, out: torch.Tensor, row_index: torch.Tensor | None, rows: int, stream) -> None:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "argmax: logits must be float32 rows")
    lib.call(
        "b200_argmax_rows", ptr(logits), c_int(rows), c_int(logits.shape[1]), c_int64(logits.stride(0)),
        ptr(row_index), ptr(out), ptr(None), ptr(None), stream,
    )


# -- norms on a branch's output, scaled embedding, PolyNorm --------------------------------------------


def embedding_scaled(ctx: StepContext, table: torch.Tensor, scale: float, out: torch.Tensor, cast: torch.Tensor | None) -> torch.Tensor:
    """``out[t] = table[token[t]] * scale`` in 32-bit; ``cast`` also receives it in the table's dtype."""
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, hidden) and out.dtype == torch.float32, "embedding: bad output")
    _need(cast is None or (cast.dtype == table.dtype and cast.shape == out.shape), "embedding: bad cast buffer")
    ctx.lib.call(
        "b200_embedding_scaled", ptr(table), ptr(ctx.token_ids), c_float(scale), ptr(out), ptr(cast), c_int(ctx.num_tokens),
        c_int(hidden), c_int(vocab), c_int(dtype_code(table.dtype)), ptr(ctx.err), ctx.stream,
    )
    return out


def branch_norm_add(
    ctx: StepContext,
    x_in: torch.Tensor,
    branch: torch.Tensor,
    weight: torch.Tensor,
    scale: torch.Tensor | None,
    mult: float,
    groups: int,
    eps: float,
    x_out: torch.Tensor,
    *,
    copy_in: torch.Tensor | None = None,
    history: torch.Tensor | None = None,
    mix: torch.Tensor | None = None,
    mixed: torch.Tensor | None = None,
    cast: torch.Tensor | None = None,
) -> None:
    """``x_out = x_in + mult * scale * weight * branch / rms_groups(branch)``. With ``mix`` (``n`` weights) and
    ``history`` (``[>= n, rows, hidden]``, whose slice ``n - 1`` is ``x_out``) also
    ``mixed = sum_j mix[j] * history[j]``; ``cast`` receives the row that travels on (``mixed`` if there
    is a mix, else ``x_out``) in the compute dtype; ``copy_in`` receives ``x_in`` unchanged."""
    rows, hidden = x_in.shape
    _need(x_in.dtype == torch.float32 and x_out.dtype == torch.float32 and x_in.is_contiguous() and x_out.is_contiguous(), "branch_norm_add: the stream is contiguous float32")
    _need(tuple(branch.shape) == (rows, hidden) and branch.is_contiguous(), "branch_norm_add: bad branch output")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "branch_norm_add: weight must be float32 [hidden]")
    _need(scale is None or (scale.dtype == torch.float32 and scale.numel() == hidden), "branch_norm_add: scale must be float32 [hidden]")
    _need(cast is None or (cast.dtype == branch.dtype and cast.shape == x_in.shape), "branch_norm_add: bad cast buffer")
    count = 0
    stride = 0
    if mix is not None:
        count = mix.numel()
        _need(mix.dtype == torch.float32 and mixed is not None and mixed.dtype == torch.float32 and mixed.shape == x_in.shape, "branch_norm_add: bad mix")
        _need(history is not None and history.dtype == torch.float32 and history.is_contiguous() and history.shape[0] >= count, "branch_norm_add: bad history")
        _need(history[count - 1].data_ptr() == x_out.data_ptr(), "branch_norm_add: the newest history entry is the output")
        stride = history.stride(0)
    ctx.lib.call(
        "b200_branch_norm_add", ptr(x_in), ptr(branch), ptr(weight), ptr(scale), c_float(mult), c_int(rows), c_int(hidden),
        c_int(groups), c_float(eps), ptr(x_out), ptr(copy_in), ptr(history), c_int64(stride), ptr(mix), c_int(count),
        ptr(mixed), ptr(cast), c_int(dtype_code(branch.dtype)), ctx.stream,
    )


def grouped_rmsnorm(
    ctx: StepContext, x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor, rows: torch.Tensor | None = None
) -> torch.Tensor:
    hidden = x.shape[1]
    num_rows = x.shape[0] if rows is None else rows.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "grouped_rmsnorm: the stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "grouped_rmsnorm: weight must be float32 [hidden]")
    _need(tuple(out.shape) == (num_rows, hidden) and out.is_contiguous(), "grouped_rmsnorm: bad output shape")
    ctx.lib.call(
        "b200_grouped_rmsnorm", ptr(x), ptr(weight), ptr(rows), c_int(num_rows), c_int(hidden), c_int(groups), c_float(eps),
        ptr(out), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def poly_norm(ctx: StepContext, z: torch.Tensor, coefficients: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    rows, width = z.shape
    _need(z.is_contiguous() and out.is_contiguous() and out.shape == z.shape and out.dtype == z.dtype, "poly_norm: bad operands")
    _need(coefficients.dtype == torch.float32 and coefficients.numel() == 4, "poly_norm: four float32 coefficients")
    ctx.lib.call(
        "b200_poly_norm", ptr(z), ptr(coefficients), c_int(rows), c_int(width), c_float(eps), ptr(out), c_int(dtype_code(z.dtype)),
        ctx.stream,
    )
    return out


def linear_per_head(ctx: StepContext, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[h] = x[h] @ weight[h].T`` for every head: ``x`` is ``[heads, rows, k]``, ``weight``
    ``[heads, n, k]``, ``out`` ``[heads, rows, n]``; ``x`` and ``out`` may be views with any head and
    row strides (a head's slice of wider rows) as long as their last dimension is dense. bfloat16
    goes to the vendor library's batched product, float32 to this engine's FMA kernel."""
    heads, rows, k = x.shape
    n = weight.shape[1]
    _need(tuple(weight.shape) == (heads, n, k) and weight.is_contiguous(), "linear_per_head: bad weight")
    _need(tuple(out.shape) == (heads, rows, n) and x.stride(2) == 1 and out.stride(2) == 1, "linear_per_head: bad operands")
    if rows == 0:
        return out
    if x.dtype == torch.float32:
        _need(weight.dtype == torch.float32 and out.dtype == torch.float32, "linear_per_head: float32 path needs float32 operands")
        ctx.lib.call(
            "b200_gemm_f32_batched", ptr(x), ptr(weight), ptr(out), c_int(rows), c_int(n), c_int(k), c_int(x.stride(1)),
            c_int(k), c_int(out.stride(1)), c_int(heads), c_int64(x.stride(0)), c_int64(n * k), c_int64(out.stride(0)),
            ctx.stream,
        )
        return out
    _need(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "linear_per_head: bfloat16 path needs bfloat16 operands")
    torch.bmm(x, weight.transpose(1, 2), out=out)
    return out


# -- attention over cached latents ------------------------------------------------------------------------


def latent_kv_write(
    ctx: StepContext, cache: CacheView, proj: torch.Tensor, q_offset: int, kv_offset: int, heads: int, dim: int, rot_dim: int,
    rank: int, norm_weight: torch.Tensor, eps: float, inv_freq: torch.Tensor, q_rot: torch.Tensor, *, q_proj: torch.Tensor | None = None,
    halves: bool = False, magnitude: float = 1.0,
) -> None:
    """``q_proj``: the matrix that holds the queries when it is not ``proj`` itself (queries that come out of a latent of
    their own); ``halves``: number i of a rotated part pairs with i + half instead of 2i with 2i + 1; ``magnitude``
    multiplies sine and cosine."""
    tokens, ld = proj.shape
    queries = proj if q_proj is None else q_proj
    _need(queries.is_contiguous() and queries.dtype == proj.dtype and queries.shape[0] == tokens and queries.shape[1] >= q_offset + heads * (dim + rot_dim),
          "latent_kv_write: bad queries")
    _need(proj.is_contiguous() and cache.keys.dtype == proj.dtype and q_rot.dtype == proj.dtype, "latent_kv_write: bad operands")
    _need(tuple(q_rot.shape) == (tokens, heads * rot_dim) and q_rot.is_contiguous(), "latent_kv_write: bad q_rot")
    _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == rank and inv_freq.dtype == torch.float32, "latent_kv_write: bad constants")
    _need(tuple(cache.keys.shape[1:]) == (1, cache.page_size, rank + rot_dim), "latent_kv_write: the cache rows are [latent | rotated key part]")
    ctx.lib.call(
        "b200_latent_kv_write", ptr(queries), c_int(queries.shape[1]), ptr(proj), c_int(ld), c_int(q_offset), c_int(kv_offset), c_int(tokens),
        c_int(heads), c_int(dim), c_int(rot_dim), c_int(rank), ptr(norm_weight), c_float(eps), ptr(inv_freq), c_int(2 * inv_freq.numel()),
        c_int(1 if halves else 0), c_float(magnitude),
        ptr(ctx.positions), ptr(ctx.token_seq), ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages),
        ptr(cache.keys), c_int(cache.page_size), c_int(1 if cache.writes else 0), ptr(q_rot), c_int(dtype_code(proj.dtype)),
        ptr(ctx.err), ctx.stream,
    )


def latent_attention_plain(
    ctx: StepContext, cache: CacheView, q_lat: torch.Tensor, q_rot: torch.Tensor, sink: torch.Tensor | None,
    gate: torch.Tensor | None, out: torch.Tensor, heads: int, rank: int, rot_dim: int, scale: float,
) -> torch.Tensor:
    """``q_lat`` and ``out`` are ``[heads, tokens, rank]`` views (any head and token strides), ``q_rot``
    ``[tokens, heads * rot_dim]``, ``gate`` a ``[tokens, heads]`` view of logits with a dense last dimension."""
    tokens = q_rot.shape[0]
    _need(tuple(q_lat.shape) == (heads, tokens, rank) and q_lat.stride(2) == 1, "latent attention: bad q_lat")
    _need(tuple(out.shape) == (heads, tokens, rank) and out.stride(2) == 1 and out.dtype == q_lat.dtype, "latent attention: bad output")
    _need(q_rot.is_contiguous() and q_rot.dtype == q_lat.dtype and cache.keys.dtype == q_lat.dtype, "latent attention: dtypes differ")
    _need(sink is None or (sink.dtype == torch.float32 and sink.numel() == heads), "latent attention: sink must be float32 [heads]")
    _need(gate is None or (tuple(gate.shape) == (tokens, heads) and gate.stride(1) == 1 and gate.dtype == q_lat.dtype), "latent attention: bad gate")
    ctx.lib.call(
        "b200_latent_attention_plain", ptr(q_lat), c_int64(q_lat.stride(1)), c_int64(q_lat.stride(0)), ptr(q_rot), ptr(cache.keys),
        ptr(ctx.positions), ptr(ctx.token_seq), ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages), ptr(sink),
        ptr(gate), c_int64(gate.stride(0) if gate is not None else 0), ptr(out), c_int64(out.stride(1)), c_int64(out.stride(0)),
        c_int(tokens), c_int(heads), c_int(rank), c_int(rot_dim), c_int(cache.page_size), c_int(cache.window), c_float(scale),
        c_int(dtype_code(q_lat.dtype)), ptr(ctx.err), ctx.stream,
    )
    return out


def latent_attention_mma_supported(ctx: StepContext, heads: int, rank: int, rot_dim: int, page_size: int) -> bool:
    return bool(ctx.lib.lib.b200_latent_attention_mma_supported(heads, rank, rot_dim, page_size))


def latent_attention_pieces(num_seqs: int, heads: int, max_kv_len: int, num_sms: int = NUM_SMS) -> int:
    """Into how many pieces a step of single tokens cuts each request's keys: enough blocks for two
    per SM, every piece at least four tiles of 32 keys, at most 64 pieces. Measured on a B200 (12 heads,
    rows of 512 + 64, 2,048 keys): 8 requests take 56 / 36 / 31 / 38 us in 4 / 8 / 16 / 32 pieces, 64
    requests 60 / 72 / 95 us in 4 / 8 / 16."""
    rows_per_block = 16 if heads <= 16 else (32 if heads <= 32 else 64)
    blocks = max(1, num_seqs * ((heads + rows_per_block - 1) // rows_per_block))
    tiles = max(1, (max_kv_len + 31) // 32)
    return max(1, min(2 * num_sms // blocks, tiles // 4, 64))


def latent_attention_mma(
    ctx: StepContext, cache: CacheView, q_lat: torch.Tensor, q_rot: torch.Tensor, sink: torch.Tensor | None,
    gate: torch.Tensor | None, out: torch.Tensor, heads: int, rank: int, rot_dim: int, scale: float, *,
    first_seq: int, num_seqs: int, max_q_len: int, pieces: int = 1,
) -> torch.Tensor:
    """The tensor-core kernel (bfloat16) for requests ``first_seq .. first_seq + num_seqs`` of the step; operands as
    for :func:`latent_attention_plain`. With ``pieces`` > 1 every request's keys are cut and merged through scratch."""
    if num_seqs <= 0:
        return out
    tokens = q_rot.shape[0]
    _need(q_lat.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.keys.dtype == torch.bfloat16, "latent attention (tensor cores) is bfloat16 only")
    _need(tuple(q_lat.shape) == (heads, tokens, rank) and q_lat.stride(2) == 1 and tuple(out.shape) == (heads, tokens, rank) and out.stride(2) == 1, "latent attention: bad operands")
    _need(q_rot.is_contiguous() and cache.window == 0, "latent attention (tensor cores): dense rotated queries, no window")
    _need(gate is None or (tuple(gate.shape) == (tokens, heads) and gate.stride(1) == 1 and gate.dtype == torch.bfloat16), "latent attention: bad gate")
    scratch = None
    if pieces > 1:
        floats = int(ctx.lib.lib.b200_latent_attention_mma_scratch(num_seqs, max_q_len, heads, rank, pieces))
        scratch = ctx.buffer("latent_partials", (floats,), torch.float32, per_token=False)
    ctx.lib.call(
        "b200_latent_attention_mma", ptr(q_lat), c_int64(q_lat.stride(1)), c_int64(q_lat.stride(0)), ptr(q_rot), ptr(cache.keys),
        ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages), c_int(cache.page_size), ptr(ctx.seq_q_start),
        ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(first_seq), c_int(num_seqs), c_int(max_q_len), ptr(sink), ptr(gate),
        c_int64(gate.stride(0) if gate is not None else 0), ptr(out), c_int64(out.stride(1)), c_int64(out.stride(0)), c_int(heads),
        c_int(rank), c_int(rot_dim), c_float(scale), c_int(pieces), ptr(scratch), ptr(ctx.err), ctx.stream,
    )
    if scratch is not None:
        ctx.lib.calls += 1  # the merge kernel is a launch of its own
    return out


# -- the gated delta rule -----------------------------------------------------------------------------------


def delta_prepare(
    ctx: StepContext, proj: torch.Tensor, decay_in: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, a_log: torch.Tensor,
    dt_bias: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    beta: torch.Tensor, decay: torch.Tensor,
) -> None:
    """Convolution + silu of the q, k, v columns of ``proj`` (continuing each request's slot of
    ``conv_state``, which is then moved on), unit vectors, beta and the decay factors, all 32-bit."""
    tokens = proj.shape[0]
    channels = 2 * kv_heads * dk + heads * dv
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels + heads, "delta_prepare: bad projections")
    _need(decay_in.stride(1) == 1 and decay_in.shape[1] >= heads * dk and decay_in.dtype == proj.dtype, "delta_prepare: bad decay input")
    _need(taps.dtype == torch.float32 and taps.shape[0] == channels and taps.is_contiguous(), "delta_prepare: taps are float32 [channels, taps]")
    _need(conv_state.dtype == proj.dtype and tuple(conv_state.shape[1:]) == (max(taps.shape[1] - 1, 0), channels), "delta_prepare: bad convolution state")
    for tensor, width in ((q, kv_heads * dk), (k, kv_heads * dk), (v, heads * dv), (beta, heads), (decay, heads * dk)):
        _need(tensor.dtype == torch.float32 and tuple(tensor.shape) == (tokens, width) and tensor.is_contiguous(), "delta_prepare: bad output")
    ctx.lib.call(
        "b200_delta_prepare", ptr(proj), c_int(proj.stride(0)), ptr(decay_in), c_int(decay_in.stride(0)), ptr(taps),
        c_int(taps.shape[1]), ptr(conv_state), ptr(a_log), ptr(dt_bias), ptr(ctx.token_seq), ptr(ctx.seq_q_start),
        ptr(ctx.seq_q_len), ptr(ctx.seq_slot), c_int(tokens), c_int(ctx.num_seqs), c_int(heads), c_int(kv_heads), c_int(dk),
        c_int(dv), ptr(q), ptr(k), ptr(v), ptr(beta), ptr(decay), c_int(dtype_code(proj.dtype)), ctx.stream,
    )
    ctx.lib.calls += 1  # the slot update is a launch of its own


def delta_recurrence(
    ctx: StepContext, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor,
    state: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int,
) -> torch.Tensor:
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dk, dv) and state.is_contiguous(), "delta_recurrence: the state is float32 [slots, heads, dk, dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (q.shape[0], heads * dv) and out.is_contiguous(), "delta_recurrence: bad output")
    ctx.lib.call(
        "b200_delta_recurrence", ptr(q), ptr(k), ptr(v), ptr(beta), ptr(decay), ptr(ctx.seq_q_start), ptr(ctx.seq_q_len),
        ptr(ctx.seq_slot), c_int(ctx.num_seqs), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), ptr(state), ptr(out),
        ctx.stream,
    )
    return out


def delta_output(
    ctx: StepContext, o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, heads: int, dv: int, eps: float, out: torch.Tensor
) -> torch.Tensor:
    rows = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and tuple(out.shape) == (rows, heads * dv) and out.is_contiguous(), "delta_output: bad operands")
    _need(gate.stride(1) == 1 and gate.shape[1] == heads * dv and gate.dtype == out.dtype, "delta_output: bad gate")
    _need(weight.dtype == torch.float32 and weight.numel() == dv, "delta_output: weight must be float32 [dv]")
    ctx.lib.call(
        "b200_delta_output", ptr(o), ptr(weight), ptr(gate), c_int(gate.stride(0)), c_int(rows), c_int(heads), c_int(dv),
        c_float(eps), ptr(out), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


# -- several residual streams per token, sinusoidal embedding, soft cap -----------------------------------


@dataclass
class PendingBranch:
    """A sublayer's output that is not in the residual streams yet, with the weights that put it
    there: ``x_t <- sum_s mix[s, t] x_s + out[t] * y`` (``mix`` None: the identity). The norm kernel
    that reads the streams next does the write on its way."""

    y: torch.Tensor
    mix: torch.Tensor | None
    out: torch.Tensor | None


def embedding_sinusoid(ctx: StepContext, table: torch.Tensor, inv_freq: torch.Tensor, scale: float, streams: int, out: torch.Tensor) -> torch.Tensor:
    """``out[t, s] = table[token[t]] * scale + e(position[t])`` for every stream ``s``; ``e`` alternates the
    sine and cosine of ``position * inv_freq[i]``. ``out`` is ``[tokens, streams * hidden]`` float32."""
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, streams * hidden) and out.dtype == torch.float32 and out.is_contiguous(), "embedding: bad output")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == hidden // 2 and hidden % 2 == 0, "embedding: one frequency per column pair")
    ctx.lib.call(
        "b200_embedding_sinusoid", ptr(table), ptr(ctx.token_ids), ptr(ctx.positions), ptr(inv_freq), c_float(scale), ptr(out),
        c_int(ctx.num_tokens), c_int(streams), c_int(hidden), c_int(vocab), c_int(dtype_code(table.dtype)), ptr(ctx.err), ctx.stream,
    )
    return out


def hyper_norm(
    ctx: StepContext, x: torch.Tensor, pending: PendingBranch | None, in_w: torch.Tensor | None, weight: torch.Tensor, streams: int,
    eps: float, out: torch.Tensor, rows: torch.Tensor | None = None,
) -> torch.Tensor:
    """Writes ``pending`` into the streams ``x`` (``[tokens, streams * hidden]``; stored back unless ``rows``
    gathers), then ``out = rms_norm(sum_s in_w[s] x_s) * weight`` (``in_w`` None: the plain sum)."""
    hidden = weight.numel()
    count = x.shape[0] if rows is None else rows.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == streams * hidden, "hyper_norm: the streams are contiguous float32")
    _need(weight.dtype == torch.float32 and tuple(out.shape) == (count, hidden) and out.is_contiguous(), "hyper_norm: bad weight or output")
    y = mix = out_w = None
    if pending is not None:
        y, mix, out_w = pending.y, pending.mix, pending.out
        _need(tuple(y.shape) == (x.shape[0], hidden) and y.is_contiguous() and y.dtype == out.dtype, "hyper_norm: bad branch output")
        _need(mix is not None and mix.dtype == torch.float32 and mix.numel() == streams * streams and out_w.dtype == torch.float32 and out_w.numel() == streams, "hyper_norm: bad mixing weights")
    _need(in_w is None or (in_w.dtype == torch.float32 and in_w.numel() == streams), "hyper_norm: bad read weights")
    ctx.lib.call(
        "b200_hyper_norm", ptr(x), ptr(y), ptr(mix), ptr(out_w), ptr(in_w), ptr(weight), ptr(rows), c_int(count), c_int(streams),
        c_int(hidden), c_float(eps), ptr(out), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def softcap(ctx: StepContext, logits: torch.Tensor, cap: float) -> torch.Tensor:
    """``logits <- cap * tanh(logits / cap)`` in place (float32)."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "softcap: logits are contiguous float32")
    ctx.lib.call("b200_softcap", ptr(logits), c_int64(logits.numel()), c_float(cap), ctx.stream)
    return logits


# -- the recurrent mixer with a decay per channel and a bonus for the current token ----------------------


def wkv_shift_mix(ctx: StepContext, h: torch.Tensor, shift: torch.Tensor, mu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]`` (a request's first token of the step takes its slot of
    ``shift`` for ``h[t - 1]``); the slot then moves on to the request's last input of the step."""
    tokens, hidden = h.shape
    blends = mu.shape[0]
    _need(h.is_contiguous() and tuple(out.shape) == (blends, tokens, hidden) and out.is_contiguous() and out.dtype == h.dtype, "wkv_shift_mix: bad operands")
    _need(mu.dtype == torch.float32 and mu.is_contiguous() and mu.shape[1] == hidden, "wkv_shift_mix: blends are float32 [n, hidden]")
    _need(shift.dtype == h.dtype and tuple(shift.shape[1:]) == (hidden,) and shift.is_contiguous(), "wkv_shift_mix: bad slot array")
    ctx.lib.call(
        "b200_wkv_shift_mix", ptr(h), ptr(shift), ptr(mu), ptr(ctx.token_seq), ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_slot),
        c_int(tokens), c_int(ctx.num_seqs), c_int(hidden), c_int(blends), ptr(out), c_int(dtype_code(h.dtype)), ctx.stream,
    )
    ctx.lib.calls += 1  # the slot update is a launch of its own
    return out


def tanh_rows(ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
    """``x <- tanh(x)`` in place."""
    _need(x.is_contiguous(), "tanh_rows: a contiguous buffer")
    ctx.lib.call("b200_tanh_rows", ptr(x), c_int64(x.numel()), c_int(dtype_code(x.dtype)), ctx.stream)
    return x


def wkv_prepare(
    ctx: StepContext, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_decay: torch.Tensor, w0: torch.Tensor, bonus_w: torch.Tensor,
    heads: int, dim: int, r32: torch.Tensor, k32: torch.Tensor, v32: torch.Tensor, decay: torch.Tensor, bonus: torch.Tensor,
) -> None:
    tokens = r.shape[0]
    width = heads * dim
    for tensor in (r, k, v):
        _need(tuple(tensor.shape) == (tokens, width) and tensor.is_contiguous() and tensor.dtype == r.dtype, "wkv_prepare: bad projections")
    _need(log_decay.dtype == torch.float32 and tuple(log_decay.shape) == (tokens, width) and log_decay.is_contiguous(), "wkv_prepare: the decay's logarithm is float32")
    _need(w0.dtype == torch.float32 and w0.numel() == width and bonus_w.dtype == torch.float32 and bonus_w.numel() == width, "wkv_prepare: bad constants")
    for tensor in (r32, k32, v32, decay):
        _need(tensor.dtype == torch.float32 and tuple(tensor.shape) == (tokens, width) and tensor.is_contiguous(), "wkv_prepare: bad output")
    _need(bonus.dtype == torch.float32 and tuple(bonus.shape) == (tokens, heads) and bonus.is_contiguous(), "wkv_prepare: bad bonus output")
    ctx.lib.call(
        "b200_wkv_prepare", ptr(r), ptr(k), ptr(v), ptr(log_decay), ptr(w0), ptr(bonus_w), c_int(tokens), c_int(heads), c_int(dim),
        ptr(r32), ptr(k32), ptr(v32), ptr(decay), ptr(bonus), c_int(dtype_code(r.dtype)), ctx.stream,
    )


def wkv_recurrence(
    ctx: StepContext, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bonus: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
    out: torch.Tensor, heads: int, dk: int, dv: int,
) -> torch.Tensor:
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dk, dv) and state.is_contiguous(), "wkv_recurrence: the state is float32 [slots, heads, dk, dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (r.shape[0], heads * dv) and out.is_contiguous(), "wkv_recurrence: bad output")
    ctx.lib.call(
        "b200_wkv_recurrence", ptr(r), ptr(k), ptr(v), ptr(bonus), ptr(decay), ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_slot),
        c_int(ctx.num_seqs), c_int(heads), c_int(dk), c_int(dv), ptr(state), ptr(out), ctx.stream,
    )
    return out


def wkv_output(ctx: StepContext, o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, heads: int, dv: int, eps: float, out: torch.Tensor,
               sigmoid_gate: bool = False) -> torch.Tensor:
    """``out[t, h] = o[t, h] / rms(o[t, h]) * weight[h] * silu(gate[t, h])`` (``sigmoid`` instead of ``silu`` with
    ``sigmoid_gate``); ``gate`` may be a column slice of a wider buffer."""
    rows = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and tuple(out.shape) == (rows, heads * dv) and out.is_contiguous(), "wkv_output: bad operands")
    _need(gate.stride(1) == 1 and gate.shape[1] == heads * dv and gate.dtype == out.dtype, "wkv_output: bad gate")
    _need(weight.dtype == torch.float32 and weight.numel() == heads * dv, "wkv_output: weight must be float32 [heads * dv]")
    ctx.lib.call(
        "b200_wkv_output", ptr(o), ptr(weight), ptr(gate), c_int(gate.stride(0)), c_int(rows), c_int(heads), c_int(dv), c_float(eps),
        c_int(1 if sigmoid_gate else 0), ptr(out), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


# -- attention without position encoding: unit-RMS queries and keys, blended values, a gate per head -----


def norm_kv_write(
    ctx: StepContext, cache: CacheView, proj: torch.Tensor, q_out: torch.Tensor, q_heads: int, kv_heads: int, dim: int, vdim: int,
    row_dim: int, normalise: bool, eps: float, shared_values: torch.Tensor | None = None, blend: torch.Tensor | None = None,
    publish: bool = False,
) -> torch.Tensor:
    """Per token of ``proj`` (rows ``[q | k | v | ...]``): queries and keys divided by their root mean square
    per head (if ``normalise``), queries to ``q_out`` and keys and values to the token's page, all in rows
    of ``row_dim`` numbers padded with zeros. ``publish``: the raw values also go to ``shared_values``;
    ``blend`` (one float32 on the device): values become ``(1 - blend) v + blend * shared_values``."""
    tokens, ld = proj.shape
    _need(proj.is_contiguous() and cache.keys.dtype == proj.dtype and cache.values is not None, "norm_kv_write: bad operands")
    _need(tuple(q_out.shape) == (tokens, q_heads * row_dim) and q_out.is_contiguous() and q_out.dtype == proj.dtype, "norm_kv_write: bad q_out")
    _need(tuple(cache.keys.shape[1:]) == (kv_heads, cache.page_size, row_dim), "norm_kv_write: the cache rows differ from the padded head size")
    mode = 1 if publish else (2 if blend is not None else 0)
    if mode:
        _need(shared_values is not None and tuple(shared_values.shape) == (tokens, kv_heads * vdim) and shared_values.dtype == proj.dtype and shared_values.is_contiguous(), "norm_kv_write: bad shared values")
        _need(blend is None or (blend.dtype == torch.float32 and blend.numel() == 1), "norm_kv_write: the blend factor is one float32")
    ctx.lib.call(
        "b200_norm_kv_write", ptr(proj), c_int(ld), ptr(ctx.positions), ptr(ctx.token_seq), ptr(ctx.seq_kv_len), ptr(cache.block_table),
        c_int(cache.max_pages), c_int(cache.num_pages), ptr(cache.keys), ptr(cache.values), ptr(q_out), ptr(shared_values if mode else None),
        ptr(blend if mode == 2 else None), c_int(mode), c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(dim), c_int(vdim),
        c_int(row_dim), c_int(cache.page_size), c_int(1 if normalise else 0), c_float(eps), c_int(1 if cache.writes else 0),
        c_int(dtype_code(proj.dtype)), ptr(ctx.err), ctx.stream,
    )
    return q_out


def head_gate(ctx: StepContext, attn: torch.Tensor, proj: torch.Tensor | None, gate_offset: int, heads: int, vdim: int, row_dim: int, out: torch.Tensor) -> torch.Tensor:
    """``out[t, h, :] = attn[t, h, :vdim] * sigmoid(proj[t, gate_offset + h])`` (``proj`` None: no gate; the
    kernel then only drops the padding)."""
    tokens = attn.shape[0]
    _need(tuple(attn.shape) == (tokens, heads * row_dim) and attn.is_contiguous() and tuple(out.shape) == (tokens, heads * vdim) and out.is_contiguous() and out.dtype == attn.dtype, "head_gate: bad operands")
    _need(proj is None or (proj.is_contiguous() and proj.dtype == attn.dtype and proj.shape[1] >= gate_offset + heads), "head_gate: bad gate logits")
    ctx.lib.call(
        "b200_head_gate", ptr(attn), ptr(proj), c_int(proj.shape[1] if proj is not None else 0), c_int(gate_offset), c_int(tokens), c_int(heads),
        c_int(vdim), c_int(row_dim), ptr(out), c_int(dtype_code(attn.dtype)), ctx.stream,
    )
    return out


# -- the routed feed-forward --------------------------------------------------------------------------------


def moe_route(ctx: StepContext, logits: torch.Tensor, groups: int, keep: int, top: int, scale: float, ids: torch.Tensor, weights: torch.Tensor,
              *, bias: torch.Tensor | None = None, softmax_chosen: bool = False) -> None:
    """``bias`` (float32 ``[experts]``) is added to the logits first. ``softmax_chosen``: an expert's score is its logit
    and the chosen experts' weights are the softmax over their logits alone (times ``scale``); otherwise the score is
    the logit's sigmoid and the weights are the chosen scores over their sum."""
    tokens, experts = logits.shape
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == experts and bias.is_contiguous()), "moe_route: the bias is float32 [experts]")
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "moe_route: router logits are contiguous float32")
    _need(ids.dtype == torch.int32 and tuple(ids.shape) == (tokens, top) and ids.is_contiguous(), "moe_route: bad ids")
    _need(weights.dtype == torch.float32 and tuple(weights.shape) == (tokens, top) and weights.is_contiguous(), "moe_route: bad weights")
    ctx.lib.call(
        "b200_moe_route", ptr(logits), ptr(bias), c_int(1 if softmax_chosen else 0), c_int(tokens), c_int(experts), c_int(groups), c_int(keep), c_int(top), c_float(scale), ptr(ids),
        ptr(weights), ctx.stream,
    )


def moe_tile_rows(ctx: StepContext) -> int:
    return int(ctx.lib.lib.b200_moe_tile_rows())


def moe_experts(
    ctx: StepContext, h: torch.Tensor, ids: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, limit: float, out: torch.Tensor
) -> torch.Tensor:
    """``out[t * top + j] = expert ids[t, j] applied to h[t]`` (float32, not yet weighted). ``w_gate_up`` is
    ``[experts, 2 * ff, width]`` (gate rows, then up rows), ``w_down`` ``[experts, width, ff]``. The slots are sorted by
    expert into runs of whole tiles, then the two products walk the tiles (tall tiles on tcgen05 read rows that a
    gather pass has put into sorted order)."""
    tokens, width = h.shape
    top = ids.shape[1]
    experts, twice, _ = w_gate_up.shape
    ff = twice // 2
    slots = tokens * top
    _need(h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.dtype == h.dtype and w_down.dtype == h.dtype, "moe_experts: bad operands")
    _need(tuple(w_gate_up.shape) == (experts, 2 * ff, width) and tuple(w_down.shape) == (experts, width, ff), "moe_experts: bad weights")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (slots, width) and out.is_contiguous(), "moe_experts: bad output")
    # bfloat16 runs on tensor cores where the sizes allow, and a step with many slots per expert sorts them into tiles
    # four times as tall (128 places), which the tcgen05 form takes; short steps keep tiles of 32 and mma.sync.
    # options["moe"]: "auto", "mma" (mma.sync for tall tiles too) or "plain" (the FMA kernels).
    choice = ctx.options.get("moe", "auto")
    tensor_cores = h.dtype == torch.bfloat16 and choice != "plain" and bool(ctx.lib.lib.b200_moe_mma_supported(width, ff))
    tile = moe_tile_rows(ctx)
    tall = tensor_cores and slots >= 2 * 4 * tile * experts
    if tall:
        tile *= 4
    max_tiles = (slots + experts * (tile - 1)) // tile + 1
    capacity = max_tiles * tile
    place_slot = ctx.buffer("moe_place_slot", (capacity,), torch.int32, per_token=False)
    tile_expert = ctx.buffer("moe_tile_expert", (max_tiles + 1,), torch.int32, per_token=False)
    act = ctx.buffer("moe_act", (capacity, ff), per_token=False)
    num_tiles = tile_expert[max_tiles:]
    ctx.lib.call("b200_moe_sort", ptr(ids), c_int(slots), c_int(experts), c_int(capacity), c_int(tile), ptr(place_slot), ptr(tile_expert), ptr(num_tiles), ctx.stream)
    if tall and choice == "auto" and bool(ctx.lib.lib.b200_moe_tcgen05_supported(width, ff)):
        sorted_rows = ctx.buffer("moe_sorted_rows", (capacity, width), per_token=False)
        ctx.lib.call("b200_moe_gather_rows", ptr(h), ptr(place_slot), c_int(capacity), c_int(top), c_int(width), ptr(sorted_rows), ctx.stream)
        stages = c_int(int(ctx.options.get("moe_stages", 0)))
        ctx.lib.call(
            "b200_moe_product_tcgen05", ptr(w_gate_up), ptr(sorted_rows), ptr(place_slot), ptr(tile_expert), ptr(num_tiles), c_int(max_tiles),
            c_int(experts), c_int(2 * ff), c_int(ff), c_int(ff), c_int(width), c_int(2), c_float(limit), ptr(act), stages, ptr(ctx.err), ctx.stream,
        )
        ctx.lib.call(
            "b200_moe_product_tcgen05", ptr(w_down), ptr(act), ptr(place_slot), ptr(tile_expert), ptr(num_tiles), c_int(max_tiles),
            c_int(experts), c_int(width), c_int(0), c_int(width), c_int(ff), c_int(1), c_float(limit), ptr(out), stages, ptr(ctx.err), ctx.stream,
        )
        return out
    code, use = c_int(dtype_code(h.dtype)), c_int(1 if tensor_cores else 0)
    ctx.lib.call(
        "b200_moe_gate_up", ptr(h), ptr(w_gate_up), ptr(place_slot), ptr(tile_expert), ptr(num_tiles), c_int(max_tiles), c_int(tile), c_int(top),
        c_int(width), c_int(ff), c_float(limit), ptr(act), code, use, ctx.stream,
    )
    ctx.lib.call(
        "b200_moe_down", ptr(act), ptr(w_down), ptr(place_slot), ptr(tile_expert), ptr(num_tiles), c_int(max_tiles), c_int(tile), c_int(width),
        c_int(ff), ptr(out), code, use, ctx.stream,
    )
    return out


def moe_combine(ctx: StepContext, expert_out: torch.Tensor, weights: torch.Tensor, shared: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    tokens, top = weights.shape
    width = out.shape[1]
    _need(expert_out.dtype == torch.float32 and tuple(expert_out.shape) == (tokens * top, width) and expert_out.is_contiguous(), "moe_combine: bad expert outputs")
    _need(out.is_contiguous() and out.shape[0] == tokens and (shared is None or (shared.shape == out.shape and shared.dtype == out.dtype and shared.is_contiguous())), "moe_combine: bad operands")
    ctx.lib.call(
        "b200_moe_combine", ptr(expert_out), ptr(weights), ptr(shared), c_int(tokens), c_int(top), c_int(width), ptr(out),
        c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def clamped_glu(ctx: StepContext, gate_up: torch.Tensor, limit: float, out: torch.Tensor) -> torch.Tensor:
    """``out = g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``; rows of
    ``gate_up`` are ``[gate | up]``. A ``limit`` of zero is the unclamped form ``silu(gate) * up``, for the experts'
    products (``moe_experts``) as well."""
    rows, twice = gate_up.shape
    ff = twice // 2
    _need(twice == 2 * ff and tuple(out.shape) == (rows, ff) and gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "clamped_glu: bad operands")
    ctx.lib.call("b200_clamped_glu", ptr(gate_up), c_int(rows), c_int(ff), c_float(limit), ptr(out), c_int(dtype_code(out.dtype)), ctx.stream)
    return out


# -- minGRU, the generalized delta rule, attention with weights mixed over heads, a pair of mixers, bigram embedding --


@dataclass
class BranchPair:
    """The outputs of two mixers that ran side by side, not yet combined: the layer's result is
    ``(wa * a / rms(a) + wb * b / rms(b)) / 2``. The norm that adds it into the stream combines them."""

    a: torch.Tensor
    b: torch.Tensor
    wa: torch.Tensor
    wb: torch.Tensor
    eps: float


MINGRU_PIECE = 64  # tokens per piece of the three-pass form (csrc/kernels/mingru.cu)


def mingru(ctx: StepContext, proj: torch.Tensor, bias: torch.Tensor, state: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``proj`` rows are ``[pz | px | pg]``; ``bias`` is ``[bz | bx]`` (float32); ``state`` the slots ``[slots, width]``.
    Steps whose longest run has more than two pieces of tokens run their prompt portions in three passes
    (pieces at the same time), everything else in one pass per request."""
    tokens, width = out.shape
    _need(proj.is_contiguous() and proj.shape == (tokens, 3 * width) and out.is_contiguous() and out.dtype == proj.dtype, "mingru: bad operands")
    _need(bias.dtype == torch.float32 and bias.numel() == 2 * width and bias.is_contiguous(), "mingru: the biases are float32 [2 * width]")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (width,) and state.is_contiguous(), "mingru: the state is float32 [slots, width]")
    first_long = ctx.num_seqs
    maps = None
    if ctx.max_q_len > 2 * MINGRU_PIECE and not ctx.captured:
        first_long = ctx.num_decode_seqs
        count = int(ctx.lib.lib.b200_mingru_scratch(ctx.num_seqs - first_long, ctx.max_q_len, width))
        maps = ctx.buffer("mingru_maps", (count,), torch.float32, per_token=False)
    ctx.lib.call(
        "b200_mingru", ptr(proj), c_int(proj.stride(0)), ptr(bias), ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_slot),
        c_int(first_long), c_int(ctx.num_seqs), c_int(max(ctx.max_q_len, 1)), c_int(width), ptr(state), ptr(maps), ptr(out),
        c_int(dtype_code(proj.dtype)), ctx.stream,
    )
    if maps is not None:
        ctx.lib.calls += 2 + (1 if first_long else 0)
    return out


def delta_general_prepare(
    ctx: StepContext, proj: torch.Tensor, offsets: tuple[int, int, int, int], log_decay: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor,
    heads: int, dim: int, outs: tuple[torch.Tensor, ...],
) -> None:
    """From ``proj`` (columns r, k, v, a at ``offsets``) and the decay's low-rank image ``log_decay`` (float32):
    the 32-bit r, k, v, ``w = exp(-e^(-1/2) sigmoid(log_decay + w0))``, ``sigmoid(a + a_bias) * u`` and ``u = k / |k|`` per head."""
    tokens = proj.shape[0]
    inner = heads * dim
    _need(proj.stride(1) == 1, "delta_general_prepare: bad projections")
    _need(log_decay.dtype == torch.float32 and tuple(log_decay.shape) == (tokens, inner) and log_decay.is_contiguous(), "delta_general_prepare: bad decay input")
    _need(w0.dtype == torch.float32 and w0.numel() == inner and a_bias.dtype == torch.float32 and a_bias.numel() == inner, "delta_general_prepare: bad constants")
    _need(len(outs) == 6 and all(o.dtype == torch.float32 and tuple(o.shape) == (tokens, inner) and o.is_contiguous() for o in outs), "delta_general_prepare: bad outputs")
    ctx.lib.call(
        "b200_delta_general_prepare", ptr(proj), c_int(proj.stride(0)), *(c_int(o) for o in offsets), ptr(log_decay), ptr(w0), ptr(a_bias),
        c_int(tokens), c_int(heads), c_int(dim), *(ptr(o) for o in outs), c_int(dtype_code(proj.dtype)), ctx.stream,
    )


def delta_general_recurrence(
    ctx: StepContext, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, au: torch.Tensor, u: torch.Tensor,
    state: torch.Tensor, out: torch.Tensor, heads: int, dk: int, dv: int,
) -> torch.Tensor:
    """``S <- diag(w) S - au (u^T S) + k v^T``, ``o = S^T r`` per head and token, each request from its slot of ``state``."""
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dk, dv) and state.is_contiguous(), "delta_general_recurrence: the state is float32 [slots, heads, dk, dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (r.shape[0], heads * dv) and out.is_contiguous(), "delta_general_recurrence: bad output")
    ctx.lib.call(
        "b200_delta_general_recurrence", ptr(r), ptr(k), ptr(v), ptr(w), ptr(au), ptr(u), ptr(ctx.seq_q_start), ptr(ctx.seq_q_len),
        ptr(ctx.seq_slot), c_int(ctx.num_seqs), c_int(max(ctx.max_q_len, 1)), c_int(heads), c_int(dk), c_int(dv), ptr(state), ptr(out), ctx.stream,
    )
    return out


def conv_norm_rope_write(
    ctx: StepContext, cache: CacheView, conv_state: torch.Tensor, proj: torch.Tensor, bias: torch.Tensor | None, taps: torch.Tensor,
    q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, inv_freq: torch.Tensor | None, rot_dims: int, q_out: torch.Tensor,
    q_heads: int, kv_heads: int, dim: int, vdim: int, row_dim: int,
) -> torch.Tensor:
    """Per token of ``proj`` (rows ``[q | k | v | ...]``): bias, the short convolution over time (continuing each
    request's slot of ``conv_state``, which is then moved on), one RMS norm over all of q and one over all of k,
    rotation of the first ``rot_dims`` dims of every head in neighbouring pairs, queries to ``q_out`` and keys
    and values to the token's page, all in rows of ``row_dim`` numbers padded with zeros."""
    tokens, ld = proj.shape
    channels = (q_heads + kv_heads) * dim + kv_heads * vdim
    _need(proj.is_contiguous() and cache.keys.dtype == proj.dtype and cache.values is not None, "conv_norm_rope_write: bad operands")
    _need(tuple(q_out.shape) == (tokens, q_heads * row_dim) and q_out.is_contiguous() and q_out.dtype == proj.dtype, "conv_norm_rope_write: bad q_out")
    _need(tuple(cache.keys.shape[1:]) == (kv_heads, cache.page_size, row_dim), "conv_norm_rope_write: the cache rows differ from the padded head size")
    _need(taps.dtype == torch.float32 and taps.shape[0] == channels and taps.is_contiguous(), "conv_norm_rope_write: taps are float32 [channels, taps]")
    _need(conv_state.dtype == proj.dtype and tuple(conv_state.shape[1:]) == (taps.shape[1] - 1, channels), "conv_norm_rope_write: bad convolution state")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == channels), "conv_norm_rope_write: bad bias")
    _need(q_weight.dtype == torch.float32 and q_weight.numel() == q_heads * dim and k_weight.dtype == torch.float32 and k_weight.numel() == kv_heads * dim, "conv_norm_rope_write: bad norm weights")
    _need(rot_dims == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2), "conv_norm_rope_write: bad frequency table")
    ctx.lib.call(
        "b200_conv_norm_rope_write", ptr(proj), c_int(ld), ptr(bias), ptr(taps), c_int(taps.shape[1]), ptr(conv_state), ptr(q_weight),
        ptr(k_weight), c_float(eps), ptr(inv_freq if rot_dims else None), c_int(rot_dims), ptr(ctx.positions), ptr(ctx.token_seq),
        ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_slot), ptr(ctx.seq_kv_len), ptr(cache.block_table), c_int(cache.max_pages),
        c_int(cache.num_pages), ptr(cache.keys), ptr(cache.values), ptr(q_out), c_int(tokens), c_int(ctx.num_seqs), c_int(q_heads),
        c_int(kv_heads), c_int(dim), c_int(vdim), c_int(row_dim), c_int(cache.page_size), c_int(1 if cache.writes else 0),
        c_int(dtype_code(proj.dtype)), ptr(ctx.err), ctx.stream,
    )
    if taps.shape[1] > 1:
        ctx.lib.calls += 1  # the slot update is a launch of its own
    return q_out


def mix_heads_gate(
    ctx: StepContext, attn: torch.Tensor, mix: torch.Tensor, gate: torch.Tensor | None, heads: int, kv_heads: int, vdim: int, row_dim: int,
    out: torch.Tensor,
) -> torch.Tensor:
    """``out[t, h] = sigmoid(gate[t, h]) * sum_g mix[h, g] * attn[c(h), t, g, :vdim]``; ``attn`` is ``[kv_heads, tokens,
    heads * row_dim]`` (plane ``c``: every head's weights applied to the values of kv head ``c``)."""
    tokens = out.shape[0]
    _need(tuple(attn.shape) == (kv_heads, tokens, heads * row_dim) and attn.is_contiguous() and tuple(out.shape) == (tokens, heads * vdim) and out.is_contiguous() and out.dtype == attn.dtype, "mix_heads_gate: bad operands")
    _need(mix.dtype == torch.float32 and tuple(mix.shape) == (heads, heads) and mix.is_contiguous(), "mix_heads_gate: the mix is float32 [heads, heads]")
    _need(gate is None or (gate.stride(1) == 1 and gate.shape[1] == heads * vdim and gate.dtype == attn.dtype), "mix_heads_gate: bad gate")
    ctx.lib.call(
        "b200_mix_heads_gate", ptr(attn), ptr(mix), ptr(gate), c_int(gate.stride(0) if gate is not None else 0), c_int(tokens), c_int(heads),
        c_int(kv_heads), c_int(vdim), c_int(row_dim), ptr(out), c_int(dtype_code(attn.dtype)), ctx.stream,
    )
    return out


def pair_norm_add(ctx: StepContext, x_in: torch.Tensor, pair: BranchPair, weight: torch.Tensor, eps: float, x_out: torch.Tensor,
                  cast: torch.Tensor | None = None) -> None:
    """``x_out = x_in + weight * y / rms(y)`` with ``y`` the combination of the pair (see :class:`BranchPair`)."""
    rows, hidden = x_in.shape
    _need(x_in.dtype == torch.float32 and x_out.dtype == torch.float32 and x_in.is_contiguous() and x_out.is_contiguous(), "pair_norm_add: the stream is contiguous float32")
    for t in (pair.a, pair.b):
        _need(tuple(t.shape) == (rows, hidden) and t.is_contiguous() and t.dtype == pair.a.dtype, "pair_norm_add: bad branch outputs")
    for w in (pair.wa, pair.wb, weight):
        _need(w.dtype == torch.float32 and w.numel() == hidden, "pair_norm_add: weights are float32 [hidden]")
    _need(cast is None or (cast.dtype == pair.a.dtype and cast.shape == x_in.shape), "pair_norm_add: bad cast buffer")
    ctx.lib.call(
        "b200_pair_norm_add", ptr(x_in), ptr(pair.a), ptr(pair.b), ptr(pair.wa), ptr(pair.wb), ptr(weight), c_int(rows), c_int(hidden),
        c_float(pair.eps), c_float(eps), ptr(x_out), ptr(cast), c_int(dtype_code(pair.a.dtype)), ctx.stream,
    )


def embedding_bigram(
    ctx: StepContext, table: torch.Tensor, pairs: torch.Tensor, last_token: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int,
    out: torch.Tensor, cast: torch.Tensor | None,
) -> torch.Tensor:
    """``out[t] = table[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets]`` (row ``buckets`` for a
    request's first token) in 32-bit; ``last_token`` ``[slots, 1]`` int32 carries each request's last token."""
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, hidden) and out.dtype == torch.float32, "embedding_bigram: bad output")
    _need(tuple(pairs.shape) == (buckets + 1, hidden) and pairs.dtype == table.dtype and pairs.is_contiguous(), "embedding_bigram: the pair table is [buckets + 1, hidden]")
    _need(last_token.dtype == torch.int32 and last_token.is_contiguous(), "embedding_bigram: the slots hold int32")
    _need(cast is None or (cast.dtype == table.dtype and cast.shape == out.shape), "embedding_bigram: bad cast buffer")
    ctx.lib.call(
        "b200_embedding_bigram", ptr(table), ptr(pairs), ptr(ctx.token_ids), ptr(ctx.positions), ptr(ctx.token_seq), ptr(ctx.seq_q_start),
        ptr(ctx.seq_q_len), ptr(ctx.seq_slot), ptr(last_token), c_int(buckets), c_int64(mul_prev), c_int64(mul_cur), ptr(out), ptr(cast),
        c_int(ctx.num_tokens), c_int(ctx.num_seqs), c_int(hidden), c_int(vocab), c_int(dtype_code(table.dtype)), ptr(ctx.err), ctx.stream,
    )
    ctx.lib.calls += 1  # the slot update is a launch of its own
    return out


# -- layer norm, the embedding that ends in one, and the row kernels of layers built around them ----------------------


@dataclass
class BranchSum:
    """The outputs of two sublayers that read the same normed rows and are both still to be added to the stream
    (``b`` may be None): the norm kernel that runs next adds them in 32-bit."""

    a: torch.Tensor
    b: torch.Tensor | None


def layernorm(ctx: StepContext, x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor,
              rows: torch.Tensor | None = None) -> torch.Tensor:
    """``v = x + delta`` (a tensor, a :class:`BranchSum` or None; written back into ``x`` unless ``rows`` is given), ``out
    = (v - mean) / sqrt(mean((v - mean)^2) + eps) * weight``."""
    hidden = x.shape[1]
    count = x.shape[0] if rows is None else rows.shape[0]
    a, b = (delta.a, delta.b) if isinstance(delta, BranchSum) else (delta, None)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "layernorm: the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "layernorm: weight must be float32 [hidden]")
    _need(tuple(out.shape) == (count, hidden) and out.is_contiguous(), "layernorm: bad output shape")
    for d in (a, b):
        _need(d is None or (d.shape == x.shape and d.dtype == out.dtype and d.is_contiguous()), "layernorm: bad pending branch output")
    ctx.lib.call(
        "b200_layernorm", ptr(x), ptr(a), ptr(b), ptr(weight), ptr(rows), c_int(count), c_int(hidden), c_float(eps), ptr(out),
        c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def embedding_layernorm(ctx: StepContext, table: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """``out[t] = layer norm of table[token[t]]`` in 32-bit."""
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, hidden) and out.dtype == torch.float32, "embedding: bad output")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "embedding: the norm's weight is float32 [hidden]")
    ctx.lib.call(
        "b200_embedding_layernorm", ptr(table), ptr(ctx.token_ids), ptr(weight), c_float(eps), ptr(out), c_int(ctx.num_tokens), c_int(hidden),
        c_int(vocab), c_int(dtype_code(table.dtype)), ptr(ctx.err), ctx.stream,
    )
    return out


def rms_rows(ctx: StepContext, rows_in: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """``out = v / sqrt(mean(v^2) + eps) * weight`` per row of ``rows_in`` (a view with any row stride)."""
    count, width = rows_in.shape
    _need(rows_in.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (count, width) and out.dtype == rows_in.dtype, "rms_rows: bad operands")
    _need(weight.dtype == torch.float32 and weight.numel() == width, "rms_rows: weight must be float32 [width]")
    ctx.lib.call(
        "b200_rms_rows", ptr(rows_in), c_int64(rows_in.stride(0)), ptr(weight), c_float(eps), c_int(count), c_int(width), ptr(out),
        c_int64(out.stride(0)), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def sigmoid_mul(ctx: StepContext, a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = a * sigmoid(gate)`` element by element; ``gate`` may be a view of wider rows."""
    rows, width = a.shape
    _need(a.is_contiguous() and out.is_contiguous() and out.shape == a.shape and out.dtype == a.dtype, "sigmoid_mul: bad operands")
    _need(tuple(gate.shape) == (rows, width) and gate.stride(1) == 1 and gate.dtype == a.dtype, "sigmoid_mul: bad gate")
    ctx.lib.call("b200_sigmoid_mul", ptr(a), ptr(gate), c_int64(gate.stride(0)), c_int(rows), c_int(width), ptr(out), c_int(dtype_code(a.dtype)), ctx.stream)
    return out


def scale_values(ctx: StepContext, values: torch.Tensor, scale: float) -> torch.Tensor:
    _need(values.dtype == torch.float32 and values.is_contiguous(), "scale_values: contiguous float32")
    ctx.lib.call("b200_scale_values", ptr(values), c_int64(values.numel()), c_float(scale), ctx.stream)
    return values


def qk_norm_rope_write(
    ctx: StepContext, cache: CacheView, proj: torch.Tensor, bias: torch.Tensor | None, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
    eps: float, inv_freq: torch.Tensor | None, magnitude: float, values_from_keys: bool, q_out: torch.Tensor, q_heads: int, kv_heads: int,
    dim: int, vdim: int, row_dim: int,
) -> torch.Tensor:
    """Per token of ``proj`` (rows ``[q | k | v | ...]``, no v part with ``values_from_keys``): bias; one RMS norm over all of
    q and one over all of k (``q_weight`` / ``k_weight``; None: no norm); the first ``2 * len(inv_freq)`` numbers of every
    head rotated in halves by ``position * inv_freq``, sine and cosine times ``magnitude``; queries to ``q_out``, keys and
    values (the keys as projected, with ``values_from_keys``) to the token's page, rows padded to ``row_dim``."""
    tokens, ld = proj.shape
    width = (q_heads + kv_heads) * dim + (0 if values_from_keys else kv_heads * vdim)
    rot_dims = 2 * inv_freq.numel() if inv_freq is not None else 0
    _need(proj.is_contiguous() and cache.keys.dtype == proj.dtype and cache.values is not None, "qk_norm_rope_write: bad operands")
    _need(tuple(q_out.shape) == (tokens, q_heads * row_dim) and q_out.is_contiguous() and q_out.dtype == proj.dtype, "qk_norm_rope_write: bad q_out")
    _need(tuple(cache.keys.shape[1:]) == (kv_heads, cache.page_size, row_dim), "qk_norm_rope_write: the cache rows differ from the padded head size")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "qk_norm_rope_write: the bias is float32 over q, k (and v)")
    _need(q_weight is None or (q_weight.dtype == torch.float32 and q_weight.numel() == q_heads * dim), "qk_norm_rope_write: bad q weight")
    _need(k_weight is None or (k_weight.dtype == torch.float32 and k_weight.numel() == kv_heads * dim), "qk_norm_rope_write: bad k weight")
    _need(inv_freq is None or inv_freq.dtype == torch.float32, "qk_norm_rope_write: bad frequency table")
    ctx.lib.call(
        "b200_qk_norm_rope_write", ptr(proj), c_int(ld), ptr(bias), ptr(q_weight), ptr(k_weight), c_float(eps), ptr(inv_freq), c_int(rot_dims),
        c_float(magnitude), c_int(1 if values_from_keys else 0), ptr(ctx.positions), ptr(ctx.token_seq), ptr(ctx.seq_kv_len), ptr(cache.block_table),
        c_int(cache.max_pages), c_int(cache.num_pages), ptr(cache.keys), ptr(cache.values), ptr(q_out), c_int(tokens), c_int(q_heads),
        c_int(kv_heads), c_int(dim), c_int(vdim), c_int(row_dim), c_int(cache.page_size), c_int(1 if cache.writes else 0),
        c_int(dtype_code(proj.dtype)), ptr(ctx.err), ctx.stream,
    )
    return q_out
