"""A recurrent mixer: the gated delta rule with a decay per head and key channel."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, StateSpec, register_part
from .context import CacheView, StepContext


class ChannelDeltaRule(Part):
    """Per head a state ``S [dim, vdim]`` (32-bit, zero at a request's start) is carried from token
    to token: ``S = g (.) S`` (``g`` scales the rows, one factor per key channel);
    ``u = beta (v - S^T k)``; ``S = S + k u^T``; ``o = S^T q``.

    ``q, k`` (``kv_heads x dim``, head ``n`` uses q/k head ``n // (heads / kv_heads)``) and ``v``
    (``heads x vdim``) are projections of ``h`` that pass a causal convolution over ``taps`` tokens
    per channel and silu; q and k then become unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``),
    q also times ``dim^-1/2``. ``beta = sigmoid(W_b h)``;
    ``g = exp(-exp(A_log[n]) * softplus(W_a2 W_a1 h + dt_bias))``. Each head's ``o`` is divided by
    its root mean square over ``vdim``, times ``norm`` (shared by the heads), times
    ``sigmoid(W_g2 W_g1 h)``; then ``W_o``. The inner sizes of the two low-rank pairs
    (``decay_rank``, ``gate_rank``) are the checkpoint's; a configuration names them only to draw
    random weights.

    Per-request state: ``S`` and the convolution's last ``taps - 1`` inputs. Three matrix products
    read ``h`` and its low-rank images: ``[q | k | v | b]``, ``[a1 | g1]``, and ``a2`` and ``g2`` as
    one block-diagonal matrix. Tensor names are ``prefix + q | q.conv | k | k.conv | v | v.conv | b |
    A_log | norm | a1 | a2 | dt_bias | g1 | g2 | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: int | None = None, gate_rank: int | None = None) -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} heads cannot share {kv_heads} q/k heads")
        if taps < 1:
            raise ValueError("the convolution needs at least the current token's tap")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = heads, kv_heads, dim, vdim, int(taps), float(eps)
        self.decay_rank = -1 if decay_rank is None else int(decay_rank)
        self.gate_rank = -1 if gate_rank is None else int(gate_rank)
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.dtype = torch.bfloat16
        self.w_main = self.w_low = self.w_high = self.w_o = None
        self.taps_w = self.a_log = self.dt_bias = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec(
            ((self.heads, self.dim, self.vdim), (self.taps - 1, self.channels)), (torch.float32, self.dtype)
        )

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        qk, vw = self.kv_heads * self.dim, self.heads * self.vdim
        return [
            TensorSpec(p + "q", (qk, d)), TensorSpec(p + "q.conv", (qk, self.taps), init="half_plus_normal"),
            TensorSpec(p + "k", (qk, d)), TensorSpec(p + "k.conv", (qk, self.taps), init="half_plus_normal"),
            TensorSpec(p + "v", (vw, d)), TensorSpec(p + "v.conv", (vw, self.taps), init="half_plus_normal"),
            TensorSpec(p + "b", (self.heads, d)),
            TensorSpec(p + "A_log", (self.heads,)),
            TensorSpec(p + "norm", (self.vdim,), init="one_plus_normal"),
            TensorSpec(p + "a1", (self.decay_rank, d)), TensorSpec(p + "a2", (self.heads * self.dim, self.decay_rank)),
            TensorSpec(p + "dt_bias", (self.heads * self.dim,)),
            TensorSpec(p + "g1", (self.gate_rank, d)), TensorSpec(p + "g2", (vw, self.gate_rank)),
            TensorSpec(p + "o", (d, vw)),
        ]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        self.dtype = dtype

        def get(name: str, to=dtype) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=to)

        self.w_main = torch.cat([get("q"), get("k"), get("v"), get("b")]).contiguous()
        a1, a2, g1, g2 = get("a1"), get("a2"), get("g1"), get("g2")
        self.w_low = torch.cat([a1, g1]).contiguous()
        ra, rg = a1.shape[0], g1.shape[0]
        high = torch.zeros((a2.shape[0] + g2.shape[0], ra + rg), dtype=dtype, device=device)
        high[: a2.shape[0], :ra] = a2
        high[a2.shape[0] :, ra:] = g2
        self.w_high = high
        self.w_o = get("o").contiguous()
        f32 = torch.float32
        self.taps_w = torch.cat([get("q.conv", f32), get("k.conv", f32), get("v.conv", f32)]).contiguous()
        self.a_log, self.dt_bias, self.norm_weight = get("A_log", f32).contiguous(), get("dt_bias", f32).contiguous(), get("norm", f32).contiguous()

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_main, self.w_low, self.w_high, self.w_o))

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, kvh, dk, dv = ctx.num_tokens, self.heads, self.kv_heads, self.dim, self.vdim
        state, conv_state = cache.state
        main = ops.linear(ctx, h, self.w_main, ctx.buffer("delta_main", (t, self.w_main.shape[0])))
        low = ops.linear(ctx, h, self.w_low, ctx.buffer("delta_low", (t, self.w_low.shape[0])))
        high = ops.linear(ctx, low, self.w_high, ctx.buffer("delta_high", (t, self.w_high.shape[0])))
        f32 = torch.float32
        q, k = ctx.buffer("delta_q", (t, kvh * dk), f32), ctx.buffer("delta_k", (t, kvh * dk), f32)
        v, beta = ctx.buffer("delta_v", (t, heads * dv), f32), ctx.buffer("delta_beta", (t, heads), f32)
        decay = ctx.buffer("delta_decay", (t, heads * dk), f32)
        ops.delta_prepare(ctx, main, high[:, : heads * dk], self.taps_w, conv_state, self.a_log, self.dt_bias, heads, kvh, dk, dv, q, k, v, beta, decay)
        o = ops.delta_recurrence(ctx, q, k, v, beta, decay, state, ctx.buffer("delta_o", (t, heads * dv), f32), heads, kvh, dk, dv)
        y = ops.delta_output(ctx, o, self.norm_weight, high[:, heads * dk :], heads, dv, self.eps, ctx.buffer("attn", (t, heads * dv)))
        return ops.linear(ctx, y, self.w_o, ctx.buffer("branch", (t, self.hidden_size)))


class GeneralDeltaRule(Part):
    """Per head a state ``S [dim, dim]`` (32-bit, zero at a request's start) is carried from token to token:
    ``S <- diag(w) S - (a * u) (u^T S) + k v^T`` (both terms read the old state), ``o = S^T r`` (the new one), with
    ``u = k / sqrt(sum k^2 + 1e-6)`` the key's direction per head.

    ``r, k, v`` (``heads x dim`` each) are projections of ``h`` without biases;
    ``w = exp(-e^(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0))`` is the decay and ``a = sigmoid(W_a h + b_a)`` the share
    removed, both per head and key channel. Each head's ``o`` is divided by its root mean square, times ``norm``
    (all heads' size), times ``sigmoid(W_g h)``; then ``W_o``. The inner size of the decay's low-rank pair
    (``decay_rank``) is the checkpoint's; a configuration names it only to draw random weights.

    Per-request state: ``S``. Two matrix products read ``h``: ``[r | k | v | a | g]`` and ``w1``; the second small
    product has a 32-bit result. Decays, shares, directions and the recurrence are 32-bit. Tensor names:
    ``prefix + r | k | v | a | a.b | g | w1 | w2 | w0 | norm | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, dim: int, eps: float, decay_rank: int | None = None,
                 out_name: str = "branch") -> None:
        self.prefix, self.hidden_size, self.heads, self.dim, self.eps = prefix, hidden_size, int(heads), int(dim), float(eps)
        self.decay_rank = -1 if decay_rank is None else int(decay_rank)
        self.out_name = out_name
        self.w_main = self.w_low = self.w_high = self.w_o = self.w0 = self.a_bias = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec(((self.heads, self.dim, self.dim),), (torch.float32,))

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, inner = self.prefix, self.hidden_size, self.heads * self.dim
        specs = [TensorSpec(p + s, (inner, d)) for s in ("r", "k", "v", "a", "g")]
        return specs + [
            TensorSpec(p + "a.b", (inner,)), TensorSpec(p + "w1", (self.decay_rank, d)), TensorSpec(p + "w2", (inner, self.decay_rank)),
            TensorSpec(p + "w0", (inner,)), TensorSpec(p + "norm", (inner,), init="one_plus_normal"), TensorSpec(p + "o", (d, inner)),
        ]

    def load(self, tensors, dtype, device) -> None:
        p, f32 = self.prefix, torch.float32

        def get(name: str, to=dtype) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=to).contiguous()

        self.w_main = torch.cat([get(s) for s in ("r", "k", "v", "a", "g")]).contiguous()
        self.w_low, self.w_high, self.w_o = get("w1"), get("w2"), get("o")
        self.w0, self.a_bias, self.norm_weight = get("w0", f32), get("a.b", f32), get("norm", f32)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_main, self.w_low, self.w_high, self.w_o))

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, dim = ctx.num_tokens, self.heads, self.dim
        inner = heads * dim
        f32 = torch.float32
        main = ops.linear(ctx, h, self.w_main, ctx.buffer("gdelta_main", (t, 5 * inner)))
        low = ops.linear(ctx, h, self.w_low, ctx.buffer("gdelta_low", (t, self.w_low.shape[0])))
        low = ops.tanh_rows(ctx, low)
        log_decay = ops.linear(ctx, low, self.w_high, ctx.buffer("gdelta_log_decay", (t, inner), f32))
        outs = tuple(ctx.buffer("gdelta_" + name, (t, inner), f32) for name in ("r", "k", "v", "w", "au", "u"))
        ops.delta_general_prepare(ctx, main, (0, inner, 2 * inner, 3 * inner), log_decay, self.w0, self.a_bias, heads, dim, outs)
        o = ops.delta_general_recurrence(ctx, *outs, cache.state[0], ctx.buffer("gdelta_o", (t, inner), f32), heads, dim, dim)
        y = ops.wkv_output(ctx, o, self.norm_weight, main[:, 4 * inner:], heads, dim, self.eps, ctx.buffer("attn", (t, inner)), sigmoid_gate=True)
        return ops.linear(ctx, y, self.w_o, ctx.buffer(self.out_name, (t, self.hidden_size)))


register_part("mixer", "channel_delta", ChannelDeltaRule)
register_part("mixer", "general_delta", GeneralDeltaRule)
