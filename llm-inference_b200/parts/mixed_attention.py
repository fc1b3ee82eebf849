"""An attention mixer whose softmax weights are mixed over heads, with short convolutions and a norm over all heads in front."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import CacheSpecs, KVCacheSpec, Part, PartSpec, StateSpec, build_part, register_part
from .context import CacheView, StepContext
from .gated_attention import padded_head_size


class MixedHeadAttention(Part):
    """Causal grouped-query attention over a paged cache.

    ``q = W_q h + b_q`` (``heads x dim``), ``k = W_k h + b_k`` (``kv_heads x dim``), ``v = W_v h + b_v`` (``kv_heads x
    vdim``). Each channel of q, k and v then passes a causal convolution over ``taps`` tokens (weights
    ``[channels, taps]``, the last tap on the current token, zeros in front of a request's first token). The whole
    of q, all heads together, is divided by its root mean square and multiplied by a weight per channel, and so
    is the whole of k. The ``position`` part rotates queries and keys. Head ``g``'s weights are
    ``softmax_j(q_g . k_j * scale)`` over the keys up to the token's own, with the keys of kv head
    ``g // (heads / kv_heads)``; the weights are then mixed over heads, ``weight_h <- sum_g talk[h, g] weight_g``, and
    head ``h`` applies its mixed weights to the values of its own kv head. The concatenated heads are multiplied by
    ``sigmoid(W_g h)`` element by element; then ``W_o``.

    Since the mix acts on normalised weights, head ``h``'s output is ``sum_g talk[h, g] A[c(h)][g]`` with
    ``A[c][g]`` = head ``g``'s own softmax applied to the values of kv head ``c``: the attention kernels run once
    per kv head ``c`` (``value_head``) and one small kernel mixes and gates.

    Per-request state: the cache pages, and the last ``taps - 1`` projections (without bias, in the compute dtype).
    The four projections are one matrix ``[q | k | v | g]``. Tensor names: ``prefix + q | q.b | q.conv | q.norm | k |
    k.b | k.conv | k.norm | v | v.b | v.conv | talk | g | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, scale: float,
                 eps: float, position: PartSpec, out_name: str = "branch") -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads cannot share {kv_heads} kv heads")
        if taps < 1:
            raise ValueError("the convolution needs at least the current token's tap")
        self.prefix, self.hidden_size, self.out_name = prefix, hidden_size, out_name
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps = int(heads), int(kv_heads), int(dim), int(vdim), int(taps)
        self.scale, self.eps = float(scale), float(eps)
        self.row_dim = padded_head_size(self.dim, self.vdim)
        self.channels = (self.heads + self.kv_heads) * self.dim + self.kv_heads * self.vdim
        self.position = build_part("position", position)
        self.graph_safe = self.position.graph_safe
        self.dtype = torch.bfloat16
        self.w_in = self.bias = self.taps_w = self.q_weight = self.k_weight = self.talk = self.w_o = None

    def cache_spec(self) -> CacheSpecs:
        return CacheSpecs((KVCacheSpec(self.kv_heads, self.row_dim, 0), StateSpec(((self.taps - 1, self.channels),), (self.dtype,))))

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        specs = []
        for name, width in (("q", self.heads * self.dim), ("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)):
            specs += [TensorSpec(p + name, (width, d)), TensorSpec(p + name + ".b", (width,)),
                      TensorSpec(p + name + ".conv", (width, self.taps), init="half_plus_normal")]
        specs += [
            TensorSpec(p + "q.norm", (self.heads * self.dim,), init="one_plus_normal"),
            TensorSpec(p + "k.norm", (self.kv_heads * self.dim,), init="one_plus_normal"),
            TensorSpec(p + "talk", (self.heads, self.heads), init="half_plus_normal"),
            TensorSpec(p + "g", (self.heads * self.vdim, d)), TensorSpec(p + "o", (d, self.heads * self.vdim)),
        ]
        return specs + self.position.tensor_specs()

    def load(self, tensors, dtype, device) -> None:
        p, f32 = self.prefix, torch.float32
        self.dtype = dtype

        def get(name: str, to=dtype) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=to)

        self.w_in = torch.cat([get("q"), get("k"), get("v"), get("g")]).contiguous()
        self.bias = torch.cat([get(n + ".b", f32) for n in ("q", "k", "v")]).contiguous()
        self.taps_w = torch.cat([get(n + ".conv", f32) for n in ("q", "k", "v")]).contiguous()
        self.q_weight, self.k_weight = get("q.norm", f32).contiguous(), get("k.norm", f32).contiguous()
        self.talk = get("talk", f32).contiguous()
        self.w_o = get("o").contiguous()
        self.position.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        from . import attention_dispatch

        t, heads, kvh, row = ctx.num_tokens, self.heads, self.kv_heads, self.row_dim
        pages, slots = cache.members
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("mixed_proj", (t, self.w_in.shape[0])))
        q = ctx.buffer("q", (t, heads * row))
        self.position.apply_after_conv_norm(ctx, pages, slots.state[0], proj, self.bias, self.taps_w, self.q_weight, self.k_weight,
                                            self.eps, q, heads, kvh, self.dim, self.vdim, row)
        planes = ctx.buffer("mixed_attn", (kvh, t, heads * row))
        attention_dispatch.attend_value_planes(ctx, pages, q, planes, heads, kvh, row, self.scale)
        gated = ops.mix_heads_gate(ctx, planes, self.talk, proj[:, self.channels:], heads, kvh, self.vdim, row,
                                   ctx.buffer("attn", (t, heads * self.vdim)))
        return ops.linear(ctx, gated, self.w_o, ctx.buffer(self.out_name, (t, self.hidden_size)))


register_part("mixer", "mixed_head_attention", MixedHeadAttention)
