"""Attention whose keys and values are expanded from one cached low-rank latent per token."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import KVCacheSpec, Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class LatentAttention(Part):
    """Causal attention over cached latents.

    Per token ``W_dkv h`` gives ``rank`` numbers, RMS-normed into the latent ``c``, plus
    ``rot_dim`` numbers that, rotated at the token's position, are a key part shared by all heads;
    only these ``rank + rot_dim`` numbers are cached. Head ``n`` has the query
    ``[q_plain (dim) | q_rot (rot_dim)]`` from ``W_q h``, the key ``[W_uk[n] c | k_rot]`` and the
    value ``W_uv[n] c``; the score is ``(q_plain . W_uk[n] c + q_rot . k_rot) * scale``. Since
    ``q_plain . W_uk[n] c = (W_uk[n]^T q_plain) . c``, the query is carried into the latent space by
    one small product per head, the attention kernel works on the cached rows as they are, and its
    result ``sum_j p_j c_j`` is expanded by ``W_uv[n]`` afterwards. With ``sink`` the softmax's
    denominator also holds ``exp(sink[n])`` (no key, no value, not scaled); with ``gate`` a head's
    output is multiplied by ``sigmoid(W_g h)[n]``. Then ``W_o`` on the concatenated heads.

    With ``q_rank`` the queries come out of a latent of their own: ``q = W_uq rmsnorm(W_dq h)`` (weight ``dq.norm``)
    instead of ``W_q h``. With ``gate_per="element"`` the gate is one number per output number: the concatenated heads are
    multiplied element by element by ``sigmoid(W_g h)`` (``W_g`` is ``[heads * vdim, hidden]``) after the expansion by
    ``W_uv``. The position part may pair neighbours or halves of the rotated part.

    The query (or its latent), latent and gate projections are one matrix product. Tensor names are
    ``prefix + q | dq | dq.norm | uq | dkv | dkv.norm | uk | uv | sink | g | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, rank: int,
                 scale: float, eps: float, position: PartSpec, sink: bool = True, gate: bool = True, window: int = 0,
                 q_rank: int | None = None, gate_per: str = "head", out_name: str = "branch") -> None:
        if gate_per not in ("head", "element"):
            raise ValueError(f"gate_per={gate_per!r} must be 'head' or 'element'")
        self.prefix, self.hidden_size, self.out_name = prefix, hidden_size, out_name
        self.q_rank = int(q_rank) if q_rank else 0
        self.gate_per_element = bool(gate) and gate_per == "element"
        self.w_uq = self.q_norm_weight = None
        self.heads, self.dim, self.rot_dim, self.vdim, self.rank = heads, dim, rot_dim, vdim, rank
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.has_sink, self.has_gate = bool(sink), bool(gate)
        self.position = build_part("position", position)
        self.graph_safe = self.position.graph_safe
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.sink = self.norm_weight = None

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(1, self.rank + self.rot_dim, self.window, planes=1)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        q_width = self.heads * (self.dim + self.rot_dim)
        if self.q_rank:
            specs = [TensorSpec(p + "dq", (self.q_rank, d)), TensorSpec(p + "dq.norm", (self.q_rank,), init="one_plus_normal"),
                     TensorSpec(p + "uq", (q_width, self.q_rank))]
        else:
            specs = [TensorSpec(p + "q", (q_width, d))]
        specs += [
            TensorSpec(p + "dkv", (self.rank + self.rot_dim, d)),
            TensorSpec(p + "dkv.norm", (self.rank,), init="one_plus_normal"),
            TensorSpec(p + "uk", (self.heads * self.dim, self.rank)),
            TensorSpec(p + "uv", (self.heads * self.vdim, self.rank)),
            TensorSpec(p + "o", (d, self.heads * self.vdim)),
        ]
        if self.has_sink:
            specs.append(TensorSpec(p + "sink", (self.heads,)))
        if self.has_gate:
            specs.append(TensorSpec(p + "g", (self.heads * self.vdim if self.gate_per_element else self.heads, d)))
        return specs + self.position.tensor_specs()

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        names = ["dq" if self.q_rank else "q", "dkv"] + (["g"] if self.has_gate else [])
        if self.q_rank:
            self.w_uq = tensors[p + "uq"].to(device=device, dtype=dtype).contiguous()
            self.q_norm_weight = tensors[p + "dq.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.w_in = torch.cat([tensors[p + n].to(device=device, dtype=dtype) for n in names]).contiguous()
        # [heads, rank, dim]: the product that carries a query into the latent space reads W_uk[n]^T.
        self.w_uk_t = tensors[p + "uk"].to(device=device, dtype=dtype).view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[p + "uv"].to(device=device, dtype=dtype).view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors[p + "o"].to(device=device, dtype=dtype).contiguous()
        self.norm_weight = tensors[p + "dkv.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.sink = tensors[p + "sink"].to(device=device, dtype=torch.float32).contiguous() if self.has_sink else None
        self.position.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.w_uq) if w is not None)

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, rank, rot = ctx.num_tokens, self.heads, self.rank, self.rot_dim
        q_width = heads * (self.dim + rot)
        width = self.w_in.shape[0]
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("latent_in", (t, width)))
        q_rot = ctx.buffer("latent_q_rot", (t, heads * rot))
        if self.q_rank:
            # queries through their own latent: norm of the first q_rank columns, then one more product
            latent_q = ops.rms_rows(ctx, proj[:, : self.q_rank], self.q_norm_weight, self.eps, ctx.buffer("latent_cq", (t, self.q_rank)))
            queries = ops.linear(ctx, latent_q, self.w_uq, ctx.buffer("latent_queries", (t, q_width)))
            kv_offset = self.q_rank
            self.position.apply_latent(ctx, cache, proj, 0, kv_offset, heads, self.dim, rank, self.norm_weight, self.eps, q_rot, q_proj=queries)
        else:
            queries, kv_offset = proj[:, :q_width], q_width
            self.position.apply_latent(ctx, cache, proj, 0, kv_offset, heads, self.dim, rank, self.norm_weight, self.eps, q_rot)
        q_plain = queries.view(t, heads, self.dim + rot)[:, :, : self.dim].transpose(0, 1)
        q_lat = ops.linear_per_head(ctx, q_plain, self.w_uk_t, ctx.buffer("latent_q", (heads, t, rank)))
        gate = proj[:, kv_offset + rank + rot :] if self.has_gate else None
        mixed = ctx.buffer("latent_out", (heads, t, rank))
        self.attend(ctx, cache, q_lat, q_rot, None if self.gate_per_element else gate, mixed)
        attn = ctx.buffer("attn", (t, heads * self.vdim))
        ops.linear_per_head(ctx, mixed, self.w_uv, attn.view(t, heads, self.vdim).transpose(0, 1))
        if self.gate_per_element:
            attn = ops.sigmoid_mul(ctx, attn, gate, ctx.buffer("attn_gated", (t, heads * self.vdim)))
        return ops.linear(ctx, attn, self.w_o, ctx.buffer(self.out_name, (t, self.hidden_size)))

    def attend(self, ctx: StepContext, cache: CacheView, q_lat, q_rot, gate, out) -> None:
        from . import attention_dispatch

        attention_dispatch.attend_latent(ctx, cache, q_lat, q_rot, self.sink, gate, out, self.heads, self.rank, self.rot_dim, self.scale)


register_part("mixer", "latent_attention", LatentAttention)
