"""An attention mixer whose queries and keys are normed as whole vectors and whose scores are shaped before the softmax."""

from __future__ import annotations

import math

import numpy as np
import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import KVCacheSpec, Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext
from .gated_attention import padded_head_size


def distance_buckets(rows: int, reach: int) -> np.ndarray:
    """For every distance ``0 .. reach`` the row of a bias table of ``rows`` rows: distances below ``rows // 2`` have a
    row each; from there on rows are spaced evenly in the logarithm of the distance, ``half + floor(ln(n / half) /
    ln(reach / half) * (rows - half))``, and the last row takes everything from where that reaches it. Worked out in
    64-bit on the host; a kernel looks up ``min(distance, reach)``."""
    half = rows // 2
    if half < 1 or reach <= half:
        raise ValueError(f"a bias table of {rows} rows cannot spread its upper half up to a distance of {reach}")
    out = np.empty(reach + 1, dtype=np.int64)
    for n in range(reach + 1):
        out[n] = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))
    return out


class ShapedAttention(Part):
    """Causal grouped-query attention over a paged cache with whole-vector norms in front and shaped scores.

    ``q = W_q h`` (``heads x dim``), ``k = W_k h`` (``kv_heads x dim``), with biases ``q.b`` / ``k.b`` if ``qk_bias``. Values:
    ``v = W_v h`` (``kv_heads x vdim``), or, with ``values="keys"``, the keys as projected (bias added, before norm and
    rotation; there is no ``W_v`` then and ``vdim = dim``). With ``qk_norm`` all of q is divided by its root mean square
    over its ``heads * dim`` numbers and multiplied by the weight ``q.norm`` of that size, and likewise all of k
    (``k.norm``). ``position`` (a rotary part, or None) then rotates part of every head of q and k. Query head ``n`` uses
    key/value head ``n // (heads / kv_heads)``; its score for a key at or before its own position is ``q . k * scale``,
    then, with ``softcap``, ``c * tanh(score / c)``, then, with ``distance_bias = {"rows": B, "reach": D}`` (``rows`` None: the checkpoint's), plus
    ``rel[bucket(distance), n]`` (``rel`` is ``[B, heads]``, see :func:`distance_buckets`); with ``chunk`` only keys of the
    query's own chunk of ``chunk`` positions (counted from the start of the request) are visible. Softmax over the
    visible keys. With ``gate="head"`` head ``n``'s output is multiplied by ``sigmoid(W_g h)_n``. Then ``W_o``.

    The projections are one matrix ``[q | k | (v) | (g)]``; bias, norms, rotation and the cache write are one kernel.
    Keys and values share one arena row width (``padded_head_size``), as in the other mixers with ``dim`` and ``vdim``.
    Tensor names: ``prefix + q | q.b | q.norm | k | k.b | k.norm | v | rel | g | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 qk_norm: bool = True, qk_bias: bool = False, values: str = "projected", position: PartSpec | None = None,
                 softcap: float | None = None, distance_bias: dict | None = None, chunk: int = 0, gate: str | None = None,
                 out_name: str = "branch") -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads cannot share {kv_heads} kv heads")
        if values not in ("projected", "keys"):
            raise ValueError(f"values={values!r} must be 'projected' or 'keys'")
        if values == "keys" and vdim != dim:
            raise ValueError("values that are the keys have the keys' size")
        if gate not in (None, "head"):
            raise ValueError(f"gate={gate!r} must be None or 'head'")
        self.prefix, self.hidden_size, self.out_name = prefix, hidden_size, out_name
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps = float(scale), float(eps)
        self.qk_norm, self.qk_bias, self.values_from_keys, self.gate = bool(qk_norm), bool(qk_bias), values == "keys", gate
        self.softcap = float(softcap) if softcap else 0.0
        self.chunk = int(chunk or 0)
        # rows None: the table's row count is the checkpoint's (random weights need it named)
        self.has_bias = bool(distance_bias)
        self.bias_rows = int(distance_bias.get("rows") or -1) if distance_bias else 0
        self.bias_reach = int(distance_bias["reach"]) if distance_bias else 0
        if self.bias_rows > 0:
            distance_buckets(self.bias_rows, self.bias_reach)  # refuses sizes that do not fit, before any weights are read
        self.row_dim = padded_head_size(self.dim, self.vdim)
        self.position = build_part("position", position) if position is not None else None
        self.graph_safe = self.position.graph_safe if self.position is not None else True
        self.w_in = self.bias = self.q_weight = self.k_weight = self.w_o = self.bias_table = None
        self.shape = ops.NO_SHAPE

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(self.kv_heads, self.row_dim, 0)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        widths = [("q", self.heads * self.dim), ("k", self.kv_heads * self.dim)]
        specs = []
        for name, width in widths:
            specs.append(TensorSpec(p + name, (width, d)))
            if self.qk_bias:
                specs.append(TensorSpec(p + name + ".b", (width,)))
            if self.qk_norm:
                specs.append(TensorSpec(p + name + ".norm", (width,), init="one_plus_normal"))
        if not self.values_from_keys:
            specs.append(TensorSpec(p + "v", (self.kv_heads * self.vdim, d)))
        if self.has_bias:
            specs.append(TensorSpec(p + "rel", (self.bias_rows, self.heads)))
        if self.gate:
            specs.append(TensorSpec(p + "g", (self.heads, d)))
        specs.append(TensorSpec(p + "o", (d, self.heads * self.vdim)))
        return specs + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, dtype, device) -> None:
        p, f32 = self.prefix, torch.float32

        def get(name: str, to=dtype) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=to)

        names = ["q", "k"] + ([] if self.values_from_keys else ["v"]) + (["g"] if self.gate else [])
        self.w_in = torch.cat([get(n) for n in names]).contiguous()
        self.w_o = get("o").contiguous()
        if self.qk_bias:
            parts = [get("q.b", f32), get("k.b", f32)]
            if not self.values_from_keys:
                parts.append(torch.zeros(self.kv_heads * self.vdim, dtype=f32, device=device))  # the values carry no bias
            self.bias = torch.cat(parts).contiguous()
        if self.qk_norm:
            self.q_weight, self.k_weight = get("q.norm", f32).contiguous(), get("k.norm", f32).contiguous()
        if self.has_bias:
            # [heads, reach + 1]: a head's biases by distance lie side by side; the kernels clamp the distance to `reach`.
            rel = get("rel", f32)
            buckets = distance_buckets(rel.shape[0], self.bias_reach)
            self.bias_table = rel[torch.from_numpy(buckets).to(device)].t().contiguous()
        peak = self.bias_table.max(dim=1).values.contiguous() if self.bias_table is not None else None
        self.shape = ops.ScoreShape(self.softcap, self.bias_table, self.chunk, peak)
        if self.position is not None:
            self.position.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        from . import attention_dispatch

        t, heads, kvh, row = ctx.num_tokens, self.heads, self.kv_heads, self.row_dim
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("shaped_proj", (t, self.w_in.shape[0])))
        q = ctx.buffer("q", (t, heads * row))
        if self.position is not None:
            self.position.apply_after_norm(ctx, cache, proj, self.bias, self.q_weight, self.k_weight, self.eps, self.values_from_keys, q,
                                           heads, kvh, self.dim, self.vdim, row)
        else:
            ops.qk_norm_rope_write(ctx, cache, proj, self.bias, self.q_weight, self.k_weight, self.eps, None, 1.0, self.values_from_keys, q,
                                   heads, kvh, self.dim, self.vdim, row)
        attn = ctx.buffer("attn_rows", (t, heads * row))
        attention_dispatch.attend(ctx, cache, q, attn, heads, kvh, row, self.scale, shape=self.shape)
        if self.gate or row != self.vdim:
            gate_offset = (heads + kvh) * self.dim + (0 if self.values_from_keys else kvh * self.vdim)
            attn = ops.head_gate(ctx, attn, proj if self.gate else None, gate_offset, heads, self.vdim, row, ctx.buffer("attn", (t, heads * self.vdim)))
        return ops.linear(ctx, attn, self.w_o, ctx.buffer(self.out_name, (t, self.hidden_size)))


register_part("mixer", "shaped_attention", ShapedAttention)
