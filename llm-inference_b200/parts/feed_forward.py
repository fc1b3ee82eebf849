"""Feed-forward parts."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, register_part
from .context import StepContext


class SwiGLU(Part):
    """``down(silu(gate(h)) * up(h))`` without biases (python/instinct/backends/dense.py:124-128).
    The gate and up matrices are stored as one ``[2 * intermediate, hidden]`` matrix with their
    rows interleaved (row 2j is gate_j, row 2j + 1 is up_j), so one matrix product yields each
    gate next to its up value and the activation can run in that product's epilogue."""

    def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int) -> None:
        self.prefix, self.hidden_size, self.intermediate_size = prefix, hidden_size, intermediate_size
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(f"{p}gate_proj.weight", (i, h)),
            TensorSpec(f"{p}up_proj.weight", (i, h)),
            TensorSpec(f"{p}down_proj.weight", (h, i)),
        ]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        gate, up = (tensors[f"{p}{n}.weight"].to(device=device, dtype=dtype) for n in ("gate_proj", "up_proj"))
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size).contiguous()
        self.w_down = tensors[f"{p}down_proj.weight"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    takes_folded = True  # `h` may be ops.FoldedRows: the gate/up product applies the norm's 1 / rms
    takes_sink = True  # with a sink the down product adds into the residual stream itself

    def forward(self, ctx: StepContext, h, sink: ops.ResidualSink | None = None):
        t, i = ctx.num_tokens, self.intermediate_size
        act = ctx.buffer("act", (t, i))
        if not ops.linear_swiglu(ctx, h, self.w_gate_up, act):
            gate_up = ops.linear(ctx, h, self.w_gate_up, ctx.buffer("gate_up", (t, 2 * i)))
            ops.silu_mul(ctx, gate_up, act)
        if sink is not None:
            folded = ops.linear_into_residual(ctx, act, self.w_down, sink)
            if folded is not None:
                return folded
        return ops.linear(ctx, act, self.w_down, ctx.buffer("branch", (t, self.hidden_size)))


class PolyNormFeedForward(Part):
    """``down(act(up(h)))`` without biases, ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with powers
    taken element by element and ``N`` dividing a token's row by its root mean square
    (``eps`` inside the root); ``a, b, c, e`` are the four numbers of the ``act`` tensor."""

    def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int, eps: float) -> None:
        self.prefix, self.hidden_size, self.intermediate_size, self.eps = prefix, hidden_size, intermediate_size, float(eps)
        self.w_up = self.w_down = self.coefficients = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(f"{p}up", (i, h)), TensorSpec(f"{p}down", (h, i)), TensorSpec(f"{p}act", (4,), init="half_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        self.w_up = tensors[f"{p}up"].to(device=device, dtype=dtype).contiguous()
        self.w_down = tensors[f"{p}down"].to(device=device, dtype=dtype).contiguous()
        self.coefficients = tensors[f"{p}act"].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        t, i = ctx.num_tokens, self.intermediate_size
        z = ops.linear(ctx, h, self.w_up, ctx.buffer("ff_up", (t, i)))
        act = ops.poly_norm(ctx, z, self.coefficients, self.eps, ctx.buffer("act", (t, i)))
        return ops.linear(ctx, act, self.w_down, ctx.buffer("branch", (t, self.hidden_size)))


class ClampedGLU(Part):
    """``down(y)`` with ``g = min(gate(h), limit)``, ``u = clamp(up(h), -limit, limit)``, ``y = g * sigmoid(1.702 g) * (u + 1)``,
    no biases. The gate and up matrices are one ``[2 * intermediate, hidden]`` matrix (gate rows first), so one
    product gives both. Tensor names: ``prefix + gate | up | down``."""

    def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int, limit: float) -> None:
        self.prefix, self.hidden_size, self.intermediate_size, self.limit = prefix, hidden_size, int(intermediate_size), float(limit)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate", (i, h)), TensorSpec(p + "up", (i, h)), TensorSpec(p + "down", (h, i))]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate"].to(device=device, dtype=dtype), tensors[p + "up"].to(device=device, dtype=dtype)]).contiguous()
        self.w_down = tensors[p + "down"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        t, i = ctx.num_tokens, self.intermediate_size
        gate_up = ops.linear(ctx, h, self.w_gate_up, ctx.buffer("gate_up", (t, 2 * i)))
        act = ops.clamped_glu(ctx, gate_up, self.limit, ctx.buffer("act", (t, i)))
        return ops.linear(ctx, act, self.w_down, ctx.buffer("branch", (t, self.hidden_size)))


class RoutedExperts(Part):
    """A mixture of ``experts`` small gated feed-forward layers of which each token uses ``top``, plus an
    optional shared expert that every token uses.

    Expert (no biases): ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``,
    ``y = g * sigmoid(1.702 g) * (u + 1)``, output ``W_down y``. Router, in 32-bit: ``s = sigmoid(W_router h)``;
    the experts form ``group_count`` equal groups of neighbours, a group scores the sum of its two
    largest ``s``, and only experts of the ``group_keep`` best groups can be chosen; the ``top`` largest
    ``s`` among them are chosen and weighted ``s / (sum of the chosen s + 1e-20) * route_scale``. The output
    is the weighted sum of the chosen experts' outputs plus the shared expert's.

    ``router="softmax_chosen"`` is another router: the ``top`` largest logits ``W_router h`` (+ ``router.b`` with
    ``router_bias``) are chosen and weighted by the softmax over the chosen logits alone (times ``route_scale``); it has no
    groups. A ``limit`` of zero makes an expert ``W_down (silu(W_gate h) * (W_up h))``, without clamps. ``out_name`` is the
    buffer the result goes to (a layer that runs its feed-forward beside its mixer gives it one of its own).

    The experts' matrices are stacked (``[experts, 2 ff, hidden]`` with the gate rows first, and
    ``[experts, hidden, ff]``); a step sorts its (token, choice) pairs by expert and the two products
    walk the sorted runs, so only chosen experts' weights are read. Tensor names: ``prefix + router |
    e<j>.{gate,up,down} | shared.{gate,up,down}``."""

    def __init__(self, *, prefix: str, hidden_size: int, experts: int, top: int, intermediate_size: int, limit: float,
                 route_scale: float = 1.0, group_count: int = 1, group_keep: int = 1, shared_size: int | None = None,
                 shared_limit: float | None = None, router: str = "sigmoid_groups", router_bias: bool = False,
                 out_name: str = "branch") -> None:
        if router not in ("sigmoid_groups", "softmax_chosen"):
            raise ValueError(f"router={router!r} must be 'sigmoid_groups' or 'softmax_chosen'")
        if router == "softmax_chosen" and (group_count != 1 or group_keep != 1):
            raise ValueError("the router that weighs by a softmax over the chosen logits has no groups")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.router, self.router_bias, self.out_name = router, bool(router_bias), out_name
        self.b_router = None
        self.experts, self.top, self.intermediate_size, self.limit = int(experts), int(top), int(intermediate_size), float(limit)
        self.route_scale, self.group_count, self.group_keep = float(route_scale), int(group_count), int(group_keep)
        self.shared_size = int(shared_size) if shared_size else 0
        self.shared_limit = float(shared_limit) if shared_limit is not None else self.limit
        self.w_router = self.w_gate_up = self.w_down = self.w_shared_gate_up = self.w_shared_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        specs = [TensorSpec(p + "router", (self.experts, h))]
        if self.router_bias:
            specs.append(TensorSpec(p + "router.b", (self.experts,)))
        for e in range(self.experts):
            specs += [TensorSpec(f"{p}e{e}.gate", (i, h)), TensorSpec(f"{p}e{e}.up", (i, h)), TensorSpec(f"{p}e{e}.down", (h, i))]
        if self.shared_size:
            s = self.shared_size
            specs += [TensorSpec(p + "shared.gate", (s, h)), TensorSpec(p + "shared.up", (s, h)), TensorSpec(p + "shared.down", (h, s))]
        return specs

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix

        def get(name: str) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=dtype)

        self.w_router = get("router").contiguous()
        if self.router_bias:
            self.b_router = tensors[p + "router.b"].to(device=device, dtype=torch.float32).contiguous()
        self.w_gate_up = torch.stack([torch.cat([get(f"e{e}.gate"), get(f"e{e}.up")]) for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([get(f"e{e}.down") for e in range(self.experts)]).contiguous()
        if self.shared_size:
            self.w_shared_gate_up = torch.cat([get("shared.gate"), get("shared.up")]).contiguous()
            self.w_shared_down = get("shared.down").contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router, the shared expert and ``top`` experts per token is the
        least; counted here is the router, the shared expert and every expert once."""
        tensors = [self.w_router, self.w_gate_up, self.w_down, self.w_shared_gate_up, self.w_shared_down]
        return sum(w.numel() * w.element_size() for w in tensors if w is not None)

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        t, width = ctx.num_tokens, self.hidden_size
        logits = ops.linear(ctx, h, self.w_router, ctx.buffer("moe_logits", (t, self.experts), torch.float32))
        # Every routed layer keeps the step's choices in a buffer of its own, so that they can be read after
        # the step (expert load statistics, tests), also when the step was replayed from a captured graph.
        ids = ctx.buffer("moe_ids:" + self.prefix, (t, self.top), torch.int32)
        weights = ctx.buffer("moe_weights", (t, self.top), torch.float32)
        ops.moe_route(ctx, logits, self.group_count, self.group_keep, self.top, self.route_scale, ids, weights, bias=self.b_router,
                      softmax_chosen=self.router == "softmax_chosen")
        expert_out = ops.moe_experts(
            ctx, h, ids, self.w_gate_up, self.w_down, self.limit, ctx.buffer("moe_expert_out", (t * self.top, width), torch.float32, per_token=False)
        )
        shared = None
        if self.shared_size:
            gate_up = ops.linear(ctx, h, self.w_shared_gate_up, ctx.buffer("gate_up", (t, 2 * self.shared_size)))
            act = ops.clamped_glu(ctx, gate_up, self.shared_limit, ctx.buffer("act", (t, self.shared_size)))
            shared = ops.linear(ctx, act, self.w_shared_down, ctx.buffer("moe_shared", (t, width)))
        return ops.moe_combine(ctx, expert_out, weights, shared, ctx.buffer(self.out_name, (t, width)))


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "poly_norm", PolyNormFeedForward)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "clamped_glu", ClampedGLU)
