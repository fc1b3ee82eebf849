"""Zetizen as a recipe of parts.

``x = layernorm(table[token])``. Each layer is a parallel block, ``h = layernorm(x); x += mixer(h) + feed_forward(h)``, with
one of three attention mixers: grouped-query attention without rotation whose scores are soft-capped and get a learned
bias by distance; grouped-query attention whose values are its keys, partly rotated (frequencies stretched by a ramp), with
soft-capped scores, keys visible inside the query's chunk of positions only and a sigmoid gate per head (both as
``shaped_attention``, both with one RMS norm over all of q and one over all of k); or attention over cached low-rank latents
with queries out of a latent of their own and an element-wise output gate. The feed-forward is a routed mixture of
unclamped gated experts (the chosen experts' weights are the softmax over their logits alone) plus a shared expert, or
absent. A last layer norm, then logits against the embedding table times a constant. Every size, constant and the order
of the layers come from the configuration; the row count of a bias table comes from the checkpoint.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zetizen_config import ZetizenConfig
from ..parts.base import PartSpec
from ..parts.model import ModelRecipe


def _rotary(rot: dict, head_dim: int) -> PartSpec:
    return PartSpec("rotary", dict(head_dim=head_dim, theta=rot["base"], rotary_dims=rot["dims"], scaling=rot.get("scaling")))


def zetizen_mixer(kind: str, sizes: dict, prefix: str, hidden: int, eps: float) -> PartSpec:
    """The mixer of one layer."""
    if kind == "latent_attention":
        return PartSpec(
            "latent_attention",
            dict(
                prefix=prefix, hidden_size=hidden, heads=sizes["heads"], dim=sizes["dim"], rot_dim=sizes["rot_dim"], vdim=sizes["vdim"],
                rank=sizes["kv_rank"], q_rank=sizes["q_rank"], scale=sizes["scale"], eps=eps, position=_rotary(sizes["rot"], sizes["rot_dim"]),
                sink=False, gate=True, gate_per="element",
            ),
        )
    common = dict(
        prefix=prefix, hidden_size=hidden, heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"], vdim=sizes["vdim"],
        scale=sizes["scale"], eps=eps, qk_norm=True, softcap=sizes.get("softcap"),
    )
    if kind == "attention":
        reach = sizes.get("bias_max")
        return PartSpec("shaped_attention", dict(common, distance_bias={"rows": sizes.get("bias_rows"), "reach": reach} if reach else None))
    rot = sizes.get("rot")
    return PartSpec(
        "shaped_attention",
        dict(
            common, qk_bias=True, values="keys", gate="head", chunk=sizes["mask"]["size"] if sizes.get("mask") else 0,
            position=_rotary(rot, sizes["dim"]) if rot and rot["dims"] else None,
        ),
    )


def zetizen_feed_forward(mlp: dict | None, prefix: str, hidden: int) -> PartSpec | None:
    if mlp is None:
        return None
    shared = mlp.get("shared")
    return PartSpec(
        "routed_experts",
        dict(
            prefix=prefix, hidden_size=hidden, experts=mlp["router"]["experts"], top=mlp["router"]["top"], intermediate_size=mlp["expert"]["ff"],
            limit=0.0, router="softmax_chosen", router_bias=True, shared_size=shared["ff"] if shared else None, shared_limit=0.0,
            out_name="branch_ff",  # beside the mixer's output, not over it
        ),
    )


def zetizen_recipe(config: ZetizenConfig) -> ModelRecipe:
    hidden, eps = config.hidden_size, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        layers.append(
            PartSpec(
                "parallel_residual",
                dict(
                    mixer=zetizen_mixer(layer["type"], layer["mixer"], prefix + "mix.", hidden, eps),
                    feed_forward=zetizen_feed_forward(layer.get("mlp"), prefix + "mlp.", hidden),
                    norm=PartSpec("layernorm", dict(name=prefix + "norm1", hidden_size=hidden, eps=eps)),
                ),
            )
        )
    return ModelRecipe(
        config=config,
        embedding=PartSpec("normed_embedding", dict(name="embed", norm_name="embed.norm", vocab_size=config.vocab_size, hidden_size=hidden, eps=eps)),
        layers=layers,
        final_norm=PartSpec("layernorm", dict(name="final.norm", hidden_size=hidden, eps=eps)),
        head=PartSpec("linear_head", dict(name="head", suffix="", tied_to="embed", vocab_size=config.vocab_size, hidden_size=hidden, scale=config.logit_scale)),
    )


register_architecture(ZetizenConfig.ARCHITECTURE, ZetizenConfig.from_json_dict, zetizen_recipe, model_types=(ZetizenConfig.MODEL_TYPE,))
