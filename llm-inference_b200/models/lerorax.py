"""Lerorax as a recipe of parts.

``x = table[token] + pairs[hash(previous token, token)]``. Each layer adds the RMS norm (weight stored as an
offset from one) of its branches' outputs to a 32-bit stream that the branches read directly:
``x += norm1(mixer(x)); x += norm2(ff(x))``. The mixer is a minGRU, or two mixers side by side whose normed
outputs are averaged: attention with short convolutions, a norm over all heads, partial interleaved rotation
with stretched long wavelengths, softmax weights mixed over heads and an output gate; and a generalized delta
rule with a decay and a removal share per key channel. The feed-forward is a clamped gated unit or absent. A
layer may run another layer's tensors against a cache and state of its own. A last norm, then an untied head.
Every size, constant and the order of the layers come from the configuration.
"""

from __future__ import annotations

from ..config.lerorax_config import LeroraxConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import LayerCall, ModelRecipe


def lerorax_recipe(config: LeroraxConfig) -> ModelRecipe:
    hidden, eps = config.hidden_size, config.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("grouped_rmsnorm", dict(name=name, hidden_size=hidden, groups=1, eps=eps, around_zero=True))

    layers: list[PartSpec] = []
    block_of: dict[int, int] = {}  # layer that owns tensors -> its place among the blocks
    for index, layer in enumerate(config.layers):
        if config.owner(index) != index:
            continue
        prefix = f"l{index}."
        sizes = layer["mixer"]
        if layer["type"] == "mingru":
            mixer = PartSpec("mingru", dict(prefix=prefix + "mix.", hidden_size=hidden, width=sizes["width"]))
        else:
            left, right = sizes["left"], sizes["right"]
            rot = left.get("rot") or {}
            first = PartSpec(
                "mixed_head_attention",
                dict(
                    prefix=prefix + "mix.left.", hidden_size=hidden, heads=left["heads"], kv_heads=left["kv_heads"], dim=left["dim"],
                    vdim=left["vdim"], taps=left["conv"], scale=left["scale"], eps=eps,
                    position=PartSpec(
                        "rotary",
                        dict(head_dim=left["dim"], theta=rot.get("base", 10000.0), rotary_dims=rot.get("dims", 0), interleaved=True,
                             scaling=rot.get("scaling")),
                    ),
                ),
            )
            second = PartSpec(
                "general_delta",
                dict(prefix=prefix + "mix.right.", hidden_size=hidden, heads=right["heads"], dim=right["dim"], eps=eps,
                     decay_rank=right.get("decay_rank")),
            )
            mixer = PartSpec(
                "parallel_mixers",
                dict(first=first, second=second, names=(prefix + "mix.left.out", prefix + "mix.right.out"), hidden_size=hidden, eps=eps),
            )
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            feed_forward = PartSpec("clamped_glu", dict(prefix=prefix + "mlp.", hidden_size=hidden, intermediate_size=mlp["ff"], limit=mlp["limit"]))
        block_of[index] = len(layers)
        layers.append(
            PartSpec(
                "post_norm_residual",
                dict(
                    mixer=mixer, feed_forward=feed_forward, mixer_norm=norm(prefix + "norm1"),
                    feed_forward_norm=norm(prefix + "norm2") if mlp is not None else None, hidden_size=hidden,
                    unused=() if mlp is not None else (prefix + "norm2",),
                ),
            )
        )
    # Every layer of the configuration is one call; a layer that names another's tensors runs that block
    # against the cache entry with its own number.
    schedule = [LayerCall(block_of[config.owner(index)], cache=index) for index in range(len(config.layers))]
    if config.bigram is not None:
        embedding = PartSpec(
            "bigram_embedding",
            dict(name="embed", pairs_name="bigram", vocab_size=config.vocab_size, hidden_size=hidden, cast=True, **config.bigram),
        )
    else:
        embedding = PartSpec("token_embedding", dict(name="embed", suffix="", vocab_size=config.vocab_size, hidden_size=hidden, cast=True))
    return ModelRecipe(
        config=config,
        embedding=embedding,
        layers=layers,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(name="head", suffix="", vocab_size=config.vocab_size, hidden_size=hidden)),
        schedule=schedule,
    )


register_architecture(LeroraxConfig.ARCHITECTURE, LeroraxConfig.from_json_dict, lerorax_recipe, model_types=(LeroraxConfig.MODEL_TYPE,))
