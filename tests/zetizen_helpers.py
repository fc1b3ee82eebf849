"""Small Zetizen configurations and weights drawn here (not by the engine)."""

from __future__ import annotations

import numpy as np
import torch


def scaling(factor=3.0, original=64, fast=8.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def biased_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.6, softcap=8.0, bias=(40, 12)):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        mixer["softcap"] = softcap
    if bias:
        mixer["bias_max"], mixer["bias_rows"] = bias
    return {"type": "attention", "mixer": mixer}


def chunked_layer(heads=4, kv_heads=1, dim=24, scale=0.5, softcap=5.0, chunk=20, rot=(8, 100.0, scaling())):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if softcap:
        mixer["softcap"] = softcap
    if chunk:
        mixer["mask"] = {"size": chunk}
    if rot:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
        if rot[2]:
            mixer["rot"]["scaling"] = rot[2]
    return {"type": "attention_2", "mixer": mixer}


def latent_layer(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, q_rank=10, scale=0.5, base=50.0, scale_rule=scaling(2.0, 32, 4.0, 0.5)):
    rot = {"dims": rot_dim, "base": base}
    if scale_rule:
        rot["scaling"] = scale_rule
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}}


def moe(experts=6, top=2, ff=20, shared=12):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def with_mlp(layer: dict, mlp: dict | None) -> dict:
    return dict(layer, mlp=mlp)


def config_of(width, vocab, layers, eps=1e-5, logit_scale=0.5) -> dict:
    out = {"architecture": "Zetizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if logit_scale is not None:
        out["logit_scale"] = logit_scale
    return out


# Three configurations that differ in every size. ALPHA: one layer of each kind and a fourth without cap, bias or
# feed-forward partner sizes of the first; keys and values of different sizes; a chunk that ends inside a page; every
# expert chosen in one layer. BETA: the latent layer first, with an odd latent size, unscaled frequencies and one head;
# a chunked layer without chunks, rotation or cap; heads that each have their own key/value head and values wider than
# 128; one expert per token, no shared expert, a layer without feed-forward, no logit scale. GAMMA: sizes the
# tensor-core kernels take (heads of 64 and 128, a latent of 64 + 16), whole heads rotated, a chunk that is no multiple
# of the page.
ALPHA = config_of(
    48, 97,
    [
        with_mlp(biased_layer(), moe()),
        with_mlp(chunked_layer(), None),
        with_mlp(latent_layer(), moe(experts=5, top=3, ff=28, shared=None)),
        with_mlp(biased_layer(heads=2, kv_heads=2, dim=8, vdim=8, scale=1.0, softcap=None, bias=None), moe(experts=4, top=4, ff=36, shared=8)),
        with_mlp(chunked_layer(heads=6, kv_heads=2, dim=16, scale=0.7, softcap=3.0, chunk=9, rot=(16, 30.0, None)), moe(experts=3, top=1, ff=16)),
    ],
)
BETA = config_of(
    40, 131,
    [
        with_mlp(latent_layer(heads=1, dim=6, rot_dim=2, vdim=5, kv_rank=7, q_rank=3, scale=0.9, scale_rule=None), moe(experts=7, top=1, ff=70, shared=None)),
        with_mlp(chunked_layer(heads=5, kv_heads=5, dim=8, scale=1.1, softcap=None, chunk=0, rot=None), None),
        with_mlp(biased_layer(heads=3, kv_heads=3, dim=8, vdim=136, scale=0.8, softcap=2.0, bias=(9, 6)), moe(experts=2, top=2, ff=33, shared=40)),
        with_mlp(latent_layer(heads=5, dim=24, rot_dim=8, vdim=8, kv_rank=12, q_rank=30, scale=0.3, base=1000.0), None),
    ],
    eps=3e-4, logit_scale=None,
)
GAMMA = config_of(
    64, 113,
    [
        with_mlp(biased_layer(heads=3, kv_heads=1, dim=64, vdim=64, scale=0.3, softcap=12.0, bias=(70, 20)), moe(experts=12, top=3, ff=32, shared=64)),
        with_mlp(chunked_layer(heads=2, kv_heads=2, dim=128, scale=0.2, softcap=15.0, chunk=44, rot=(128, 10000.0, scaling(4.0, 48, 16.0, 1.0))), moe(experts=8, top=2, ff=48)),
        with_mlp(latent_layer(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=32, scale=0.25, base=500.0, scale_rule=scaling(2.0, 40, 8.0, 1.0)), moe(experts=2, top=1, ff=16, shared=None)),
        with_mlp(biased_layer(heads=4, kv_heads=2, dim=64, vdim=32, scale=0.3, softcap=None, bias=(33, 8)), None),
    ],
    logit_scale=2.0,
)
# DELTA: sizes that are multiples of nothing in particular (a width of 50, heads of 10 and 14, a latent of 10 + 6, values of 7,
# an odd vocabulary, expert widths of 18 and 9, a table of 7 rows, chunks of 5, a chunk of one position).
DELTA = config_of(
    50, 101,
    [
        with_mlp(chunked_layer(heads=3, kv_heads=3, dim=10, scale=0.6, softcap=4.0, chunk=5, rot=(6, 77.0, scaling(1.5, 20, 3.0, 0.7))), moe(experts=3, top=2, ff=18, shared=9)),
        with_mlp(latent_layer(heads=2, dim=10, rot_dim=6, vdim=7, kv_rank=10, q_rank=5, scale=0.45, base=123.0, scale_rule=scaling(5.0, 16, 2.0, 0.25)), moe(experts=9, top=4, ff=10, shared=None)),
        with_mlp(biased_layer(heads=5, kv_heads=1, dim=14, vdim=6, scale=0.55, softcap=6.5, bias=(25, 7)), None),
        with_mlp(chunked_layer(heads=2, kv_heads=1, dim=18, scale=0.5, softcap=None, chunk=1, rot=(2, 9.0, None)), moe(experts=2, top=1, ff=26, shared=5)),
    ],
    eps=2e-6, logit_scale=1.75,
)
CONFIGS = {"alpha": ALPHA, "beta": BETA, "gamma": GAMMA, "delta": DELTA}


def draw_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 weights at the scales of a trained model, by tensor name: linear weights N(0, 1/in) times a gain, norm
    weights around one, biases of a size that shows, distance biases of order one, router logits wide enough that
    choices are clear. Scores come out a few units wide (see the layers' ``scale``), so that single keys carry weight."""
    rng = np.random.default_rng(seed)
    width, vocab = config["width"], config["vocab"]
    out: dict[str, np.ndarray] = {}

    def linear(name, rows, cols, gain=1.0):
        out[name] = rng.normal(0.0, gain / np.sqrt(cols), (rows, cols))

    def near_one(name, count, spread=0.2):
        out[name] = 1.0 + rng.normal(0.0, spread, count)

    out["embed"] = rng.normal(0.0, 1.0, (vocab, width)) + rng.normal(0.0, 0.5, (vocab, 1))  # rows with a mean of their own
    near_one("embed.norm", width), near_one("final.norm", width)
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        near_one(p + "norm1", width)
        heads = m["heads"]
        if layer["type"] == "latent_attention":
            dim, rot, vdim, rank, q_rank = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            linear(p + "mix.dq", q_rank, width), near_one(p + "mix.dq.norm", q_rank)
            linear(p + "mix.uq", heads * (dim + rot), q_rank, 2.0)
            linear(p + "mix.dkv", rank + rot, width, 2.0), near_one(p + "mix.dkv.norm", rank)
            linear(p + "mix.uk", heads * dim, rank, 2.0), linear(p + "mix.uv", heads * vdim, rank)
            linear(p + "mix.g", heads * vdim, width, 2.0), linear(p + "mix.o", width, heads * vdim)
        else:
            kvh, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
            linear(p + "mix.q", heads * dim, width), linear(p + "mix.k", kvh * dim, width)
            near_one(p + "mix.q.norm", heads * dim, 0.3), near_one(p + "mix.k.norm", kvh * dim, 0.3)
            if layer["type"] == "attention":
                linear(p + "mix.v", kvh * vdim, width)
                if m.get("bias_max"):
                    out[p + "mix.rel"] = rng.normal(0.0, 1.0, (m["bias_rows"], heads))
            else:
                out[p + "mix.q.b"] = rng.normal(0.0, 0.5, heads * dim)
                out[p + "mix.k.b"] = rng.normal(0.0, 0.5, kvh * dim)
                linear(p + "mix.g", heads, width, 2.0)
            linear(p + "mix.o", width, heads * vdim)
        mlp = layer.get("mlp")
        if mlp is not None:
            experts, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            linear(p + "mlp.router", experts, width, 3.0)
            out[p + "mlp.router.b"] = rng.normal(0.0, 0.5, experts)
            for e in range(experts):
                linear(f"{p}mlp.e{e}.gate", ff, width, 2.0), linear(f"{p}mlp.e{e}.up", ff, width, 2.0), linear(f"{p}mlp.e{e}.down", width, ff)
            if mlp.get("shared"):
                s = mlp["shared"]["ff"]
                linear(p + "mlp.shared.gate", s, width, 2.0), linear(p + "mlp.shared.up", s, width, 2.0), linear(p + "mlp.shared.down", width, s)
    return {name: torch.from_numpy(np.ascontiguousarray(value)).to(torch.bfloat16) for name, value in out.items()}
