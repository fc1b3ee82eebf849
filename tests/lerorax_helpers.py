"""Small Lerorax configurations and weights drawn here (not by the engine)."""

from __future__ import annotations

import numpy as np
import torch


def mingru_layer(width=56):
    return {"type": "mingru", "mixer": {"width": width}}


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, scale=0.3, rot=(8, 100.0), scaling=None, right_heads=3, right_dim=8, decay_rank=5):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale}
    if rot is not None:
        left["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling is not None:
            left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    right = {"heads": right_heads, "dim": right_dim}
    if decay_rank is not None:  # the key only serves to draw random weights from a configuration; a checkpoint's shapes say it too
        right["decay_rank"] = decay_rank
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def with_mlp(layer: dict, ff: int | None, limit: float = 2.5) -> dict:
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff, "limit": limit})


def same_as(layers: list[dict], index: int) -> dict:
    """A layer that runs layer ``index``'s tensors against a cache and state of its own."""
    return dict(layers[index], weights_of=index)


def config_of(width, vocab, layers, bigram=(61, 31, 5), eps=1e-5) -> dict:
    out = {"architecture": "Lerorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram is not None:
        out["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    return out


# Four configurations that differ in every size. ALPHA: the pair of mixers first, keys and values of different
# widths, half of each head rotated with stretched long wavelengths (the three ranges of wavelengths all occur),
# a layer without a feed-forward, a layer that runs an earlier layer's tensors, a delta rule with other heads than
# the attention. BETA: the minGRU first, all query heads on one key/value head, a single tap (no convolution
# state), no rotation at all, one head per key/value head with whole heads rotated and plain frequencies, a
# chain of two layers on the same tensors, no bigram table, a clamp that bites often. GAMMA: heads of 64 over
# pages that the tensor-core attention kernels take, five taps, one delta head of a width that is no multiple of four.
_ALPHA = [
    with_mlp(parallel_layer(scaling=(4.0, 1.0, 4.0, 64)), 80),
    with_mlp(mingru_layer(), 64, limit=1.5),
    with_mlp(parallel_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=2, scale=0.6, rot=(8, 50.0), right_heads=1, right_dim=20, decay_rank=3), None),
]
ALPHA = config_of(48, 97, _ALPHA + [same_as(_ALPHA, 0), with_mlp(mingru_layer(40), None)])
_BETA = [
    with_mlp(mingru_layer(24), 72, limit=0.4),
    with_mlp(parallel_layer(heads=5, kv_heads=1, dim=12, vdim=6, conv=1, scale=0.45, rot=None, right_heads=2, right_dim=40, decay_rank=None), 48),
    with_mlp(parallel_layer(heads=3, kv_heads=3, dim=8, vdim=20, conv=4, scale=0.5, rot=(8, 1e4), right_heads=5, right_dim=6, decay_rank=7), None),
]
BETA = config_of(40, 131, _BETA + [same_as(_BETA, 1), same_as(_BETA, 0), dict(same_as(_BETA, 1), weights_of=3)], bigram=None, eps=3e-4)
_GAMMA = [
    with_mlp(parallel_layer(heads=6, kv_heads=2, dim=64, vdim=64, conv=5, scale=0.11, rot=(48, 2e5), scaling=(6.0, 1.0, 3.0, 256), right_heads=1, right_dim=30, decay_rank=4), 96),
    with_mlp(mingru_layer(200), 64),
]
GAMMA = config_of(64, 113, _GAMMA + [same_as(_GAMMA, 0)], bigram=(7, 1, 1))
# DELTA: heads of 128 on two key/value heads (prompt portions take the tcgen05 attention kernel), two taps.
_DELTA = [
    with_mlp(mingru_layer(72), 56),
    with_mlp(parallel_layer(heads=4, kv_heads=2, dim=128, vdim=128, conv=2, scale=0.07, rot=(64, 1e4), right_heads=2, right_dim=16, decay_rank=3), 64),
]
DELTA = config_of(56, 101, _DELTA + [same_as(_DELTA, 1)], bigram=(13, 5, 3))
CONFIGS = {"alpha": ALPHA, "beta": BETA, "gamma": GAMMA, "delta": DELTA}


def owner(config: dict, index: int) -> int:
    while config["layers"][index].get("weights_of") is not None:
        index = config["layers"][index]["weights_of"]
    return index


def draw_weights(config: dict, seed: int, sharp: float = 3.0) -> dict[str, torch.Tensor]:
    """bfloat16 weights at the scales of a trained model, by tensor name: linear weights N(0, 1/in), query norm
    weights ``sharp`` times those of the keys (so that a softmax picks few keys and a wrong or missing key moves
    the result), a head mix with negative entries, taps around "the current token", decays and update gates
    spread between channels that forget in a few tokens and channels that keep hundreds."""
    rng = np.random.default_rng(seed)
    width, vocab = config["width"], config["vocab"]
    out: dict[str, np.ndarray] = {}

    def linear(name, rows, cols, gain=1.0):
        out[name] = rng.normal(0.0, gain / np.sqrt(cols), (rows, cols))

    def near_one(name, n, spread=0.2, centre=1.0):
        out[name] = centre + rng.normal(0.0, spread, n)

    out["embed"] = rng.normal(0.0, 1.0, (vocab, width))
    big = config.get("embedding", {}).get("bigram")
    if big:
        out["bigram"] = rng.normal(0.0, 1.0, (big["buckets"] + 1, width))
    linear("head", vocab, width, 2.0)
    near_one("final.norm", width, centre=0.0)
    for index, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{index}.", layer["mixer"]
        near_one(p + "norm1", width, centre=0.0)
        if layer["type"] == "mingru":
            w = m["width"]
            linear(p + "mix.z", w, width, 2.0), linear(p + "mix.x", w, width, 2.0), linear(p + "mix.g", w, width, 2.0), linear(p + "mix.o", width, w)
            out[p + "mix.z.b"] = rng.permutation(np.linspace(-5.0, 1.0, w))
            out[p + "mix.x.b"] = rng.normal(0.0, 0.5, w)
        else:
            left, right = m["left"], m["right"]
            heads, kvh, dim, vdim, taps = left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["conv"]
            q = p + "mix.left."
            for name, rows in (("q", heads * dim), ("k", kvh * dim), ("v", kvh * vdim)):
                linear(q + name, rows, width, 2.0)
                out[q + name + ".b"] = rng.normal(0.0, 0.3, rows)
                out[q + name + ".conv"] = rng.normal(0.0, 0.4, (rows, taps)) + np.eye(1, taps, taps - 1)
            near_one(q + "q.norm", heads * dim, centre=sharp), near_one(q + "k.norm", kvh * dim)
            out[q + "talk"] = np.eye(heads) * 0.7 + rng.normal(0.0, 0.35, (heads, heads))
            linear(q + "g", heads * vdim, width, 2.0), linear(q + "o", width, heads * vdim)
            r = p + "mix.right."
            inner = right["heads"] * right["dim"]
            for name in ("r", "k", "v", "a"):
                linear(r + name, inner, width, 2.0)
            linear(r + "g", inner, width, 2.0)
            out[r + "a.b"] = rng.normal(0.0, 1.5, inner)
            rank = right.get("decay_rank") or 4
            linear(r + "w1", rank, width), linear(r + "w2", inner, rank, 2.0)
            out[r + "w0"] = rng.permutation(np.linspace(-7.0, 2.0, inner))
            near_one(r + "norm", inner), linear(r + "o", width, inner)
            near_one(p + "mix.left.out", width), near_one(p + "mix.right.out", width)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            near_one(p + "norm2", width, centre=0.0)
            linear(p + "mlp.gate", ff, width, 2.0), linear(p + "mlp.up", ff, width, 2.0), linear(p + "mlp.down", width, ff)
    return {name: torch.from_numpy(np.ascontiguousarray(value)).to(torch.bfloat16) for name, value in out.items()}
