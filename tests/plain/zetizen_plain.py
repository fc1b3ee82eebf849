"""A plain, slow Zetizen forward pass in NumPy: one function per mechanism, float64 throughout.

It imports nothing from the engine and the engine imports nothing from here. ``config`` is the
model's config.json as a dict, ``weights`` maps tensor names to arrays. Attention keeps what it has
seen in an explicit per-layer state (lists of rows), so a sequence can be fed whole, in portions or
token by token.

Notation: ``T`` new tokens, ``D`` the model's width, ``H`` query heads, ``G`` key/value heads; a linear
weight is ``[out, in]`` and is applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def linear(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    y = x.astype(F64) @ weight.astype(F64).T
    return y if bias is None else y + bias.astype(F64)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-x))


def silu(x: np.ndarray) -> np.ndarray:
    return x * sigmoid(x)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis."""
    x = x.astype(F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight.astype(F64)


def layer_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``(x - mean) / sqrt(var + eps) * weight``, the variance being the mean squared deviation; no bias."""
    x = x.astype(F64)
    centred = x - np.mean(x, axis=-1, keepdims=True)
    return centred / np.sqrt(np.mean(centred * centred, axis=-1, keepdims=True) + eps) * weight.astype(F64)


def softmax(scores: np.ndarray) -> np.ndarray:
    e = np.exp(scores - np.max(scores, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


def soft_cap(scores: np.ndarray, cap: float | None) -> np.ndarray:
    return scores if not cap else cap * np.tanh(scores / cap)


# -- positions ------------------------------------------------------------------------------------------


def distance_bucket(n: int, rows: int, reach: int) -> int:
    """Row of the distance-bias table for a key ``n`` positions back: one row per distance below ``rows / 2``,
    then rows spaced evenly in the logarithm of the distance up to ``reach``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def rotary_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[np.ndarray, float]:
    """``dims / 2`` angular frequencies and the factor on sine and cosine. Without ``scaling``: ``base^(-2i / dims)``
    and 1. With it, frequencies of long wavelengths are divided by ``factor``, short ones kept, a linear ramp between."""
    i = np.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turning_point(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turning_point(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turning_point(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: np.ndarray, positions: np.ndarray, dims: int, base: float, scaling: dict | None) -> np.ndarray:
    """``x`` is ``[T, heads, size]``; the first ``dims`` numbers of every head are rotated, number ``i`` with
    number ``i + dims / 2``, by the angle ``position * f_i``."""
    if not dims:
        return x
    f, magnitude = rotary_frequencies(dims, base, scaling)
    angle = np.asarray(positions, dtype=F64)[:, None] * f[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# -- attention over explicit keys and values ------------------------------------------------------------


def attend(q: np.ndarray, keys: np.ndarray, values: np.ndarray, positions: np.ndarray, scale: float, cap: float | None = None,
           bias=None, chunk: int = 0) -> np.ndarray:
    """``q`` ``[T, H, d]`` at ``positions``; ``keys`` ``[N, G, d]`` and ``values`` ``[N, G, e]`` of positions ``0 .. N - 1``.
    ``bias(distance, head)`` is added after the cap; with ``chunk`` a query sees only keys of its own chunk of positions."""
    t_count, heads, _ = q.shape
    groups = keys.shape[1]
    out = np.zeros((t_count, heads, values.shape[2]), dtype=F64)
    for t in range(t_count):
        p = int(positions[t])
        first = (p // chunk) * chunk if chunk else 0
        for h in range(heads):
            g = h // (heads // groups)
            scores = soft_cap(keys[first : p + 1, g] @ q[t, h] * scale, cap)
            if bias is not None:
                scores = scores + np.array([bias(p - j, h) for j in range(first, p + 1)])
            out[t, h] = softmax(scores) @ values[first : p + 1, g]
    return out


def _grow(state: dict, name: str, rows: np.ndarray) -> np.ndarray:
    state[name] = rows if name not in state else np.concatenate([state[name], rows])
    return state[name]


def biased_attention(h: np.ndarray, w: dict, p: str, m: dict, eps: float, positions, state: dict) -> np.ndarray:
    """Grouped-query attention without rotation: one RMS norm over all of q and one over all of k, capped scores
    (with ``softcap``), a learned bias by distance (with ``bias_max``)."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t_count = h.shape[0]
    q = rms_norm(linear(h, w[p + "q"]), w[p + "q.norm"], eps).reshape(t_count, heads, dim)
    k = rms_norm(linear(h, w[p + "k"]), w[p + "k.norm"], eps).reshape(t_count, groups, dim)
    v = linear(h, w[p + "v"]).reshape(t_count, groups, vdim)
    keys, values = _grow(state, "k", k), _grow(state, "v", v)
    bias = None
    if m.get("bias_max"):
        table = w[p + "rel"].astype(F64)
        rows = table.shape[0]

        def bias(distance: int, head: int) -> float:
            return table[distance_bucket(distance, rows, m["bias_max"]), head]

    out = attend(q, keys, values, positions, m["scale"], m.get("softcap"), bias)
    return linear(out.reshape(t_count, heads * vdim), w[p + "o"])


def chunked_attention(h: np.ndarray, w: dict, p: str, m: dict, eps: float, positions, state: dict) -> np.ndarray:
    """Grouped-query attention whose values are its keys as projected; biases on q and k, norms over all of q and all
    of k, part of each head rotated, capped scores, keys visible inside the query's chunk only, a gate per head."""
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    t_count = h.shape[0]
    q_raw = linear(h, w[p + "q"], w[p + "q.b"])
    k_raw = linear(h, w[p + "k"], w[p + "k.b"])
    v = k_raw.reshape(t_count, groups, dim)
    q = rms_norm(q_raw, w[p + "q.norm"], eps).reshape(t_count, heads, dim)
    k = rms_norm(k_raw, w[p + "k.norm"], eps).reshape(t_count, groups, dim)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, positions, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_halves(k, positions, rot["dims"], rot["base"], rot.get("scaling"))
    keys, values = _grow(state, "k", k), _grow(state, "v", v)
    size = m["mask"]["size"] if m.get("mask") else 0
    out = attend(q, keys, values, positions, m["scale"], m.get("softcap"), None, size)
    out = out * sigmoid(linear(h, w[p + "g"]))[:, :, None]
    return linear(out.reshape(t_count, heads * dim), w[p + "o"])


def latent_attention(h: np.ndarray, w: dict, p: str, m: dict, eps: float, positions, state: dict) -> np.ndarray:
    """Attention whose keys and values are expanded from a cached latent row per token, queries through a latent of
    their own, one rotated key part shared by all heads, an element-wise output gate."""
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t_count = h.shape[0]
    rot = m["rot"]
    q = linear(rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps), w[p + "uq"]).reshape(t_count, heads, dim + rot_dim)
    q_plain = q[..., :dim]
    q_rot = rotate_halves(q[..., dim:].copy(), positions, rot_dim, rot["base"], rot.get("scaling"))
    down = linear(h, w[p + "dkv"])
    latent = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_halves(down[:, None, rank:].copy(), positions, rot_dim, rot["base"], rot.get("scaling"))
    latents, shared = _grow(state, "c", latent), _grow(state, "r", k_rot)
    n = latents.shape[0]
    k_plain = linear(latents, w[p + "uk"]).reshape(n, heads, dim)
    values = linear(latents, w[p + "uv"]).reshape(n, heads, vdim)
    keys = np.concatenate([k_plain, np.broadcast_to(shared, (n, heads, rot_dim))], axis=-1)
    queries = np.concatenate([q_plain, q_rot], axis=-1)
    out = attend(queries, keys, values, positions, m["scale"], m.get("softcap"))
    out = out.reshape(t_count, heads * vdim) * sigmoid(linear(h, w[p + "g"]))
    return linear(out, w[p + "o"])


MIXERS = {"attention": biased_attention, "attention_2": chunked_attention, "latent_attention": latent_attention}


# -- feed-forward ---------------------------------------------------------------------------------------


def gated_unit(h: np.ndarray, w: dict, p: str) -> np.ndarray:
    return linear(silu(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def route(logits: np.ndarray, top: int) -> tuple[np.ndarray, np.ndarray]:
    """The ``top`` largest logits of every row (ties: the lower index) and the softmax over just those."""
    order = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    return order, softmax(np.take_along_axis(logits, order, axis=-1))


def routed_experts(h: np.ndarray, w: dict, p: str, mlp: dict, choices=None, margins=None, free=None) -> np.ndarray:
    """``choices`` (``[T, top]`` expert ids) replaces the router's own choice of experts (their weights are still the
    softmax over the chosen logits); ``margins`` (a list) receives one array per call, per token the gap between the
    last chosen and the first rejected logit, and ``free`` (a list) the router's own choices."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = linear(h, w[p + "router"], w[p + "router.b"])
    ids, weights = route(logits, top)
    if margins is not None:
        ordered = -np.sort(-logits, axis=-1)
        margins.append(ordered[:, top - 1] - ordered[:, top] if top < experts else np.full(h.shape[0], np.inf))
    if free is not None:
        free.append(ids.copy())
    if choices is not None:
        ids = np.asarray(choices, dtype=np.int64)
        weights = softmax(np.take_along_axis(logits, ids, axis=-1))
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F64)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += weights[t, j] * gated_unit(h[t : t + 1], w, f"{p}e{ids[t, j]}.")[0]
    if mlp.get("shared"):
        out += gated_unit(h, w, p + "shared.")
    return out


# -- the model ------------------------------------------------------------------------------------------


def new_state(config: dict) -> dict:
    return {"position": 0, "layers": [dict() for _ in config["layers"]]}


def forward(config: dict, weights: dict, tokens, state: dict | None = None, *, layer_outputs: list | None = None,
            choices: dict | None = None, margins: list | None = None, free: list | None = None) -> tuple[np.ndarray, dict]:
    """Feed ``tokens`` (the next ones of the sequence ``state`` belongs to; None: a new sequence). Returns the logits
    ``[T, vocab]`` and the state. ``layer_outputs`` receives the stream after every layer; ``choices`` maps a layer index
    to the experts to use (``[T, top]``); ``margins`` and ``free`` receive one entry per routed layer (see
    :func:`routed_experts`)."""
    state = new_state(config) if state is None else state
    eps = config["norm"]["eps"]
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = state["position"] + np.arange(tokens.shape[0])
    state["position"] += tokens.shape[0]
    table = weights["embed"].astype(F64)
    x = layer_norm(table[tokens], weights["embed.norm"], eps)
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = layer_norm(x, weights[p + "norm1"], eps)
        branch = MIXERS[layer["type"]](h, weights, p + "mix.", layer["mixer"], eps, positions, state["layers"][index])
        if layer.get("mlp") is not None:
            branch = branch + routed_experts(h, weights, p + "mlp.", layer["mlp"], None if choices is None else choices.get(index), margins, free)
        x = x + branch
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    logits = linear(layer_norm(x, weights["final.norm"], eps), table) * config.get("logit_scale", 1.0)
    return logits, state


def greedy(config: dict, weights: dict, prompt, count: int) -> list[int]:
    """``count`` tokens, each the arg-max of the last position's logits, fed back one by one."""
    logits, state = forward(config, weights, prompt)
    out = []
    for _ in range(count):
        out.append(int(np.argmax(logits[-1])))
        logits, state = forward(config, weights, [out[-1]], state)
    return out
