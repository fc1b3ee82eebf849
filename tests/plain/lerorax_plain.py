"""Lerorax in plain NumPy, float64, one function per mechanism.

Written from the design's equations; it shares no code with the engine. Every function that carries
something from token to token takes and returns that state explicitly, so a sequence can be fed in
any cutting: ``PlainLerorax.forward(tokens, state)`` runs the next tokens of one sequence.

Notation: ``h`` is a sublayer's input ``[n, width]`` (rows are tokens), matrices are stored
``[out, in]`` and applied as ``h @ W.T``.
"""

from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """Rows of ``x`` divided by their root mean square, ``eps`` inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    """The layers' norm: the stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def bigram_rows(tokens, previous, buckets, mul_prev, mul_cur):
    """Row of the bigram table for each token; ``previous`` is the token in front of the first one,
    None at a sequence's start (which takes the table's last row, number ``buckets``)."""
    rows = []
    for t in tokens:
        rows.append(buckets if previous is None else (int(previous) * mul_prev + int(t) * mul_cur) % buckets)
        previous = int(t)
    return np.array(rows, dtype=np.int64), previous


def mingru(h, state, wz, bz, wx, bx, wg, wo):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t with gates and candidates that read only token t."""
    z = sigmoid(h @ wz.T + bz)
    u = h @ wx.T + bx
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ wg.T)
    out = np.empty_like(z)
    s = state
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        out[t] = s * gate[t]
    return out @ wo.T, s


def short_convolution(u, history, taps_w):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j); ``history`` holds the ``taps - 1`` inputs in front of
    ``u`` (zeros at a sequence's start). Returns y and the new history."""
    taps = taps_w.shape[1]
    full = np.concatenate([history, u], axis=0)
    n = u.shape[0]
    y = np.zeros_like(u)
    for j in range(taps):
        y += full[j : j + n] * taps_w[:, j]
    return y, full[full.shape[0] - (taps - 1) :] if taps > 1 else full[:0]


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i / dims); with ``scaling`` long wavelengths are stretched by ``factor``, short
    ones kept, and those between blended linearly in ``original / wavelength``."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(x, positions, freqs):
    """``x`` is ``[n, heads, dim]``; dims 2i and 2i + 1 of the first ``2 len(freqs)`` turn by p f_i."""
    out = x.copy()
    angle = positions[:, None].astype(np.float64) * freqs[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    d = 2 * len(freqs)
    a, b = x[..., 0:d:2], x[..., 1:d:2]
    out[..., 0:d:2] = a * c - b * s
    out[..., 1:d:2] = b * c + a * s
    return out


def mixed_head_attention(q, keys, values, positions, scale, talk):
    """Causal softmax attention whose weights are mixed over heads before they meet the values.

    ``q`` ``[n, H, dim]`` at ``positions``; ``keys`` ``[m, G, dim]`` and ``values`` ``[m, G, vdim]`` hold
    positions 0..m-1. Head h's weights become ``sum_g talk[h, g] softmax_g`` and are applied to the
    values of h's own key/value head."""
    n, heads, _ = q.shape
    group = heads // keys.shape[1]
    out = np.zeros((n, heads, values.shape[2]))
    for t in range(n):
        m = int(positions[t]) + 1
        weights = np.empty((heads, m))
        for g in range(heads):
            s = keys[:m, g // group] @ q[t, g] * scale
            e = np.exp(s - s.max())
            weights[g] = e / e.sum()
        weights = talk @ weights
        for h in range(heads):
            out[t, h] = weights[h] @ values[:m, h // group]
    return out


def delta_rule_general(r, k, v, w, a, state):
    """Per head, S <- diag(w) S - (a u)(u^T S) + k v^T with u = k / sqrt(sum k^2 + 1e-6), both terms
    reading the old S; o = S^T r. Inputs ``[n, heads, dim]``, ``state`` ``[heads, dim, dim]``."""
    n, heads, _ = r.shape
    out = np.empty_like(v)
    s = state.copy()
    for t in range(n):
        for hd in range(heads):
            u = k[t, hd] / math.sqrt(float(np.sum(k[t, hd] ** 2)) + 1e-6)
            old = s[hd]
            s[hd] = w[t, hd][:, None] * old - np.outer(a[t, hd] * u, u @ old) + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = s[hd].T @ r[t, hd]
    return out, s


def clamped_glu_ff(h, w_gate, w_up, w_down, limit):
    g = np.minimum(h @ w_gate.T, limit)
    u = np.clip(h @ w_up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


class PlainLerorax:
    def __init__(self, config: dict, tensors: dict[str, np.ndarray]) -> None:
        self.c = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]

    def owner(self, i: int) -> int:
        while "weights_of" in self.layers[i] and self.layers[i]["weights_of"] is not None:
            i = int(self.layers[i]["weights_of"])
        return i

    def new_state(self) -> dict:
        state: dict = {"previous": None, "position": 0, "layers": []}
        for entry in self.layers:
            m = entry["mixer"]
            if entry["type"] == "mingru":
                state["layers"].append({"s": np.zeros(m["width"])})
            else:
                left, right = m["left"], m["right"]
                hq, g, d, dv, taps = left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["conv"]
                state["layers"].append({
                    "conv": {"q": np.zeros((taps - 1, hq * d)), "k": np.zeros((taps - 1, g * d)), "v": np.zeros((taps - 1, g * dv))},
                    "keys": np.zeros((0, g, d)), "values": np.zeros((0, g, dv)),
                    "s": np.zeros((right["heads"], right["dim"], right["dim"])),
                })
        return state

    # -- mixers ------------------------------------------------------------------------------

    def left(self, p, m, h, st, positions):
        w, n = self.w, h.shape[0]
        hq, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        proj = {}
        for name in ("q", "k", "v"):
            u = h @ w[p + name].T + w[p + name + ".b"]
            proj[name], st["conv"][name] = short_convolution(u, st["conv"][name], w[p + name + ".conv"])
        q = unit_rms(proj["q"], self.eps) * w[p + "q.norm"]
        k = unit_rms(proj["k"], self.eps) * w[p + "k.norm"]
        rot = m.get("rot")
        q, k, v = q.reshape(n, hq, d), k.reshape(n, g, d), proj["v"].reshape(n, g, dv)
        if rot and rot.get("dims", 0):
            f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
            q, k = rotate_pairs(q, positions, f), rotate_pairs(k, positions, f)
        st["keys"] = np.concatenate([st["keys"], k])
        st["values"] = np.concatenate([st["values"], v])
        o = mixed_head_attention(q, st["keys"], st["values"], positions, m["scale"], w[p + "talk"])
        o = o.reshape(n, hq * dv) * sigmoid(h @ w[p + "g"].T)
        return o @ w[p + "o"].T

    def right(self, p, m, h, st):
        w, n = self.w, h.shape[0]
        heads, d = m["heads"], m["dim"]
        r, k, v = (h @ w[p + x].T for x in ("r", "k", "v"))
        decay = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
        a = sigmoid(h @ w[p + "a"].T + w[p + "a.b"])
        shape = (n, heads, d)
        o, st["s"] = delta_rule_general(r.reshape(shape), k.reshape(shape), v.reshape(shape), decay.reshape(shape), a.reshape(shape), st["s"])
        o = unit_rms(o, self.eps).reshape(n, heads * d) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
        return o @ w[p + "o"].T

    # -- the model -----------------------------------------------------------------------------

    def forward(self, tokens, state, want=None, layer_outputs=None):
        """Next ``tokens`` of the sequence whose ``state`` this is; logits ``[len(want), vocab]`` (all
        rows if ``want`` is None). ``layer_outputs``, a list, receives the stream after every layer."""
        w, c = self.w, self.c
        tokens = [int(t) for t in tokens]
        n = len(tokens)
        positions = np.arange(state["position"], state["position"] + n)
        x = w["embed"][tokens]
        big = c.get("embedding", {}).get("bigram")
        if big:
            rows, state["previous"] = bigram_rows(tokens, state["previous"], big["buckets"], big["mul_prev"], big["mul_cur"])
            x = x + w["bigram"][rows]
        for i, entry in enumerate(self.layers):
            p = f"l{self.owner(i)}."
            st, m = state["layers"][i], entry["mixer"]
            if entry["type"] == "mingru":
                y, st["s"] = mingru(x, st["s"], w[p + "mix.z"], w[p + "mix.z.b"], w[p + "mix.x"], w[p + "mix.x.b"], w[p + "mix.g"], w[p + "mix.o"])
            else:
                a = self.left(p + "mix.left.", m["left"], x, st, positions)
                b = self.right(p + "mix.right.", m["right"], x, st)
                y = 0.5 * (unit_rms(a, self.eps) * w[p + "mix.left.out"] + unit_rms(b, self.eps) * w[p + "mix.right.out"])
            x = x + norm_around_zero(y, w[p + "norm1"], self.eps)
            ff = entry.get("mlp")
            if ff:
                y = clamped_glu_ff(x, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], float(ff["limit"]))
                x = x + norm_around_zero(y, w[p + "norm2"], self.eps)
            if layer_outputs is not None:
                layer_outputs.append(x.copy())
        state["position"] += n
        rows = x if want is None else x[list(want)]
        return norm_around_zero(rows, w["final.norm"], self.eps) @ w["head"].T


def forward(config: dict, weights: dict, tokens, layer_outputs=None) -> np.ndarray:
    """Logits ``[len(tokens), vocab]`` of one whole sequence."""
    model = PlainLerorax(config, weights)
    return model.forward(tokens, model.new_state(), layer_outputs=layer_outputs)


def greedy(config: dict, weights: dict, prompt, count: int) -> list[int]:
    model = PlainLerorax(config, weights)
    state = model.new_state()
    row = model.forward(prompt, state)[-1]
    out = []
    for _ in range(count):
        out.append(int(np.argmax(row)))
        row = model.forward([out[-1]], state)[-1]
    return out
