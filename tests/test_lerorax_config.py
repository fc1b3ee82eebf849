"""Lerorax on the CPU: registry, configuration errors, tensor names and shapes, layers that run another
layer's tensors, seeded folders, and the plain implementation against second formulations of its mechanisms."""

from __future__ import annotations

import copy
import json

import numpy as np
import pytest

from lerorax_helpers import ALPHA, BETA, CONFIGS, GAMMA, draw_weights, owner
from plain import lerorax_plain as plain


def parsed(raw):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config.registry import parse_config

    return parse_config(json.loads(json.dumps(raw)))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    from llm_inference_b200.parts.model import Model

    raw = CONFIGS[name]
    entry, config = parsed(raw)
    assert entry.name == "Lerorax" and config.to_json_dict() == raw
    model = Model(entry.recipe(config))
    specs = {spec.name: spec for spec in model.tensor_specs()}
    weights = draw_weights(raw, 3)
    assert all(specs[n].fits(tuple(t.shape)) for n, t in weights.items())
    assert {n for n, s in specs.items() if not s.optional} == set(weights)
    # a layer that runs another's tensors has none of its own, but a cache entry of its own
    shared = [i for i in range(len(raw["layers"])) if owner(raw, i) != i]
    assert shared and not any(n.startswith(f"l{i}.") for i in shared for n in specs)
    assert [call.cache_id for call in model.schedule] == list(range(len(raw["layers"])))
    assert len({call.layer for call in model.schedule}) == len(raw["layers"]) - len(shared)


def test_recipe_reads_every_size_from_the_configuration():
    from llm_inference_b200.cache.paged_cache import flatten_specs
    from llm_inference_b200.parts.base import KVCacheSpec, StateSpec
    from llm_inference_b200.parts.model import EMBEDDING_CACHE, Model

    entry, config = parsed(BETA)
    model = Model(entry.recipe(config))
    assert [call.layer for call in model.schedule] == [0, 1, 2, 1, 0, 1]
    gru, pair = model.blocks[0], model.blocks[1]
    assert gru.mixer.width == 24 and gru.feed_forward.limit == 0.4 and gru.feed_forward.intermediate_size == 72
    left, right = pair.mixer.members
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.taps, left.scale) == (5, 1, 12, 6, 1, 0.45)
    assert left.position.rotary_dims == 0 and (right.heads, right.dim, right.decay_rank) == (2, 40, -1)
    assert model.blocks[2].feed_forward is None and model.blocks[2].mixer.members[0].position.rotary_dims == 8
    assert type(model.embedding).__name__ == "TokenEmbedding" and pair.mixer_norm.eps == 3e-4 and pair.mixer.eps == 3e-4
    flat = flatten_specs(model.cache_specs())
    assert EMBEDDING_CACHE not in flat
    assert flat[(1, 0, 0)] == KVCacheSpec(1, 64, 0) and flat[(5, 0, 0)] == flat[(1, 0, 0)] and flat[(1, 1)].shapes == ((2, 40, 40),)
    assert flat[(1, 0, 1)].shapes == ((0, 5 * 12 + 12 + 6),) and flat[0] == StateSpec(((24,),), flat[0].dtypes)
    alpha = Model(parsed(ALPHA)[0].recipe(parsed(ALPHA)[1]))
    assert alpha.embedding.buckets == 61 and (alpha.embedding.mul_prev, alpha.embedding.mul_cur) == (31, 5)
    assert EMBEDDING_CACHE in alpha.cache_specs()
    scaling = alpha.blocks[0].mixer.members[0].position.scaling
    assert scaling == {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}
    assert alpha.blocks[2].mixer.members[0].position.scaling is None
    gamma = Model(parsed(GAMMA)[0].recipe(parsed(GAMMA)[1]))
    assert gamma.blocks[0].mixer.members[0].row_dim == 64 and gamma.blocks[0].mixer.members[0].position.rotary_dims == 48


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(width=0), "width"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(high=1.0), "high"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(dim=0), "positive"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][3].update(weights_of=3), "another"),
    (lambda c: c["layers"][3].update(weights_of=9), "another"),
    (lambda c: c["layers"][3].update(weights_of=1), "equal"),
    (lambda c: c["layers"][3].update(mlp=None), "equal"),
    (lambda c: (c["layers"][0].update(weights_of=3)), "circle"),
])
def test_configuration_errors(change, message):
    from llm_inference_b200.config.model_config import ConfigError

    raw = copy.deepcopy(ALPHA)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        parsed(raw)


def test_seeded_folder_round_trip(tmp_path):
    from llm_inference_b200.config.model_config import read_config_json
    from llm_inference_b200.weights.loader import load_weights
    from llm_inference_b200.weights.random_init import write_model_folder

    entry, config = parsed(ALPHA)
    folder = write_model_folder(tmp_path / "m", config, seed=5)
    assert read_config_json(folder) == ALPHA
    tensors = load_weights(folder, entry.recipe(config).tensor_specs())
    assert tensors["bigram"].shape == (62, 48) and tensors["l0.mix.right.w1"].shape == (5, 48) and tensors["l0.mix.left.talk"].shape == (4, 4)
    assert tensors["l0.mix.left.q.conv"].shape == (64, 3) and not any(n.startswith("l3.") for n in tensors)
    # a checkpoint's own inner size of the decay pair is taken whatever it is, when the configuration does not name one
    entry, config = parsed(BETA)
    specs = {s.name: s for s in entry.recipe(config).tensor_specs()}
    assert specs["l1.mix.right.w1"].fits((9, 40)) and specs["l1.mix.right.w2"].fits((80, 9)) and not specs["l1.mix.right.w2"].fits((81, 9))
    with pytest.raises(Exception, match="decay_rank|size"):
        write_model_folder(tmp_path / "n", config, seed=5)  # random weights need the size named


# --- the plain implementation against second formulations ----------------------------------------------


def test_plain_mingru_equals_its_unrolled_sum():
    """S_t = sum_j (prod_{j<m<=t} (1 - z_m)) z_j c_j."""
    rng = np.random.default_rng(0)
    width, hidden, tokens = 5, 7, 9
    wz, wx, wg = (rng.normal(size=(width, hidden)) for _ in range(3))
    bz, bx = rng.normal(size=width), rng.normal(size=width)
    h = rng.normal(size=(tokens, hidden))
    out, last = plain.mingru(h, np.zeros(width), wz, bz, wx, bx, wg, np.eye(width))
    z = plain.sigmoid(h @ wz.T + bz)
    u = h @ wx.T + bx
    c = np.where(u >= 0, u + 0.5, plain.sigmoid(u))
    assert (u >= 0).any() and (u < 0).any()
    for t in range(tokens):
        s = sum(np.prod(1 - z[j + 1 : t + 1], axis=0) * z[j] * c[j] for j in range(t + 1))
        assert np.allclose(out[t], s * plain.silu(h[t] @ wg.T))
    assert np.allclose(last, s)
    first, carried = plain.mingru(h[:4], np.zeros(width), wz, bz, wx, bx, wg, np.eye(width))
    rest, _ = plain.mingru(h[4:], carried, wz, bz, wx, bx, wg, np.eye(width))
    assert np.allclose(np.vstack([first, rest]), out)


def test_plain_convolution_is_a_sliding_dot_product_and_is_cut_anywhere():
    rng = np.random.default_rng(1)
    u, taps = rng.normal(size=(11, 4)), rng.normal(size=(4, 3))
    y, history = plain.short_convolution(u, np.zeros((2, 4)), taps)
    padded = np.vstack([np.zeros((2, 4)), u])
    for t in range(11):
        assert np.allclose(y[t], (padded[t : t + 3].T * taps).sum(axis=1))
    assert np.allclose(history, u[-2:])
    a, carried = plain.short_convolution(u[:1], np.zeros((2, 4)), taps)
    b, _ = plain.short_convolution(u[1:], carried, taps)
    assert np.allclose(np.vstack([a, b]), y)
    lone, none = plain.short_convolution(u, np.zeros((0, 4)), taps[:, :1])
    assert np.allclose(lone, u * taps[:, 0]) and none.shape == (0, 4)


def test_plain_rotation_depends_on_the_distance_only_and_leaves_the_rest():
    rng = np.random.default_rng(2)
    f = plain.rotary_frequencies(4, 100.0)
    q, k = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    near = (plain.rotate_pairs(q, np.array([9]), f) * plain.rotate_pairs(k, np.array([4]), f)).sum()
    far = (plain.rotate_pairs(q, np.array([105]), f) * plain.rotate_pairs(k, np.array([100]), f)).sum()
    assert np.isclose(near, far)
    turned = plain.rotate_pairs(q, np.array([3]), f)
    assert np.allclose(turned[..., 4:], q[..., 4:]) and not np.allclose(turned[..., :4], q[..., :4])
    assert np.allclose(turned[0, 0, 0], q[0, 0, 0] * np.cos(3.0) - q[0, 0, 1] * np.sin(3.0))  # f_0 = 1; dims 0 and 1 are a pair


def test_plain_mixed_heads_equal_a_mix_of_plain_attention_outputs():
    """Mixing normalised weights is mixing the outputs that each head's own weights give on the same values."""
    rng = np.random.default_rng(3)
    n, heads, kvh, dim, vdim = 7, 4, 2, 5, 3
    q, k, v = rng.normal(size=(n, heads, dim)), rng.normal(size=(n, kvh, dim)), rng.normal(size=(n, kvh, vdim))
    talk = rng.normal(size=(heads, heads))
    got = plain.mixed_head_attention(q, k, v, np.arange(n), 0.7, talk)
    own = np.zeros((kvh, n, heads, vdim))  # own[c][t][g]: head g's softmax on the values of kv head c
    for c in range(kvh):
        for g in range(heads):
            scores = q[:, g] @ k[:, g // 2].T * 0.7
            scores[np.triu_indices(n, 1)] = -np.inf
            p = np.exp(scores - scores.max(axis=1, keepdims=True))
            own[c, :, g] = (p / p.sum(axis=1, keepdims=True)) @ v[:, c]
    for h in range(heads):
        assert np.allclose(got[:, h], np.einsum("g,tgd->td", talk[h], own[h // 2]))
    assert np.allclose(plain.mixed_head_attention(q, k, v, np.arange(n), 0.7, np.eye(heads))[:, 3], own[1, :, 3])


def test_plain_delta_rule_column_by_column():
    """Every column s of S follows s <- w * s - (a * u) (u . s) + k v_c on its own; with a = 0 and w = 1 the state is
    the sum of outer products."""
    rng = np.random.default_rng(4)
    n, heads, dim = 6, 2, 4
    r, k, v = (rng.normal(size=(n, heads, dim)) for _ in range(3))
    w, a = rng.uniform(0.5, 1, (n, heads, dim)), rng.uniform(0, 1, (n, heads, dim))
    out, state = plain.delta_rule_general(r, k, v, w, a, np.zeros((heads, dim, dim)))
    for hd in range(heads):
        for c in range(dim):
            s = np.zeros(dim)
            for t in range(n):
                u = k[t, hd] / np.sqrt((k[t, hd] ** 2).sum() + 1e-6)
                s = w[t, hd] * s - a[t, hd] * u * (u @ s) + k[t, hd] * v[t, hd, c]
                assert np.isclose(out[t, hd, c], s @ r[t, hd])
            assert np.allclose(state[hd][:, c], s)
    _, plain_sum = plain.delta_rule_general(r, k, v, np.ones_like(w), np.zeros_like(a), np.zeros((heads, dim, dim)))
    assert np.allclose(plain_sum[1], sum(np.outer(k[t, 1], v[t, 1]) for t in range(n)))
    # a = 1, w = 1: what the state held along the key's direction is gone before the new pair is written
    k1 = np.zeros((2, 1, 3))
    k1[:, 0, 0] = 2.0
    v1 = np.array([[[1.0, 2.0, 3.0]], [[5.0, 5.0, 5.0]]])
    _, replaced = plain.delta_rule_general(k1, k1, v1, np.ones_like(k1), np.ones_like(k1), np.zeros((1, 3, 3)))
    assert np.allclose(replaced[0][0], 2.0 * v1[1, 0], atol=1e-5)


def test_plain_bigram_rows_and_layers_on_shared_tensors():
    rows, last = plain.bigram_rows([3, 5, 5], None, 7, 2, 3)
    assert rows.tolist() == [7, (3 * 2 + 5 * 3) % 7, (5 * 2 + 5 * 3) % 7] and last == 5
    assert plain.bigram_rows([4], 5, 7, 2, 3)[0].tolist() == [(5 * 2 + 4 * 3) % 7]
    weights = {k: v.double().numpy() for k, v in draw_weights(ALPHA, 1).items()}
    tokens = list(range(12))
    layers: list = []
    whole = plain.forward(ALPHA, weights, tokens, layer_outputs=layers)
    assert len(layers) == 5
    # layer 3 runs layer 0's tensors on its own state: fed with layer 0's input it gives layer 0's output
    model = plain.PlainLerorax(ALPHA, weights)
    state = model.new_state()
    first = model.forward(tokens[:5], state)
    rest = model.forward(tokens[5:], state)
    assert np.allclose(np.vstack([first, rest]), whole)
    cut = dict(ALPHA, layers=ALPHA["layers"][:3])
    assert not np.allclose(plain.forward(cut, weights, tokens), whole)
