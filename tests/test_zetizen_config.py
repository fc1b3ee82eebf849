"""Zetizen on the CPU: registry, configuration errors, tensor names and shapes, seeded folders, the host-side tables
of the parts, and the plain implementation against second formulations of its mechanisms."""

from __future__ import annotations

import copy
import json
import math

import numpy as np
import pytest

from plain import zetizen_plain as plain
from zetizen_helpers import ALPHA, BETA, CONFIGS, GAMMA, draw_weights, scaling


def parsed(raw):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config.registry import parse_config

    return parse_config(json.loads(json.dumps(raw)))


def as_float64(weights):
    import torch

    return {name: tensor.to(torch.float64).numpy() for name, tensor in weights.items()}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    from llm_inference_b200.parts.model import Model

    raw = CONFIGS[name]
    entry, config = parsed(raw)
    assert entry.name == "Zetizen"
    assert config.to_json_dict() == (raw if "logit_scale" in raw else dict(raw, logit_scale=1.0))
    specs = {spec.name: spec for spec in Model(entry.recipe(config)).tensor_specs()}
    weights = draw_weights(raw, 3)
    assert all(specs[n].fits(tuple(t.shape)) for n, t in weights.items())
    assert {n for n, s in specs.items() if not s.optional} == set(weights)  # the head is the embedding table
    kinds = {type(s).__name__ for s in Model(entry.recipe(config)).cache_specs().values()}
    assert kinds == {"KVCacheSpec"}


def test_recipe_reads_every_size_from_the_configuration():
    from llm_inference_b200.parts.model import Model

    entry, config = parsed(BETA)
    model = Model(entry.recipe(config))
    latent, chunked, biased, second_latent = (block.mixer for block in model.blocks)
    assert (latent.heads, latent.dim, latent.rot_dim, latent.vdim, latent.rank, latent.q_rank, latent.scale) == (1, 6, 2, 5, 7, 3, 0.9)
    assert latent.gate_per_element and not latent.has_sink and latent.position.ramp is None and latent.position.magnitude == 1.0
    assert latent.cache_spec().head_dim == 9 and latent.cache_spec().planes == 1
    assert (chunked.heads, chunked.kv_heads, chunked.dim, chunked.values_from_keys, chunked.qk_bias, chunked.gate) == (5, 5, 8, True, True, "head")
    assert (chunked.chunk, chunked.softcap, chunked.position) == (0, 0.0, None)
    assert (biased.dim, biased.vdim, biased.row_dim, biased.softcap, biased.bias_reach, biased.bias_rows) == (8, 136, 144, 2.0, 9, 6)
    assert not biased.values_from_keys and biased.gate is None and not biased.qk_bias
    assert second_latent.position.theta == 1000.0 and second_latent.position.ramp["factor"] == 2.0
    first = model.blocks[0].feed_forward
    assert (first.experts, first.top, first.intermediate_size, first.shared_size, first.limit, first.router, first.router_bias) == (7, 1, 70, 0, 0.0, "softmax_chosen", True)
    assert model.blocks[1].feed_forward is None and model.blocks[2].feed_forward.shared_size == 40
    assert model.head.scale is None and model.head.tied_to == "embed"
    alpha = Model(parsed(ALPHA)[0].recipe(parsed(ALPHA)[1]))
    assert alpha.head.scale == 0.5 and alpha.blocks[1].mixer.chunk == 20 and alpha.blocks[1].mixer.position.rotary_dims == 8
    assert alpha.blocks[3].mixer.softcap == 0.0 and not alpha.blocks[3].mixer.has_bias
    gamma = Model(parsed(GAMMA)[0].recipe(parsed(GAMMA)[1]))
    assert gamma.blocks[1].mixer.position.rotary_dims == 128 and gamma.blocks[3].mixer.row_dim == 64


def test_the_row_count_of_a_bias_table_may_be_left_to_the_checkpoint():
    from llm_inference_b200.parts.model import Model

    raw = copy.deepcopy(ALPHA)
    rows = raw["layers"][0]["mixer"].pop("bias_rows")
    entry, config = parsed(raw)
    specs = {spec.name: spec for spec in Model(entry.recipe(config)).tensor_specs()}
    assert specs["l0.mix.rel"].shape == (-1, 4) and specs["l0.mix.rel"].fits((rows, 4)) and specs["l0.mix.rel"].fits((30, 4))


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.update(logit_scale=-1.0), "logit_scale"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"].update(bias_max=5), "bias_rows"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][2]["mixer"].update(softcap=4.0), "no soft cap"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["layers"][1]["mixer"].update(dim=0), "positive"),
])
def test_configuration_errors(change, message):
    from llm_inference_b200.config.model_config import ConfigError

    raw = copy.deepcopy(ALPHA)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        parsed(raw)


def test_seeded_folder_loads_back(tmp_path):
    from llm_inference_b200.weights import SafetensorsFile, write_model_folder

    _, config = parsed(GAMMA)
    folder = write_model_folder(tmp_path / "m", config, seed=5)
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Zetizen"
    with SafetensorsFile(folder / "model.safetensors") as file:
        names = set(file.tensors)
    assert {"embed", "embed.norm", "final.norm", "l0.mix.rel", "l1.mix.q.b", "l2.mix.dq.norm", "l0.mlp.router.b", "l0.mlp.shared.down"} <= names
    assert "head" not in names and "l1.mix.v" not in names and "l3.mlp.router" not in names


# --- the parts' host-side tables against the plain implementation ---------------------------------------


@pytest.mark.parametrize("rows,reach", [(12, 40), (6, 9), (20, 70), (8, 33), (2, 2), (33, 500), (32, 256)])
def test_distance_buckets_of_the_part(rows, reach):
    from llm_inference_b200.parts.shaped_attention import distance_buckets

    table = distance_buckets(rows, reach)
    assert table.shape == (reach + 1,)
    assert [int(b) for b in table] == [plain.distance_bucket(n, rows, reach) for n in range(reach + 1)]
    assert all(plain.distance_bucket(n, rows, reach) == rows - 1 for n in (reach, reach + 1, 10 * reach))  # what the clamp assumes
    assert list(table[: rows // 2]) == list(range(rows // 2)) and np.all(np.diff(table) >= 0) and table[-1] == rows - 1


@pytest.mark.parametrize("dims,base,rule", [(8, 100.0, scaling()), (16, 30.0, None), (128, 10000.0, scaling(4.0, 48, 16.0, 1.0)), (4, 50.0, scaling(2.0, 32, 4.0, 0.5)),
                                            (2, 1000.0, scaling(8.0, 4096, 32.0, 1.0)), (64, 500000.0, scaling(16.0, 8192, 32.0, 1.0))])
def test_frequency_table_of_the_rotary_part(dims, base, rule):
    from llm_inference_b200.parts.positions import RotaryEncoding

    part = RotaryEncoding(head_dim=dims + 8, theta=base, rotary_dims=dims, scaling=rule)
    f, magnitude = plain.rotary_frequencies(dims, base, rule)
    np.testing.assert_allclose(part.table(), f, rtol=1e-7)
    assert part.magnitude == pytest.approx(magnitude, rel=1e-12) and (rule is None) == (part.magnitude == 1.0)


# --- the plain implementation against second formulations -------------------------------------------------


def test_layer_norm_is_the_rms_norm_of_the_centred_row():
    rng = np.random.default_rng(0)
    x, w = rng.normal(3.0, 2.0, (5, 31)), rng.normal(1.0, 0.2, 31)
    centred = x - x.mean(-1, keepdims=True)
    np.testing.assert_allclose(plain.layer_norm(x, w, 1e-5), plain.rms_norm(centred, w, 1e-5), rtol=1e-12)
    assert abs(plain.layer_norm(x, np.ones(31), 1e-5).mean(-1)).max() < 1e-12


def test_buckets_are_exact_below_half_and_logarithmic_above():
    rows, reach = 32, 300
    half = rows // 2
    assert [plain.distance_bucket(n, rows, reach) for n in range(half)] == list(range(half))
    edges = [min(n for n in range(half, reach + 1) if plain.distance_bucket(n, rows, reach) >= b) for b in range(half, rows)]
    ratios = np.diff(np.log(edges[3:]))
    assert np.all(np.abs(ratios - math.log(reach / half) / (rows - half)) < 0.1)  # equal steps in the logarithm, up to rounding to whole distances
    assert plain.distance_bucket(reach - 1, rows, reach) == rows - 1 and plain.distance_bucket(10**6, rows, reach) == rows - 1


def test_rotation_keeps_lengths_up_to_the_magnitude_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    rule = scaling(4.0, 48, 16.0, 1.0)
    q, k = rng.normal(0, 1, (1, 2, 24)), rng.normal(0, 1, (1, 2, 24))
    _, magnitude = plain.rotary_frequencies(16, 200.0, rule)
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    turned = plain.rotate_halves(q, np.array([37]), 16, 200.0, rule)
    np.testing.assert_allclose(np.linalg.norm(turned[..., :16], axis=-1), magnitude * np.linalg.norm(q[..., :16], axis=-1), rtol=1e-12)
    np.testing.assert_array_equal(turned[..., 16:], q[..., 16:])

    def score(pq, pk):
        a = plain.rotate_halves(q, np.array([pq]), 16, 200.0, rule)
        b = plain.rotate_halves(k, np.array([pk]), 16, 200.0, rule)
        return np.einsum("thd,thd->h", a, b)

    np.testing.assert_allclose(score(50, 41), score(19, 10), rtol=1e-9)
    assert np.abs(score(50, 41) - score(50, 40)).max() > 1e-3
    # the ramp: fast frequencies kept, slow ones divided by the factor
    plain_f, _ = plain.rotary_frequencies(16, 200.0, None)
    f, _ = plain.rotary_frequencies(16, 200.0, rule)
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(plain_f[-1] / 4.0) and np.all(f <= plain_f) and np.all(f >= plain_f / 4.0)


def test_attention_as_a_masked_softmax_with_cap_bias_and_chunks():
    rng = np.random.default_rng(2)
    count, heads, groups, d, e, chunk, cap = 23, 4, 2, 6, 5, 7, 3.0
    q, k, v = rng.normal(0, 1, (count, heads, d)), rng.normal(0, 1, (count, groups, d)), rng.normal(0, 1, (count, groups, e))
    table = rng.normal(0, 1, (30, heads))
    got = plain.attend(q, k, v, np.arange(count), 0.8, cap, lambda n, h: table[n, h], chunk)
    i, j = np.arange(count)[:, None], np.arange(count)[None, :]
    visible = (j <= i) & (j // chunk == i // chunk)
    for h in range(heads):
        scores = cap * np.tanh(q[:, h] @ k[:, h // 2].T * 0.8 / cap) + table[np.clip(i - j, 0, 29), h]
        weights = np.where(visible, np.exp(scores), 0.0)
        np.testing.assert_allclose(got[:, h], weights / weights.sum(-1, keepdims=True) @ v[:, h // 2], rtol=1e-10)
    # cut anywhere: the second half alone over all keys gives the same rows
    tail = plain.attend(q[11:], k, v, np.arange(11, count), 0.8, cap, lambda n, h: table[n, h], chunk)
    np.testing.assert_allclose(tail, got[11:], rtol=1e-12)


def test_latent_attention_is_attention_over_expanded_keys_and_values_in_any_cutting():
    config = copy.deepcopy(BETA)
    w = as_float64(draw_weights(config, 4))
    m, p = config["layers"][3]["mixer"], "l3.mix."
    h = np.random.default_rng(3).normal(0, 1, (19, config["width"]))
    whole = plain.latent_attention(h, w, p, m, 1e-5, np.arange(19), {})
    state, parts = {}, []
    for a, b in ((0, 5), (5, 6), (6, 8), (8, 19)):
        parts.append(plain.latent_attention(h[a:b], w, p, m, 1e-5, np.arange(a, b), state))
    np.testing.assert_allclose(np.concatenate(parts), whole, rtol=1e-9, atol=1e-12)
    assert state["c"].shape == (19, m["kv_rank"]) and state["r"].shape == (19, 1, m["rot_dim"])  # all that is kept per token


def test_router_against_a_search_over_all_choices():
    rng = np.random.default_rng(5)
    logits = rng.normal(0, 2, (40, 7))
    for top in (1, 3, 7):
        ids, weights = plain.route(logits, top)
        for t in range(40):
            best = sorted(range(7), key=lambda e: -logits[t, e])[:top]
            assert list(ids[t]) == best
            e = np.exp(logits[t, best])
            np.testing.assert_allclose(weights[t], e / e.sum(), rtol=1e-12)
        np.testing.assert_allclose(weights.sum(-1), 1.0, rtol=1e-12)


def test_whole_model_in_portions_and_token_by_token():
    config = ALPHA
    w = as_float64(draw_weights(config, 6))
    tokens = [int(t) for t in np.random.default_rng(7).integers(0, config["vocab"], 45)]
    whole, _ = plain.forward(config, w, tokens)
    assert whole.shape == (45, config["vocab"])
    state, rows = None, []
    for a, b in ((0, 1), (1, 3), (3, 20), (20, 21), (21, 45)):
        logits, state = plain.forward(config, w, tokens[a:b], state)
        rows.append(logits)
    np.testing.assert_allclose(np.concatenate(rows), whole, rtol=1e-8, atol=1e-10)
    # the chunks of layer 1 and the logit scale show
    other = copy.deepcopy(config)
    other["layers"][1]["mixer"]["mask"]["size"] = 21
    assert np.abs(plain.forward(other, w, tokens)[0][20:] - whole[20:]).max() > 1e-3
    np.testing.assert_allclose(plain.forward(dict(config, logit_scale=1.0), w, tokens)[0] * 0.5, whole, rtol=1e-12)
