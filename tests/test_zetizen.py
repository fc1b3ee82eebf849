"""Zetizen: every mechanism alone against the plain implementation, then whole models in every cutting of the
work (whole prompts, token by token, portions down to two tokens, unequal requests in one batch, pages given back
and used again), long decoding from captured steps, the trace tool and greedy generation through the engine."""

from __future__ import annotations

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from gunedra_helpers import MEAN_TOLERANCE, TOLERANCE, Replay, as_float64, row_error, write_folder
from helpers import TRACE_RUN
from plain import zetizen_plain as plain
from test_parts import context_for
from test_tunadra import step_mixers
from zetizen_helpers import ALPHA, CONFIGS, biased_layer, chunked_layer, draw_weights, latent_layer, moe, scaling

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CLOSE = {"float32": dict(atol=2e-5, rtol=2e-5), "bfloat16": dict(atol=5e-2, rtol=3e-2)}


def rounded(array: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype)


# --- kernels and parts alone ---------------------------------------------------------------------------


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [48, 40, 257, 4100, 13000])
def test_layer_norm_adds_two_pending_outputs_and_takes_the_mean_off(name, hidden):
    from llm_inference_b200.parts import PartSpec, build_part, ops

    dtype, tokens = DTYPES[name], 9
    rng = np.random.default_rng(hidden)
    norm = build_part("norm", PartSpec("layernorm", dict(name="n", hidden_size=hidden, eps=1e-5)))
    weight = rounded(1.0 + rng.normal(0, 0.3, hidden), torch.bfloat16)
    norm.load({"n": weight}, dtype, torch.device("cuda:0"))
    x0 = rng.normal(2.5, 3.0, (tokens, hidden)).astype(np.float32)  # a mean far from zero: an RMS norm would show
    a, b = rounded(rng.normal(0, 1, (tokens, hidden)), dtype), rounded(rng.normal(0.5, 1, (tokens, hidden)), dtype)
    tolerance = dict(atol=1e-5, rtol=1e-5) if name == "float32" else dict(atol=2e-2, rtol=1e-2)
    for pending, total in ((None, x0.astype(np.float64)), (a.cuda(), x0 + a.double().numpy()),
                           (ops.BranchSum(a.cuda(), b.cuda()), x0 + a.double().numpy() + b.double().numpy()),
                           (ops.BranchSum(a.cuda(), None), x0 + a.double().numpy())):
        _, _, ctx = context_for({}, dtype, [tokens])
        x = torch.from_numpy(x0).cuda()
        got = norm.forward(ctx, x, pending)
        np.testing.assert_allclose(x.double().cpu().numpy(), total, atol=1e-6, rtol=1e-6)  # the stream holds the 32-bit sum
        want = plain.layer_norm(total, weight.double().numpy(), 1e-5)
        np.testing.assert_allclose(got.double().cpu().numpy(), want, **tolerance)
        assert np.abs(want - plain.rms_norm(total, weight.double().numpy(), 1e-5)).max() > 0.3
    # gathered rows: the pending outputs count, the stream stays
    _, _, ctx = context_for({}, dtype, [tokens])
    x = torch.from_numpy(x0).cuda()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    got = norm.forward(ctx, x, ops.BranchSum(a.cuda(), b.cuda()), rows=rows, out_name="normed_rows")
    want = plain.layer_norm((x0 + a.double().numpy() + b.double().numpy())[[7, 0, 3]], weight.double().numpy(), 1e-5)
    np.testing.assert_allclose(got.double().cpu().numpy(), want, **tolerance)
    assert torch.equal(x.cpu(), torch.from_numpy(x0))


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
def test_embedding_ends_in_a_layer_norm_and_the_tied_head_scales_its_logits(name):
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, vocab, tokens = DTYPES[name], 72, 130, 11
    rng = np.random.default_rng(3)
    weights = {"emb": rounded(rng.normal(0.4, 1.0, (vocab, hidden)), torch.bfloat16), "emb.norm": rounded(1.0 + rng.normal(0, 0.3, hidden), torch.bfloat16)}
    embedding = build_part("embedding", PartSpec("normed_embedding", dict(name="emb", norm_name="emb.norm", vocab_size=vocab, hidden_size=hidden, eps=1e-4)))
    head = build_part("head", PartSpec("linear_head", dict(name="head", suffix="", tied_to="emb", vocab_size=vocab, hidden_size=hidden, scale=0.3)))
    for part in (embedding, head):
        part.load(weights, dtype, torch.device("cuda:0"))
    head.share(embedding)
    assert head.weight.data_ptr() == embedding.table.data_ptr()
    runner, _, ctx = context_for({}, dtype, [tokens])
    ids = rng.integers(0, vocab, tokens)
    ctx.token_ids.copy_(torch.from_numpy(ids.astype(np.int32)).cuda())
    x = embedding.forward(ctx)
    w64 = as_float64(weights)
    want = plain.layer_norm(w64["emb"][ids], w64["emb.norm"], 1e-4)
    assert x.dtype == torch.float32
    np.testing.assert_allclose(x.double().cpu().numpy(), want, atol=2e-6, rtol=2e-6)  # 32-bit in both precisions
    h = rounded(rng.normal(0, 1, (4, hidden)), dtype)
    logits = head.forward(ctx, h.cuda())
    np.testing.assert_allclose(logits.double().cpu().numpy(), plain.linear(h.double().numpy(), w64["emb"]) * 0.3, atol=1e-4 if name == "float32" else 2e-2, rtol=1e-3)
    runner.check()
    ctx.token_ids[2] = vocab  # outside the table: flagged, not read
    embedding.forward(ctx)
    with pytest.raises(Exception, match="token id"):
        runner.check()


@pytest.mark.parametrize("experts,top", [(6, 2), (8, 1), (5, 5), (64, 8), (96, 40), (3, 2)])
def test_router_weighs_by_a_softmax_over_the_chosen_logits(experts, top):
    from llm_inference_b200.parts import ops

    tokens = 50
    _, _, ctx = context_for({}, torch.float32, [tokens])
    rng = np.random.default_rng(experts * 7 + top)
    logits = rng.normal(0, 2, (tokens, experts)).astype(np.float32)
    bias = rng.normal(0, 1.5, experts).astype(np.float32)  # large enough to change who wins
    ids = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    ops.moe_route(ctx, torch.from_numpy(logits).cuda(), 1, 1, top, 1.0, ids, weights, bias=torch.from_numpy(bias).cuda(), softmax_chosen=True)
    ids, weights = ids.cpu().numpy(), weights.cpu().numpy()
    want_ids, want_weights = plain.route(logits.astype(np.float64) + bias, top)
    np.testing.assert_array_equal(ids, want_ids)
    np.testing.assert_allclose(weights, want_weights, rtol=3e-6, atol=1e-9)
    np.testing.assert_allclose(weights.sum(-1), 1.0, rtol=1e-5)
    if top < experts:
        assert (want_ids != plain.route(logits.astype(np.float64), top)[0]).any()  # the bias decides some choices


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(experts=5, top=3, ff=28, shared=None), dict(experts=4, top=4, ff=36, shared=8), dict(experts=7, top=1, ff=70, shared=None),
                                   dict(experts=40, top=6, ff=8, shared=3)])
def test_unclamped_experts_alone_and_a_token_alone_equals_the_token_in_a_batch(name, sizes):
    from llm_inference_b200.models.zetizen import zetizen_feed_forward
    from llm_inference_b200.parts import build_part

    dtype, hidden, tokens = DTYPES[name], 48, 150
    mlp = moe(**sizes)
    config = dict(ALPHA, layers=[dict(biased_layer(), mlp=mlp)])
    weights = {k: v for k, v in draw_weights(config, 31).items() if k.startswith("l0.mlp.")}
    part = build_part("feed_forward", zetizen_feed_forward(mlp, "l0.mlp.", hidden))
    part.load(weights, dtype, torch.device("cuda:0"))
    h = rounded(np.random.default_rng(1).normal(0, 1, (tokens, hidden)), dtype)
    _, _, ctx = context_for({}, dtype, [tokens])
    got = part.forward(ctx, h.cuda()).clone()
    chosen = ctx.buffer("moe_ids:l0.mlp.", (tokens, part.top), torch.int32).cpu().numpy()
    free: list = []
    want = plain.routed_experts(h.double().numpy(), as_float64(weights), "l0.mlp.", mlp, choices=None if name == "float32" else chosen, free=free)
    assert (np.sort(chosen, -1) != np.sort(free[0], -1)).any(-1).mean() <= (0.0 if name == "float32" else 0.05)
    scale = np.abs(want).max()
    np.testing.assert_allclose(got.double().cpu().numpy() / scale, want / scale, atol=3e-6 if name == "float32" else 2e-2, rtol=0)
    for rows in ([7], [149, 3, 64]):
        _, _, small = context_for({}, dtype, [len(rows)])
        alone = part.forward(small, h[rows].cuda())
        assert torch.equal(alone, got[rows])


@pytest.mark.parametrize("hidden,ff,experts", [(64, 72, 4), (200, 136, 3)])
def test_unclamped_experts_on_tall_tiles(hidden, ff, experts):
    """bfloat16, 1,100 tokens over a few experts: enough slots per expert that the step sorts them into tiles of 128
    places, which run on tcgen05; the FMA kernels and the plain implementation agree within rounding."""
    from llm_inference_b200.models.zetizen import zetizen_feed_forward
    from llm_inference_b200.parts import build_part

    tokens = 1100
    mlp = moe(experts=experts, top=2, ff=ff, shared=24)
    config = dict(ALPHA, width=hidden, layers=[dict(biased_layer(), mlp=mlp)])
    weights = {k: v for k, v in draw_weights(config, 13).items() if k.startswith("l0.mlp.")}
    part = build_part("feed_forward", zetizen_feed_forward(mlp, "l0.mlp.", hidden))
    part.load(weights, torch.bfloat16, torch.device("cuda:0"))
    h = rounded(np.random.default_rng(1).normal(0, 1, (tokens, hidden)), torch.bfloat16)
    runner, _, ctx = context_for({}, torch.bfloat16, [1])
    ctx.num_tokens = tokens
    got = part.forward(ctx, h.cuda()).clone()
    runner.check()
    chosen = ctx.buffer("moe_ids:l0.mlp.", (tokens, 2), torch.int32).cpu().numpy()
    want = plain.routed_experts(h.double().numpy(), as_float64(weights), "l0.mlp.", mlp, choices=chosen)
    scale = np.abs(want).max()
    np.testing.assert_allclose(got.double().cpu().numpy() / scale, want / scale, atol=2e-2, rtol=0)
    ctx.options = dict(ctx.options, moe="plain")
    simple = part.forward(ctx, h.cuda()).clone()
    np.testing.assert_allclose(simple.double().cpu().numpy() / scale, got.double().cpu().numpy() / scale, atol=1e-2, rtol=0)


PORTIONS = (7, 1, 2, 9, 1, 1, 1, 16, 1, 1, 1, 1, 28)  # single tokens at positions 7, 19 to 21 and 38 to 41: both sides of chunk and page edges


def run_in_portions(mixer, weights, dtype, inputs, total):
    """Request 10 in PORTIONS beside request 11 (three tokens, then one by one), pages of 8 poisoned with NaN."""
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    for group in cache.groups:
        group.arena.fill_(float("nan"))  # pages are not cleared between requests: a request reads only what it wrote
    mixer.load(weights, dtype, torch.device("cuda:0"))
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other = 0, 0
    for portion in PORTIONS:
        step = [(10, slice(at, at + portion))]
        if other < 9:
            step.insert(0, (11, slice(other, other + (1 if other else 3))))
        (out,) = step_mixers(runner, cache, [mixer], step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
        other += (1 if other else 3) if other < 9 else 0
    runner.check()
    assert at == total
    return {rid: np.concatenate(parts) for rid, parts in got.items()}


SHAPED = {
    "biased": biased_layer(),
    "biased, one kv head, short reach": biased_layer(heads=5, kv_heads=1, dim=40, vdim=72, scale=0.4, softcap=3.0, bias=(9, 6)),
    "biased, heads of 64": biased_layer(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.3, softcap=10.0, bias=(60, 16)),
    "biased, narrow values in heads of 128": biased_layer(heads=2, kv_heads=2, dim=128, vdim=96, scale=0.2, softcap=None, bias=(33, 8)),
    "no cap, no bias": biased_layer(heads=3, kv_heads=3, dim=8, vdim=136, scale=1.0, softcap=None, bias=None),
    "chunked": chunked_layer(),
    "chunked, chunks of 8 (a page), heads of 64 rotated whole": chunked_layer(heads=4, kv_heads=2, dim=64, scale=0.3, softcap=6.0, chunk=8, rot=(64, 1000.0, scaling(4.0, 48, 16.0, 1.0))),
    "chunked, chunks of 21, heads of 128": chunked_layer(heads=6, kv_heads=3, dim=128, scale=0.2, softcap=20.0, chunk=21, rot=(48, 300000.0, scaling(6.0, 1024, 16.0, 2.0))),
    "chunked, one chunk for all, unscaled frequencies": chunked_layer(heads=2, kv_heads=1, dim=16, scale=0.8, softcap=None, chunk=1000, rot=(4, 10.0, None)),
    "values are keys, nothing else": chunked_layer(heads=3, kv_heads=1, dim=24, scale=0.5, softcap=None, chunk=0, rot=None),
}


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", sorted(SHAPED))
def test_shaped_attention_alone_in_portions_beside_another_request(name, case):
    """70 tokens over pages of 8 in portions that end before, on and after page and chunk edges, single tokens on both
    sides of them, a second request in the same steps. Scores are a few units wide, so single keys carry weight: the
    test itself asserts that a chunk one position longer or shorter, a bias table read one row off, a missing cap or
    the keys of the first page left out move the output far outside the tolerance."""
    from llm_inference_b200.models.zetizen import zetizen_mixer
    from llm_inference_b200.parts import build_part

    dtype, hidden, total = DTYPES[name], 48, 70
    layer = SHAPED[case]
    config = dict(ALPHA, layers=[dict(layer, mlp=None)])
    m = layer["mixer"]
    weights = {k: v for k, v in draw_weights(config, 21).items() if ".mix." in k}
    w64 = as_float64(weights)
    mixer = build_part("mixer", zetizen_mixer(layer["type"], m, "l0.mix.", hidden, 1e-5))
    rng = np.random.default_rng(8)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (9, hidden)), dtype)}
    reference = plain.MIXERS[layer["type"]]

    def expect(rows, sizes=m, first=0, table=w64):
        return reference(rows, table, "l0.mix.", sizes, 1e-5, np.arange(first, first + len(rows)), {})

    want = {rid: expect(rows.double().numpy()) for rid, rows in inputs.items()}
    long = inputs[10].double().numpy()
    size = m["mask"]["size"] if m.get("mask") else 0
    if not size or size > 30:
        assert np.abs(expect(long[8:])[-20:] - want[10][-20:]).max() > 0.05  # keys 50 and more positions back carry the last queries
    if size and size < total:
        for other in (size - 1, size + 1):
            assert np.abs(expect(long, dict(m, mask={"size": other})) - want[10]).max() > 0.2
    if m.get("softcap"):
        assert np.abs(expect(long, {k: v for k, v in m.items() if k != "softcap"}) - want[10]).max() > 0.02
    if m.get("bias_max"):
        shifted = dict(w64, **{"l0.mix.rel": np.roll(w64["l0.mix.rel"], 1, axis=0)})
        assert np.abs(expect(long, table=shifted) - want[10]).max() > 0.2
        assert np.abs(expect(long, dict(m, bias_max=m["bias_max"] + 7)) - want[10]).max() > 0.02
    if m.get("rot"):
        assert np.abs(expect(long, dict(m, rot=dict(m["rot"], base=m["rot"]["base"] * 3))) - want[10]).max() > 0.02
    got = run_in_portions(mixer, weights, dtype, inputs, total)
    np.testing.assert_allclose(got[10], want[10], **CLOSE[name])
    np.testing.assert_allclose(got[11], want[11], **CLOSE[name])


LATENT = {
    "small": latent_layer(),
    "one head, odd sizes, unscaled": latent_layer(heads=1, dim=6, rot_dim=2, vdim=5, kv_rank=7, q_rank=3, scale=0.9, scale_rule=None),
    "tensor-core sizes": latent_layer(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=32, scale=0.25, base=500.0, scale_rule=scaling(2.0, 40, 8.0, 1.0)),
    "many heads, wide latent": latent_layer(heads=20, dim=16, rot_dim=32, vdim=24, kv_rank=96, q_rank=50, scale=0.2, base=15000.0, scale_rule=scaling(3.0, 1024, 24.0, 1.0)),
}


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", sorted(LATENT))
def test_latent_attention_with_a_query_latent_alone_in_portions(name, case):
    """Queries through their own latent, the rotated part in halves with the ramp's magnitude, an element-wise gate; the
    same portions, pages and neighbour as above. The test asserts that the gate, the query latent's norm and the
    rotation show in the result."""
    from llm_inference_b200.models.zetizen import zetizen_mixer
    from llm_inference_b200.parts import build_part

    dtype, hidden, total = DTYPES[name], 48, 70
    layer = LATENT[case]
    config = dict(ALPHA, layers=[dict(layer, mlp=None)])
    m = layer["mixer"]
    weights = {k: v for k, v in draw_weights(config, 22).items() if ".mix." in k}
    w64 = as_float64(weights)
    mixer = build_part("mixer", zetizen_mixer("latent_attention", m, "l0.mix.", hidden, 1e-5))
    assert mixer.cache_spec().head_dim == m["kv_rank"] + m["rot_dim"] and mixer.cache_spec().planes == 1
    rng = np.random.default_rng(9)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (9, hidden)), dtype)}

    def expect(rows, sizes=m, table=w64):
        return plain.latent_attention(rows, table, "l0.mix.", sizes, 1e-5, np.arange(len(rows)), {})

    want = {rid: expect(rows.double().numpy()) for rid, rows in inputs.items()}
    long = inputs[10].double().numpy()
    assert np.abs(expect(long, table=dict(w64, **{"l0.mix.g": 0 * w64["l0.mix.g"]})) - want[10]).max() > 0.05
    assert np.abs(expect(long, table=dict(w64, **{"l0.mix.dq.norm": np.roll(w64["l0.mix.dq.norm"], 1)})) - want[10]).max() > 0.01
    if m["rot_dim"] > 2:  # a rotated part of two numbers has the one frequency 1, whatever the base
        assert np.abs(expect(long, dict(m, rot=dict(m["rot"], base=m["rot"]["base"] * 7))) - want[10]).max() > 0.005
    got = run_in_portions(mixer, weights, dtype, inputs, total)
    np.testing.assert_allclose(got[10], want[10], **CLOSE[name])
    np.testing.assert_allclose(got[11], want[11], **CLOSE[name])


@pytest.mark.parametrize("case", ["biased, heads of 64", "chunked, chunks of 21, heads of 128", "chunked, chunks of 8 (a page), heads of 64 rotated whole"])
def test_tensor_core_kernels_against_the_plain_kernel_far_in(case):
    """bfloat16, 600 keys over pages of 16: prompt portions run the tcgen05 kernel (heads of 128 with a cap and chunks) or
    the mma.sync prefill kernel, single tokens at a page border and just past a chunk edge the split-key kernel; the same
    steps run the plain kernel. Unwritten rows of the pages hold NaN."""
    from llm_inference_b200.models.zetizen import zetizen_mixer
    from llm_inference_b200.parts import build_part

    hidden, total = 48, 600
    layer = SHAPED[case]
    m = layer["mixer"]
    config = dict(ALPHA, layers=[dict(layer, mlp=None)])
    weights = {k: v for k, v in draw_weights(config, 23).items() if ".mix." in k}
    mixer = build_part("mixer", zetizen_mixer(layer["type"], m, "l0.mix.", hidden, 1e-5))
    rows = rounded(np.random.default_rng(5).normal(0, 1, (total, hidden)), torch.bfloat16)
    want = plain.MIXERS[layer["type"]](rows.double().numpy(), as_float64(weights), "l0.mix.", m, 1e-5, np.arange(total), {})
    results = {}
    for choice in ("auto", "plain"):
        from llm_inference_b200.cache import PagedCache
        from llm_inference_b200.engine.runner import ModelRunner
        from types import SimpleNamespace

        device = torch.device("cuda:0")
        cache = PagedCache({0: mixer.cache_spec()}, dtype=torch.bfloat16, device=device, page_size=16, max_num_sequences=4, max_model_length=1024,
                           step_tokens=1024, num_pages=64)
        for group in cache.groups:
            group.arena[:, :, :-1].fill_(float("nan"))  # every page a request can hold; the spare page that pads block tables stays finite
        runner = ModelRunner(SimpleNamespace(device=device, dtype=torch.bfloat16), cache, max_batch_tokens=1024, options={"attention": choice})
        mixer.load(weights, torch.bfloat16, device)
        cache.open(10)
        parts, at = [], 0
        for portion in (511, 1, 1, 50, 1, 1, 1, 34):
            (out,) = step_mixers(runner, cache, [mixer], [(10, slice(at, at + portion))], {10: rows})
            parts.append(out[10])
            at += portion
        runner.check()
        results[choice] = np.concatenate(parts)
    np.testing.assert_allclose(results["plain"], want, atol=5e-2, rtol=3e-2)
    np.testing.assert_allclose(results["auto"], want, atol=5e-2, rtol=3e-2)
    assert np.abs(results["auto"] - results["plain"]).max() < 4e-2 and np.abs(results["auto"] - results["plain"]).max() > 0  # other kernels ran


# --- whole models ---------------------------------------------------------------------------------------------


LENGTHS = [1, 2, 3, 9, 31, 70, 150]


@pytest.fixture(scope="module", params=["alpha", "beta", "gamma", "delta"])
def model_case(request, tmp_path_factory):
    config = CONFIGS[request.param]
    weights = draw_weights(config, seed=17 + len(request.param))
    folder = write_folder(tmp_path_factory.mktemp(request.param), config, weights)
    rng = np.random.default_rng(4)
    sequences = {f"s{n}": [int(t) for t in rng.integers(0, config["vocab"], n)] for n in LENGTHS}
    w64 = as_float64(weights)
    expected = {key: plain.forward(config, w64, tokens)[0] for key, tokens in sequences.items()}
    return request.param, config, folder, sequences, expected, w64


# A router's choice is a step function of its logits: where two candidates are closer than bfloat16 rounding moves
# them, the engine may rightly choose the other one, and that token's logits (and, through the cache, later ones) then
# differ by much more than rounding. So in bfloat16 the plain implementation is run along the engine's own choices,
# which every routed layer leaves in a buffer of its own, and each choice that differs from the plain one must have
# been a close call in that run. In float32 the plain implementation's own choices stand.
CLOSE_CALL = 0.1


class RoutedReplay(Replay):
    """A replay that also files every routed layer's choices by (request, layer, position)."""

    def __init__(self, config, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.routed = {i: layer["mlp"]["router"]["top"] for i, layer in enumerate(config["layers"]) if layer.get("mlp") is not None}
        self.chosen: dict[tuple[str, int, int], np.ndarray] = {}

    def step(self, portions, end=()):
        before = {name: self.at.get(name, 0) for name, _ in portions}
        super().step(portions, end)
        order = sorted(range(len(portions)), key=lambda i: (len(portions[i][1]) != 1, i))  # single tokens lead a batch
        for layer, top in self.routed.items():
            flat = self.runner.workspace._flat[f"moe_ids:l{layer}.mlp.:torch.int32"].cpu().numpy()
            row = 0
            for i in order:
                name, tokens = portions[i]
                for j in range(len(tokens)):
                    self.chosen[(name, layer, before[name] + j)] = flat[row * top : (row + 1) * top].copy()
                    row += 1

    def choices(self, name: str, length: int) -> dict[int, np.ndarray]:
        return {layer: np.stack([self.chosen[(name, layer, i)] for i in range(length)]) for layer in self.routed}


def expected_along(case, replay, key: str, tokens, dtype: str) -> np.ndarray:
    """The plain logits for ``tokens``: in bfloat16 along the engine's choices of experts, which may differ from the
    plain ones only where the plain run saw a close call."""
    _, config, _, _, expected, w64 = case
    if dtype == "float32":
        return expected[key] if key in expected else plain.forward(config, w64, tokens)[0]
    choices = replay.choices(key, len(tokens))
    margins, free = [], []
    logits, _ = plain.forward(config, w64, tokens, margins=margins, choices=choices, free=free)
    differing = 0
    for at, layer in enumerate(sorted(choices)):
        for t in range(len(tokens)):
            if set(choices[layer][t].tolist()) != set(free[at][t].tolist()):
                differing += 1
                assert margins[at][t] < CLOSE_CALL, f"request {key}, layer {layer}, position {t}: the engine chose {choices[layer][t]}, plain {free[at][t]} by {margins[at][t]:.3f}"
    assert differing <= 0.1 * max(1, len(choices)) * len(tokens) + 1
    return logits


def check_all(case, replay, sequences, dtype: str, what: str) -> None:
    errors = []
    for key, tokens in sequences.items():
        error = row_error(replay.of(key, len(tokens)), expected_along(case, replay, key, tokens, dtype))
        assert error.max() <= TOLERANCE[dtype], f"{what}: request {key}, position {int(error.argmax())}: error {error.max():.2e}"
        errors.append(error)
    mean = np.concatenate(errors).mean()
    assert mean <= MEAN_TOLERANCE[dtype], f"{what}: mean error over all rows {mean:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_one_by_one_against_plain(model_case, dtype):
    """The stream after every layer of a short prompt, so that a fault names its layer."""
    from llm_inference_b200.engine.runner import StepEntry
    from llm_inference_b200.parts import ops

    _, config, folder, sequences, _, w64 = model_case
    tokens = sequences["s31"]
    replay = RoutedReplay(config, folder, dtype, 64)
    replay.cache.open(1)
    replay.cache.manager.ensure(1, len(tokens))
    replay.cache.clear_new_slots()
    ctx = replay.runner._build_context([StepEntry(1, tokens)], [0], [])
    x = replay.model.embedding.forward(ctx)
    total = x.double().clone()
    pending, streams, choices = None, [], {}
    for index, call in enumerate(replay.model.schedule):
        block = replay.model.blocks[call.layer]
        pending = block.forward(ctx, replay.runner._view(call, replay.runner._tables), x, pending)
        branches = (pending.a, pending.b) if isinstance(pending, ops.BranchSum) else (pending,)
        total = total + sum(b.double() for b in branches if b is not None)
        streams.append(total.cpu().numpy())
        if block.feed_forward is not None:
            choices[index] = ctx.buffer(f"moe_ids:l{index}.mlp.", (len(tokens), block.feed_forward.top), torch.int32).cpu().numpy()
    replay.runner.check()
    layers: list = []
    plain.forward(config, w64, tokens, layer_outputs=layers, choices=None if dtype == "float32" else choices)
    for index, (got, want) in enumerate(zip(streams, layers)):
        error = np.abs(got - want).max() / np.abs(want).max()
        assert error <= (1e-5 if dtype == "float32" else 6e-2), f"layer {index} ({config['layers'][index]['type']}): {error:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_one_after_another_in_a_pool_for_one(model_case, dtype):
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        replay.step([(key, tokens)], end=(key,))
    check_all(model_case, replay, sequences, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model_case, dtype):
    """All but the last 40 tokens as one portion, the rest one by one (captured steps replayed)."""
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        head = max(0, len(tokens) - 40)
        if head:
            replay.step([(key, tokens[:head])])
        for position in range(head, len(tokens)):
            replay.step([(key, [tokens[position]])], end=(key,) if position == len(tokens) - 1 else ())
    check_all(model_case, replay, sequences, dtype, "token by token")
    assert replay.runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2,), (3, 1, 2, 8, 1, 17), (7, 9, 64)])
def test_portions_of_changing_size(model_case, dtype, sizes):
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        at, turn = 0, 0
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            replay.step([(key, tokens[at : at + size])], end=(key,) if at + size == len(tokens) else ())
            at, turn = at + size, turn + 1
    check_all(model_case, replay, sequences, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_pages_used_again(model_case, dtype):
    """Up to three live requests (38 pages of 8 for sequences that need 46 in all): portions of some beside single tokens
    of others, requests left out of steps, and every request that ends hands its pages to one that starts later."""
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 304, slots=3)
    rng = np.random.default_rng(9)
    waiting = ["s150", "s70", "s31", "s9", "s3", "s2", "s1", "again70", "again9"]
    sequences = dict(sequences, again70=sequences["s70"], again9=sequences["s9"])
    live: dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        portions, end = [], []
        for key in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            left = len(sequences[key]) - live[key]
            size = min(left, int(rng.choice([1, 1, 1, 2, 3, 8, 29])))
            portions.append((key, sequences[key][live[key] : live[key] + size]))
            live[key] += size
            if live[key] == len(sequences[key]):
                end.append(key)
                del live[key]
        if portions:
            replay.step(portions, end=tuple(end))
    check_all(model_case, replay, sequences, dtype, "mixed")
    stats = replay.cache.stats()
    assert stats["requests"] == 0 and stats["live_tokens"] == 0
    assert all(pool["used_pages"] == 0 and pool["high_water"] <= pool["capacity_pages"] for pool in stats["kv_pools"].values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_case, dtype):
    """Four tokens of prompt, then 330 single tokens: the cache after hundreds of steps, across many pages, chunks and the
    whole reach of the distance biases."""
    _, config, folder, _, _, w64 = model_case
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, config["vocab"], 334)]
    replay = RoutedReplay(config, folder, dtype, 384, slots=1)
    replay.step([("long", tokens[:4])])
    for token in tokens[4:]:
        replay.step([("long", [token])])
    error = row_error(replay.of("long", len(tokens)), expected_along(model_case, replay, "long", tokens, dtype))
    assert error.max() <= TOLERANCE[dtype], f"position {int(error.argmax())}: {error.max():.2e}"
    assert error.mean() <= MEAN_TOLERANCE[dtype] and error[-50:].mean() <= MEAN_TOLERANCE[dtype], f"mean {error.mean():.2e}, last 50 {error[-50:].mean():.2e}"
    assert replay.runner.graph_replays > 300


def test_trace_tool_mixed_schedule(model_case, tmp_path):
    """bin/trace_run itself: two requests interleaved, a third that reuses what the first gave back."""
    _, config, folder, sequences, expected, _ = model_case
    a, b, c = sequences["s70"], sequences["s31"], sequences["s9"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": [1]}, {"id": "a", "tokens": a[33:34], "want": [0]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[34:], "want": [35]}, {"id": "b", "tokens": b[2:3], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "b", "tokens": b[3:], "want": [27]}, {"id": "c", "tokens": c, "want": [8]}], "end": ["b", "c"]},
    ]
    want = [expected["s70"][[0, 32]], expected["s31"][[1]], expected["s70"][[33]], expected["s70"][[69]], expected["s31"][[30]], expected["s9"][[8]]]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        result = subprocess.run(
            [sys.executable, str(TRACE_RUN), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600,
        )
        assert result.returncode == 0, result.stderr[-3000:]
        assert [line for line in result.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(4)]
        got = np.concatenate([np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, config["vocab"]) for i in range(4)])
        error = row_error(got, np.concatenate(want))
        if dtype == "float32":
            assert error.max() <= TOLERANCE[dtype]
        else:  # the tool gives no routing choices to follow: all but a row that met a close call are within the bound
            assert np.sort(error)[-2] <= TOLERANCE[dtype]


def test_greedy_generation_through_the_engine(model_case):
    """submit / step / sample through the scheduler: float32 gives the plain implementation's tokens; two requests at once
    give what each gives alone."""
    from llm_inference_b200 import create_engine

    _, config, folder, sequences, _, w64 = model_case
    prompt, other = sequences["s31"], sequences["s9"]
    want = plain.greedy(config, w64, prompt, 12)
    with create_engine(folder, dtype="float32", max_num_sequences=3, max_model_length=128, kv_cache_bytes=4 << 20, page_size=8,
                       prefill_chunk_size=16, prefill_burst_size=16) as engine:
        assert engine.generate(prompt, 12) == want
        first, second = engine.submit(prompt, 12), engine.submit(other, 7)
        while engine.has_work():
            engine.step()
        assert engine.request(first).output == want
        assert engine.request(second).output == plain.greedy(config, w64, other, 7)
    with create_engine(folder, dtype="bfloat16", max_num_sequences=2, max_model_length=128, kv_cache_bytes=4 << 20, page_size=8) as engine:
        got = engine.generate(prompt, 12)
    tokens = list(prompt)
    for token in got:  # only a near-tie may go the other way in bfloat16
        row = plain.forward(config, w64, tokens)[0][-1]
        if token != int(np.argmax(row)):
            assert row.max() - row[token] <= 0.1 * row.std()
            break
        tokens.append(token)


def test_command_line_tools_take_the_design(tmp_path):
    """A seeded folder from the named shape, its inspection, and greedy generation from the folder and from the shape
    itself (weights drawn on the device)."""
    run = lambda *args: subprocess.run([sys.executable, "-m", *args], capture_output=True, text=True, timeout=600)
    folder = tmp_path / "model"
    made = run("llm_inference_b200.cli.random_model", "--preset", "zetizen-small", "--seed", "3", "--out", str(folder))
    assert made.returncode == 0, made.stderr[-2000:]
    seen = run("llm_inference_b200.cli.inspect_model", str(folder))
    assert seen.returncode == 0 and "architecture: Zetizen" in seen.stdout and "l2.mix.dq.norm" in seen.stdout, seen.stderr[-2000:]
    ask = ["--prompt-ids", "5,17,3,900,41", "--max-new-tokens", "6", "--max-model-length", "256", "--kv-cache-mib", "64"]
    from_folder = run("llm_inference_b200.cli.generate", "--model", str(folder), *ask)
    from_shape = run("llm_inference_b200.cli.generate", "--random", "zetizen-small", "--weights-seed", "3", *ask)
    assert from_folder.returncode == 0, from_folder.stderr[-2000:]
    assert from_shape.returncode == 0, from_shape.stderr[-2000:]
    for result in (from_folder, from_shape):
        line = json.loads(result.stdout.strip().splitlines()[-1])
        assert line["prompt_tokens"] == 5 and len(line["tokens"]) == 6 and all(0 <= t < 8192 for t in line["tokens"])
    # continuous batching with sampling through the scheduler: six requests of unequal lengths on three slots
    report = tmp_path / "bench.json"
    timed = run("llm_inference_b200.cli.benchmark", "--random", "zetizen-small", "--mix", "6", "--mix-prompt-lengths", "20", "90",
                "--mix-output-lengths", "4", "12", "--max-sequences", "3", "--max-model-length", "256", "--kv-cache-mib", "64", "--warmups", "0",
                "--repetitions", "1", "--output", str(report))
    assert timed.returncode == 0, timed.stderr[-2000:]
    assert report.exists() and json.loads(report.read_text())
