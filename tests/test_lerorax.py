"""Lerorax: every mechanism alone against the plain implementation, then whole models in every cutting of
the work (whole prompts, token by token, portions down to two tokens, unequal requests in one batch, pages
and state slots given back and used again), long decoding from captured steps, the trace tool and greedy
generation through the engine."""

from __future__ import annotations

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from gunedra_helpers import MEAN_TOLERANCE, TOLERANCE, Replay, as_float64, row_error, write_folder
from helpers import TRACE_RUN
from lerorax_helpers import ALPHA, CONFIGS, config_of, draw_weights, mingru_layer, parallel_layer, with_mlp
from plain import lerorax_plain as plain
from test_parts import context_for
from test_tunadra import step_mixers

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CLOSE = {"float32": dict(atol=3e-5, rtol=3e-5), "bfloat16": dict(atol=5e-2, rtol=3e-2)}


def rounded(array: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype)


def on_device(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()


def poison(cache) -> None:
    """A slot is cleared when it is handed out and pages are never cleared: a request reads only what it wrote
    (and the arena's last page, which no request holds: block tables are padded with it, it stays zero, and kernels
    that fetch whole tiles read it under a weight of zero)."""
    for group in cache.groups:
        group.arena[:, :, :-1].fill_(float("nan"))
    for arrays in cache.states.values():
        for array in arrays:
            array.fill_(-7 if array.dtype == torch.int32 else float("nan"))


def one_layer(layer: dict, width: int = 48) -> dict:
    return config_of(width, 97, [layer])


# --- kernels and parts alone ---------------------------------------------------------------------------


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur,hidden", [(61, 31, 5, 48), (1, 3, 2, 40), (521, 100003, 77777, 260), (7, 0, 1, 16)])
def test_bigram_embedding_keeps_the_token_in_front_across_steps(name, buckets, mul_prev, mul_cur, hidden):
    """Two requests in portions of 1, 2, 5 tokens: the row of the pair table follows from the token in front,
    which for a portion's first token comes from the request's slot; a request's very first token takes the last
    row. Products of token and multiplier beyond 32 bits are in the third case."""
    from llm_inference_b200.engine.runner import StepEntry
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, vocab = DTYPES[name], 30011
    part = build_part("embedding", PartSpec("bigram_embedding", dict(
        name="embed", pairs_name="bigram", vocab_size=vocab, hidden_size=hidden, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur, cast=True)))
    rng = np.random.default_rng(buckets)
    table, pairs = rounded(rng.normal(0, 1, (vocab, hidden)), torch.bfloat16), rounded(rng.normal(0, 1, (buckets + 1, hidden)), torch.bfloat16)
    runner, cache, _ = context_for({0: part.cache_spec()}, dtype, [1])
    part.load({"embed": table, "bigram": pairs}, dtype, runner.device)
    poison(cache)
    tokens = {10: [int(t) for t in rng.integers(vocab - 200, vocab, 19)], 11: [int(t) for t in rng.integers(0, vocab, 9)]}
    cache.open(10), cache.open(11)
    at = {10: 0, 11: 0}
    got = {10: [], 11: []}
    for sizes in ((5, 1), (1, 2), (2, 1), (1, 5), (10, 0)):
        entries = [StepEntry(rid, tokens[rid][at[rid] : at[rid] + size]) for rid, size in zip((10, 11), sizes) if size]
        entries.sort(key=lambda e: len(e.tokens) != 1)
        starts = [cache.manager.length(e.request_id) for e in entries]
        for e, s in zip(entries, starts):
            cache.manager.ensure(e.request_id, s + len(e.tokens))
        cache.clear_new_slots()
        ctx = runner._build_context(entries, starts, [])
        x = part.forward(ctx, cache.view(0, True, runner._tables)).cpu().numpy()
        if dtype != torch.float32:
            cast = ctx.buffer("stream_cast", (ctx.num_tokens, hidden)).float().cpu().numpy()
            np.testing.assert_allclose(cast, x, rtol=2 ** -8, atol=0)
        row = 0
        for e, s in zip(entries, starts):
            got[e.request_id].append(x[row : row + len(e.tokens)])
            row += len(e.tokens)
            at[e.request_id] += len(e.tokens)
            cache.manager.advance(e.request_id, s + len(e.tokens))
    runner.check()
    for rid, ids in tokens.items():
        rows, _ = plain.bigram_rows(ids, None, buckets, mul_prev, mul_cur)
        assert rows[0] == buckets and (buckets == 1 or len(set(rows.tolist())) > 2)
        want = table.double().numpy()[ids] + pairs.double().numpy()[rows]
        np.testing.assert_allclose(np.concatenate(got[rid]), want, atol=1e-6, rtol=0)


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,total", [(56, 41), (384, 250), (7, 200), (130, 129)])
def test_mingru_alone_in_portions_beside_another_request(name, width, total):
    """The state carries across steps of 5, 1, 2, ... tokens and across a portion long enough to run in pieces at
    the same time (more than 128 tokens); a second request moves through another slot. The slowest channels
    keep the first tokens to the end: without them the last outputs differ visibly."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden = DTYPES[name], 48
    config = one_layer(with_mlp(mingru_layer(width), None))
    weights = {k: v for k, v in draw_weights(config, 5).items() if k.startswith("l0.mix.")}
    w64 = as_float64(weights)
    args = [w64["l0.mix." + n] for n in ("z", "z.b", "x", "x.b", "g", "o")]
    mixer = build_part("mixer", PartSpec("mingru", dict(prefix="l0.mix.", hidden_size=hidden, width=width)))
    rng = np.random.default_rng(2)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (12, hidden)), dtype)}
    want = {rid: plain.mingru(rows.double().numpy(), np.zeros(width), *args)[0] for rid, rows in inputs.items()}
    skipped = 3 if total < 100 else total // 2
    headless = plain.mingru(inputs[10].double().numpy()[skipped:], np.zeros(width), *args)[0]
    assert np.abs(headless[-5:] - want[10][-5:]).max() > 1e-2
    mixer.load(weights, dtype, torch.device("cuda:0"))
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    poison(cache)
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other = 0, 0
    portions = [5, 1, 2, 1, 1, 17, 3, 1]
    portions.append(total - sum(portions) - 2)
    portions += [1, 1]
    for portion in portions:
        step = [(10, slice(at, at + portion))]
        if other < 12:
            size = 1 if other % 2 else 3
            step.append((11, slice(other, other + size)))
            other += size
        (out,) = step_mixers(runner, cache, [mixer], step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
    runner.check()
    assert at == total and other == 12
    scale = np.abs(want[10]).max()
    tolerance = dict(atol=(1e-5 if name == "float32" else 3e-2) * scale, rtol=0)
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **tolerance)
    np.testing.assert_allclose(np.concatenate(got[11]), want[11], **tolerance)


ATTENTION_SIZES = [
    dict(),
    dict(heads=5, kv_heads=1, dim=12, vdim=6, conv=1, scale=0.45, rot=None),
    dict(heads=3, kv_heads=3, dim=8, vdim=20, conv=4, scale=0.5, rot=(8, 1e4)),
    dict(heads=6, kv_heads=2, dim=64, vdim=64, conv=5, scale=0.11, rot=(48, 2e5), scaling=(6.0, 1.0, 3.0, 256)),
    dict(heads=6, kv_heads=3, dim=64, vdim=48, conv=2, scale=0.1, rot=(64, 300.0), scaling=(4.0, 1.0, 4.0, 64)),
    dict(heads=2, kv_heads=1, dim=128, vdim=128, conv=3, scale=0.06, rot=(16, 1e3)),
    dict(heads=2, kv_heads=1, dim=10, vdim=5, conv=2, scale=0.4, rot=(4, 1e3)),  # an odd size: numbers are loaded one by one
    dict(heads=4, kv_heads=2, dim=128, vdim=128, conv=2, scale=0.07, rot=(32, 1e4)),  # heads the tcgen05 prefill kernel takes, values of another kv head
]


def build_left(m: dict, hidden: int, eps: float):
    from llm_inference_b200.parts import PartSpec, build_part

    rot = m.get("rot") or {}
    position = PartSpec("rotary", dict(head_dim=m["dim"], theta=rot.get("base", 10000.0), rotary_dims=rot.get("dims", 0), interleaved=True, scaling=rot.get("scaling")))
    return build_part("mixer", PartSpec("mixed_head_attention", dict(
        prefix="l0.mix.left.", hidden_size=hidden, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], taps=m["conv"],
        scale=m["scale"], eps=eps, position=position)))


def plain_left(config, w64, rows, state=None):
    model = plain.PlainLerorax(config, w64)
    state = state or model.new_state()
    st = state["layers"][0]
    first = st["keys"].shape[0]
    out = model.left("l0.mix.left.", config["layers"][0]["mixer"]["left"], rows, st, np.arange(first, first + rows.shape[0]))
    return out, state


@pytest.mark.parametrize("name", ["float32", "bfloat16", "bfloat16-plain", "bfloat16-tcgen05", "bfloat16-passes"])
@pytest.mark.parametrize("sizes", ATTENTION_SIZES)
def test_attention_with_mixed_heads_alone_in_portions(name, sizes):
    """150 tokens over pages of 8 in portions that end before, on and after page borders, beside a second request
    that gets a slot and pages of its own. Token 2's key is made to match the last query of head 0 (the last input
    row is minus row 2, the key matrix of kv head 0 minus head 0's query matrix, no biases there, taps that pass the
    current token; the last token's own key then points away from its query and its value is minus token 2's): with a
    sharp softmax that one far key carries head 0, and through the mix over heads every head. The result without
    it, without the mix, without the convolution or without the gate is far outside the tolerance. In bfloat16 the
    tensor-core kernels run (every head here is padded to 64 or 128); "bfloat16-plain" asks for the plain one,
    "bfloat16-tcgen05" (heads of 128 over pages of 16) for the tcgen05 kernel in every prompt portion. Steps of single
    tokens only (the last five, and those beside the second request's single tokens) run the passes of all kv heads
    as one launch; "bfloat16-passes" runs them one by one there too."""
    name, _, kernels = name.partition("-")
    if kernels == "tcgen05" and sizes.get("dim") != 128:
        pytest.skip("the tcgen05 prefill kernel takes heads of 128")
    dtype, hidden, total = DTYPES[name], 48, 150
    config = one_layer(with_mlp(parallel_layer(**sizes), None))
    m = config["layers"][0]["mixer"]["left"]
    weights = {k: v.clone() for k, v in draw_weights(config, 21).items() if ".mix.left." in k and not k.endswith(".out")}
    dim, p = m["dim"], "l0.mix.left."
    weights[p + "k"][:dim] = -weights[p + "q"][:dim]
    weights[p + "k.b"][:dim] = weights[p + "q.b"][:dim] = 0
    weights[p + "k.norm"][:dim] = weights[p + "q.norm"][:dim] / 3
    weights[p + "q.norm"][:dim] *= 2
    for s in "qk":
        weights[p + s + ".conv"][:dim] = 0
        weights[p + s + ".conv"][:dim, -1] = 1
    w64 = as_float64(weights)
    rng = np.random.default_rng(8)
    long_rows = rng.normal(0, 1, (total, hidden))
    long_rows[-1] = -long_rows[2]
    inputs = {10: rounded(long_rows, dtype), 11: rounded(rng.normal(0, 1, (9, hidden)), dtype)}
    want = {rid: plain_left(config, w64, rows.double().numpy())[0] for rid, rows in inputs.items()}

    def changed(**replaced):
        return plain_left(config, dict(w64, **{p + k: v for k, v in replaced.items()}), inputs[10].double().numpy())[0]

    other = inputs[10].double().numpy().copy()
    other[2] = rng.normal(0, 1, hidden)
    bound = 10 * CLOSE[name]["atol"]
    spread = want[10][-1].std()
    far = np.abs(plain_left(config, w64, other)[0][-1] - want[10][-1]).max()  # the far key
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    slow = rot["dims"] * 2 <= dim and (rot["dims"] == 0 or rot["base"] >= 1000)  # the rotated dims turn the far key away, the rest still match
    assert not slow or far > spread
    assert np.abs(changed(talk=np.eye(m["heads"])) - want[10]).max() > max(bound, 0.3 * spread)
    assert np.abs(changed(g=0 * w64[p + "g"]) - want[10]).max() > bound
    if m["conv"] > 1:
        now = np.zeros_like(w64[p + "v.conv"])
        now[:, -1] = 1
        assert np.abs(changed(**{"v.conv": now}) - want[10]).max() > bound
    mixer = build_left(m, hidden, 1e-5)
    mixer.load(weights, dtype, torch.device("cuda:0"))  # the convolution's last inputs are kept in the dtype the weights were loaded in
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1], page_size=16 if kernels == "tcgen05" else 8)
    if name == "bfloat16":
        runner.options["attention"] = "flash" if kernels in ("", "passes") else kernels  # "flash" and "tcgen05" refuse a step they cannot take
        if kernels == "passes":
            runner.options["value_planes"] = "passes"
    poison(cache)
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other_at = 0, 0
    for portion in (7, 1, 2, 30, 1, 1, 8, 20, 2, 64, 9, 1, 1, 1, 1, 1):
        step = [(10, slice(at, at + portion))]
        if other_at < 9:
            size = 1 if other_at else 3
            step.insert(0, (11, slice(other_at, other_at + size)))
            other_at += size
        (out,) = step_mixers(runner, cache, [mixer], step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
    runner.check()
    assert at == total
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **CLOSE[name])
    np.testing.assert_allclose(np.concatenate(got[11]), want[11], **CLOSE[name])


DELTA_SIZES = [dict(), dict(right_heads=1, right_dim=6, decay_rank=2), dict(right_heads=2, right_dim=40, decay_rank=3), dict(right_heads=3, right_dim=130, decay_rank=4),
               dict(right_heads=1, right_dim=300, decay_rank=2), dict(right_heads=4, right_dim=64, decay_rank=16),
               dict(right_heads=2, right_dim=128, decay_rank=8), dict(right_heads=1, right_dim=256, decay_rank=4),
               dict(right_heads=2, right_dim=32, decay_rank=4), dict(right_heads=1, right_dim=12, decay_rank=2)]


def plain_right(config, w64, rows):
    model = plain.PlainLerorax(config, w64)
    return model.right("l0.mix.right.", config["layers"][0]["mixer"]["right"], rows, model.new_state()["layers"][0])


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", DELTA_SIZES)
def test_generalized_delta_rule_alone_in_portions_beside_another_request(name, sizes):
    """The matrix state carries across steps of 5, 1, 2, 1, ... tokens; a second request moves through another slot
    at the same time. The slowest channels keep the first token to the end: without it the last read-outs differ
    visibly; so they do without the removal along the key's direction and with one decay for all channels."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, total = DTYPES[name], 48, 41
    config = one_layer(with_mlp(parallel_layer(**sizes), None))
    m = config["layers"][0]["mixer"]["right"]
    p = "l0.mix.right."
    weights = {k: v for k, v in draw_weights(config, 5).items() if ".mix.right." in k and not k.endswith(".out")}
    w64 = as_float64(weights)
    mixer = build_part("mixer", PartSpec("general_delta", dict(prefix=p, hidden_size=hidden, heads=m["heads"], dim=m["dim"], eps=1e-5)))
    rng = np.random.default_rng(2)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (12, hidden)), dtype)}
    want = {rid: plain_right(config, w64, rows.double().numpy()) for rid, rows in inputs.items()}
    headless = plain_right(config, w64, inputs[10].double().numpy()[1:])
    assert np.abs(headless[-10:] - want[10][-10:]).max() > 1e-2
    keeps = plain_right(config, dict(w64, **{p + "a.b": w64[p + "a.b"] - 50.0}), inputs[10].double().numpy())
    assert np.abs(keeps - want[10]).max() > 1e-1
    flat = plain_right(config, dict(w64, **{p + "w0": 0 * w64[p + "w0"], p + "w2": 0 * w64[p + "w2"]}), inputs[10].double().numpy())
    assert np.abs(flat - want[10]).max() > 1e-1
    mixer.load(weights, dtype, torch.device("cuda:0"))
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    poison(cache)
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other = 0, 0
    for portion in (5, 1, 2, 1, 1, 17, 3, 1, 10):
        step = [(10, slice(at, at + portion))]
        if other < 12:
            size = 1 if other % 2 else 3
            step.append((11, slice(other, other + size)))
            other += size
        (out,) = step_mixers(runner, cache, [mixer], step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
    runner.check()
    assert at == total and other == 12
    scale = np.abs(want[10]).max()
    tolerance = dict(atol=(3e-5 if name == "float32" else 4e-2) * scale, rtol=0)
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **tolerance)
    np.testing.assert_allclose(np.concatenate(got[11]), want[11], **tolerance)


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [48, 40, 1030, 5000])
def test_pair_of_branches_is_combined_and_added_in_one_kernel(name, hidden):
    from llm_inference_b200.parts import ops

    dtype, rows = DTYPES[name], 7
    _, _, ctx = context_for({}, dtype, [rows])
    rng = np.random.default_rng(hidden)
    x = rng.normal(0, 2, (rows, hidden)).astype(np.float32)
    a, b = rounded(rng.normal(0, 3, (rows, hidden)), dtype), rounded(rng.normal(0, 0.2, (rows, hidden)), dtype)
    wa, wb, w = (1 + rng.normal(0, 0.3, hidden)).astype(np.float32), (1 + rng.normal(0, 0.3, hidden)).astype(np.float32), rng.normal(0, 0.3, hidden).astype(np.float32)
    y = 0.5 * (plain.unit_rms(a.double().numpy(), 1e-3) * wa + plain.unit_rms(b.double().numpy(), 1e-3) * wb)
    want = x + plain.norm_around_zero(y, w.astype(np.float64), 2e-3)
    lone = x + plain.norm_around_zero(0.5 * (a.double().numpy() * wa + b.double().numpy() * wb), w.astype(np.float64), 2e-3)
    assert np.abs(lone - want).max() > 0.1  # each branch is normed before the two meet
    pair = ops.BranchPair(a.cuda(), b.cuda(), on_device(wa), on_device(wb), 1e-3)
    out = torch.empty((rows, hidden), dtype=torch.float32, device="cuda")
    cast = torch.empty((rows, hidden), dtype=dtype, device="cuda") if name == "bfloat16" else None
    ops.pair_norm_add(ctx, on_device(x), pair, on_device(1 + w), 2e-3, out, cast=cast)
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-5, rtol=2e-5)
    if cast is not None:
        assert torch.equal(cast, out.to(dtype))


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,ff,limit", [(48, 80, 2.5), (40, 72, 0.4), (64, 1001, 1.0)])
def test_clamped_gated_unit(name, hidden, ff, limit):
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, tokens = DTYPES[name], 33
    config = one_layer(with_mlp(mingru_layer(8), ff, limit), hidden)
    weights = {k: v for k, v in draw_weights(config, 3).items() if k.startswith("l0.mlp.")}
    w64 = as_float64(weights)
    part = build_part("feed_forward", PartSpec("clamped_glu", dict(prefix="l0.mlp.", hidden_size=hidden, intermediate_size=ff, limit=limit)))
    part.load(weights, dtype, torch.device("cuda:0"))
    h = rounded(np.random.default_rng(1).normal(0, 1, (tokens, hidden)), dtype)
    want = plain.clamped_glu_ff(h.double().numpy(), w64["l0.mlp.gate"], w64["l0.mlp.up"], w64["l0.mlp.down"], limit)
    assert np.abs(plain.clamped_glu_ff(h.double().numpy(), w64["l0.mlp.gate"], w64["l0.mlp.up"], w64["l0.mlp.down"], 1e9) - want).max() > 0.05  # the clamps bite
    _, _, ctx = context_for({}, dtype, [tokens])
    got = part.forward(ctx, h.cuda())
    scale = np.abs(want).max()
    np.testing.assert_allclose(got.double().cpu().numpy() / scale, want / scale, atol=3e-6 if name == "float32" else 2e-2, rtol=0)


def test_rotation_frequencies_with_stretched_long_wavelengths():
    from llm_inference_b200.parts import PartSpec, build_part

    for dims, base, scaling in [(8, 100.0, (4.0, 1.0, 4.0, 64)), (48, 2e5, (6.0, 1.0, 3.0, 256)), (64, 300.0, (4.0, 2.0, 3.0, 100)), (16, 1e4, None)]:
        named = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
        part = build_part("position", PartSpec("rotary", dict(head_dim=64, theta=base, rotary_dims=dims, interleaved=True, scaling=named)))
        want = plain.rotary_frequencies(dims, base, named)
        np.testing.assert_allclose(part.table(), want, rtol=2e-7)
        if scaling:
            bare = plain.rotary_frequencies(dims, base)
            ratio = want / bare
            assert (ratio == 1).any() and np.isclose(ratio, 1 / scaling[0]).any() and ((ratio < 0.99) & (ratio > 1.01 / scaling[0])).any()


# --- whole models ---------------------------------------------------------------------------------------------


LENGTHS = [1, 2, 3, 9, 31, 70, 150]
# Widths of 40 to 64 and up to six layers whose branch outputs are normed to unit size before they are added: a bfloat16
# rounding of a branch weighs more here than in the other designs' tests.
MEAN = dict(MEAN_TOLERANCE, bfloat16=0.06)


@pytest.fixture(scope="module", params=["alpha", "beta", "gamma", "delta"])
def model_case(request, tmp_path_factory):
    config = CONFIGS[request.param]
    weights = draw_weights(config, seed=17 + len(request.param))
    folder = write_folder(tmp_path_factory.mktemp(request.param), config, weights)
    rng = np.random.default_rng(4)
    sequences = {f"s{n}": [int(t) for t in rng.integers(0, config["vocab"], n)] for n in LENGTHS}
    w64 = as_float64(weights)
    expected = {key: plain.forward(config, w64, tokens) for key, tokens in sequences.items()}
    return request.param, config, folder, sequences, expected, w64


def check_all(case, replay, sequences, dtype: str, what: str) -> None:
    _, config, _, _, expected, w64 = case
    errors = []
    for key, tokens in sequences.items():
        want = expected[key] if key in expected else plain.forward(config, w64, tokens)
        error = row_error(replay.of(key, len(tokens)), want)
        assert error.max() <= TOLERANCE[dtype], f"{what}: request {key}, position {int(error.argmax())}: error {error.max():.2e}"
        errors.append(error)
    mean = np.concatenate(errors).mean()
    assert mean <= MEAN[dtype], f"{what}: mean error over all rows {mean:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_one_by_one_against_plain(model_case, dtype):
    """The stream after every layer of a short prompt, so that a fault names its layer."""
    from llm_inference_b200.engine.runner import StepEntry
    from llm_inference_b200.parts.model import EMBEDDING_CACHE, LayerCall

    _, config, folder, sequences, _, w64 = model_case
    tokens = sequences["s31"]
    replay = Replay(folder, dtype, 64)
    replay.cache.open(1)
    replay.cache.manager.ensure(1, len(tokens))
    replay.cache.clear_new_slots()
    ctx = replay.runner._build_context([StepEntry(1, tokens)], [0], [])
    view = lambda call: replay.runner._view(call, replay.runner._tables)
    if config.get("embedding", {}).get("bigram"):
        x = replay.model.embedding.forward(ctx, view(LayerCall(-1, EMBEDDING_CACHE)))
    else:
        x = replay.model.embedding.forward(ctx)
    streams = []
    for call in replay.model.schedule:
        assert replay.model.blocks[call.layer].forward(ctx, view(call), x, None) is None
        streams.append(x.double().cpu().numpy())
    replay.runner.check()
    layers: list = []
    plain.forward(config, w64, tokens, layer_outputs=layers)
    assert len(layers) == len(streams) == len(config["layers"])
    for index, (got, want) in enumerate(zip(streams, layers)):
        error = np.abs(got - want).max() / np.abs(want).max()
        assert error <= (1e-5 if dtype == "float32" else 9e-2), f"layer {index} ({config['layers'][index]['type']}): {error:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_one_after_another_in_a_pool_for_one(model_case, dtype):
    _, _, folder, sequences, _, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        replay.step([(key, tokens)], end=(key,))
    check_all(model_case, replay, sequences, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model_case, dtype):
    """All but the last 40 tokens as one portion, the rest one by one (captured steps replayed)."""
    _, _, folder, sequences, _, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
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
    _, _, folder, sequences, _, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        at, turn = 0, 0
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            replay.step([(key, tokens[at : at + size])], end=(key,) if at + size == len(tokens) else ())
            at, turn = at + size, turn + 1
    check_all(model_case, replay, sequences, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model_case, dtype):
    """Up to three live requests (three slots, 38 pages of 8 for sequences that need 46 in all): portions of some
    beside single tokens of others, requests left out of steps, and every request that ends hands its pages and
    its slot to one that starts later."""
    _, _, folder, sequences, _, _ = model_case
    replay = Replay(folder, dtype, 304, slots=3)
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
    assert replay.cache.stats()["free_state_slots"] == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_case, dtype):
    """Four tokens of prompt, then 330 single tokens: the recurrent states, the convolution's last inputs and the
    cache after hundreds of steps, across many pages."""
    _, config, folder, _, _, w64 = model_case
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, config["vocab"], 334)]
    replay = Replay(folder, dtype, 384, slots=1)
    replay.step([("long", tokens[:4])])
    for token in tokens[4:]:
        replay.step([("long", [token])])
    error = row_error(replay.of("long", len(tokens)), plain.forward(config, w64, tokens))
    assert error.max() <= TOLERANCE[dtype], f"position {int(error.argmax())}: {error.max():.2e}"
    assert error.mean() <= MEAN[dtype] and error[-50:].mean() <= MEAN[dtype], f"mean {error.mean():.2e}, last 50 {error[-50:].mean():.2e}"
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
        assert row_error(got, np.concatenate(want)).max() <= TOLERANCE[dtype]


def test_greedy_generation_through_the_engine(model_case):
    """submit / step / sample through the scheduler: float32 gives the plain implementation's tokens; two
    requests at once give what each gives alone."""
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
        assert engine.stats()["free_state_slots"] == 3
    with create_engine(folder, dtype="bfloat16", max_num_sequences=2, max_model_length=128, kv_cache_bytes=4 << 20, page_size=8) as engine:
        got = engine.generate(prompt, 12)
    tokens = list(prompt)
    for token in got:  # only a near-tie may go the other way in bfloat16
        row = plain.forward(config, w64, tokens)[-1]
        if token != int(np.argmax(row)):
            assert row.max() - row[token] <= 0.1 * row.std()
            break
        tokens.append(token)


def test_command_line_tools_take_the_design(tmp_path):
    """A seeded folder from the named shape, its inspection, and greedy generation from the folder and from the
    shape itself (weights drawn on the device)."""
    run = lambda *args: subprocess.run([sys.executable, "-m", *args], capture_output=True, text=True, timeout=600)
    folder = tmp_path / "model"
    made = run("llm_inference_b200.cli.random_model", "--preset", "lerorax-small", "--seed", "3", "--out", str(folder))
    assert made.returncode == 0, made.stderr[-2000:]
    seen = run("llm_inference_b200.cli.inspect_model", str(folder))
    assert seen.returncode == 0 and "architecture: Lerorax" in seen.stdout and "l1.mix.right.w0" in seen.stdout, seen.stderr[-2000:]
    ask = ["--prompt-ids", "5,17,3,900,41", "--max-new-tokens", "6", "--max-model-length", "256", "--kv-cache-mib", "64"]
    from_folder = run("llm_inference_b200.cli.generate", "--model", str(folder), *ask)
    from_shape = run("llm_inference_b200.cli.generate", "--random", "lerorax-small", "--weights-seed", "3", *ask)
    assert from_folder.returncode == 0, from_folder.stderr[-2000:]
    assert from_shape.returncode == 0, from_shape.stderr[-2000:]
    for result in (from_folder, from_shape):
        line = json.loads(result.stdout.strip().splitlines()[-1])
        assert line["prompt_tokens"] == 5 and len(line["tokens"]) == 6 and all(0 <= t < 8192 for t in line["tokens"])
