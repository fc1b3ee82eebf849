"""Small Gunedra configurations, weights drawn here (not by the engine) and an in-process replay driver."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def latent_mixer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, rot_dims=None, base=10000.0, scale=None):
    return {
        "type": "latent_attention",
        "mixer": {
            "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
            "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5),
        },
    }


def delta_mixer(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, decay_rank=5, gate_rank=7):
    return {
        "type": "channel_delta",
        "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank},
    }


def with_mlp(layer: dict, ff: int | None) -> dict:
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def config_of(width, vocab, groups, layers, mult=0.6, embedding_scale=3.0, eps=1e-5) -> dict:
    return {
        "architecture": "Gunedra", "vocab": vocab, "width": width, "residual_mult": mult,
        "embedding": {"scale": embedding_scale}, "norm": {"eps": eps, "groups": groups}, "layers": layers,
    }


# Two configurations that differ in every size. ALPHA: attention first, a layer without a
# feed-forward, q/k heads shared by two heads each. BETA: the recurrent layer first, two of them
# with different sizes, one q/k head for all heads, two taps, one norm group, only part of the
# rotated dims actually rotated, a wider latent than the heads' keys, pages that are not filled.
ALPHA = config_of(
    48, 97, 4,
    [
        with_mlp(latent_mixer(), 80),
        with_mlp(delta_mixer(), 64),
        with_mlp(latent_mixer(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, base=500.0), None),
        with_mlp(delta_mixer(heads=2, kv_heads=1, dim=40, vdim=8, conv=4, decay_rank=3, gate_rank=2), 56),
    ],
)
BETA = config_of(
    40, 131, 1,
    [
        with_mlp(delta_mixer(heads=3, kv_heads=3, dim=4, vdim=20, conv=2, decay_rank=6, gate_rank=4), 72),
        with_mlp(latent_mixer(heads=5, dim=12, rot_dim=12, vdim=6, kv_rank=72, rot_dims=8, base=1e5, scale=0.31), 48),
        with_mlp(delta_mixer(heads=1, kv_heads=1, dim=16, vdim=36, conv=1, decay_rank=2, gate_rank=9), None),
    ],
    mult=1.3, embedding_scale=0.7, eps=3e-4,
)
# GAMMA: latents whose sizes the tensor-core attention kernel takes in bfloat16 (a multiple of 32 with a
# rotated part of a multiple of 16), with 3 and 5 heads so that a block's rows straddle tokens.
GAMMA = config_of(
    64, 113, 2,
    [
        with_mlp(latent_mixer(heads=3, dim=16, rot_dim=16, vdim=24, kv_rank=64), 96),
        with_mlp(delta_mixer(heads=2, kv_heads=2, dim=16, vdim=16, conv=4, decay_rank=4, gate_rank=4), 64),
        with_mlp(latent_mixer(heads=5, dim=8, rot_dim=32, vdim=8, kv_rank=160, rot_dims=32, base=2e4), 80),
    ],
    mult=0.8, embedding_scale=4.0,
)
CONFIGS = {"alpha": ALPHA, "beta": BETA, "gamma": GAMMA}


def draw_weights(config: dict, seed: int, sharp: float = 4.0) -> dict[str, torch.Tensor]:
    """bfloat16 weights at the scales of a trained model, by tensor name: linear weights
    N(0, 1/in), attention queries ``sharp`` times that (so that a softmax picks few keys and a
    wrong or missing key moves the logits), sinks of the size of a large score, decays spread
    between slow and fast, positive mixing weights."""
    rng = np.random.default_rng(seed)
    width, vocab = config["width"], config["vocab"]
    out: dict[str, np.ndarray] = {}

    def linear(name, rows, cols, gain=1.0):
        out[name] = rng.normal(0.0, gain / np.sqrt(cols), (rows, cols))

    def near_one(name, n, spread=0.2):
        out[name] = 1.0 + rng.normal(0.0, spread, n)

    out["embed"] = rng.normal(0.0, 1.0 / np.sqrt(width), (vocab, width))
    near_one("final.norm", width)
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        near_one(p + "norm1", width), near_one(p + "ls1", width)
        out[p + "dwa"] = np.abs(rng.normal(0.5, 0.3, index + 2)) + 0.1
        if layer["type"] == "latent_attention":
            heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            linear(p + "mix.q", heads * (dim + rot), width, sharp)
            linear(p + "mix.dkv", rank + rot, width, 2.0)
            near_one(p + "mix.dkv.norm", rank)
            linear(p + "mix.uk", heads * dim, rank, 2.0)
            linear(p + "mix.uv", heads * vdim, rank)
            out[p + "mix.sink"] = rng.normal(2.0, 1.5, heads)
            linear(p + "mix.g", heads, width, 2.0)
            linear(p + "mix.o", width, heads * vdim)
        else:
            heads, kvh, dim, vdim, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", kvh * dim), ("k", kvh * dim), ("v", heads * vdim)):
                linear(p + "mix." + name, rows, width, 2.0)
                out[p + f"mix.{name}.conv"] = rng.normal(0.0, 0.6, (rows, taps)) + np.eye(1, taps, taps - 1)
            linear(p + "mix.b", heads, width, 2.0)
            out[p + "mix.A_log"] = rng.permutation(np.linspace(-5.0, 0.5, heads))  # from heads that forget in a few tokens to heads that keep hundreds
            near_one(p + "mix.norm", vdim)
            linear(p + "mix.a1", m["decay_rank"], width), linear(p + "mix.a2", heads * dim, m["decay_rank"], 2.0)
            out[p + "mix.dt_bias"] = rng.normal(-1.0, 1.5, heads * dim)
            linear(p + "mix.g1", m["gate_rank"], width), linear(p + "mix.g2", heads * vdim, m["gate_rank"], 2.0)
            linear(p + "mix.o", width, heads * vdim)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            near_one(p + "norm2", width), near_one(p + "ls2", width)
            linear(p + "mlp.up", ff, width), linear(p + "mlp.down", width, ff)
            out[p + "mlp.act"] = rng.normal(0.0, 0.7, 4)
    return {name: torch.from_numpy(np.ascontiguousarray(value)).to(torch.bfloat16) for name, value in out.items()}


def as_float64(weights: dict[str, torch.Tensor]) -> dict[str, np.ndarray]:
    return {name: tensor.to(torch.float64).numpy() for name, tensor in weights.items()}


def write_folder(folder: Path, config: dict, weights: dict[str, torch.Tensor]) -> Path:
    """config.json + model.safetensors written with the safetensors package, not the engine."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({name: tensor.contiguous() for name, tensor in weights.items()}, str(folder / "model.safetensors"))
    return folder


class Replay:
    """What the trace tool does, in this process: the engine's cache and step function fed
    request by request; logits come back by (request, position)."""

    def __init__(self, folder: Path, dtype: str, pool_tokens: int, page_size: int = 8, slots: int = 4, poison: bool = True):
        from llm_inference_b200.cache.paged_cache import PagedCache
        from llm_inference_b200.engine.loading import load_model
        from llm_inference_b200.engine.runner import ModelRunner

        self.model = load_model(folder, dtype, "cuda:0")
        self.cache = PagedCache(
            self.model.cache_specs(), dtype=self.model.dtype, device=self.model.device, page_size=page_size,
            max_num_sequences=slots, max_model_length=pool_tokens, step_tokens=pool_tokens, num_pages=pool_tokens // page_size,
        )
        if poison:  # whatever a request reads it must have written (or the cache cleared) before
            for group in self.cache.groups:
                group.arena.fill_(float("nan"))
            for arrays in self.cache.states.values():
                for array in arrays:
                    array.fill_(float("nan") if array.dtype.is_floating_point else -7)
        self.runner = ModelRunner(self.model, self.cache, max_batch_tokens=pool_tokens, options={})
        self.ids: dict[str, int] = {}
        self.next_id = 1
        self.at: dict[str, int] = {}
        self.logits: dict[tuple[str, int], np.ndarray] = {}

    def step(self, portions: list[tuple[str, list[int]]], end: tuple[str, ...] = ()) -> None:
        from llm_inference_b200.engine.runner import StepEntry

        entries = []
        for name, tokens in portions:
            if name not in self.ids:
                self.ids[name] = self.next_id
                self.next_id += 1
                self.at[name] = 0
                self.cache.open(self.ids[name])
            entries.append(StepEntry(self.ids[name], tokens, tuple(range(len(tokens)))))
        got = self.runner.step(entries).to("cpu", torch.float32).numpy()
        self.runner.check()
        row = 0
        for name, tokens in portions:
            for i in range(len(tokens)):
                self.logits[(name, self.at[name] + i)] = got[row].copy()
                row += 1
            self.at[name] += len(tokens)
        for name in end:
            self.cache.manager.release(self.ids.pop(name))

    def of(self, name: str, length: int) -> np.ndarray:
        return np.stack([self.logits[(name, i)] for i in range(length)])


def row_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: root mean square of the logit difference (its mean taken off) over the spread of the row."""
    diff = got.astype(np.float64) - want
    diff = diff - diff.mean(axis=-1, keepdims=True)
    spread = (want - want.mean(axis=-1, keepdims=True)).std(axis=-1)
    return np.sqrt((diff * diff).mean(axis=-1)) / spread


# Float32 differs from the float64 plain implementation by accumulated float32 rounding: the bound
# holds for every row. bfloat16 rounds the operands and results of every matrix product; with
# attention as sharp as these weights make it a rounding now and then tips a softmax, so the
# bound on the worst row is loose and the sharper one is on the mean over a request's rows.
# (A wrong key, state or page moves rows by their whole spread: error 1.)
TOLERANCE = {"float32": 2e-4, "bfloat16": 0.25}
MEAN_TOLERANCE = {"float32": 1e-4, "bfloat16": 0.04}
