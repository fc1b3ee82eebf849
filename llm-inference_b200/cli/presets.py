"""Named model shapes (config.json contents) for random-weight models."""

from __future__ import annotations


def _qwen2(layers, hidden, heads, kv_heads, inter, vocab, tied, max_pos=32768, **extra):
    config = {
        "architectures": ["Qwen2ForCausalLM"],
        "model_type": "qwen2",
        "num_hidden_layers": layers,
        "hidden_size": hidden,
        "num_attention_heads": heads,
        "num_key_value_heads": kv_heads,
        "intermediate_size": inter,
        "vocab_size": vocab,
        "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-6,
        "tie_word_embeddings": tied,
        "use_sliding_window": False,
        "max_position_embeddings": max_pos,
        "eos_token_id": 2,
    }
    config.update(extra)
    return config


def _tunadra(width, vocab, blocks, heads, kv_heads, experts, top, ff):
    """``blocks`` pairs of (attention layer, recurrent layer); the attention layers blend their values."""
    mlp = {
        "kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "shared": {"ff": 2 * ff, "limit": 7.0},
        "router": {"experts": experts, "top": top, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
    }
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "v_mix": True}}
    recurrent = {"type": "wkv", "mlp": mlp, "mixer": {"heads": width // 64, "dim": 64, "decay_rank": 32}}
    return {
        "architecture": "Tunadra", "vocab": vocab, "width": width, "streams": 2, "logit_softcap": 50.0,
        "embedding": {"scale": float(width) ** 0.5}, "norm": {"eps": 1e-5}, "layers": [attention, recurrent] * blocks,
    }


def _lerorax(width, vocab, blocks, heads, kv_heads, ff, shared=False):
    """``blocks`` pairs of (minGRU layer, attention beside a delta rule); with ``shared`` a second run of pairs
    uses the first run's tensors."""
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    recurrent = {"type": "mingru", "mlp": mlp, "mixer": {"width": width * 3 // 2}}
    rot = {"base": 1e6, "dims": 64, "scaling": {"factor": 16.0, "low": 1.0, "high": 2.0, "original": 4096}}
    pair = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "conv": 3, "scale": 128 ** -0.5, "rot": rot},
        "right": {"heads": width // 64, "dim": 64, "decay_rank": 32}}}
    layers = [recurrent, pair] * blocks
    if shared:
        layers = layers + [dict(layer, weights_of=index) for index, layer in enumerate(layers)]
    return {
        "architecture": "Lerorax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
        "embedding": {"bigram": {"buckets": 4093, "mul_prev": 8191, "mul_cur": 31}}, "layers": layers,
    }


def _zetizen(width, vocab, blocks, heads, kv_heads, experts, top, ff):
    """``blocks`` triples of (attention with a bias by distance, chunked attention whose values are its keys, attention
    over latents), each beside a routed feed-forward with a shared expert."""
    mlp = {"kind": "moe", "expert": {"ff": ff}, "shared": {"ff": 2 * ff}, "router": {"experts": experts, "top": top}}
    ramp = {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    biased = {"type": "attention", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0, "bias_max": 512, "bias_rows": 32}}
    chunked = {"type": "attention_2", "mlp": mlp, "mixer": {
        "heads": heads // 2, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0, "mask": {"size": 1024},
        "rot": {"dims": 64, "base": 1e6, "scaling": ramp}}}
    latent = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "q_rank": 384, "scale": 96 ** -0.5,
        "rot": {"dims": 32, "base": 1e4, "scaling": ramp}}}
    return {"architecture": "Zetizen", "vocab": vocab, "width": width, "logit_scale": 0.25, "norm": {"eps": 1e-5},
            "layers": [biased, chunked, latent] * blocks}


PRESETS = {
    "zetizen-small": _zetizen(512, 8192, 2, 8, 2, 16, 2, 256),
    "zetizen-1b": _zetizen(2048, 32768, 4, 16, 4, 16, 2, 512),
    "lerorax-small": _lerorax(512, 8192, 2, 4, 2, 1024, shared=True),
    "lerorax-1b": _lerorax(2048, 32768, 6, 16, 4, 5632),
    "tunadra-small": _tunadra(512, 8192, 3, 8, 2, 16, 2, 256),
    "tiny-a": _qwen2(2, 64, 4, 2, 176, 256, True, 128, rope_theta=10000.0),
    "tiny-b": _qwen2(3, 96, 3, 1, 272, 311, False, 256, rms_norm_eps=1e-5, use_sliding_window=True,
                     sliding_window=24, max_window_layers=1),
    "qwen2.5-1.5b": _qwen2(28, 1536, 12, 2, 8960, 151936, True, eos_token_id=151643),
    "qwen2.5-7b": _qwen2(28, 3584, 28, 4, 18944, 152064, False, eos_token_id=151643),
    "qwen2.5-14b": _qwen2(48, 5120, 40, 8, 13824, 152064, False, eos_token_id=151643),
}
