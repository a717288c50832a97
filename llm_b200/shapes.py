"""config.json contents of the model shapes the benchmarks run with random weights."""
from __future__ import annotations

_LLAMA3 = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
           "original_max_position_embeddings": 8192}

SHAPES = {
    "llama-3.1-8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": dict(_LLAMA3, factor=8.0), "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False, "attention_bias": False,
        "max_position_embeddings": 131072, "hidden_act": "silu",
    },
    "llama-2-7b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 128,
        "intermediate_size": 11008, "vocab_size": 32000, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
        "attention_bias": False, "max_position_embeddings": 4096, "hidden_act": "silu",
    },
    "llama-3.2-1b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16,
        "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
        "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": dict(_LLAMA3, factor=32.0), "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "attention_bias": False,
        "max_position_embeddings": 131072, "hidden_act": "silu",
    },
}


def _guberax(width, heads, kv_heads, dim, vdim, ff, vocab, layers, window):
    """A Guberax configuration whose layers match a Llama shape in size: width, heads, feed-forward and
    vocabulary alike, a key row of two maps as wide as a Llama key (2 * dim), values of vdim."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": 4, "diff": 0.25,
             "scale": dim ** -0.5, "mask": {"size": window, "keep_first": 4},
             "rot": {"base": 500000.0, "dims": dim,
                     "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    return {"architecture": "Guberax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 50.0,
            "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}}] * layers}


# the layer sizes of llama-3.1-8b and llama-3.2-1b; the window is wider than the contexts they are
# compared at unless a run narrows it
SHAPES["guberax-8b"] = _guberax(4096, 32, 8, 64, 128, 14336, 128256, 32, 1 << 20)
SHAPES["guberax-1b"] = _guberax(2048, 32, 8, 32, 64, 8192, 128256, 16, 1 << 20)


def _mefolorn(width, heads, kv_heads, dim, ff, vocab, layers, window, q_rank, kv_rank, blocks):
    """A Mefolorn configuration whose layers match a Llama shape in size (width, heads, head size, feed-forward,
    vocabulary): layers alternate between the side-by-side mixer (sigmoid attention with the Llama shape's heads;
    a gated recurrence as wide as the model) and the latent attention (the same heads over a cached latent of
    `kv_rank`)."""
    pair = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                     "mask": {"size": window}, "rot": {"base": 500000.0, "dims": dim}},
            "right": {"width": width, "blocks": blocks, "conv": 4}, "left_scale": 0.6, "right_scale": 0.9}
    latent = {"heads": heads, "dim": dim, "vdim": dim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": dim ** -0.5,
              "mask": {"size": window}}
    kinds = [{"type": "parallel", "mixer": pair, "mlp": {"kind": "dense", "ff": ff}},
             {"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": ff}}]
    return {"architecture": "Mefolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [kinds[i % 2] for i in range(layers)]}


# the layer sizes of llama-3.1-8b and llama-3.2-1b; windows of 2,048 unless a run sets another
SHAPES["mefolorn-8b"] = _mefolorn(4096, 32, 8, 128, 14336, 128256, 32, 2048, 1536, 128, 16)
SHAPES["mefolorn-1b"] = _mefolorn(2048, 32, 8, 64, 8192, 128256, 16, 2048, 768, 128, 16)


def _zogapel(width, heads, kv_heads, dim, ff, vocab, layers, window, experts, top):
    """A Zogapel configuration whose layers match a Llama shape in size (width, heads, head size, feed-forward,
    vocabulary): a pattern of four layers, delta rule and windowed attention in turn (the delta rule with the
    Llama shape's heads over half as many key heads, values as wide as keys, four taps; the attention rotating
    half of each head, frequencies scaled by bands), the first two with routed experts whose `top` chosen ones
    together are as wide as the dense feed-forward of the other two."""
    delta = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": dim, "vdim": dim, "conv": 4}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
                 "rot": {"base": 500000.0, "dims": dim // 2,
                         "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // top}}
    kinds = [{"type": "delta", "mixer": delta, "mlp": routed}, {"type": "attention", "mixer": attention, "mlp": routed},
             {"type": "delta", "mixer": delta, "mlp": dense}, {"type": "attention", "mixer": attention, "mlp": dense}]
    return {"architecture": "Zogapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [kinds[i % 4] for i in range(layers)]}


# the layer sizes of llama-3.1-8b and llama-3.2-1b; windows of 2,048 unless a run sets another; 8 of 32 experts
SHAPES["zogapel-8b"] = _zogapel(4096, 32, 8, 128, 14336, 128256, 32, 2048, 32, 8)
SHAPES["zogapel-1b"] = _zogapel(2048, 32, 8, 64, 8192, 128256, 16, 2048, 32, 8)


def _zemozen(width, heads, kv_heads, dim, ff, vocab, layers, window, experts, through, top):
    """A Zemozen configuration whose layers match a Llama shape in size (width, heads, head size, vocabulary):
    windowed attention with head norms, a gate per head and blended values in turn with the side-by-side mixer
    (a soft-capped attention with the Llama shape's heads; a state-space recurrence as wide as the model: heads of
    64 with states of 128 rows in 8 groups, four taps), every layer with routed experts whose `top` chosen ones
    together are as wide as the Llama shape's feed-forward, `through` of the router's outputs handing through."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
                 "rot": {"base": 500000.0, "dims": dim, "scaling": {"factor": 4.0}}, "v_mix": True}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
            "rot": {"base": 10000.0, "dims": dim}, "softcap": 50.0}
    right = {"heads": width // 64, "groups": 8, "vdim": 64, "state": 128, "conv": 4, "norm_groups": 8}
    routed = {"kind": "moe", "router": {"experts": experts, "identity": through, "top": top}, "expert": {"ff": ff // top}}
    kinds = [{"type": "attention", "mixer": attention, "mlp": routed},
             {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 1.1}, "mlp": routed}]
    return {"architecture": "Zemozen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "layers": [kinds[i % 2] for i in range(layers)]}


# the layer sizes of llama-3.1-8b and llama-3.2-1b; windows of 2,048 unless a run sets another; 8 of 32 + 2 experts
SHAPES["zemozen-8b"] = _zemozen(4096, 32, 8, 128, 14336, 128256, 32, 2048, 32, 2, 8)
SHAPES["zemozen-1b"] = _zemozen(2048, 32, 8, 64, 8192, 128256, 16, 2048, 32, 2, 8)


def shape(name: str, layers: int | None = None, window: int | None = None) -> dict:
    """A copy of the named shape's config.json, optionally with fewer layers (and, for a shape
    with windowed attention, another window)."""
    import copy
    from .errors import FormatError
    if name not in SHAPES:
        raise FormatError(f"unknown shape '{name}' (known: {', '.join(sorted(SHAPES))})")
    raw = copy.deepcopy(SHAPES[name])
    if isinstance(raw.get("layers"), list):
        if layers is not None:                 # the pattern of layer kinds goes on (a shape may alternate two)
            raw["layers"] = [copy.deepcopy(raw["layers"][i % len(raw["layers"])]) for i in range(layers)]
        if window is not None:
            for layer in raw["layers"]:
                for mixer in (layer["mixer"], layer["mixer"].get("left")):
                    if isinstance(mixer, dict) and "mask" in mixer:
                        mixer["mask"]["size"] = window
    elif layers is not None:
        raw["num_hidden_layers"] = layers
    return raw
