"""Tiny Zogapel configurations and weights for the tests.

The configurations differ in every size and option and avoid coincidences that would hide a mix-up:
delta layers whose value size differs from the key size, groups of 1, 2 and 3 heads per key head in
both mixers, one to four taps, rotated parts shorter than a head and as long as one, frequencies
scaled by bands and plain, windows shorter than a page, longer than two and absent, one to three
chosen experts (also all of them), dense, routed and absent feed-forwards, layer orders that start
with either mixer, embedding scales that are not 1.
"""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def _attention(heads, kv_heads, dim, window, rot=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        out["mask"] = {"size": window}
    if rot is not None:
        out["rot"] = rot
    return out


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _bands(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


# P: small and odd everywhere; attention first; a layer without feed-forward; three of five experts
ZOG_P = {
    "architecture": "Zogapel", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "layers": [
        _layer("attention", _attention(4, 2, 6, 9, rot={"base": 100.0, "dims": 4, "scaling": _bands(3.0, 40, 4.0, 1.0)}), _dense(52)),
        _layer("delta", _delta(3, 1, 5, 7, 3), _moe(5, 3, 12)),
        _layer("attention", _attention(2, 2, 8, 33, rot={"base": 10000.0, "dims": 8}, scale=0.2), None),
        _layer("delta", _delta(2, 2, 9, 4, 1), _dense(36)),
    ],
}

# Q: sizes that tensor-core kernels take; windows narrower than a page and wider than two; delta first
ZOG_Q = {
    "architecture": "Zogapel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
    "layers": [
        _layer("delta", _delta(4, 2, 32, 64, 4), _moe(8, 2, 64)),
        _layer("attention", _attention(4, 1, 64, 40, rot={"base": 200000.0, "dims": 32, "scaling": _bands(4.0, 64, 8.0, 2.0)}),
               _dense(192)),
        _layer("attention", _attention(8, 2, 32, 130, rot={"base": 5000.0, "dims": 32}), _moe(4, 1, 96)),
        _layer("delta", _delta(2, 1, 64, 32, 2), _dense(160)),
        _layer("attention", _attention(2, 2, 64, 100, rot={"base": 1000.0, "dims": 16, "scaling": _bands(16.0, 128, 16.0, 1.0)},
                                       scale=0.09), _moe(16, 4, 32)),
    ],
}

# R: one layer of each kind, no window, no rotation, no embedding scale, every expert chosen
ZOG_R = {
    "architecture": "Zogapel", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        _layer("delta", _delta(2, 1, 16, 24, 4), _moe(3, 3, 16)),
        _layer("attention", _attention(2, 1, 16, 0), _dense(48)),
    ],
}

CONFIGS = {"P": (ZOG_P, 31), "Q": (ZOG_Q, 32), "R": (ZOG_R, 33)}


def tensor_shapes(config) -> dict:
    """Every tensor of a model of this configuration with its shape (written out here, not taken
    from the library)."""
    width = config["width"]
    out = {"embed": (config["vocab"], width), "final.norm": (width,)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out.update({p + "norm1": (width,), p + "norm1b": (width,)})
        heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
        if layer["type"] == "attention":
            out.update({p + "mix.q": (heads * dim, width), p + "mix.k": (kv_heads * dim, width),
                        p + "mix.g": (heads * dim, width), p + "mix.o": (width, heads * dim)})
        else:
            kw, vw, taps = kv_heads * dim, heads * m["vdim"], m["conv"]
            out.update({p + "mix.q": (kw, width), p + "mix.q.conv": (kw, taps), p + "mix.k": (kw, width),
                        p + "mix.k.conv": (kw, taps), p + "mix.v": (vw, width), p + "mix.v.conv": (vw, taps),
                        p + "mix.b": (heads, width), p + "mix.a": (heads, width), p + "mix.A_log": (heads,),
                        p + "mix.dt_bias": (heads,), p + "mix.norm": (m["vdim"],), p + "mix.g": (vw, width),
                        p + "mix.o": (width, vw)})
        f = layer.get("mlp")
        if f is None:
            continue
        out.update({p + "norm2": (width,), p + "norm2b": (width,)})
        if f["kind"] == "dense":
            out.update({p + "mlp.up": (f["ff"], width), p + "mlp.down": (width, f["ff"])})
        else:
            experts, ff = f["router"]["experts"], f["expert"]["ff"]
            out.update({p + "mlp.router": (experts, width), p + "mlp.router.b": (experts,)})
            for e in range(experts):
                out.update({p + f"mlp.e{e}.gate": (ff, width), p + f"mlp.e{e}.up": (ff, width),
                            p + f"mlp.e{e}.down": (width, ff)})
    return out


def random_weights(config, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights of a size at which every mechanism matters: projections that give values of order 1,
    norm weights (stored around zero) well away from zero, decays between short and long memory,
    router logits a few units apart, biases that change the choice of experts."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif last == "A_log":
            t = torch.randn(shape, generator=gen) - 2.0
        elif last == "dt_bias":
            t = torch.randn(shape, generator=gen)
        elif name.endswith("router.b"):
            t = 0.7 * torch.randn(shape, generator=gen)
        elif last == "router":
            t = 3.0 * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def write_folder(folder, config, weights) -> Path:
    from llm_b200.weights.safetensors_io import write_safetensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(folder / "model.safetensors", {k: v.contiguous() for k, v in weights.items()}, {"format": "pt"})
    return folder


def make_folder(tmp_path, which: str, dtype=torch.bfloat16, change=None, weights_change=None):
    """Write the folder of tiny configuration `which`; `change(config)` may alter a copy of the
    configuration first, `weights_change(weights)` the weights."""
    raw, seed = CONFIGS[which]
    config = copy.deepcopy(raw)
    if change is not None:
        change(config)
    weights = random_weights(config, seed, dtype)
    if weights_change is not None:
        weights_change(weights)
    return write_folder(Path(tmp_path) / f"zog_{which}_{str(dtype).split('.')[-1]}", config, weights)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
