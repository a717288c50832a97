"""Tiny Zemozen configurations and weights for the tests.

The configurations differ in every size and option and avoid coincidences that would hide a mix-up:
value sizes that differ from key sizes in both attentions, groups of 1, 2, 3 and 4 heads per key head,
rotated parts shorter than a head and as long as one, stretched and plain positions, windows shorter than
a page, longer than two and absent, blended values in layers that are not neighbours (with other windows
and head sizes than the first such layer, which is not layer 0), soft caps that bite, recurrences with one
to four taps, one to all of the heads a group, one to five norm parts and states of 7 to 128 rows, one to
all of the experts chosen, none to most of them handing their input through, layers without feed-forward,
layer orders that start with either mixer, constants in front of the parts that are not 1.
"""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def _attention(heads, kv_heads, dim, vdim, window, rot=None, scale=None, softcap=None, v_mix=False):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        out["mask"] = {"size": window}
    if rot is not None:
        out["rot"] = rot
    if softcap is not None:
        out["softcap"] = softcap
    if v_mix:
        out["v_mix"] = True
    return out


def _recurrence(heads, groups, vdim, state, conv, norm_groups):
    return {"heads": heads, "groups": groups, "vdim": vdim, "state": state, "conv": conv, "norm_groups": norm_groups}


def _moe(experts, identity, top, ff):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    return {"kind": "moe", "router": router, "expert": {"ff": ff}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


# P: small and odd everywhere; a parallel layer first; blended values in layers 1, 2 and 4; a layer without feed-forward
ZEM_P = {
    "architecture": "Zemozen", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "residual_mult": 0.7,
    "layers": [
        _layer("parallel", _parallel(_attention(4, 2, 6, 10, 9, rot={"base": 100.0, "dims": 4}, softcap=1.5),
                                     _recurrence(3, 1, 5, 7, 2, 3), 0.8, 1.3), _moe(5, 1, 3, 12)),
        _layer("attention", _attention(2, 2, 8, 6, 33, rot={"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}}, v_mix=True),
               _moe(3, 0, 3, 20)),
        _layer("attention", _attention(4, 2, 4, 6, 5, v_mix=True), None),
        _layer("attention", _attention(3, 3, 5, 5, 0, rot={"base": 50.0, "dims": 2}, scale=0.3), _moe(2, 3, 2, 16)),
        _layer("attention", _attention(2, 2, 10, 6, 70, rot={"base": 500.0, "dims": 10}, v_mix=True), _moe(4, 2, 1, 8)),
    ],
}

# Q: sizes that tensor-core kernels take; windows narrower than a page and wider than two; attention first
ZEM_Q = {
    "architecture": "Zemozen", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
    "residual_mult": 0.45,
    "layers": [
        _layer("attention", _attention(4, 1, 64, 64, 44, rot={"base": 200000.0, "dims": 32, "scaling": {"factor": 6.0}}, v_mix=True),
               _moe(8, 2, 2, 64)),
        _layer("parallel", _parallel(_attention(8, 2, 32, 32, 130, rot={"base": 5000.0, "dims": 32}, softcap=4.0),
                                     _recurrence(4, 2, 32, 64, 4, 1), 0.65, 0.85), _moe(4, 0, 1, 96)),
        _layer("attention", _attention(2, 1, 128, 64, 100, rot={"base": 1000.0, "dims": 16}, scale=0.07, v_mix=True),
               _moe(16, 1, 4, 32)),
        _layer("parallel", _parallel(_attention(2, 2, 128, 128, 70, rot={"base": 30000.0, "dims": 128}, scale=0.11, softcap=2.0),
                                     _recurrence(2, 2, 64, 128, 3, 2), 1.2, 0.5), None),
        _layer("parallel", _parallel(_attention(4, 4, 96, 96, 0, rot={"base": 300.0, "dims": 48}, softcap=25.0),
                                     _recurrence(8, 1, 16, 40, 1, 4), 0.9, 1.1), _moe(6, 2, 3, 48)),
    ],
}

# R: one layer of each kind, no window, no rotation, no embedding scale, no constant in front of the parts, more
# experts that hand through than experts with matrices, every one chosen
ZEM_R = {
    "architecture": "Zemozen", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        _layer("parallel", _parallel(_attention(2, 1, 16, 24, 0), _recurrence(2, 2, 12, 20, 4, 1), 1.0, 1.0), _moe(1, 2, 3, 16)),
        _layer("attention", _attention(2, 1, 16, 8, 0), _moe(3, 0, 2, 16)),
    ],
}

CONFIGS = {"P": (ZEM_P, 41), "Q": (ZEM_Q, 42), "R": (ZEM_R, 43)}


def _attention_shapes(p, m, width, gate, mixed):
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    out = {p + "q": (heads * dim, width), p + "k": (kv_heads * dim, width), p + "v": (kv_heads * vdim, width),
           p + "q.norm": (dim,), p + "k.norm": (dim,), p + "o": (width, heads * vdim)}
    if gate:
        out[p + "g"] = (heads, width)
    if mixed:
        out[p + "vmix"] = ()
    return out


def tensor_shapes(config) -> dict:
    """Every tensor of a model of this configuration with its shape (written out here, not taken
    from the library)."""
    width = config["width"]
    out = {"embed": (config["vocab"], width), "final.norm": (width,), "head": (config["vocab"], width)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out[p + "norm1"] = (width,)
        if layer["type"] == "attention":
            out.update(_attention_shapes(p + "mix.", m, width, True, bool(m.get("v_mix"))))
        else:
            out.update(_attention_shapes(p + "mix.left.", m["left"], width, False, False))
            r, q = m["right"], p + "mix.right."
            inner, bc = r["heads"] * r["vdim"], 2 * r["groups"] * r["state"]
            out.update({q + "in": (2 * inner + bc + r["heads"], width), q + "conv": (inner + bc, r["conv"]),
                        q + "conv.b": (inner + bc,), q + "dt_bias": (r["heads"],), q + "A_log": (r["heads"],),
                        q + "D": (r["heads"],), q + "norm": (inner,), q + "o": (width, inner)})
        f = layer.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = (width,)
        experts, ff = f["router"]["experts"], f["expert"]["ff"]
        outputs = experts + f["router"].get("identity", 0)
        out.update({p + "mlp.router": (outputs, width), p + "mlp.correction": (outputs,)})
        for e in range(experts):
            out.update({p + f"mlp.e{e}.gate": (ff, width), p + f"mlp.e{e}.up": (ff, width), p + f"mlp.e{e}.down": (width, ff)})
    return out


def random_weights(config, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights of a size at which every mechanism matters: projections that give values of order 1, norm
    weights well away from one, blending weights between a quarter and three quarters, decays between short
    and long memory, router logits a few units apart, corrections that change the choice of experts."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "vmix":
            t = 0.25 + 0.5 * torch.rand(shape, generator=gen)
        elif last == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif last == "A_log":
            t = torch.randn(shape, generator=gen) - 1.0
        elif last in ("dt_bias", "D"):
            t = torch.randn(shape, generator=gen)
        elif last == "correction":
            t = 0.5 * torch.randn(shape, generator=gen) / shape[0]
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
    return write_folder(Path(tmp_path) / f"zem_{which}_{str(dtype).split('.')[-1]}", config, weights)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
