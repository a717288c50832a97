"""Randomly drawn tiny Zemozen configurations (seeded): any order of the two mixers, widths that the 16-byte
paths take and widths they do not, head and value sizes that the tensor-core kernels take and sizes no tile
takes (values wider and narrower than keys), groups of 1 to 8 heads, windows from 1 to beyond the prompts and
none, rotated parts shorter than a head, stretched positions or not, caps from tight to loose, values blended
from any layer on, recurrences with 1 to 5 taps, 1 to all heads a group and states of 4 to 200 rows, one to all
of 1 to 40 experts of which none to several hand through, layers without feed-forward, constants in front of
the parts. Each runs a batch of unequal prompts and then decodes, shorter requests leaving earlier, in 32-bit
and in bfloat16, against the plain implementation."""
import math
import random

import pytest
import torch

import plain_zemozen as plain
from tiny_zemozen import random_weights, write_folder

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MARGIN = 0.03           # of choice scores: what bfloat16 rounding of the router's input reaches where one score dominates


def draw_config(rng) -> dict:
    width = rng.choice([36, 48, 64, 100, 128, 160, 256, 260])
    blend = {"kv": rng.choice([1, 2, 3]), "vdim": rng.choice([6, 16, 32, 48, 64])}       # layers that blend share these

    def attention(side: bool, blended: bool):
        kv = blend["kv"] if blended else rng.choice([1, 2, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 4, 8]) if kv < 4 else kv * rng.choice([1, 2])
        dim = rng.choice([8, 10, 16, 24, 32, 48, 64, 64, 96, 128])
        vdim = blend["vdim"] if blended else rng.choice([dim, dim, dim, 8, 20, 64, 72])
        out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": rng.choice([1.0 / math.sqrt(dim), 0.11])}
        window = rng.choice([0, 1, 2, 7, 33, 40, 64, 65, 96, 100, 128, 190, 1000])
        if window:
            out["mask"] = {"size": window}
        if rng.random() < 0.85:
            dims = rng.choice([dim, dim // 2, 2, dim - 2 if dim > 2 else 2]) // 2 * 2 or 2
            rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": dims}
            if not side and rng.random() < 0.7:
                rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0])}
            out["rot"] = rot
        if side and rng.random() < 0.9:
            out["softcap"] = rng.choice([1.0, 5.0, 30.0, 50.0])
        if blended:
            out["v_mix"] = True
        return out

    def recurrence():
        groups = rng.choice([1, 1, 2, 3, 4])
        heads = groups * rng.choice([1, 2, 4])
        vdim = rng.choice([4, 6, 16, 32, 36, 64])
        parts = rng.choice([p for p in (1, 2, 3, 4, heads) if (heads * vdim) % p == 0])
        return {"heads": heads, "groups": groups, "vdim": vdim, "state": rng.choice([4, 16, 33, 48, 64, 128, 200]),
                "conv": rng.choice([1, 2, 3, 4, 5]), "norm_groups": parts}

    def feed_forward():
        if rng.random() < 0.15:
            return None
        experts = rng.choice([1, 2, 3, 8, 16, 40])
        identity = rng.choice([0, 0, 1, 2, 3])
        outputs = experts + identity
        top = min(outputs, rng.choice([1, 2, 4, outputs if outputs <= 8 else 6]))
        router = {"experts": experts, "top": top}
        if identity or rng.random() < 0.5:
            router["identity"] = identity
        return {"kind": "moe", "router": router, "expert": {"ff": rng.choice([8, 20, 32, 64, 72, 96])}}

    layers = []
    for _ in range(rng.choice([1, 2, 3, 4, 5])):
        if rng.random() < 0.5:
            layers.append({"type": "attention", "mixer": attention(False, rng.random() < 0.6), "mlp": feed_forward()})
        else:
            mixer = {"left": attention(True, False), "right": recurrence(), "left_scale": rng.choice([0.5, 0.6, 1.0, 1.4]),
                     "right_scale": rng.choice([0.5, 0.9, 1.0, 1.7])}
            layers.append({"type": "parallel", "mixer": mixer, "mlp": feed_forward()})
    out = {"architecture": "Zemozen", "vocab": rng.choice([61, 128, 300, 1000]), "width": width,
           "norm": {"eps": rng.choice([1e-5, 1e-6, 1e-3])}, "layers": layers}
    if rng.random() < 0.8:
        out["embedding"] = {"scale": rng.choice([0.5, 4.0, 12.0])}
    if rng.random() < 0.8:
        out["residual_mult"] = rng.choice([0.3, 0.5, 1.0, 1.5])
    return out


def close(got, want, dtype, sure=None) -> bool:
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:              # rounding goes with the size of the logits (an embedding scale of 12 makes them large)
        return bool(torch.allclose(got, want, atol=max(6e-4, 2e-5 * float(want.max() - want.min())), rtol=2e-4))
    if got.dim() == 1:
        got, want = got[None], want[None]
        sure = None if sure is None else torch.as_tensor(sure).reshape(1)
    if sure is not None:
        got, want = got[sure], want[sure]
    if got.numel() == 0:
        return True
    span = float(want.max() - want.min())
    error = (got - want).abs()
    return float(error.max()) <= 0.07 * span and float(error.mean()) <= 0.015 * span


@pytest.mark.parametrize("case", range(100, 130))
def test_random_configuration(tmp_path, case):
    from llm_b200.engine import Engine, Entry, load_model
    rng = random.Random(31700 + case)
    raw = draw_config(rng)
    folder = write_folder(tmp_path / "model", raw, random_weights(raw, 900 + case))
    config, weights = plain.read_model(folder)
    lengths = [rng.choice([1, 3, 17, 64, 65, 127, 128, 129, 200, 300]) for _ in range(rng.choice([1, 2, 3, 5]))]
    extra = [rng.choice([1, 2, 8, 33]) for _ in lengths]
    gen = torch.Generator().manual_seed(case)
    seqs = [torch.randint(0, raw["vocab"], (n + e,), generator=gen).tolist() for n, e in zip(lengths, extra)]
    expected, margins = [], []
    for s in seqs:
        per_layer = []
        expected.append(plain.forward(config, weights, s, margins=per_layer))
        # bfloat16: from the first position on at which an expert was chosen by less than rounding reaches, a sequence is
        # not compared (another expert there changes what every later position reads from the state and the cache)
        margins.append(torch.cummin(torch.stack(per_layer).min(dim=0).values, dim=0).values > MARGIN if per_layer
                       else torch.ones(len(s), dtype=torch.bool))
    for dtype in (torch.float32, torch.bfloat16):
        sure = [None if dtype == torch.float32 else m for m in margins]
        engine = Engine(load_model(folder, dtype, DEV), max_tokens=64 * 7 * len(seqs), max_slots=len(seqs))
        slots = engine.acquire(len(seqs))
        logits = engine.step([Entry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lengths)])
        at = 0
        for b, n in enumerate(lengths):
            assert close(logits[at:at + n], expected[b][:n], dtype, None if sure[b] is None else sure[b][:n]), \
                (raw, dtype, "prompt", b, lengths)
            at += n
        live = list(range(len(seqs)))
        for k in range(max(extra)):
            ended = [b for b in live if k >= extra[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
            if not live:
                break
            logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
            for row, b in enumerate(live):
                p = lengths[b] + k
                assert close(logits[row], expected[b][p], dtype, None if sure[b] is None else sure[b][p]), \
                    (raw, dtype, "step", k, b, lengths)
        engine.release([slots[b] for b in live])
        engine.cache.check()
        engine.check()
