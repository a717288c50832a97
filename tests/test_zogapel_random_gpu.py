"""Randomly drawn tiny Zogapel configurations (seeded): any order of the two mixers and the three
kinds of feed-forward, widths that the 16-byte paths take and widths they do not, head and value
sizes that the tensor-core kernels take and sizes no tile takes, groups of 1 to 8 heads, windows
from 1 to beyond the prompts and none, rotated parts shorter than a head, bands and no bands, one
to five taps, one to all of 2 to 40 experts. Each runs a batch of unequal prompts and then decodes,
shorter requests leaving earlier, in 32-bit and in bfloat16, against the plain implementation."""
import math
import random

import pytest
import torch

import plain_zogapel as plain
from tiny_zogapel import random_weights, write_folder

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def draw_config(rng) -> dict:
    width = rng.choice([36, 48, 64, 100, 128, 160, 256, 260])

    def attention():
        kv = rng.choice([1, 2, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 4, 8]) if kv < 4 else kv * rng.choice([1, 2])
        dim = rng.choice([8, 10, 16, 24, 32, 64, 64, 96, 128])
        out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": rng.choice([1.0 / math.sqrt(dim), 0.11])}
        window = rng.choice([0, 1, 2, 7, 33, 64, 65, 100, 128, 190, 1000])
        if window:
            out["mask"] = {"size": window}
        if rng.random() < 0.85:
            dims = rng.choice([dim, dim // 2, 2, dim - 2 if dim > 2 else 2]) // 2 * 2 or 2
            rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": dims}
            if rng.random() < 0.7:
                rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "original": rng.choice([16, 64, 512, 4096]),
                                  "fast": rng.choice([4.0, 32.0]), "slow": rng.choice([0.5, 1.0, 2.0])}
            out["rot"] = rot
        return out

    def delta():
        kv = rng.choice([1, 2, 3, 4])
        return {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": rng.choice([4, 12, 16, 32, 40, 64, 128]),
                "vdim": rng.choice([4, 6, 16, 32, 36, 64, 128]), "conv": rng.choice([1, 2, 3, 4, 5])}

    def feed_forward():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": rng.choice([32, 80, 100, 128, 200])}
        experts = rng.choice([2, 3, 8, 16, 40])
        top = rng.choice([1, 2, min(4, experts), experts if experts <= 8 else 6])
        return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": rng.choice([8, 20, 32, 64, 72])}}

    layers = []
    for _ in range(rng.choice([1, 2, 3, 4])):
        kind = rng.choice(["attention", "delta"])
        layers.append({"type": kind, "mixer": attention() if kind == "attention" else delta(), "mlp": feed_forward()})
    out = {"architecture": "Zogapel", "vocab": rng.choice([61, 128, 300, 1000]), "width": width,
           "norm": {"eps": rng.choice([1e-5, 1e-6, 1e-3])}, "layers": layers}
    if rng.random() < 0.8:
        out["embedding"] = {"scale": rng.choice([0.5, 4.0, 12.0])}
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


@pytest.mark.parametrize("case", range(100, 124))
def test_random_configuration(tmp_path, case):
    from llm_b200.engine import Engine, Entry, load_model
    rng = random.Random(20400 + case)
    raw = draw_config(rng)
    folder = write_folder(tmp_path / "model", raw, random_weights(raw, 700 + case))
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
        margins.append(torch.cummin(torch.stack(per_layer).min(dim=0).values, dim=0).values > 0.15 if per_layer
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
