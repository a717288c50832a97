"""Zogapel on the CPU: configuration, the plain statement's own mechanisms, and the engine's
host-side logic (packing, positions, pages, slots, the delta rule's and the convolutions' state, the
norms on both sides of a part, the experts' rows) with the kernels replaced by their plain
statements, against the plain whole-sequence implementation."""
import copy
import math

import pytest
import torch

import plain_zogapel as plain
from tiny_zogapel import CONFIGS, ZOG_P, ZOG_Q, ZOG_R, make_folder, random_tokens, tensor_shapes

from llm_b200.config import ZogapelConfig, config_from_dict
from llm_b200.engine import Engine, Entry, declared_parameters, load_model
from llm_b200.errors import FormatError, MissingKey, Unsupported, WeightError

TOL = dict(atol=4e-4, rtol=1e-4)


def _setup(tmp_path, which, change=None, **engine_options):
    folder = make_folder(tmp_path, which, torch.float32, change)
    config, weights = plain.read_model(folder)
    engine = Engine(load_model(folder, torch.float32, "cpu"), **{"max_tokens": 2048, **engine_options})
    return config, weights, engine


# ----------------------------------------------------------------------------- configuration

def test_config_gives_the_layers_and_names():
    config = config_from_dict(copy.deepcopy(ZOG_P))
    assert isinstance(config, ZogapelConfig)
    spec = config.model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and spec.head is None and spec.embedding_scale == 2.5
    attention, delta = spec.blocks[0].mixer, spec.blocks[1].mixer
    assert attention.kind == "gated_attention" and delta.kind == "delta_rule"
    assert (attention.n_heads, attention.n_kv_heads, attention.head_dim, attention.window) == (4, 2, 6, 9)
    assert attention.values_are_keys and attention.out_gate and attention.position.rotary_dim == 4
    assert attention.position.pairing == "half" and dict(attention.position.scaling)["factor"] == 3.0
    assert spec.blocks[2].mixer.position.scaling is None and spec.blocks[2].mixer.scale == 0.2
    assert (delta.n_heads, delta.n_kv_heads, delta.head_dim, delta.value_dim, delta.conv_taps) == (3, 1, 5, 7, 3)
    assert delta.eps == 1e-5 and delta.unit_eps == 1e-6
    routed = spec.blocks[1].feed_forward
    assert (routed.n_experts, routed.top, routed.intermediate, routed.router_bias) == (5, 3, 12, True)
    assert spec.blocks[0].feed_forward.activation == "gelu_tanh" and spec.blocks[0].feed_forward.intermediate == 52
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].ffn_norm is None and spec.blocks[2].ffn_post_norm is None
    assert spec.blocks[0].mixer_post_norm.weight == "l0.norm1b" and spec.blocks[0].ffn_post_norm.weight == "l0.norm2b"
    nothing = config_from_dict(copy.deepcopy(ZOG_R)).model_spec()
    assert nothing.blocks[1].mixer.position is None and nothing.blocks[1].mixer.window == 0 and nothing.embedding_scale == 1.0
    for raw in (ZOG_P, ZOG_Q, ZOG_R):
        spec = config_from_dict(copy.deepcopy(raw)).model_spec()
        declared = {name: tuple(p.shape) for name, p in declared_parameters(spec).items()}
        assert declared == tensor_shapes(raw)
    assert config_from_dict(config.to_dict()).model_spec() == config.model_spec()


def test_config_errors_name_the_key():
    for path, value, error in [(("layers", 0, "mixer", "heads"), 3, FormatError),          # 3 heads, 2 kv heads
                               (("layers", 0, "type"), "parallel", Unsupported),
                               (("layers", 0, "mlp", "kind"), "gated", Unsupported),
                               (("layers", 0, "mixer", "rot", "dims"), 7, FormatError),
                               (("layers", 0, "mixer", "vdim"), 8, FormatError),             # the values are the keys
                               (("layers", 1, "mlp", "router", "top"), 6, FormatError),
                               (("layers", 1, "mixer", "conv"), 0, FormatError)]:
        raw = copy.deepcopy(ZOG_P)
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            config_from_dict(raw)
    raw = copy.deepcopy(ZOG_P)
    del raw["layers"][1]["mixer"]["vdim"]
    with pytest.raises(MissingKey) as info:
        config_from_dict(raw)
    assert "vdim" in str(info.value)


def test_a_missing_tensor_is_reported(tmp_path):
    def drop(weights):
        del weights["l1.mix.A_log"]
        weights["l1.mlp.e2.down"] = weights["l1.mlp.e2.down"][:3]
    folder = make_folder(tmp_path, "P", torch.float32, weights_change=drop)
    with pytest.raises(WeightError) as info:
        load_model(folder, torch.float32, "cpu")
    assert "l1.mix.A_log" in str(info.value) and "l1.mlp.e2.down" in str(info.value)


# ----------------------------------------------------------------------------- the plain statement's mechanisms

def test_plain_mechanisms():
    gen = torch.Generator().manual_seed(0)
    F = plain.F
    # the norm's weight is stored around zero: zero is the plain norm
    x = torch.randn((7, 12), generator=gen, dtype=F)
    y = plain.rms_norm(x, torch.zeros(12, dtype=F), 1e-5)
    assert torch.allclose((y * y).mean(-1), torch.ones(7, dtype=F), atol=1e-3)
    assert torch.allclose(plain.rms_norm(x, torch.full((12,), -1.0, dtype=F), 1e-5), torch.zeros_like(x))
    # the convolution: the last column is the current token's tap, zeros before the start
    u = torch.randn((5, 2), generator=gen, dtype=F)
    c = plain.causal_conv(u, torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=F))
    assert torch.allclose(c[:, 0], u[:, 0]) and torch.allclose(c[2:, 1], u[:3, 1]) and torch.allclose(c[:2, 1], torch.zeros(2, dtype=F))
    # rotation: position 0 is scaled only, elements beyond the rotated part stay, pairs are (i, i + half)
    h = torch.randn((2, 6), generator=gen, dtype=F)
    freq, magnitude = plain.rotary_frequencies({"base": 50.0, "dims": 4})
    assert magnitude == 1.0 and torch.allclose(freq, torch.tensor([1.0, 50.0 ** -0.5], dtype=F))
    r = plain.rotate(h, 1.0, freq, magnitude)
    assert torch.allclose(plain.rotate(h, 0.0, freq, magnitude), h) and torch.allclose(r[..., 4:], h[..., 4:])
    assert torch.allclose(r[0, 0], h[0, 0] * math.cos(1.0) - h[0, 2] * math.sin(1.0))
    assert torch.allclose(r[0, 2], h[0, 2] * math.cos(1.0) + h[0, 0] * math.sin(1.0))
    # bands: dims 8, base 100, original 100: dim(10) = 0.40 -> lo 0, dim(1) = 2.40 -> hi 3; pairs 0..3 ramp 0, 1/3, 2/3, 1
    freq, magnitude = plain.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 100, "fast": 10.0, "slow": 1.0}})
    plain_freq = torch.tensor([100.0 ** (-2.0 * i / 8) for i in range(4)], dtype=F)
    ramp = torch.tensor([0.0, 1 / 3, 2 / 3, 1.0], dtype=F)
    assert torch.allclose(freq, plain_freq / 4.0 * ramp + plain_freq * (1 - ramp)) and abs(magnitude - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    # the experts: a chosen expert's weight is the softmax over the chosen logits only
    f = {"router": {"experts": 3, "top": 2}}
    w = {"r.router": torch.zeros((3, 2), dtype=F), "r.router.b": torch.tensor([1.0, 3.0, 2.0], dtype=F)}
    for e in range(3):
        w[f"r.e{e}.gate"] = torch.full((1, 2), 50.0, dtype=F)           # silu(large) = itself
        w[f"r.e{e}.up"] = torch.full((1, 2), float(e + 1), dtype=F)
        w[f"r.e{e}.down"] = torch.ones((2, 1), dtype=F)
    margins = []
    out = plain.routed_ff(torch.tensor([[1.0, 1.0]], dtype=F), f, w, "r.", margins)
    share = math.exp(3.0) / (math.exp(3.0) + math.exp(2.0))
    assert torch.allclose(out[0, 0], torch.tensor(100.0 * (share * 4.0 + (1 - share) * 6.0), dtype=F)) and float(margins[0][0]) == 1.0


def test_plain_delta_rule_stores_and_reads_back():
    """beta = 1, no decay, orthogonal unit keys: reading with a stored key gives its value back."""
    F = plain.F
    big = 40.0
    w = {"d.q": torch.eye(4, dtype=F), "d.k": torch.eye(4, dtype=F), "d.v": torch.zeros((3, 4), dtype=F),
         "d.q.conv": torch.ones((4, 1), dtype=F), "d.k.conv": torch.ones((4, 1), dtype=F), "d.v.conv": torch.ones((3, 1), dtype=F),
         "d.b": torch.zeros((1, 4), dtype=F), "d.a": torch.zeros((1, 4), dtype=F), "d.A_log": torch.tensor([-40.0], dtype=F),
         "d.dt_bias": torch.zeros(1, dtype=F), "d.norm": torch.ones(3, dtype=F), "d.g": torch.zeros((3, 4), dtype=F),
         "d.o": torch.eye(3, dtype=F)}
    w["d.v"][:, :3] = torch.eye(3, dtype=F)
    w["d.b"][0] = big                                                   # sigmoid(large) = 1
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "conv": 1}
    h = torch.zeros((3, 4), dtype=F)
    h[0, 0], h[1, 1], h[2, 0] = big, big, big                           # token 2 asks with token 0's key
    w["d.g"][:, 0] = 1.0
    out = plain.delta_mixer(h, m, w, "d.", 1e-12)
    # token 0 wrote v = (silu(big), 0, 0) under key e0; token 2 overwrites with the same and reads it: only element 0 is non-zero
    assert float(out[2, 0].abs()) > 1.0 and float(out[2, 1:].abs().max()) < 1e-9


# ----------------------------------------------------------------------------- the engine with plain kernels

@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_whole_prompt_matches_plain(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(150, config["vocab"], 1)
    streams = []
    want = plain.forward(config, weights, tokens, streams).float()
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    assert torch.allclose(got, want, **TOL), float((got - want).abs().max())


@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_token_by_token_equals_prefill(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(80, config["vocab"], 2)
    want = plain.forward(config, weights, tokens).float()
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):                      # from the very first token on
        got = engine.step([Entry(slot, [token], [0])])
        assert torch.allclose(got[0], want[p], **TOL), (p, float((got[0] - want[p]).abs().max()))


@pytest.mark.parametrize("piece", [2, 3, 7, 64])
def test_prompts_cut_into_pieces(tmp_path, plain_kernels, piece):
    config, weights, engine = _setup(tmp_path, "P")
    tokens = random_tokens(131, config["vocab"], 3)
    want = plain.forward(config, weights, tokens).float()
    (slot,) = engine.acquire()
    for start in range(0, len(tokens), piece):
        part = tokens[start:start + piece]
        got = engine.step([Entry(slot, part, list(range(len(part))))])
        assert torch.allclose(got, want[start:start + len(part)], **TOL), start
    # the engine's own cutting of a long prompt into passes
    config, weights, engine = _setup(tmp_path, "Q", step_tokens=piece * 8)
    tokens = random_tokens(140, config["vocab"], 4)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, [0, 70, 139])])
    assert torch.allclose(got, plain.forward(config, weights, tokens).float()[[0, 70, 139]], **TOL)


def test_unequal_batch_slot_reuse_and_early_ends(tmp_path, plain_kernels):
    config, weights, engine = _setup(tmp_path, "P", max_tokens=1024)
    lengths = [70, 1, 33, 12]
    for again in range(3):                                   # slots, pages and states are taken again
        seqs = [random_tokens(n, config["vocab"], 10 * again + n) for n in lengths]
        want = [plain.forward(config, weights, s).float() for s in seqs]
        slots = engine.acquire(len(seqs))
        heads = [max(1, n - 5 - i) for i, n in enumerate(lengths)]
        got = engine.step([Entry(s, q[:h], [h - 1]) for s, q, h in zip(slots, seqs, heads)])
        for b, h in enumerate(heads):
            assert torch.allclose(got[b], want[b][h - 1], **TOL), (again, b)
        live = [b for b in range(len(seqs)) if heads[b] < lengths[b]]
        engine.release([slots[b] for b in range(len(seqs)) if b not in live])
        done = 0
        while live:
            got = engine.step([Entry(slots[b], [seqs[b][heads[b] + done]], [0]) for b in live])
            for r, b in enumerate(live):
                assert torch.allclose(got[r], want[b][heads[b] + done], **TOL), (again, b, done)
            done += 1
            ended = [b for b in live if heads[b] + done == lengths[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


def test_a_mixed_step(tmp_path, plain_kernels):
    """Two sequences go on by one token while a third brings the rest of its prompt."""
    config, weights, engine = _setup(tmp_path, "Q")
    a, b, c = (random_tokens(n, config["vocab"], 40 + n) for n in (30, 9, 90))
    sa, sb, sc = engine.acquire(3)
    engine.step([Entry(sa, a[:29], []), Entry(sb, b[:8], []), Entry(sc, c[:20], [])])
    got = engine.step([Entry(sa, [a[29]], [0]), Entry(sc, c[20:], [0, 69]), Entry(sb, [b[8]], [0])])
    wa, wb, wc = (plain.forward(config, weights, s).float() for s in (a, b, c))
    want = torch.stack([wa[29], wc[20], wc[89], wb[8]])
    assert torch.allclose(got, want, **TOL), float((got - want).abs().max())


def test_random_model_writer_round_trip(tmp_path, plain_kernels):
    from llm_b200.weights import write_random_model
    config = config_from_dict(copy.deepcopy(ZOG_P))
    folder = write_random_model(tmp_path / "random", config, seed=5, dtype=torch.float32, std=0.3)
    raw, weights = plain.read_model(folder)
    assert {k: tuple(v.shape) for k, v in weights.items()} == tensor_shapes(ZOG_P)
    engine = Engine(load_model(folder, torch.float32, "cpu"), max_tokens=256)
    tokens = random_tokens(40, raw["vocab"], 6)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(40)))])
    assert torch.allclose(got, plain.forward(raw, weights, tokens).float(), **TOL)


def test_inspect_and_random_commands(tmp_path, capsys):
    import json
    from llm_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(ZOG_Q))
    assert main(["random", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    text = capsys.readouterr().out
    assert "Zogapel" in text and "delta" in text
