"""Zemozen on the CPU: configuration, the plain statement's own mechanisms, and the engine's host-side
logic (packing, positions, pages, slots, the recurrence's and the convolution's state, values blended
across layers, the experts' rows) with the kernels replaced by their plain statements, against the plain
whole-sequence implementation."""
import copy
import math

import pytest
import torch

import plain_zemozen as plain
from tiny_zemozen import CONFIGS, ZEM_P, ZEM_Q, ZEM_R, make_folder, random_tokens, tensor_shapes

from llm_b200.config import ZemozenConfig, config_from_dict
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
    config = config_from_dict(copy.deepcopy(ZEM_P))
    assert isinstance(config, ZemozenConfig)
    spec = config.model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4] and spec.head == "head" and spec.embedding_scale == 2.5
    pair, attention = spec.blocks[0].mixer, spec.blocks[1].mixer
    assert pair.kind == "side_by_side" and attention.kind == "gated_attention"
    left, right = pair.left, pair.right
    assert (left.n_heads, left.n_kv_heads, left.head_dim, left.value_dim, left.window) == (4, 2, 6, 10, 9)
    assert left.unit_sink and left.softcap == 1.5 and not left.head_gate and left.head_norm and left.value_mix is None
    assert left.position.pairing == "interleaved" and left.position.rotary_dim == 4 and left.position.scaling is None
    assert abs(left.out_scale - 0.7 * 0.8) < 1e-12 and abs(right.out_scale - 0.7 * 1.3) < 1e-12
    assert (right.n_heads, right.groups, right.value_dim, right.state, right.conv_taps, right.norm_groups) == (3, 1, 5, 7, 2, 3)
    assert right.kind == "state_space" and right.eps == 1e-5
    assert attention.head_gate and not attention.unit_sink and attention.softcap == 0.0 and attention.out_scale == 0.7
    assert attention.position.pairing == "half" and dict(attention.position.scaling) == {"type": "linear", "factor": 4.0}
    assert attention.norm_eps == 1e-5 and not attention.values_are_keys and not attention.out_gate
    # the first layer that blends values is layer 1; layer 3 does not blend
    mixes = [(b.mixer.value_mix, b.mixer.value_mix_first) for b in spec.blocks[1:]]
    assert mixes == [("v_mix", True), ("v_mix", False), (None, False), ("v_mix", False)]
    assert spec.blocks[3].mixer.window == 0 and spec.blocks[3].mixer.scale == 0.3 and spec.blocks[2].mixer.position is None
    routed = spec.blocks[0].feed_forward
    assert (routed.n_experts, routed.pass_through, routed.top, routed.intermediate) == (5, 1, 3, 12)
    assert routed.scoring == "all" and routed.correction and not routed.router_bias and routed.out_scale == 0.7
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].ffn_norm is None
    nothing = config_from_dict(copy.deepcopy(ZEM_R)).model_spec()
    assert nothing.embedding_scale == 1.0 and nothing.blocks[1].mixer.out_scale == 1.0
    assert nothing.blocks[1].mixer.position is None and nothing.blocks[1].mixer.window == 0
    for raw in (ZEM_P, ZEM_Q, ZEM_R):
        spec = config_from_dict(copy.deepcopy(raw)).model_spec()
        declared = {name: tuple(p.shape) for name, p in declared_parameters(spec).items()}
        assert declared == tensor_shapes(raw)
    assert config_from_dict(config.to_dict()).model_spec() == config.model_spec()


def test_config_errors_name_the_key():
    for path, value, error in [(("layers", 1, "mixer", "heads"), 3, FormatError),           # 3 heads, 2 kv heads
                               (("layers", 0, "type"), "delta", Unsupported),
                               (("layers", 0, "mlp", "kind"), "dense", Unsupported),
                               (("layers", 1, "mixer", "rot", "dims"), 7, FormatError),
                               (("layers", 0, "mixer", "right", "groups"), 2, FormatError),    # 3 heads in 2 groups
                               (("layers", 0, "mixer", "right", "norm_groups"), 4, FormatError),
                               (("layers", 0, "mlp", "router", "top"), 7, FormatError),
                               (("layers", 0, "mixer", "right", "conv"), 0, FormatError)]:
        raw = copy.deepcopy(ZEM_P)
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            config_from_dict(raw)
    raw = copy.deepcopy(ZEM_P)
    del raw["layers"][0]["mixer"]["right"]["state"]
    with pytest.raises(MissingKey) as info:
        config_from_dict(raw)
    assert "state" in str(info.value)


def test_a_missing_tensor_is_reported(tmp_path):
    def drop(weights):
        del weights["l0.mix.right.A_log"]
        weights["l0.mlp.correction"] = weights["l0.mlp.correction"][:3]
    folder = make_folder(tmp_path, "P", torch.float32, weights_change=drop)
    with pytest.raises(WeightError) as info:
        load_model(folder, torch.float32, "cpu")
    assert "l0.mix.right.A_log" in str(info.value) and "l0.mlp.correction" in str(info.value)


# ----------------------------------------------------------------------------- the plain statement's mechanisms

def test_plain_mechanisms():
    gen = torch.Generator().manual_seed(0)
    F = plain.F
    x = torch.randn((7, 12), generator=gen, dtype=F)
    y = plain.rms_norm(x, torch.ones(12, dtype=F), 1e-9)
    assert torch.allclose((y * y).mean(-1), torch.ones(7, dtype=F), atol=1e-6)
    # the convolution: the last column is the current token's tap, zeros before the start, then the bias
    u = torch.randn((5, 2), generator=gen, dtype=F)
    c = plain.causal_conv(u, torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=F), torch.tensor([0.0, 2.0], dtype=F))
    assert torch.allclose(c[:, 0], u[:, 0]) and torch.allclose(c[2:, 1], u[:3, 1] + 2.0) and torch.allclose(c[:2, 1], torch.full((2,), 2.0, dtype=F))
    # rotation: both pairings, elements beyond the rotated part stay, stretched positions divide the frequencies
    h = torch.randn((2, 6), generator=gen, dtype=F)
    freq = plain.rotary_frequencies({"base": 50.0, "dims": 4})
    assert torch.allclose(freq, torch.tensor([1.0, 50.0 ** -0.5], dtype=F))
    assert torch.allclose(plain.rotary_frequencies({"base": 50.0, "dims": 4, "scaling": {"factor": 8.0}}), freq / 8.0)
    for interleaved, partner in ((False, 2), (True, 1)):
        r = plain.rotate(h, 1.0, freq, interleaved)
        assert torch.allclose(plain.rotate(h, 0.0, freq, interleaved), h) and torch.allclose(r[..., 4:], h[..., 4:])
        assert torch.allclose(r[0, 0], h[0, 0] * math.cos(1.0) - h[0, partner] * math.sin(1.0))
        assert torch.allclose(r[0, partner], h[0, partner] * math.cos(1.0) + h[0, 0] * math.sin(1.0))
    # the router: scores over all outputs, the correction decides the choice but not the weights, an output beyond
    # the experts with matrices hands the input through
    f = {"router": {"experts": 2, "identity": 1, "top": 2}}
    w = {"r.router": torch.zeros((3, 2), dtype=F), "r.correction": torch.tensor([0.0, -1.0, 0.5], dtype=F)}
    w["r.router"][:, 0] = torch.tensor([1.0, 3.0, 2.0], dtype=F)
    for e in range(2):
        w[f"r.e{e}.gate"] = torch.full((1, 2), 50.0, dtype=F)           # silu(large) = itself
        w[f"r.e{e}.up"] = torch.full((1, 2), float(e + 1), dtype=F)
        w[f"r.e{e}.down"] = torch.ones((2, 1), dtype=F)
    margins = []
    hh = torch.tensor([[1.0, 0.0]], dtype=F)
    out = plain.routed_ff(hh, f, w, "r.", margins)
    s = torch.softmax(torch.tensor([1.0, 3.0, 2.0], dtype=F), 0)
    share0, share2 = s[0] / (s[0] + s[2]), s[2] / (s[0] + s[2])       # expert 1 has the largest score and is not chosen
    want = share0 * 50.0 * 1.0 * torch.ones(2, dtype=F) + share2 * hh[0]
    assert torch.allclose(out[0], want) and abs(float(margins[0][0]) - float(s[0] - (s[1] - 1.0))) < 1e-12


def test_plain_recurrence_remembers_and_fades():
    """One head, one state row: with x = 1 at the first token only, y_t = C_t * prod(decay) * dt_0 * B_0."""
    F = plain.F
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    big = 40.0
    w = {"s.in": torch.zeros((5, 5), dtype=F), "s.conv": torch.ones((3, 1), dtype=F), "s.conv.b": torch.zeros(3, dtype=F),
         "s.dt_bias": torch.zeros(1, dtype=F), "s.A_log": torch.zeros(1, dtype=F), "s.D": torch.zeros(1, dtype=F),
         "s.norm": torch.ones(1, dtype=F), "s.o": torch.ones((1, 1), dtype=F)}
    w["s.in"] = torch.eye(5, dtype=F)                        # h = [z, x, B, C, dt] itself
    h = torch.zeros((4, 5), dtype=F)
    h[:, 0] = big                                            # silu(z) = z
    h[0, 1] = big                                            # x: silu(big) = big at the first token, 0 after
    h[:, 2], h[:, 3] = big, big                              # B = C = big
    h[:, 4] = 1.0
    states = []
    plain.state_space_mixer(h, m, w, "s.", 1e-30, states)
    dt = math.log1p(math.e)
    assert abs(float(states[0][0, 0, 0]) - math.exp(-dt) ** 3 * dt * big * big) < 1e-6 * big * big


# ----------------------------------------------------------------------------- the engine with plain kernels

@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_whole_prompt_matches_plain(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(150, config["vocab"], 1)
    want = plain.forward(config, weights, tokens).float()
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
    config = config_from_dict(copy.deepcopy(ZEM_P))
    folder = write_random_model(tmp_path / "random", config, seed=5, dtype=torch.float32, std=0.3)
    raw, weights = plain.read_model(folder)
    assert {k: tuple(v.shape) for k, v in weights.items()} == tensor_shapes(ZEM_P)
    engine = Engine(load_model(folder, torch.float32, "cpu"), max_tokens=256)
    tokens = random_tokens(40, raw["vocab"], 6)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(40)))])
    assert torch.allclose(got, plain.forward(raw, weights, tokens).float(), **TOL)


def test_inspect_and_random_commands(tmp_path, capsys):
    import json
    from llm_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(ZEM_Q))
    assert main(["random", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    text = capsys.readouterr().out
    assert "Zemozen" in text and "residual_mult" in text and "attention" in text
