"""Zogapel on the GPU: every new kernel beside its plain statement (also with weights and inputs
made so that one key, a window's edge, a stored value or a lost state shows), and the model through
the engine, the generation entry point and the trace-replay program against the plain
whole-sequence implementation, in 32-bit and in bfloat16."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_ops
import plain_zogapel as plain
from test_mefolorn_gpu import BATCHES, Batch, _close, only_generic
from tiny_zogapel import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

PAGE = 64
DEV = "cuda:0"


def _ops():
    from llm_b200 import ops
    return ops


# ----------------------------------------------------------------------------- norms on both sides of a part

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 97, 128, 1024, 4100])
def test_norm_add(out_dtype, width):
    ops = _ops()
    gen = torch.Generator().manual_seed(width)
    for terms in (1, 2, 3):
        for n in (1, 9, 70):
            x = (2.0 * torch.randn((n, width), generator=gen)).to(DEV)
            y = (5.0 * torch.randn((n * terms, width), generator=gen)).to(DEV)
            y[0] *= 1e-4                                       # a row whose mean square is of the order of eps
            g1, g2 = (1.0 + 0.3 * torch.randn(width, generator=gen)).to(DEV), torch.randn(width, generator=gen).to(DEV)
            xa, xb = x.clone(), x.clone()
            assert ops.norm_add_(xa, y, g1, 1e-5, terms) is None
            plain_ops.norm_add_(xb, y, g1, 1e-5, terms)
            _close(xa, xb, torch.float32, (terms, n, "x"))
            xa, xb = x.clone(), x.clone()
            out = torch.zeros((n, width), dtype=out_dtype, device=DEV)
            got = ops.norm_add_(xa, y, g1, 1e-5, terms, g2, 1e-3, out=out, out_dtype=out_dtype)
            want = plain_ops.norm_add_(xb, y, g1, 1e-5, terms, g2, 1e-3, out_dtype=out_dtype)
            assert got.data_ptr() == out.data_ptr()
            _close(xa, xb, torch.float32, (terms, n, "x with next"))
            _close(got, want, out_dtype, (terms, n, "next"))


def test_norm_add_sums_a_token_s_rows_in_their_order():
    """Three rows a token whose sum in another order would round differently: 1e8 - 1e8 + 1 is 1, not 0."""
    ops = _ops()
    width = 64
    y = torch.zeros((3, width), device=DEV)
    y[0], y[1], y[2] = 1e8, -1e8, 1.0
    x = torch.zeros((1, width), device=DEV)
    ops.norm_add_(x, y, torch.ones(width, device=DEV), 0.0, 3)
    assert torch.allclose(x, torch.ones_like(x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gate_terms_and_fill(dtype):
    ops = _ops()
    gen = torch.Generator().manual_seed(3)
    for n, width in ((1, 5), (7, 52), (70, 320), (33, 4100)):
        a = (3.0 * torch.randn((n, width), generator=gen)).to(dtype).to(DEV)
        _close(ops.gelu_(a.clone()), plain_ops.gelu_(a.clone()), dtype, ("gelu", n, width))
        wide = torch.randn((n, 2 * width + 11), generator=gen).to(dtype).to(DEV)
        outs = [wide.clone(), wide.clone()]
        gate = wide[:, width + 3:2 * width + 3]
        ops.sigmoid_gate_(outs[0][:, 2:2 + width], gate)
        plain_ops.sigmoid_gate_(outs[1][:, 2:2 + width], gate)
        _close(outs[0], outs[1], dtype, ("gate", n, width))                    # nothing beside the gated columns moves
        x = torch.randn((n, width), generator=gen).to(DEV)
        y = torch.randn((n * 3, width), generator=gen).to(DEV)
        _close(ops.add_terms_(x.clone(), y, 3), plain_ops.add_terms_(x.clone(), y, 3), torch.float32, ("terms", n, width))
        assert float((ops.fill_(x.clone(), 0.25) - 0.25).abs().max()) == 0.0
    z = torch.tensor([-30.0, -1.0, 0.0, 0.5, 30.0], device=DEV)
    want = torch.tensor([0.0, -0.15880801, 0.0, 0.34571401, 30.0], device=DEV)          # the tanh form's values
    assert torch.allclose(ops.gelu_(z.clone()), want, atol=1e-6)


# ----------------------------------------------------------------------------- frequencies scaled by bands

@pytest.mark.parametrize("rot", [
    {"base": 100.0, "dims": 4, "scaling": {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 1.0}},
    {"base": 200000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}},
    {"base": 1000.0, "dims": 16, "scaling": {"factor": 16.0, "original": 128, "fast": 16.0, "slow": 1.0}},
    {"base": 10.0, "dims": 6, "scaling": {"factor": 2.0, "original": 4096, "fast": 1.0, "slow": 0.5}},          # lo = hi
    {"base": 5000.0, "dims": 32}])
def test_rotation_table_with_bands(rot):
    from llm_b200.parts.base import build_position
    from llm_b200.parts.spec import PositionSpec
    scaling = tuple(sorted({"type": "ramp", **rot["scaling"]}.items())) if "scaling" in rot else None
    position = build_position(PositionSpec(head_dim=40, theta=rot["base"], max_positions=4096, scaling=scaling,
                                           pairing="half", rotary_dim=rot["dims"]))
    position.prepare(3000, DEV)
    freq, magnitude = plain.rotary_frequencies(rot)
    angle = torch.arange(3000, dtype=torch.float64)[:, None] * freq[None, :]
    want = torch.cat([angle.cos(), angle.sin()], dim=1) * magnitude
    assert position.table.shape[1] == rot["dims"] and not position.interleaved
    assert torch.allclose(position.table[:3000].cpu().double(), want, atol=2e-6)


# ----------------------------------------------------------------------------- keys that are also the values

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [(4, 2, 6, 4, 24), (2, 2, 8, 8, 0), (4, 1, 64, 32, 256), (8, 2, 32, 32, 5), (2, 1, 128, 0, 256)])
def test_cache_write_takes_the_values_from_the_unrotated_keys(dtype, case):
    ops = _ops()
    heads, groups, dim, n_rot, behind = case
    qw, kw = heads * dim, groups * dim
    gen = torch.Generator().manual_seed(5)
    for lengths, new in BATCHES:
        batch = Batch(lengths, new, seed=len(lengths))
        wide = torch.randn((batch.n_tokens, qw + kw + behind), generator=gen).to(dtype).to(DEV)
        table = None
        if n_rot:
            angle = torch.arange(400, dtype=torch.float64)[:, None] * torch.rand(n_rot // 2, generator=gen, dtype=torch.float64)
            table = (1.2 * torch.cat([angle.cos(), angle.sin()], dim=1)).float().to(DEV)
        results = []
        for fn in (ops.norm_rope_cache_write, plain_ops.norm_rope_cache_write):
            k_cache, v_cache = batch.caches(groups, dim, dim, dtype, seed=5)
            queries = torch.zeros((batch.n_tokens, qw), dtype=dtype, device=DEV)
            fn(wide, qw, kw, kw, None, None, 0.0, table, dim, False, batch.tok_pos, batch.tok_seq, queries, batch.table,
               batch.width, k_cache, v_cache, value_source=qw)
            results.append((queries, k_cache, v_cache))
        torch.cuda.synchronize()
        for got, want, what in zip(results[0], results[1], ("queries", "keys", "values")):
            _close(got, want, dtype, (case, lengths, what))
        # the cached values are the projection's key columns themselves, bit for bit
        k_cache, v_cache = results[0][1], results[0][2]
        for row in (0, batch.n_tokens - 1):
            b, p = int(batch.tok_seq[row]), int(batch.tok_pos[row])
            page, at = batch.place(b, p)
            assert torch.equal(v_cache[page, :, at].reshape(-1), wide[row, qw:qw + kw])
            if n_rot and p > 0:
                assert not torch.equal(k_cache[page, :, at].reshape(-1), wide[row, qw:qw + kw])


def test_attention_over_rotated_keys_and_unrotated_values_at_the_window_s_edges():
    """Keys and values in caches of their own: one key is made to stand out, and the result is that
    position's VALUE row exactly when the key is inside the window (far back, at page borders, at both
    edges), in a prompt's portion and in decoding, in 32-bit, bfloat16 and with the generic kernels."""
    ops = _ops()
    heads, dim, window, length = 2, 64, 100, 331
    for dtype, generic in ((torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)):
        for decode in (False, True):
            batch = Batch([length, 40], [1, 1] if decode else [length, 40], seed=11)
            last = 0 if decode else length - 1
            gen = torch.Generator().manual_seed(4)
            for planted in (length - 1, length - window, length - window - 1, 256, 255, 0, length - 2):
                k_cache, v_cache = batch.caches(1, dim, dim, dtype, seed=6, std=0.1)
                v_cache *= 0.1
                page, row = batch.place(0, planted)
                k_cache[page, 0, row] = 0.0
                k_cache[page, 0, row, :4] = torch.tensor([3.0, -2.0, 1.0, 2.0])
                v_cache[page, 0, row, :2] = torch.tensor([5.0, -7.0])
                q = (0.1 * torch.randn((batch.n_tokens, heads * dim), generator=gen)).to(dtype).to(DEV)
                q[last] = 0.0
                q[last, :4] = torch.tensor([3.0, -2.0, 1.0, 2.0]) * 8.0
                args = (q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, 1, dim, 1.0 / 8.0, window)
                with only_generic(generic):
                    got = ops.attention(*args, **batch.extra())
                want = plain_ops.attention(*args, **batch.extra())
                torch.cuda.synchronize()
                seen = length - 1 - planted < window
                if seen:
                    assert abs(float(got[last, 0]) - 5.0) < 0.1 and abs(float(got[last, 1]) + 7.0) < 0.1, (planted, got[last, :2])
                else:
                    assert float(got[last, :2].float().abs().max()) < 0.5, (planted, got[last, :2])
                _close(got, want, dtype, (planted, decode, generic))


# ----------------------------------------------------------------------------- the gated delta rule

def _delta_inputs(H, G, D, V, K, n_tokens, n_slots, dtype, seed, memory="mixed"):
    gen = torch.Generator().manual_seed(seed)
    C = 2 * G * D + H * V
    width = (C + H * V + 2 * H + 7) // 8 * 8 + 8
    proj = torch.randn((n_tokens, width), generator=gen).to(dtype).to(DEV)
    a_log = torch.randn(H, generator=gen) - (2.0 if memory == "mixed" else 9.0)
    params = dict(taps=torch.randn((C, K), generator=gen) / K ** 0.5, rate=-torch.exp(a_log), dt_bias=torch.randn(H, generator=gen),
                  norm_weight=1.0 + 0.3 * torch.randn(V, generator=gen))
    state = (0.3 * torch.randn((n_slots, (K - 1) * C + H * D * V + 3), generator=gen)).to(DEV)
    return proj, {k: v.to(DEV).contiguous() for k, v in params.items()}, state


def _delta(fn, proj, params, state, batch, H, G, D, V, dtype, unit_eps=1e-6, eps=1e-5):
    ops = _ops()
    n = batch.n_tokens
    work = torch.zeros((n, ops.delta_rule_work_width(H, G, D, V)), device=DEV)
    o = torch.zeros((n, H * V), device=DEV)
    mixed_wide = torch.zeros((n, H * V + 9), dtype=dtype, device=DEV)
    fn(proj, params["taps"], state, batch.tok_seq, batch.cu, batch.slots, params["rate"], params["dt_bias"], unit_eps,
       params["norm_weight"], eps, work, o, mixed_wide[:, 4:4 + H * V], H, G, D, V)
    return mixed_wide


DELTA_CASES = [(3, 1, 5, 7, 3), (2, 2, 9, 4, 1), (4, 2, 32, 64, 4), (2, 1, 64, 32, 2), (2, 1, 16, 24, 4), (1, 1, 128, 128, 4),
               (6, 2, 48, 40, 5), (4, 4, 17, 300, 2), (2, 1, 256, 16, 4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", DELTA_CASES)
def test_delta_rule(dtype, case):
    ops = _ops()
    H, G, D, V, K = case
    for lengths, new in BATCHES + [([130, 64, 129, 5, 2], [130, 3, 129, 5, 1])]:
        batch = Batch(lengths, new, seed=1)
        proj, params, state = _delta_inputs(H, G, D, V, K, batch.n_tokens, len(lengths) + 2, dtype, seed=D + V)
        states = [state.clone(), state.clone()]
        got = _delta(ops.delta_rule, proj, params, states[0], batch, H, G, D, V, dtype)
        want = _delta(plain_ops.delta_rule, proj, params, states[1], batch, H, G, D, V, dtype)
        torch.cuda.synchronize()
        _close(got, want, dtype, (case, lengths, "out"))
        _close(states[0], states[1], torch.float32, (case, lengths, "state"))          # also the slots and columns that no one owns


def test_delta_rule_carries_its_state_across_any_cut():
    """A sequence in one step, and the same cut at every place into two steps (the second also token by
    token): the same results to the last bit in 32-bit, and the state that the cuts leave is the same."""
    ops = _ops()
    H, G, D, V, K, n = 4, 2, 12, 20, 4, 21
    proj, params, state = _delta_inputs(H, G, D, V, K, n, 3, torch.float32, seed=9)
    state.zero_()
    first_state = state.clone()
    want = _delta(ops.delta_rule, proj, params, first_state, Batch([n], [n]), H, G, D, V, torch.float32)
    for cut in range(1, n):
        held = state.clone()
        head = _delta(ops.delta_rule, proj[:cut], params, held, Batch([cut], [cut]), H, G, D, V, torch.float32)
        if cut % 2:
            tail = _delta(ops.delta_rule, proj[cut:], params, held, Batch([n], [n - cut]), H, G, D, V, torch.float32)
        else:
            tail = torch.cat([_delta(ops.delta_rule, proj[t:t + 1], params, held, Batch([t + 1], [1]), H, G, D, V, torch.float32)
                              for t in range(cut, n)])
        assert torch.equal(torch.cat([head, tail]), want), cut
        assert torch.equal(held, first_state), cut


def test_delta_rule_reads_back_a_value_stored_hundreds_of_tokens_ago():
    """Almost no decay, a step size of one: token 0 stores a value under a key of its own, the keys of the
    400 tokens between lie in other dimensions, and the last token asks with token 0's key: its result is
    token 0's value (up to the head's norm). With the state lost (zeroed) on the way it is not."""
    ops = _ops()
    H, G, D, V, K, n = 1, 1, 32, 8, 1, 402
    C = 2 * D + V
    big = 30.0
    proj = torch.zeros((n, (C + V + 2 + 7) // 8 * 8), device=DEV)
    gen = torch.Generator().manual_seed(2)
    proj[:, D + 1:2 * D] = torch.rand((n, D - 1), generator=gen).to(DEV) * big              # keys away from dimension 0
    proj[:, 1:D] = torch.rand((n, D - 1), generator=gen).to(DEV)
    proj[:, 2 * D:C] = torch.randn((n, V), generator=gen).to(DEV)
    proj[0, D:2 * D] = 0.0
    proj[0, D] = big                                                                        # token 0's key: dimension 0
    proj[0, 2 * D:C] = torch.tensor([4.0, -3.0, 2.0, 5.0, -1.0, 6.0, 3.0, -2.0])
    proj[n - 1, :D] = 0.0
    proj[n - 1, 0] = big                                                                    # the last query: dimension 0
    proj[n - 1, D:2 * D] = 0.0
    proj[n - 1, D + 5] = big
    proj[n - 1, 2 * D:C] = 0.0                                                              # and it writes nothing itself
    proj[:, C:C + V] = big                                                                  # silu(gate) = gate
    proj[:, C + V] = big                                                                    # beta = 1
    proj[:, C + V + 1] = 0.0
    params = dict(taps=torch.ones((C, 1), device=DEV), rate=torch.tensor([-1e-6], device=DEV), dt_bias=torch.zeros(1, device=DEV),
                  norm_weight=torch.ones(V, device=DEV))
    silu = lambda z: z / (1.0 + torch.exp(-z))
    stored = silu(proj[0, 2 * D:C])
    want = stored / torch.sqrt((stored * stored).mean()) * big
    state = torch.zeros((1, D * V), device=DEV)
    batch = Batch([n], [n])
    batch.slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = _delta(ops.delta_rule, proj, params, state, batch, H, G, D, V, torch.float32, eps=1e-12)[n - 1, 4:4 + V]
    assert torch.allclose(got, want, rtol=2e-3, atol=1e-2), (got, want)
    # the same in two steps with the state zeroed between them: the stored value is gone
    state.zero_()
    half = Batch([200], [200])
    half.slots = batch.slots
    _delta(ops.delta_rule, proj[:200], params, state, half, H, G, D, V, torch.float32, eps=1e-12)
    state.zero_()
    rest = Batch([n], [n - 200])
    rest.slots = batch.slots
    lost = _delta(ops.delta_rule, proj[200:], params, state, rest, H, G, D, V, torch.float32, eps=1e-12)[n - 201, 4:4 + V]
    assert float((lost - want).abs().max()) > 1.0


# ----------------------------------------------------------------------------- routed experts

def _experts(fn, h, router, bias, w_up, w_down, top):
    ops = _ops()
    n, hidden = h.shape
    E, a = router.shape[0], n * top
    ids = torch.zeros(a, dtype=torch.int32, device=DEV)
    weights = torch.zeros(a, device=DEV)
    order = torch.zeros(a, dtype=torch.int32, device=DEV)
    plan = torch.zeros(ops.routed_experts_plan_ints(n, top, E), dtype=torch.int32, device=DEV)
    act = torch.zeros((a, w_down.shape[2]), dtype=h.dtype, device=DEV)
    y = torch.zeros((a, hidden), device=DEV)
    gathered = torch.zeros((a, hidden), dtype=h.dtype, device=DEV)
    fn(h, router, bias, w_up, w_down, top, ids, weights, order, plan, act, y, gathered)
    return ids, weights, y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [(40, 12, 5, 3), (128, 64, 8, 2), (128, 96, 4, 1), (32, 16, 3, 3), (256, 128, 32, 4), (136, 40, 7, 7),
                                  (64, 200, 2, 1), (1024, 256, 16, 2)])
def test_routed_experts(dtype, case):
    ops = _ops()
    hidden, F, E, top = case
    gen = torch.Generator().manual_seed(hidden + E)
    router = (3.0 * torch.randn((E, hidden), generator=gen) / hidden ** 0.5).to(DEV)
    bias = (0.7 * torch.randn(E, generator=gen)).to(DEV)
    w_up = (torch.randn((E, 2 * F, hidden), generator=gen) / hidden ** 0.5).to(dtype).to(DEV)
    w_down = (torch.randn((E, hidden, F), generator=gen) / F ** 0.5).to(dtype).to(DEV)
    for n in (1, 2, 33, 70, 300, 1000):                      # the larger steps of bfloat16 take the tiles of 128 rows
        wide = torch.randn((n, hidden + 8), generator=gen).to(dtype).to(DEV)
        h = wide[:, :hidden]
        if dtype == torch.bfloat16 and hidden % 8 == 0 and F % 8 == 0:
            assert ops.routed_experts_wide(n, top, E, hidden, F, dtype) == (n * top >= 32 * E)
        for b in (bias, None):
            ids, weights, y = _experts(ops.routed_experts, h, router, b, w_up, w_down, top)
            want_ids, want_weights, want_y = _experts(plain_ops.routed_experts, h, router, b, w_up, w_down, top)
            torch.cuda.synchronize()
            assert torch.equal(ids, want_ids), (case, n)
            _close(weights, want_weights, torch.float32, (case, n, "weights"))
            _close(y, want_y, dtype, (case, n, "rows"))
            assert torch.allclose(weights.view(n, top).sum(-1), torch.ones(n, device=DEV), atol=1e-5)


def test_routed_experts_on_wide_tiles_agree_with_narrow_ones():
    """The same step through the tiles of 128 rows and, with those switched off, through the tiles of 32: equal up
    to the order of the sums; experts with no row, one row, and more rows than a tile holds."""
    ops = _ops()
    from llm_b200.ops import tactics
    hidden, F, E, top, n = 192, 72, 6, 2, 700
    gen = torch.Generator().manual_seed(3)
    router = (3.0 * torch.randn((E, hidden), generator=gen) / hidden ** 0.5).to(DEV)
    bias = torch.tensor([2.0, 2.0, 0.0, -9.0, -60.0, 1.0], device=DEV)         # expert 4 is never chosen, expert 3 rarely
    w_up = (torch.randn((E, 2 * F, hidden), generator=gen) / hidden ** 0.5).bfloat16().to(DEV)
    w_down = (torch.randn((E, hidden, F), generator=gen) / F ** 0.5).bfloat16().to(DEV)
    h = torch.randn((n, hidden), generator=gen).bfloat16().to(DEV)
    assert ops.routed_experts_wide(n, top, E, hidden, F, torch.bfloat16)
    ids, weights, y = _experts(ops.routed_experts, h, router, bias, w_up, w_down, top)
    counts = torch.bincount(ids.long(), minlength=E).tolist()
    assert counts[4] == 0 and max(counts) > 256 and 0 < counts[3] < 128, counts
    tactics.disable("routed_experts_wide")
    try:
        assert not ops.routed_experts_wide(n, top, E, hidden, F, torch.bfloat16)
        ids_narrow, weights_narrow, y_narrow = _experts(ops.routed_experts, h, router, bias, w_up, w_down, top)
    finally:
        tactics.enable("routed_experts_wide")
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(ids, ids_narrow) and torch.equal(weights, weights_narrow)
    _close(y, y_narrow, torch.bfloat16, "rows")
    assert float((y - y_narrow).abs().max()) <= 2e-2 * float(y_narrow.abs().max())


def test_routed_experts_on_tiles_of_256_columns():
    """Long lists (1,024 rows an expert and more) take tiles of 256 accumulator columns: the same step with those switched
    off, and with all tcgen05 tiles switched off; sizes that are no multiple of any tile."""
    ops = _ops()
    from llm_b200.ops import tactics
    hidden, F, E, top, n = 328, 136, 2, 1, 2300
    gen = torch.Generator().manual_seed(5)
    router = (3.0 * torch.randn((E, hidden), generator=gen) / hidden ** 0.5).to(DEV)
    w_up = (torch.randn((E, 2 * F, hidden), generator=gen) / hidden ** 0.5).bfloat16().to(DEV)
    w_down = (torch.randn((E, hidden, F), generator=gen) / F ** 0.5).bfloat16().to(DEV)
    h = torch.randn((n, hidden), generator=gen).bfloat16().to(DEV)
    ids, weights, y = _experts(ops.routed_experts, h, router, None, w_up, w_down, top)
    results = []
    for name in ("routed_experts_wide256", "routed_experts_wide"):
        tactics.disable(name)
        try:
            results.append(_experts(ops.routed_experts, h, router, None, w_up, w_down, top))
        finally:
            tactics.enable(name)
    torch.cuda.synchronize()
    ops.check_device_status()
    for other_ids, other_weights, other_y in results:
        assert torch.equal(ids, other_ids) and torch.equal(weights, other_weights)
        _close(y, other_y, torch.bfloat16, "rows")
        assert float((y - other_y).abs().max()) <= 2e-2 * float(other_y.abs().max())
    want = _experts(plain_ops.routed_experts, h[:64].contiguous(), router, None, w_up, w_down, top)[2]
    _close(y[:64], want, torch.bfloat16, "rows against the plain statement")


def test_routed_experts_choice_ties_and_batch_independence():
    """The bias alone decides when the router's matrix is zero; equal logits go to the lower index; a
    token's rows do not depend on what else is in the step (bit for bit in 32-bit)."""
    ops = _ops()
    hidden, F, E, top = 48, 24, 6, 2
    gen = torch.Generator().manual_seed(1)
    w_up = torch.randn((E, 2 * F, hidden), generator=gen).to(DEV) / hidden ** 0.5
    w_down = torch.randn((E, hidden, F), generator=gen).to(DEV) / F ** 0.5
    h = torch.randn((50, hidden), generator=gen).to(DEV)
    zero = torch.zeros((E, hidden), device=DEV)
    bias = torch.tensor([0.0, 2.0, -1.0, 3.0, 2.0, -5.0], device=DEV)
    ids, weights, y = _experts(ops.routed_experts, h, zero, bias, w_up, w_down, top)
    assert ids.view(50, top).tolist() == [[3, 1]] * 50                              # 3.0 first, then the lower of the two 2.0
    share = math.exp(3.0) / (math.exp(3.0) + math.exp(2.0))
    assert torch.allclose(weights.view(50, top), torch.tensor([share, 1.0 - share], device=DEV).expand(50, top), atol=1e-6)
    x = h[7].double().cpu()
    gate_up = w_up[3].double().cpu() @ x
    expert = w_down[3].double().cpu() @ (gate_up[:F] / (1.0 + torch.exp(-gate_up[:F])) * gate_up[F:])
    assert torch.allclose(y[7 * top].double().cpu(), share * expert, atol=1e-5)
    router = torch.randn((E, hidden), generator=gen).to(DEV)
    _, _, all_rows = _experts(ops.routed_experts, h, router, bias, w_up, w_down, top)
    for rows in ([7], [49, 3, 7, 20]):
        _, _, some = _experts(ops.routed_experts, h[rows].contiguous(), router, bias, w_up, w_down, top)
        for i, r in enumerate(rows):
            assert torch.equal(some[i * top:(i + 1) * top], all_rows[r * top:(r + 1) * top]), (rows, r)


# ----------------------------------------------------------------------------- the model through the engine

def _setup(tmp_path, which, dtype, change=None, weights_change=None, **engine_options):
    from llm_b200.engine import Engine, load_model
    folder = make_folder(tmp_path, which, torch.bfloat16, change, weights_change)
    config, weights = plain.read_model(folder)
    engine = Engine(load_model(folder, dtype, DEV), **{"max_tokens": 4096, **engine_options})
    return config, weights, engine


def _check_logits(got, want, dtype, what="", sure=None):
    """32-bit: element by element. bfloat16: against the span of the logits; a row at which the plain
    model chose its experts by less than a rounding's reach (`sure` False) is not looked at."""
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=4e-4, rtol=1e-4), (what, float((got - want).abs().max()))
        return
    if got.dim() == 1:
        got, want = got[None], want[None]
        sure = None if sure is None else torch.as_tensor(sure).reshape(1)
    if sure is not None:
        got, want = got[sure], want[sure]
    if got.numel() == 0:
        return
    span = float(want.max() - want.min())
    assert float((got - want).abs().max()) <= 0.06 * span, (what, float((got - want).abs().max()), span)
    assert float((got - want).abs().mean()) <= 0.012 * span, what


def _sure(config, weights, tokens, dtype):
    """Per position: True where every routed layer's choice has a margin that bfloat16 rounding does not reach."""
    if dtype == torch.float32:
        return torch.ones(len(tokens), dtype=torch.bool)
    return plain.closest_call(config, weights, tokens) > 0.15


def test_every_layer_agrees_with_plain(tmp_path):
    """The residual stream after each layer in 32-bit (a model of the first k layers, for every k, whose
    last norm is made the identity up to the row's scale, and its last layer also without feed-forward)."""
    from llm_b200.engine import Entry
    for which in sorted(CONFIGS):
        depth = len(CONFIGS[which][0]["layers"])
        for k in range(1, depth + 1):
            for mixer_only in (True, False):
                def cut(config, k=k, mixer_only=mixer_only):
                    config["layers"] = config["layers"][:k]
                    if mixer_only:
                        config["layers"][-1]["mlp"] = None
                def plain_final(weights):
                    weights["final.norm"].fill_(0.0)
                config, weights, engine = _setup(tmp_path / f"{which}{k}{mixer_only}", which, torch.float32, cut, plain_final)
                tokens = random_tokens(90, config["vocab"], k)
                want = plain.forward(config, weights, tokens)
                (slot,) = engine.acquire()
                got = engine.step([Entry(slot, tokens, list(range(90)))])
                _check_logits(got, want, torch.float32, (which, k, mixer_only))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["P", "Q", "R"])
def test_whole_decode_pieces_and_batches_agree_with_plain(tmp_path, which, dtype):
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, which, dtype, step_tokens=48)
    lengths = [150, 1, 67, 20]
    seqs = [random_tokens(n, config["vocab"], 30 + n) for n in lengths]
    expected = [plain.forward(config, weights, s) for s in seqs]
    sure = [_sure(config, weights, s, dtype) for s in seqs]
    for again in range(2):                                       # the second time reuses slots, pages and states
        slots = engine.acquire(len(seqs))
        heads = [max(1, n - 9 - 2 * i) for i, n in enumerate(lengths)]          # unequal prompts, cut into passes of 48
        logits = engine.step([Entry(s, q[:h], list(range(h))) for s, q, h in zip(slots, seqs, heads)])
        row = 0
        for b, h in enumerate(heads):
            _check_logits(logits[row:row + h], expected[b][:h], dtype, ("prompt", b), sure[b][:h])
            row += h
        live = [b for b in range(len(seqs)) if heads[b] < lengths[b]]
        engine.release([slots[b] for b in range(len(seqs)) if b not in live])
        done = 0
        while live:                                              # decoding together; shorter sequences end earlier
            logits = engine.step([Entry(slots[b], [seqs[b][heads[b] + done]], [0]) for b in live])
            for r, b in enumerate(live):
                at = heads[b] + done
                _check_logits(logits[r], expected[b][at], dtype, ("decode", b, done), sure[b][at])
            done += 1
            ended = [b for b in live if heads[b] + done == lengths[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_passes_the_windows_and_page_edges(tmp_path, dtype):
    """One token a step from the first on, 300 steps: windows of 40, 100 and 130 slide over decoded tokens,
    pages fill and follow each other, the delta rule's state is carried 300 times, and steps are replayed
    from graphs."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", dtype)
    tokens = random_tokens(300, config["vocab"], 77)
    expected = plain.forward(config, weights, tokens)
    sure = _sure(config, weights, tokens, dtype)
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):
        logits = engine.step([Entry(slot, [token], [0])])
        _check_logits(logits[0], expected[p], dtype, p, sure[p])
    assert engine.graph_replays > 200
    assert int(sure.sum()) > 150


@pytest.mark.parametrize("piece", [2, 5, 64])
def test_pieces_down_to_two_tokens(tmp_path, piece):
    from llm_b200.engine import Entry
    for which in ("P", "Q"):
        config, weights, engine = _setup(tmp_path, which, torch.float32)
        tokens = random_tokens(140, config["vocab"], 8)
        expected = plain.forward(config, weights, tokens)
        (slot,) = engine.acquire()
        for start in range(0, len(tokens), piece):
            part = tokens[start:start + piece]
            logits = engine.step([Entry(slot, part, list(range(len(part))))])
            _check_logits(logits, expected[start:start + len(part)], torch.float32, (which, start))


def test_batch_and_cut_change_nothing_in_32_bit(tmp_path):
    """A position's logits alone, among neighbours, and with its prompt cut: equal to the last bit in the
    32-bit path (every reduction's order depends only on the position; states are carried exactly; an
    expert's rows do not depend on the tile they fall into)."""
    from llm_b200.engine import Entry
    for which in ("P", "Q"):
        config, weights, engine = _setup(tmp_path, which, torch.float32)
        seqs = [random_tokens(n, config["vocab"], 60 + n) for n in (50, 13, 31)]
        a, b, c, d = engine.acquire(4)
        alone = engine.step([Entry(a, seqs[0], [49, 20])]).clone()
        together = engine.step([Entry(b, seqs[1], [12]), Entry(c, seqs[0], [49, 20]), Entry(d, seqs[2], [])])
        assert torch.equal(alone, together[1:3]), which
        engine.release([a])
        (e,) = engine.acquire()
        engine.step([Entry(e, seqs[0][:17], [])])
        engine.step([Entry(e, seqs[0][17:21], [])])
        for t in range(21, 30):
            engine.step([Entry(e, [seqs[0][t]], [])])
        cut = engine.step([Entry(e, seqs[0][30:], [49 - 30])])
        assert torch.equal(alone[0], cut[0]), which


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_passes_walked_from_their_record_agree_with_plain_passes(tmp_path, dtype):
    """The same shape of step five times on other slots, pages and states: the first pass runs through the parts,
    the second is recorded, the later ones are walked natively from the record; a mixed step likewise."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", dtype)
    for again in range(5):
        seqs = [random_tokens(n, config["vocab"], 100 * again + n) for n in (90, 33)]
        sure = [_sure(config, weights, s, dtype) for s in seqs]
        slots = engine.acquire(2)
        logits = engine.step([Entry(slots[0], seqs[0][:80], [0, 79]), Entry(slots[1], seqs[1][:30], [29])])
        want = [plain.forward(config, weights, s) for s in seqs]
        _check_logits(logits, torch.stack([want[0][0], want[0][79], want[1][29]]), dtype, ("prompt", again),
                      torch.stack([sure[0][0], sure[0][79], sure[1][29]]))
        mixed = engine.step([Entry(slots[0], seqs[0][80:], [9]), Entry(slots[1], [seqs[1][30]], [0])])
        _check_logits(mixed, torch.stack([want[0][89], want[1][30]]), dtype, ("mixed", again), torch.stack([sure[0][89], sure[1][30]]))
        engine.release(slots)
    assert engine.records_run >= 4


def test_what_a_fault_would_change_shows_in_the_logits(tmp_path):
    """Changes that a fault would make, made on purpose in the plain model: each must move the logits by far
    more than the library differs from the unchanged plain model."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", torch.float32)
    tokens = random_tokens(200, config["vocab"], 5)
    want = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(200)))]).cpu()
    error = float((got - want).abs().max())
    changes = ("window wider", "window narrower", "decay", "taps", "step size", "bands", "rotated part", "gate", "router bias",
               "post norm", "nothing")
    for change in changes:
        other, w = json.loads(json.dumps(config)), dict(weights)
        if change == "window wider":
            other["layers"][1]["mixer"]["mask"]["size"] += 1
        elif change == "window narrower":
            other["layers"][2]["mixer"]["mask"]["size"] -= 1
        elif change == "decay":
            w["l0.mix.A_log"] = weights["l0.mix.A_log"] + 1.0                 # a state that fades faster
        elif change == "taps":
            w["l3.mix.k.conv"] = weights["l3.mix.k.conv"].flip(1)             # the taps in the other order
        elif change == "step size":
            w["l0.mix.b"] = weights["l0.mix.b"] * 0.0                          # beta = 1/2 everywhere
        elif change == "bands":
            del other["layers"][1]["mixer"]["rot"]["scaling"]
        elif change == "rotated part":
            other["layers"][4]["mixer"]["rot"]["dims"] = 32
        elif change == "gate":
            w["l2.mix.g"] = weights["l2.mix.g"] * 0.0
        elif change == "router bias":
            w["l0.mlp.router.b"] = weights["l0.mlp.router.b"] * 0.0
        elif change == "post norm":
            w["l1.norm1b"] = weights["l1.norm1b"] * 0.0
        else:
            other["layers"][3]["mixer"]["dim"] = 64                             # as it was: the control
        moved = float((plain.forward(other, w, tokens) - want).abs().max())
        if change == "nothing":
            assert moved == 0.0
        else:
            assert moved > 50 * error, (change, moved, error)


def test_greedy_generation_through_the_entry_point(tmp_path):
    import llm_b200
    folder = make_folder(tmp_path, "Q", torch.bfloat16)
    config, weights = plain.read_model(folder)
    prompts = [random_tokens(n, config["vocab"], 90 + n) for n in (5, 70, 23)]
    llm = llm_b200.LLM(str(folder), dtype="float32", device=DEV, context=256, batch=3)
    got = llm.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[], repeat_penalty=1.0)
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain.greedy(config, weights, prompt, 8)
    llm16 = llm_b200.LLM(str(folder), dtype="bfloat16", device=DEV, context=256, batch=3)
    for prompt, tokens in zip(prompts, llm16.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[],
                                                      repeat_penalty=1.0)):
        sequence = list(prompt)
        for token in tokens:                                    # every token is a maximum of the plain logits up to rounding
            if not bool(_sure(config, weights, sequence, torch.bfloat16).all()):
                break                                           # an expert chosen by a hair: the plain model may go another way
            logits = plain.forward(config, weights, sequence)[-1]
            assert logits[token] >= logits.max() - 0.06 * float(logits.max() - logits.min())
            sequence.append(token)


def test_trace_replay_program(tmp_path):
    folder = make_folder(tmp_path, "P", torch.bfloat16)
    config, weights = plain.read_model(folder)
    a, b = random_tokens(40, config["vocab"], 1), random_tokens(9, config["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a"]}]
    program = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    result = subprocess.run([sys.executable, str(program), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                             "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    assert [line for line in result.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    read = lambda n: torch.frombuffer(bytearray((out / f"{n}.f32").read_bytes()), dtype=torch.float32).view(-1, config["vocab"])
    wa, wb = plain.forward(config, weights, a), plain.forward(config, weights, b)
    _check_logits(read(0), wa[[0, 29]], torch.float32)
    _check_logits(read(1), torch.stack([wa[30], wb[8]]), torch.float32)
    _check_logits(read(2), wa[39:40], torch.float32)
