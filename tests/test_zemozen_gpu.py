"""Zemozen on the GPU: every new kernel and kernel option beside its plain statement (also with weights and
inputs made so that one key, a window's edge, the one in the softmax's denominator, a blended value or a
lost state shows), and the model through the engine, the generation entry point and the trace-replay
program against the plain whole-sequence implementation, in 32-bit and in bfloat16."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_ops
import plain_zemozen as plain
from test_mefolorn_gpu import BATCHES, Batch, _close, only_generic
from tiny_zemozen import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

PAGE = 64
DEV = "cuda:0"


def _ops():
    from llm_b200 import ops
    return ops


# ----------------------------------------------------------------------------- head norms, rotation, blended values

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # query heads, key heads, head size, value size, rotated, interleaved, blended, columns behind
    (4, 2, 6, 10, 4, True, False, 0), (2, 2, 8, 6, 8, False, True, 5), (4, 1, 64, 64, 32, False, True, 8),
    (8, 2, 32, 32, 32, True, False, 4), (2, 1, 128, 64, 16, False, True, 0), (3, 3, 5, 5, 2, False, False, 1),
    (2, 2, 128, 128, 128, True, True, 0), (4, 4, 96, 40, 0, False, True, 0), (1, 1, 48, 48, 48, False, True, 3)])
def test_head_norms_rotation_and_blended_values(dtype, case):
    ops = _ops()
    heads, groups, dim, vdim, n_rot, interleaved, blended, behind = case
    qw, kw, vw = heads * dim, groups * dim, groups * vdim
    gen = torch.Generator().manual_seed(dim + vdim)
    for lengths, new in BATCHES:
        batch = Batch(lengths, new, seed=len(lengths))
        other = Batch(lengths, new, seed=len(lengths) + 7, slack_pages=5)       # the first layer's pages: another table
        wide = torch.randn((batch.n_tokens, qw + kw + vw + behind), generator=gen).to(dtype).to(DEV)
        q_gain = (1.0 + 0.3 * torch.randn(dim, generator=gen)).to(DEV)
        k_gain = (1.0 + 0.3 * torch.randn(dim, generator=gen)).to(DEV)
        table = None
        if n_rot:
            angle = torch.arange(400, dtype=torch.float64)[:, None] * torch.rand(n_rot // 2, generator=gen, dtype=torch.float64)
            table = torch.cat([angle.cos(), angle.sin()], dim=1).float().to(DEV)
        _, first_values = other.caches(groups, dim, vdim, dtype, seed=9)
        blend = dict(mix_cache=first_values, mix_table=other.table, mix_ring=other.width, mix=0.37) if blended else {}
        results = []
        for fn in (ops.norm_rope_cache_write, plain_ops.norm_rope_cache_write):
            k_cache, v_cache = batch.caches(groups, dim, vdim, dtype, seed=5)
            q_wide = torch.zeros((batch.n_tokens, qw + 8), dtype=dtype, device=DEV)
            fn(wide, qw, kw, vw, q_gain, k_gain, 1e-3, table, dim, interleaved, batch.tok_pos, batch.tok_seq,
               q_wide[:, :qw], batch.table, batch.width, k_cache, v_cache, norm_unit=dim, **blend)
            results.append((q_wide, k_cache, v_cache))
        torch.cuda.synchronize()
        for got, want, what in zip(results[0], results[1], ("queries", "keys", "values")):
            _close(got, want, dtype, (case, lengths, what))
        assert float(results[0][0][:, qw:].abs().max()) == 0.0           # nothing written beside the queries
        # a head's norm is its own: scaling one head's columns of the input changes no other head's queries
        scaled = wide.clone()
        scaled[:, dim:2 * dim] *= 3.0
        k_cache, v_cache = batch.caches(groups, dim, vdim, dtype, seed=5)
        q_again = torch.zeros((batch.n_tokens, qw), dtype=dtype, device=DEV)
        ops.norm_rope_cache_write(scaled, qw, kw, vw, q_gain, k_gain, 1e-3, table, dim, interleaved, batch.tok_pos,
                                  batch.tok_seq, q_again, batch.table, batch.width, k_cache, v_cache, norm_unit=dim, **blend)
        assert torch.equal(q_again[:, :dim], results[0][0][:, :dim])
        if heads > 1:
            # (the scaled head itself norms to nearly the same: eps is all that keeps it from equal)
            assert torch.allclose(q_again[:, dim:2 * dim].float(), results[0][0][:, dim:2 * dim].float(), atol=3e-2, rtol=3e-2)
        if blended:                                                      # the cached value is the blend, not the projection
            row = batch.n_tokens - 1
            b, p = int(batch.tok_seq[row]), int(batch.tok_pos[row])
            page, at = batch.place(b, p)
            first_page, first_at = other.place(b, p)
            want = 0.63 * wide[row, qw + kw:qw + kw + vw].float() + 0.37 * first_values[first_page, :, first_at].reshape(-1).float()
            _close(results[0][2][page, :, at].reshape(-1), want, dtype, (case, "blend"))


# ----------------------------------------------------------------------------- attention: soft cap, the one in the denominator, head gate, value size

def _attention(fn, batch, heads, groups, dim, vdim, dtype, window, cap, unit, gated, out_scale=1.0, seed=2, q=None, caches=None,
               q_std=1.0):
    gen = torch.Generator().manual_seed(seed)
    if q is None:
        q = (q_std * torch.randn((batch.n_tokens, heads * dim), generator=gen)).to(dtype).to(DEV)
    k_cache, v_cache = caches if caches is not None else batch.caches(groups, dim, vdim, dtype, seed=seed + 1)
    gate_wide = torch.randn((batch.n_tokens, heads + 3), generator=gen).to(dtype).to(DEV)
    sinks = torch.zeros(heads, device=DEV) if unit else None
    out_wide = torch.zeros((batch.n_tokens, heads * vdim + 16), dtype=dtype, device=DEV)
    fn(q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, groups, dim, dim ** -0.5,
       window, out=out_wide[:, 8:8 + heads * vdim], sinks=sinks, gate=gate_wide[:, 2:2 + heads] if gated else None,
       out_scale=out_scale, softcap=cap, value_dim=vdim, **batch.extra())
    return out_wide


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # heads, kv heads, head size, value size, window, soft cap, one in the denominator, head gate
    (8, 2, 96, 64, 80, 25.0, True, False), (6, 2, 48, 48, 50, 0.0, False, True), (4, 2, 6, 10, 9, 1.5, True, False),
    (8, 2, 32, 32, 130, 4.0, True, False), (2, 2, 128, 128, 70, 2.0, True, False), (4, 4, 96, 96, 0, 30.0, True, False),
    (4, 1, 64, 64, 40, 0.0, False, True), (2, 1, 128, 64, 100, 0.0, False, True), (16, 2, 64, 64, 1000, 0.7, True, True),
    (3, 3, 5, 300, 21, 3.0, False, True), (2, 1, 16, 24, 0, 0.0, True, False), (24, 2, 128, 128, 63, 5.0, True, False),
    (2, 1, 300, 8, 64, 9.0, True, True)])
def test_attention_with_soft_cap_unit_sink_head_gate_and_value_size(dtype, case, generic):
    ops = _ops()
    heads, groups, dim, vdim, window, cap, unit, gated = case
    if generic and dtype == torch.float32:
        pytest.skip("the 32-bit path is the generic kernel already")
    dtype_ = torch.bfloat16 if generic else dtype
    for lengths, new in BATCHES + [([700, 64, 129], [700, 3, 129]), ([1500, 1, 64, 65, 700], [1] * 5)]:
        batch = Batch(lengths, new, seed=3 + len(lengths))
        with only_generic(generic):
            got = _attention(ops.attention, batch, heads, groups, dim, vdim, dtype_, window, cap, unit, gated, 0.8, q_std=3.0)
        want = _attention(plain_ops.attention, batch, heads, groups, dim, vdim, dtype_, window, cap, unit, gated, 0.8, q_std=3.0)
        torch.cuda.synchronize()
        _close(got, want, dtype_, (case, lengths))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "generic"])
@pytest.mark.parametrize("decode", [False, True])
def test_attention_planted_keys_at_the_window_s_edges_under_a_soft_cap(dtype, decode):
    """One key stands out (its capped score is near the cap, far above the others): the result is that key's
    value times e^c / (1 + e^c + ..) exactly when the key is inside the window: far back, at page borders, at both
    edges of the window, in a prompt's portion and in decoding."""
    ops = _ops()
    generic = dtype == "generic"
    dtype = torch.bfloat16 if generic else dtype
    heads, dim, window, length, cap = 2, 64, 100, 331, 12.0
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
        q[last, :4] = torch.tensor([3.0, -2.0, 1.0, 2.0]) * 8.0          # score 18 before the cap, 12 tanh(1.5) = 10.9 behind it
        args = (q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, 1, dim, 1.0 / 8.0, window)
        extra = dict(sinks=torch.zeros(heads, device=DEV), softcap=cap, **batch.extra())
        with only_generic(generic):
            got = ops.attention(*args, **extra)
        want = plain_ops.attention(*args, **extra)
        torch.cuda.synchronize()
        seen = length - 1 - planted < window
        if seen:
            assert abs(float(got[last, 0]) - 5.0) < 0.1 and abs(float(got[last, 1]) + 7.0) < 0.1, (planted, got[last, :2])
        else:
            assert float(got[last, :2].float().abs().max()) < 0.5, (planted, got[last, :2])
        _close(got, want, dtype, (planted, decode, generic))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "generic"])
def test_the_one_in_the_denominator_and_the_cap_show(dtype):
    """Queries of zero: every score is 0, so with n visible keys every weight is 1 / (n + 1), not 1 / n; the first
    token's result is half its value. And a score far above the cap weighs e^cap, not e^score."""
    ops = _ops()
    generic = dtype == "generic"
    dtype = torch.bfloat16 if generic else dtype
    heads, dim, window = 4, 64, 10
    for lengths, new in (([25, 1, 3], [25, 1, 3]), ([25, 1, 3], [1, 1, 1])):
        batch = Batch(lengths, new, seed=2)
        k_cache, v_cache = batch.caches(1, dim, dim, dtype, seed=3)
        v_cache[:] = 1.0
        q = torch.zeros((batch.n_tokens, heads * dim), dtype=dtype, device=DEV)
        with only_generic(generic):
            got = ops.attention(q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, 1, dim,
                                0.125, window, sinks=torch.zeros(heads, device=DEV), softcap=5.0, **batch.extra())
        torch.cuda.synchronize()
        for t in range(batch.n_tokens):
            n = min(int(batch.tok_pos[t]) + 1, window)
            assert torch.allclose(got[t].float(), torch.full((heads * dim,), n / (n + 1.0), device=DEV), atol=8e-3), (t, n)
    # two keys: one with a raw score of 40 (capped to 5 tanh(8) = 5), one with 0: weights e^5 and 1 beside the one
    batch = Batch([2], [2], seed=1)
    k_cache, v_cache = batch.caches(1, dim, dim, dtype, seed=3)
    k_cache.zero_()
    v_cache.zero_()
    page, row = batch.place(0, 0)
    k_cache[page, 0, row, 0] = 4.0
    v_cache[page, 0, row, 0] = 1.0
    q = torch.zeros((2, heads * dim), dtype=dtype, device=DEV)
    q[1, 0] = 10.0
    with only_generic(generic):
        got = ops.attention(q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, 1, dim, 1.0, 0,
                            sinks=torch.zeros(heads, device=DEV), softcap=5.0, **batch.extra())
    capped = math.exp(5.0 * math.tanh(8.0))
    assert abs(float(got[1, 0]) - capped / (capped + 2.0)) < 4e-3


# ----------------------------------------------------------------------------- the state-space recurrence

def _ssm_inputs(H, G, N, V, K, n_tokens, n_slots, dtype, seed, memory="mixed"):
    gen = torch.Generator().manual_seed(seed)
    inner = H * V
    C = inner + 2 * G * N
    width = (inner + C + H + 7) // 8 * 8 + 8
    proj = torch.randn((n_tokens, width), generator=gen).to(dtype).to(DEV)
    a_log = torch.randn(H, generator=gen) - (1.0 if memory == "mixed" else 9.0)
    params = dict(taps=torch.randn((C, K), generator=gen) / K ** 0.5, conv_bias=0.3 * torch.randn(C, generator=gen),
                  rate=-torch.exp(a_log), dt_bias=torch.randn(H, generator=gen), skip=torch.randn(H, generator=gen),
                  norm_weight=1.0 + 0.3 * torch.randn(inner, generator=gen))
    state = (0.3 * torch.randn((n_slots, (K - 1) * C + H * N * V + 3), generator=gen)).to(DEV)
    return proj, {k: v.to(DEV).contiguous() for k, v in params.items()}, state


def _ssm(fn, proj, params, state, batch, H, G, N, V, dtype, parts=1, eps=1e-5, out_scale=1.0):
    ops = _ops()
    n = batch.n_tokens
    work = torch.zeros((n, ops.state_space_work_width(H, G, N, V)), device=DEV)
    y = torch.zeros((n, H * V), device=DEV)
    mixed_wide = torch.zeros((n, H * V + 9), dtype=dtype, device=DEV)
    fn(proj, params["taps"], params["conv_bias"], state, batch.tok_seq, batch.cu, batch.slots, params["rate"], params["dt_bias"],
       params["skip"], params["norm_weight"], eps, parts, out_scale, work, y, mixed_wide[:, 4:4 + H * V], H, G, N, V)
    return mixed_wide


# heads, groups, state, value size, taps, norm parts
SSM_CASES = [(3, 1, 7, 5, 2, 3), (4, 2, 48, 40, 3, 2), (4, 2, 64, 32, 4, 1), (2, 2, 128, 64, 3, 2), (8, 1, 40, 16, 1, 4),
             (2, 2, 20, 12, 4, 1), (1, 1, 256, 7, 2, 1), (6, 3, 33, 18, 5, 9), (2, 1, 130, 130, 2, 4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", SSM_CASES)
def test_state_space(dtype, case):
    ops = _ops()
    H, G, N, V, K, parts = case
    for lengths, new in BATCHES + [([130, 64, 129, 5, 2], [130, 3, 129, 5, 1])]:
        batch = Batch(lengths, new, seed=1)
        proj, params, state = _ssm_inputs(H, G, N, V, K, batch.n_tokens, len(lengths) + 2, dtype, seed=N + V)
        states = [state.clone(), state.clone()]
        got = _ssm(ops.state_space, proj, params, states[0], batch, H, G, N, V, dtype, parts, out_scale=0.7)
        want = _ssm(plain_ops.state_space, proj, params, states[1], batch, H, G, N, V, dtype, parts, out_scale=0.7)
        torch.cuda.synchronize()
        _close(got, want, dtype, (case, lengths, "out"))
        _close(states[0], states[1], torch.float32, (case, lengths, "state"))          # also the slots and columns that no one owns


def test_state_space_carries_its_state_across_any_cut():
    """A sequence in one step, and the same cut at every place into two steps (the second also token by
    token): the same results to the last bit in 32-bit, and the state that the cuts leave is the same."""
    ops = _ops()
    H, G, N, V, K, n = 4, 2, 12, 10, 4, 21
    proj, params, state = _ssm_inputs(H, G, N, V, K, n, 3, torch.float32, seed=9)
    state.zero_()
    first_state = state.clone()
    want = _ssm(ops.state_space, proj, params, first_state, Batch([n], [n]), H, G, N, V, torch.float32, 2)
    for cut in range(1, n):
        held = state.clone()
        head = _ssm(ops.state_space, proj[:cut], params, held, Batch([cut], [cut]), H, G, N, V, torch.float32, 2)
        if cut % 2:
            tail = _ssm(ops.state_space, proj[cut:], params, held, Batch([n], [n - cut]), H, G, N, V, torch.float32, 2)
        else:
            tail = torch.cat([_ssm(ops.state_space, proj[t:t + 1], params, held, Batch([t + 1], [1]), H, G, N, V, torch.float32, 2)
                              for t in range(cut, n)])
        assert torch.equal(torch.cat([head, tail]), want), cut
        assert torch.equal(held, first_state), cut


def test_state_space_reads_back_what_it_stored_hundreds_of_tokens_ago():
    """Almost no decay: token 0 writes x under a B of its own (state row 0), the 400 tokens between write under
    other rows, and the last token reads row 0 only: it gets token 0's x back. With the state lost on the way it
    does not."""
    ops = _ops()
    H, G, N, V, K, n = 1, 1, 32, 8, 1, 402
    inner, big = V, 30.0
    C = inner + 2 * N
    gen = torch.Generator().manual_seed(2)
    proj = torch.zeros((n, (inner + C + H + 7) // 8 * 8), device=DEV)
    proj[:, :inner] = big                                                                   # z: silu(z) = z, the gate is a constant
    proj[:, inner:2 * inner] = torch.randn((n, V), generator=gen).to(DEV) * 3.0             # x
    proj[:, 2 * inner + 1:2 * inner + N] = torch.rand((n, N - 1), generator=gen).to(DEV) * 3.0   # B away from row 0
    proj[:, 2 * inner + N + 1:2 * inner + 2 * N] = torch.rand((n, N - 1), generator=gen).to(DEV)  # C likewise
    proj[0, 2 * inner:2 * inner + N] = 0.0
    proj[0, 2 * inner] = big                                                                 # token 0 writes under row 0
    proj[-1, 2 * inner + N:2 * inner + 2 * N] = 0.0
    proj[-1, 2 * inner + N] = big                                                            # the last token reads row 0
    proj[-1, 2 * inner:2 * inner + N] = -big                                                 # and writes nothing (silu = 0)
    proj[:, inner + C] = 0.0                                                                 # dt = softplus(0) = ln 2
    params = dict(taps=torch.ones((C, 1), device=DEV), conv_bias=None, rate=torch.tensor([-1e-6], device=DEV),
                  dt_bias=torch.zeros(1, device=DEV), skip=None, norm_weight=torch.ones(inner, device=DEV))
    silu = lambda t: t / (1.0 + torch.exp(-t))
    stored = silu(proj[0, inner:2 * inner])

    def run(lose_at=None):
        state = torch.zeros((2, H * N * V), device=DEV)
        outs = []
        for lo, hi in ((0, 150), (150, 151), (151, 300), (300, n)):
            if lose_at == lo:
                state.zero_()
            outs.append(_ssm(ops.state_space, proj[lo:hi], params, state, Batch([hi], [hi - lo]), H, G, N, V, torch.float32,
                             eps=1e-12)[:, 4:4 + inner])
        return torch.cat(outs)[-1]

    got = run()
    want = stored / torch.sqrt((stored * stored).mean())            # the norm takes every constant factor away
    assert torch.allclose(got, want, atol=2e-3), (got, want)
    lost = run(lose_at=300)
    assert float((lost - want).abs().max()) > 0.3


# ----------------------------------------------------------------------------- routed experts scored over all outputs

def _experts(fn, h, router, correction, w_up, w_down, top, pass_through, scale=0.7):
    ops = _ops()
    n, hidden = h.shape
    E, F = w_up.shape[0], w_up.shape[1] // 2
    a = n * top
    ids = torch.zeros(a, dtype=torch.int32, device=DEV)
    weights = torch.zeros(a, device=DEV)
    order = torch.zeros(a, dtype=torch.int32, device=DEV)
    plan = torch.zeros(ops.routed_experts_plan_ints(n, top, E), dtype=torch.int32, device=DEV)
    act = torch.zeros((a, F), dtype=h.dtype, device=DEV)
    y = torch.full((a, hidden), 77.0, device=DEV)
    gathered = torch.zeros((a, hidden), dtype=h.dtype, device=DEV)
    fn(h, router, None, w_up, w_down, top, ids, weights, order, plan, act, y, gathered, scoring=1, correction=correction,
       pass_through=pass_through, weight_scale=scale)
    return y, ids, weights


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # width, expert width, experts with matrices, experts that hand through, chosen
    (40, 12, 5, 1, 3), (128, 64, 8, 2, 2), (128, 96, 4, 0, 1), (32, 16, 1, 2, 3), (256, 128, 16, 2, 4), (136, 40, 2, 5, 7),
    (320, 104, 12, 2, 4), (64, 32, 3, 0, 3)])
def test_routed_experts_scored_over_all_outputs(dtype, case):
    ops = _ops()
    hidden, F, E, through, top = case
    gen = torch.Generator().manual_seed(hidden + E)
    router = (3.0 * torch.randn((E + through, hidden), generator=gen) / hidden ** 0.5).to(DEV)
    correction = (0.5 * torch.randn(E + through, generator=gen) / (E + through)).to(DEV)
    w_up = (torch.randn((E, 2 * F, hidden), generator=gen) / hidden ** 0.5).to(dtype).to(DEV)
    w_down = (torch.randn((E, hidden, F), generator=gen) / F ** 0.5).to(dtype).to(DEV)
    for n in (1, 7, 70, 600, 48 * max(E, 1)):                      # few rows an expert, and enough for the tiles of 128 rows
        h = torch.randn((n, hidden), generator=gen).to(dtype).to(DEV)
        got, got_ids, got_weights = _experts(ops.routed_experts, h, router, correction, w_up, w_down, top, through)
        want, want_ids, want_weights = _experts(plain_ops.routed_experts, h, router, correction, w_up, w_down, top, through)
        torch.cuda.synchronize()
        # a choice by less than rounding reaches may fall either way: compare the tokens whose choice is the same
        same = (got_ids.view(n, top) == want_ids.view(n, top)).all(dim=1)
        assert int(same.sum()) >= 0.97 * n, (case, n)
        rows = same.repeat_interleave(top)
        assert torch.allclose(got_weights[rows], want_weights[rows], atol=2e-6, rtol=2e-5)
        _close(got[rows], want[rows], dtype, (case, n))
        if through:
            assert int((got_ids >= E).sum()) > 0 or n < 7           # the experts that hand through are chosen somewhere


def test_the_correction_decides_the_choice_and_not_the_weights():
    """A router of zeros: every score is 1 / outputs, so the correction alone chooses (its largest entries, the lower
    index on a tie), and every weight is scale / top whatever the correction is. An expert that hands through
    returns its input times that weight."""
    ops = _ops()
    hidden, F, E, through, top = 64, 32, 4, 2, 3
    gen = torch.Generator().manual_seed(1)
    router = torch.zeros((E + through, hidden), device=DEV)
    correction = torch.tensor([0.1, 0.5, 0.1, -1.0, 0.3, 0.1], device=DEV)
    w_up = torch.randn((E, 2 * F, hidden), generator=gen).to(DEV) / 8
    w_down = torch.randn((E, hidden, F), generator=gen).to(DEV) / 6
    h = torch.randn((5, hidden), generator=gen).to(DEV)
    y, ids, weights = _experts(ops.routed_experts, h, router, correction, w_up, w_down, top, through, scale=0.9)
    assert ids.view(5, top).tolist() == [[1, 4, 0]] * 5                 # 0.5, 0.3, then the first of the three 0.1
    assert torch.allclose(weights, torch.full_like(weights, 0.9 / 3), atol=1e-7)
    assert torch.allclose(y.view(5, top, hidden)[:, 1], h * (0.9 / 3), atol=1e-6)        # output 4 is the first that hands through
    # and the same rows whatever else is in the batch
    alone, _, _ = _experts(ops.routed_experts, h[2:3], router, correction, w_up, w_down, top, through, scale=0.9)
    assert torch.equal(alone, y.view(5, top, hidden)[2])


# ----------------------------------------------------------------------------- the model

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


MARGIN = 0.004          # of choice scores (softmax scores plus correction): what bfloat16 rounding of the input reaches


def _sure(config, weights, tokens, dtype):
    """Per position: True where every routed layer's choice has a margin that bfloat16 rounding does not reach."""
    if dtype == torch.float32:
        return torch.ones(len(tokens), dtype=torch.bool)
    return plain.closest_call(config, weights, tokens) > MARGIN


def test_every_layer_agrees_with_plain(tmp_path):
    """The residual stream after each layer in 32-bit (a model of the first k layers, for every k, whose
    last norm has a weight of one, and its last layer also without feed-forward)."""
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
                    weights["final.norm"].fill_(1.0)
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
    """One token a step from the first on, 300 steps: windows of 44, 70, 100 and 130 slide over decoded tokens,
    pages fill and follow each other, the recurrences' states are carried 300 times, values are blended with the
    first layer's step by step, and steps are replayed from graphs."""
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
    changes = ("window wider", "window narrower", "decay", "taps", "step bias", "stretch", "rotated part", "gate", "correction",
               "blend", "cap", "head norm", "skip", "norm parts", "constant", "hand through", "nothing")
    for change in changes:
        other, w = json.loads(json.dumps(config)), dict(weights)
        if change == "window wider":
            other["layers"][0]["mixer"]["mask"]["size"] += 1
        elif change == "window narrower":
            other["layers"][1]["mixer"]["left"]["mask"]["size"] -= 1
        elif change == "decay":
            w["l1.mix.right.A_log"] = weights["l1.mix.right.A_log"] + 1.0          # a state that fades faster
        elif change == "taps":
            w["l3.mix.right.conv"] = weights["l3.mix.right.conv"].flip(1)           # the taps in the other order
        elif change == "step bias":
            w["l1.mix.right.dt_bias"] = weights["l1.mix.right.dt_bias"] * 0.0
        elif change == "stretch":
            del other["layers"][0]["mixer"]["rot"]["scaling"]
        elif change == "rotated part":
            other["layers"][2]["mixer"]["rot"]["dims"] = 32
        elif change == "gate":
            w["l2.mix.g"] = weights["l2.mix.g"] * 0.0
        elif change == "correction":
            w["l0.mlp.correction"] = weights["l0.mlp.correction"] * 0.0
        elif change == "blend":
            w["l2.mix.vmix"] = weights["l2.mix.vmix"] * 0.0
        elif change == "cap":
            other["layers"][3]["mixer"]["left"]["softcap"] = 20.0
        elif change == "head norm":
            w["l1.mix.left.k.norm"] = weights["l1.mix.left.k.norm"].flip(0)
        elif change == "skip":
            w["l4.mix.right.D"] = weights["l4.mix.right.D"] * 0.0
        elif change == "norm parts":
            other["layers"][4]["mixer"]["right"]["norm_groups"] = 2
        elif change == "constant":
            other["residual_mult"] = 0.46
        elif change == "hand through":
            other["layers"][2]["mlp"]["router"]["identity"] = 0                     # the last output would be an expert with matrices
            other["layers"][2]["mlp"]["router"]["experts"] = 17
            for role, shape in (("gate", (32, 128)), ("up", (32, 128)), ("down", (128, 32))):
                w[f"l2.mlp.e16.{role}"] = torch.zeros(shape, dtype=plain.F)
        else:
            other["layers"][3]["mixer"]["left"]["dim"] = 128                        # as it was: the control
        moved = float((plain.forward(other, w, tokens) - want).abs().max())
        if change == "nothing":
            assert moved == 0.0
        else:
            assert moved > 30 * error, (change, moved, error)


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
