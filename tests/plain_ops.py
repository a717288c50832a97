"""Plain PyTorch statements of what every kernel of `llm_b200.ops` computes.

Each function has the signature of the op it restates and works on any
device in 32-bit arithmetic (results are rounded to the op's output dtype at
the end). The GPU tests compare every CUDA kernel with its function here;
the CPU tests put these functions in the kernels' place (`install`) to check
the host-side logic of the engine: packing, positions, pages, slots, chunked
steps. Nothing in the `llm_b200` package imports this file.
"""
from __future__ import annotations

import torch

PAGE = 64


def embed(tokens, table, out=None, scale=1.0, emit=None):
    x = table[tokens.long()].to(torch.float32) * scale
    if emit is not None:
        cast_sumsq(x, emit)
    return x


def cast_sumsq(x, emit):
    """The next norm's input: the rows as bfloat16 and their sums of squares (one part)."""
    emit.rows.copy_(x.to(torch.bfloat16))
    emit.sumsq[:, 0] = (x.float() * x.float()).sum(dim=-1)
    emit.parts = 1
    return emit


def scale_(x, scale):
    x *= scale
    return x


def rmsnorm(x, gain, eps, out_dtype, rows=None, out=None):
    if rows is not None:
        x = x[rows.long()]
    x = x.to(torch.float32)
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * scale * gain.to(torch.float32)).to(out_dtype)


def swiglu(gate_up, out=None):
    width = gate_up.shape[1] // 2
    g = gate_up[:, :width].to(torch.float32)
    u = gate_up[:, width:].to(torch.float32)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear(a, w, bias=None, out_dtype=None, residual=None, out=None, glu=False, norm=None, emit=None,
           rope=None):
    product = a.to(torch.float32) @ w.to(torch.float32).T
    if norm is not None:
        # a folded norm: rows scaled by 1 / sqrt(mean square + eps) from the partial sums of squares
        mean_square = norm.sumsq[:, :norm.parts].sum(dim=-1, keepdim=True) / norm.width
        product = product / torch.sqrt(mean_square + norm.eps)
    if rope is not None:
        if bias is not None:
            product = product + bias.to(torch.float32)
        qkv = product.to(out_dtype or a.dtype)
        rope_cache_write(qkv, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                         rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                         rope.interleaved, rope.write_cache)
        return qkv
    if glu:
        # rows of w alternate 16 gate rows, 16 up rows
        m = product.shape[0]
        blocks = product.view(m, -1, 2, 16)
        g, u = blocks[:, :, 0, :].reshape(m, -1), blocks[:, :, 1, :].reshape(m, -1)
        return (g / (1.0 + torch.exp(-g)) * u).to(a.dtype)
    if bias is not None:
        product = product + bias.to(torch.float32)
    if residual is not None:
        residual += product
        if emit is not None:
            cast_sumsq(residual, emit)
        return residual
    if out is not None:
        out.copy_(product.to(out.dtype))
        return out
    return product.to(out_dtype or a.dtype)


def _rotate(x, cos, sin, interleaved):
    """x [n, heads, D] float32; cos, sin [n, n_rot/2]: the first n_rot elements of a head rotate,
    the rest passes through."""
    half = cos.shape[-1]
    n_rot = 2 * half
    cos, sin = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    if interleaved:
        low, high = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
        out[..., 0:n_rot:2] = low * cos - high * sin
        out[..., 1:n_rot:2] = low * sin + high * cos
    else:
        low, high = x[..., :half], x[..., half:n_rot]
        out[..., :half] = low * cos - high * sin
        out[..., half:n_rot] = low * sin + high * cos
    return out


def rope_cache_write(qkv, rope_table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache,
                     n_heads, n_kv_heads, head_dim, interleaved=False, write_cache=True):
    n = qkv.shape[0]
    if n == 0:
        return
    qw, kw = n_heads * head_dim, n_kv_heads * head_dim
    pos = tok_pos.long()
    q = qkv[:, :qw].to(torch.float32).view(n, n_heads, head_dim)
    k = qkv[:, qw:qw + kw].to(torch.float32).view(n, n_kv_heads, head_dim)
    v = qkv[:, qw + kw:].view(n, n_kv_heads, head_dim)
    if rope_table is not None:
        half = rope_table.shape[1] // 2
        cos, sin = rope_table[pos, :half], rope_table[pos, half:]
        q = _rotate(q, cos, sin, interleaved)
        k = _rotate(k, cos, sin, interleaved)
    qkv[:, :qw] = q.reshape(n, qw).to(qkv.dtype)
    if not write_cache:
        return
    pages = block_table.long()[tok_seq.long(), (pos // PAGE) % ring_pages]
    rows = pos % PAGE
    k_cache[pages, :, rows, :] = k.to(k_cache.dtype)
    v_cache[pages, :, rows, :] = v.to(v_cache.dtype)


def attention(qkv, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads,
              n_kv_heads, head_dim, scale, window=0, out=None, decode=False, seq_lens=None,
              max_len=0, cu_seqlens=None, max_new=0, seq_order=None, sinks=None, gate=None, out_scale=1.0,
              softcap=0.0, value_dim=None):
    """`sinks` (float32 [heads]): e^sink is one more term of a head's softmax denominator. `gate`
    ([T, heads]): head a of token t is multiplied by sigmoid(gate[t, a]). `out_scale` multiplies all.
    `softcap` c > 0: score <- c tanh(score / c). `value_dim`: the size of a value (default head_dim)."""
    n = qkv.shape[0]
    value_dim = value_dim or head_dim
    result = torch.zeros((n, n_heads * value_dim), dtype=torch.float32, device=qkv.device)
    group = n_heads // n_kv_heads
    table = block_table.long()
    for t in range(n):
        pos, b = int(tok_pos[t]), int(tok_seq[t])
        first = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(first, pos + 1, device=qkv.device)
        pages = table[b, (js // PAGE) % ring_pages]
        keys = k_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, Hkv, D]
        vals = v_cache[pages, :, js % PAGE, :].to(torch.float32)
        q = qkv[t, :n_heads * head_dim].to(torch.float32).view(n_heads, head_dim)
        for h in range(n_heads):
            scores = (keys[:, h // group, :] @ q[h]) * scale
            if softcap > 0.0:
                scores = softcap * torch.tanh(scores / softcap)
            if sinks is None:
                p = torch.softmax(scores, dim=0)
            else:
                top = torch.maximum(scores.max(), sinks[h].to(torch.float32))
                e = torch.exp(scores - top)
                p = e / (e.sum() + torch.exp(sinks[h] - top))
            o = (p @ vals[:, h // group, :]) * out_scale
            if gate is not None:
                o = o * torch.sigmoid(gate[t, h].to(torch.float32))
            result[t, h * value_dim:(h + 1) * value_dim] = o
    if out is not None:
        out.copy_(result.to(out.dtype))
        return out
    return result.to(qkv.dtype)


def tanh_norm(x, alpha, gain, bias, out_dtype, rows=None, out=None, second=None):
    if rows is not None:
        x = x[rows.long()]
    if second is not None:
        alpha2, gain2, bias2, out2 = second
        out2.copy_((torch.tanh(x.to(torch.float32) * alpha2) * gain2 + bias2).to(out_dtype))
    y = (torch.tanh(x.to(torch.float32) * alpha) * gain + bias).to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def norm_rope_cache_write(u, q_width, k_width, v_width, q_gain, k_gain, eps, rope_table, rot_unit, interleaved,
                          tok_pos, tok_seq, q_out, block_table, ring_pages, k_cache, v_cache, write_cache=True,
                          value_source=None, norm_unit=0, mix_cache=None, mix_table=None, mix_ring=0, mix=0.0):
    """The first q_width columns of u are the queries, the next k_width the keys, the next v_width
    the values (or, with value_source, the v_width columns from there on: q_width makes the values
    the keys as projected). With a gain, queries (keys) are divided by the root mean square of the
    whole segment (or, with norm_unit, of every unit of that many columns, all units sharing a gain of
    that size) and multiplied by the gain; then every unit of rot_unit columns of both rotates. With
    mix_cache the values become (1 - mix) v + mix * (what that cache holds at the token's place)."""
    n = u.shape[0]
    if n == 0:
        return q_out
    pos = tok_pos.long()

    def segment(first, width, gain):
        x = u[:, first:first + width].to(torch.float32)
        if gain is not None and norm_unit:
            x = x.reshape(n, -1, norm_unit)
            x = (x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain).reshape(n, width)
        elif gain is not None:
            x = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain
        if rope_table is not None:
            half = rope_table.shape[1] // 2
            x = _rotate(x.reshape(n, -1, rot_unit), rope_table[pos, :half], rope_table[pos, half:], interleaved)
        return x.reshape(n, width)

    q_out.copy_(segment(0, q_width, q_gain).to(q_out.dtype))
    if write_cache:
        pages = block_table.long()[tok_seq.long(), (pos // PAGE) % ring_pages]
        rows = pos % PAGE
        k = segment(q_width, k_width, k_gain)
        k_cache[pages, :, rows, :] = k.reshape(n, k_cache.shape[1], k_cache.shape[3]).to(k_cache.dtype)
        if v_width:
            start = q_width + k_width if value_source is None else value_source
            v = u[:, start:start + v_width].reshape(n, v_cache.shape[1], v_cache.shape[3])
            if mix_cache is not None:
                first_pages = mix_table.long()[tok_seq.long(), (pos // PAGE) % mix_ring]
                v = (1.0 - mix) * v.to(torch.float32) + mix * mix_cache[first_pages, :, rows, :].to(torch.float32)
            v_cache[pages, :, rows, :] = v.to(v_cache.dtype)
    return q_out


def sigmoid_attention(q, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads, n_kv_heads, dim, vdim,
                      scale, window, talk, head_bias, out_scale, out, decode=False, seq_lens=None, max_len=0,
                      cu_seqlens=None, max_new=0, seq_order=None):
    n = q.shape[0]
    group = n_heads // n_kv_heads
    table = block_table.long()
    result = torch.zeros((n, n_heads * vdim), dtype=torch.float32, device=q.device)
    for t in range(n):
        pos, b = int(tok_pos[t]), int(tok_seq[t])
        first = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(first, pos + 1, device=q.device)
        pages = table[b, (js // PAGE) % ring_pages]
        keys = k_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, G, dim]
        vals = v_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, G, vdim]
        heads = q[t].to(torch.float32).view(n_heads, dim)
        scores = torch.stack([keys[:, a // group, :] @ heads[a] for a in range(n_heads)]) * scale    # [H, n_keys]
        if talk is not None:
            scores = talk.to(torch.float32) @ scores
        if head_bias is not None:
            scores = scores + head_bias.to(torch.float32)[:, None]
        weights = torch.sigmoid(scores)
        for a in range(n_heads):
            result[t, a * vdim:(a + 1) * vdim] = (weights[a] @ vals[:, a // group, :]) * out_scale
    out.copy_(result.to(out.dtype))
    return out


def gated_recurrence(y, x, conv_w, conv_b, gate_a, gate_a_bias, gate_i, gate_i_bias, rate, state, tok_seq,
                     cu_seqlens, slot_ids, out, out_scale, work, single_tokens=False):
    """Sequence by sequence and token by token. state [slots, taps, C] float32: rows 0 .. taps - 2
    are the convolution's last inputs (oldest first), the last row is S."""
    n, channels = y.shape
    if n == 0:
        return out
    taps, blocks = conv_w.shape[1], gate_a.shape[0]
    cu = cu_seqlens.tolist()
    result = torch.zeros((n, channels), dtype=torch.float32, device=y.device)
    for b in range(len(cu) - 1):
        slot = int(slot_ids[b])
        history = state[slot, :taps - 1].clone()
        s = state[slot, taps - 1].clone()
        for t in range(cu[b], cu[b + 1]):
            rows = torch.cat([history, x[t].to(torch.float32)[None]])                     # [taps, C]
            u = conv_b + (conv_w.T * rows).sum(dim=0)
            history = rows[1:]
            parts = u.view(blocks, -1)
            r = torch.sigmoid(torch.einsum("boi,bi->bo", gate_a, parts).reshape(-1) + gate_a_bias)
            i = torch.sigmoid(torch.einsum("boi,bi->bo", gate_i, parts).reshape(-1) + gate_i_bias)
            a = torch.exp(rate * r)
            s = a * s + torch.sqrt(1.0 - a * a) * i * u
            z = y[t].to(torch.float32)
            gelu = 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))
            result[t] = s * gelu * out_scale
        state[slot, :taps - 1] = history
        state[slot, taps - 1] = s
    out.copy_(result.to(out.dtype))
    return out


def norm_add_(x, y, gain_post, eps_post, terms=1, gain_next=None, eps_next=0.0, out=None, out_dtype=None):
    """x[t] += norm(sum of the token's `terms` rows of y); with gain_next also the norm of the new x."""
    n, hidden = x.shape
    s = y[:n * terms].view(n, terms, hidden)[:, 0].clone()
    for k in range(1, terms):                       # the terms in index order
        s = s + y[:n * terms].view(n, terms, hidden)[:, k]
    x += s / torch.sqrt((s * s).mean(dim=-1, keepdim=True) + eps_post) * gain_post
    if gain_next is None:
        return None
    normed = (x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps_next) * gain_next)
    dtype = out_dtype or (out.dtype if out is not None else torch.float32)
    if out is None:
        return normed.to(dtype)
    out.copy_(normed.to(dtype))
    return out


def gelu_(a):
    z = a.to(torch.float32)
    a.copy_((0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))).to(a.dtype))
    return a


def sigmoid_gate_(out, gate):
    out.copy_((out.to(torch.float32) * torch.sigmoid(gate.to(torch.float32))).to(out.dtype))
    return out


def add_terms_(x, y, terms):
    n, hidden = x.shape
    rows = y.reshape(-1)[:n * terms * hidden].view(n, terms, hidden)
    for k in range(terms):
        x += rows[:, k]
    return x


def fill_(x, value):
    x.fill_(value)
    return x


def delta_rule_work_width(n_heads, n_kv_heads, dim, vdim):
    return (2 * n_kv_heads * dim + n_heads * vdim + 2 * n_heads + n_kv_heads + 3) // 4 * 4


def delta_rule(proj, taps, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, unit_eps, norm_weight, eps, work, o,
               mixed, n_heads, n_kv_heads, dim, vdim):
    """Sequence by sequence, token by token, head by head. A token's row of proj is
    [q (G D) | k (G D) | v (H V) | gate (H V) | b (H) | a (H) | ...]; a slot's row of state is the
    convolution's last K - 1 inputs [K - 1, C] (oldest first), then S [H, D, V]."""
    H, G, D, V = n_heads, n_kv_heads, dim, vdim
    n = proj.shape[0]
    if n == 0:
        return mixed
    C, K = 2 * G * D + H * V, taps.shape[1]
    cu = cu_seqlens.tolist()
    result = torch.zeros((n, H * V), dtype=torch.float32, device=proj.device)

    def silu(z):
        return z / (1.0 + torch.exp(-z))

    for b in range(len(cu) - 1):
        slot = int(slot_ids[b])
        history = state[slot, :(K - 1) * C].view(K - 1, C).clone()
        S = state[slot, (K - 1) * C:(K - 1) * C + H * D * V].view(H, D, V).clone()
        for t in range(cu[b], cu[b + 1]):
            row = proj[t].to(torch.float32)
            rows = torch.cat([history, row[None, :C]])                                    # [K, C]
            u = silu((taps.T * rows).sum(dim=0))
            history = rows[1:]
            q, k, v = u[:G * D].view(G, D), u[G * D:2 * G * D].view(G, D), u[2 * G * D:].view(H, V)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) / (D ** 0.5)
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
            gate = row[C:C + H * V].view(H, V)
            beta = torch.sigmoid(row[C + H * V:C + H * V + H])
            z = row[C + H * V + H:C + H * V + 2 * H] + dt_bias
            decay = torch.exp(rate * torch.where(z > 20.0, z, torch.log1p(torch.exp(torch.clamp(z, max=20.0)))))
            for a in range(H):
                g = a // (H // G)
                S[a] = decay[a] * S[a]
                w = beta[a] * (v[a] - S[a].T @ k[g])
                S[a] = S[a] + torch.outer(k[g], w)
                read = S[a].T @ q[g]
                read = read / torch.sqrt((read * read).mean() + eps) * norm_weight
                result[t, a * V:(a + 1) * V] = read * silu(gate[a])
        state[slot, :(K - 1) * C] = history.reshape(-1)
        state[slot, (K - 1) * C:(K - 1) * C + H * D * V] = S.reshape(-1)
    mixed.copy_(result.to(mixed.dtype))
    return mixed


def routed_experts_plan_ints(n_tokens, top, n_experts):
    return n_experts + 2 + 3 * ((n_tokens * top + 31) // 32 + n_experts)


def routed_experts_wide(n_tokens, top, n_experts, hidden, intermediate, dtype):
    return False


def routed_experts(h, router, router_bias, w_up, w_down, top, ids, weights, order, plan, act, y, gathered=None,
                   scoring=0, correction=None, pass_through=0, weight_scale=1.0):
    """Token by token: 32-bit router logits, the `top` largest, the softmax over them, and one row
    weight * expert(h) per choice, in the order of choice (largest logit first). scoring 1: the scores are the
    softmax over all outputs, the choice is by score + correction, the weights are the chosen scores over
    their sum (+ 1e-20). The router's last `pass_through` outputs are experts whose result is h."""
    n, hidden = h.shape
    F = w_up.shape[1] // 2
    x = h.to(torch.float32)
    logits = x @ router.T
    if router_bias is not None:
        logits = logits + router_bias
    E = w_up.shape[0]
    for t in range(n):
        if scoring == 1:
            scores = torch.softmax(logits[t], 0)
            choice = scores + correction if correction is not None else scores
            chosen = torch.sort(choice, descending=True, stable=True).indices[:top]
            share = scores[chosen] / (scores[chosen].sum() + 1e-20) * weight_scale
        else:
            chosen = torch.topk(logits[t], top).indices
            share = torch.softmax(logits[t, chosen], 0) * weight_scale
        for k in range(top):
            e = int(chosen[k])
            ids[t * top + k] = e
            weights[t * top + k] = share[k]
            if e >= E:
                y[t * top + k] = share[k] * x[t]
                continue
            gate_up = x[t] @ w_up[e].to(torch.float32).T
            g, u = gate_up[:F], gate_up[F:]
            a = (g / (1.0 + torch.exp(-g)) * u).to(h.dtype).to(torch.float32)
            y[t * top + k] = share[k] * (a @ w_down[e].to(torch.float32).T)
    return y


def state_space_work_width(n_heads, groups, state, vdim):
    return (n_heads * vdim + 2 * groups * state + 2 * n_heads + 3) // 4 * 4


def state_space(proj, taps, conv_bias, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, skip, norm_weight, eps,
                norm_groups, out_scale, work, y, mixed, n_heads, groups, n_state, vdim):
    """Sequence by sequence, token by token, head by head. A token's row of proj is
    [z (H V) | x (H V) | B (G N) | C (G N) | dt (H) | ...]; a slot's row of state is the convolution's last
    K - 1 inputs [K - 1, C] (oldest first, C = H V + 2 G N), then S [H, V, N] (a value element's N rows together)."""
    H, G, N, V = n_heads, groups, n_state, vdim
    n = proj.shape[0]
    if n == 0:
        return mixed
    inner = H * V
    C, K = inner + 2 * G * N, taps.shape[1]
    cu = cu_seqlens.tolist()
    result = torch.zeros((n, inner), dtype=torch.float32, device=proj.device)

    def silu(z):
        return z / (1.0 + torch.exp(-z))

    for b in range(len(cu) - 1):
        slot = int(slot_ids[b])
        history = state[slot, :(K - 1) * C].view(K - 1, C).clone()
        S = state[slot, (K - 1) * C:(K - 1) * C + H * N * V].view(H, V, N).transpose(1, 2).clone()       # as [H, N, V]
        for t in range(cu[b], cu[b + 1]):
            row = proj[t].to(torch.float32)
            rows = torch.cat([history, row[None, inner:inner + C]])                       # [K, C]
            u = (taps.T * rows).sum(dim=0)
            u = silu(u + conv_bias if conv_bias is not None else u)
            history = rows[1:]
            x, B, Cm = u[:inner].view(H, V), u[inner:inner + G * N].view(G, N), u[inner + G * N:].view(G, N)
            z = row[inner + C:inner + C + H] + dt_bias
            dt = torch.where(z > 20.0, z, torch.log1p(torch.exp(torch.clamp(z, max=20.0))))
            decay = torch.exp(rate * dt)
            out = torch.zeros((H, V), dtype=torch.float32, device=proj.device)
            for a in range(H):
                g = a // (H // G)
                S[a] = decay[a] * S[a] + dt[a] * torch.outer(B[g], x[a])
                out[a] = S[a].T @ Cm[g] + (skip[a] * x[a] if skip is not None else 0.0)
            gated = (out.reshape(inner) * silu(row[:inner])).view(norm_groups, inner // norm_groups)
            gated = gated / torch.sqrt((gated * gated).mean(-1, keepdim=True) + eps)
            result[t] = gated.reshape(inner) * norm_weight * out_scale
        state[slot, :(K - 1) * C] = history.reshape(-1)
        state[slot, (K - 1) * C:(K - 1) * C + H * N * V] = S.transpose(1, 2).reshape(-1)
    mixed.copy_(result.to(mixed.dtype))
    return mixed


def softcap_(x, cap):
    x.copy_(cap * torch.tanh(x / cap))
    return x


def add_rows_(x, y, emit=None):
    x += y
    if emit is not None:
        cast_sumsq(x, emit)
    return x


def conv_rope_cache_write(u, conv_w, state, tok_pos, tok_seq, cu_seqlens, seq_lens, slot_ids, rope_table,
                          rot_unit, interleaved, q_out, k_width, v_width, block_table, ring_pages, k_cache,
                          v_cache, write_cache=True, single_tokens=False, conv_w_rows=None):
    """Sequence by sequence: the rows before the step's first token come from the state, the
    convolution is a plain sum over taps, then every unit of `rot_unit` channels of q and k rotates."""
    n, q_width = q_out.shape
    if n == 0:
        return q_out
    y = torch.empty((n, u.shape[1]), dtype=torch.float32, device=u.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        first, last = cu[b], cu[b + 1]
        rows = u[first:last].to(torch.float32)
        if conv_w is None:
            y[first:last] = rows
            continue
        taps = conv_w.shape[1]
        if taps > 1:
            slot = int(slot_ids[b])
            history = torch.cat([state[slot].to(torch.float32), rows])
            state[slot] = history[-(taps - 1):].to(state.dtype)
        else:
            history = rows
        count = last - first
        total = torch.zeros_like(rows)
        for j in range(taps):
            total += conv_w[:, j].to(torch.float32)[None, :] * history[j:j + count]
        y[first:last] = total
    pos = tok_pos.long()
    k_end = q_width + k_width
    q = y[:, :q_width].reshape(n, -1, rot_unit)
    k = y[:, q_width:k_end].reshape(n, -1, rot_unit)
    if rope_table is not None:
        half = rope_table.shape[1] // 2
        cos, sin = rope_table[pos, :half], rope_table[pos, half:]
        q = _rotate(q, cos, sin, interleaved)
        k = _rotate(k, cos, sin, interleaved)
    q_out.copy_(q.reshape(n, q_width).to(q_out.dtype))
    if write_cache:
        pages = block_table.long()[tok_seq.long(), (pos // PAGE) % ring_pages]
        rows = pos % PAGE
        k_cache[pages, :, rows, :] = k.reshape(n, k_cache.shape[1], k_cache.shape[3]).to(k_cache.dtype)
        v_cache[pages, :, rows, :] = y[:, k_end:].reshape(n, v_cache.shape[1], v_cache.shape[3]).to(v_cache.dtype)
    return q_out


def diff_attention(q, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads, n_kv_heads, dim,
                   vdim, scale, window, keep_first, lam, eps, out_scale, head_norm=True, out=None, decode=False,
                   seq_lens=None, max_len=0, cu_seqlens=None, max_new=0, seq_order=None):
    n = q.shape[0]
    result = torch.zeros((n, n_heads * vdim), dtype=torch.float32, device=q.device)
    group = n_heads // n_kv_heads
    table = block_table.long()
    for t in range(n):
        pos, b = int(tok_pos[t]), int(tok_seq[t])
        js = torch.arange(0, pos + 1, device=q.device)
        if window > 0:
            js = js[(pos - js < window) | (js < keep_first)]
        pages = table[b, (js // PAGE) % ring_pages]
        keys = k_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, G, 2 * dim]
        vals = v_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, G, vdim]
        maps = q[t].to(torch.float32).view(n_kv_heads, group, 2, dim)
        split_keys = keys.view(-1, n_kv_heads, 2, dim)
        scores = torch.einsum("ghmd,jgmd->ghmj", maps, split_keys) * scale       # per kv head, head of its group, map
        a = torch.einsum("ghmj,jgv->ghmv", torch.softmax(scores, dim=-1), vals)
        o = a[:, :, 0] - lam * a[:, :, 1]                                         # [G, group, vdim]
        if head_norm:
            o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
        result[t] = (o * out_scale).reshape(-1)
    return result.to(q.dtype)


def argmax_rows(logits, out=None):
    best = logits.max(dim=1, keepdim=True).values
    first = (logits == best).to(torch.int32).argmax(dim=1)
    return first.to(torch.int32)


MASK64 = (1 << 64) - 1


def _next_uniform(state):
    x = state & MASK64
    x ^= x >> 12
    x ^= (x << 25) & MASK64
    x ^= x >> 27
    value = (x * 0x2545F4914F6CDD1D) & MASK64
    return x, float(value >> 40) / float(1 << 24)


def _sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status):
    """Row by row, the chain of csrc/sampling.cu in 32-bit host arithmetic."""
    n, vocab = logits.shape
    f32 = torch.float32
    for r in range(n):
        temperature, top_p, min_p, penalty = (float(v) for v in params[r])
        top_k, last_n = (int(v) for v in iparams[r])
        row = logits[r]
        status[r] = 0
        if penalty != 1.0 and last_n > 0 and recent is not None:
            cap = recent.shape[1]
            total = int(recent_len[r])
            span = min(total, last_n, cap)
            pen = torch.tensor(penalty, dtype=f32)
            for i in range(total - span, total):
                token = int(recent[r, i % cap])
                if 0 <= token < vocab:
                    row[token] = row[token] / pen if row[token] > 0 else row[token] * pen
        if not temperature > 0.0:
            out[r] = int(argmax_rows(row[None])[0])
            continue
        row *= (torch.tensor(1.0, dtype=f32) / torch.tensor(temperature, dtype=f32))
        state = int(rng_state[r]) & MASK64
        if (top_k <= 0 or top_k >= vocab) and vocab > 1024:
            if top_k > 0 or 0.0 <= top_p < 1.0:
                status[r], out[r] = 1, 0
                continue
            p = torch.exp(row - row.max())
            p = torch.where(p >= max(min_p, 0.0), p, torch.zeros_like(p))
            state, u = _next_uniform(state)
            target = torch.tensor(u, dtype=f32) * p.sum()
            pick = int((torch.cumsum(p, 0) >= target).nonzero()[0])
        else:
            if top_k > 1024:
                status[r], out[r] = 1, 0
                continue
            k = vocab if top_k <= 0 or top_k >= vocab else top_k
            order = sorted(range(vocab), key=lambda i: (-float(row[i]), i))[:k]
            probs = torch.exp(row[order] - row[order[0]])
            total = torch.tensor(0.0, dtype=f32)
            for v in probs:
                total = total + v
            if total > 0:
                probs = probs / total
            kept = len(order)
            if 0.0 <= top_p < 1.0:
                cumulative = torch.tensor(0.0, dtype=f32)
                for i, v in enumerate(probs):
                    cumulative = cumulative + v
                    if cumulative > top_p:
                        kept = i + 1
                        break
            if min_p > 0.0:
                cut = probs[0] * torch.tensor(min_p, dtype=f32)
                keep = 0
                while keep < kept and probs[keep] >= cut:
                    keep += 1
                kept = keep
            total = torch.tensor(0.0, dtype=f32)
            for v in probs[:kept]:
                total = total + v
            pick = order[0]
            if total > 0:
                state, u = _next_uniform(state)
                target = torch.tensor(u, dtype=f32) * total
                for i in range(kept):
                    target = target - probs[i]
                    if target <= 0:
                        pick = order[i]
                        break
        rng_state[r] = state - (1 << 64) if state >= (1 << 63) else state
        out[r] = pick
    return out


def sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status, record=False,
                state_rows=None):
    """The chain for every row; with `record`, the drawn tokens then enter the rows' windows.
    `state_rows`: row i of the logits belongs to the sequence in row state_rows[i] of the state."""
    if state_rows is not None:
        index = state_rows.long()
        taken = [t[index].clone() if t is not None else None
                 for t in (params, iparams, recent, recent_len, rng_state, status)]
        sample_rows(logits, taken[0], taken[1], taken[2], taken[3], taken[4], out, taken[5], record)
        for whole, part in zip((recent, recent_len, rng_state, status), (taken[2], taken[3], taken[4], taken[5])):
            if whole is not None:
                whole[index] = part
        return out
    _sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status)
    if record and recent is not None:
        cap = recent.shape[1]
        for r in range(logits.shape[0]):
            recent[r, int(recent_len[r]) % cap] = int(out[r])
            recent_len[r] += 1
    return out



OPS = {"embed": embed, "scale_": scale_, "cast_sumsq": cast_sumsq, "rmsnorm": rmsnorm, "swiglu": swiglu, "linear": linear,
       "rope_cache_write": rope_cache_write, "attention": attention, "argmax_rows": argmax_rows,
       "softcap_": softcap_, "add_rows_": add_rows_, "conv_rope_cache_write": conv_rope_cache_write,
       "diff_attention": diff_attention, "tanh_norm": tanh_norm, "norm_rope_cache_write": norm_rope_cache_write,
       "sigmoid_attention": sigmoid_attention, "gated_recurrence": gated_recurrence,
       "sample_rows": sample_rows, "norm_add_": norm_add_, "gelu_": gelu_, "sigmoid_gate_": sigmoid_gate_,
       "add_terms_": add_terms_, "fill_": fill_, "delta_rule": delta_rule, "delta_rule_work_width": delta_rule_work_width,
       "routed_experts": routed_experts, "routed_experts_plan_ints": routed_experts_plan_ints,
       "routed_experts_wide": routed_experts_wide, "state_space": state_space,
       "state_space_work_width": state_space_work_width}


def install(monkeypatch):
    """Put the plain functions in the kernels' place (CPU tests of host logic)."""
    import llm_b200.ops as ops
    for name, fn in OPS.items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "ensure_built", lambda names: None)
    monkeypatch.setattr(ops, "check_device_status", lambda: None)
    monkeypatch.setattr(ops, "glu_fusable", lambda n, k, dtype: dtype == torch.bfloat16 and n % 32 == 0)
