"""The gated delta rule: a linear recurrence with a matrix state per head."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import register_mixer, to_float32, to_run_dtype
from .projected import ProjectedMixer


class DeltaRuleMixer(ProjectedMixer):
    """Per head a state M [head_dim, value_dim], token by token
        M_t = a_t M_{t-1} + k_t w_t^T,   w_t = b_t (v_t - a_t M_{t-1}^T k_t),   o_t = M_t^T q_t
    (the read-out sees the token's own write), with q, k (n_kv_heads heads, each serving a group of
    heads) and v behind a causal convolution per channel and silu, q and k of unit length (q also
    times head_dim^-1/2), b_t = sigmoid(W_b h), a_t = exp(-exp(A_log) softplus(W_a h + dt_bias)), and
    o / rms(o) * weight * silu(W_g h) per head before the output product.

    One product [q; k; v; gate; b; a] (rows padded to a multiple of 8), then ops.delta_rule (the
    convolution with its state, unit norms, gates, the scan over each sequence's tokens, the heads'
    norm and gate), then the output product. Per sequence the cache holds one float32 row: the
    convolution's last taps - 1 inputs [taps - 1, C], then M [heads, head_dim, value_dim]; zeroed
    when a slot is taken. Everything behind the projection is 32-bit in every run."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "delta_rule")

    def __init__(self, spec):
        s = spec
        if min(s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim, s.conv_taps) < 1 or s.n_heads % s.n_kv_heads:
            raise FormatError("a delta rule needs positive sizes, at least one tap and heads in whole groups")
        self.spec = spec
        self.taps = self.rate = self.dt_bias = self.norm_weight = None

    @property
    def channels(self):
        s = self.spec
        return 2 * s.n_kv_heads * s.head_dim + s.n_heads * s.value_dim

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.value_dim

    @property
    def in_width(self):
        return (self.channels + self.out_width + 2 * self.spec.n_heads + 7) // 8 * 8

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        kw, vw = s.n_kv_heads * s.head_dim, self.out_width
        return {t["q"]: ParamSpec((kw, s.hidden)), t["k"]: ParamSpec((kw, s.hidden)), t["v"]: ParamSpec((vw, s.hidden)),
                t["q_conv"]: ParamSpec((kw, s.conv_taps), "taps"), t["k_conv"]: ParamSpec((kw, s.conv_taps), "taps"),
                t["v_conv"]: ParamSpec((vw, s.conv_taps), "taps"),
                t["beta"]: ParamSpec((s.n_heads, s.hidden)), t["decay"]: ParamSpec((s.n_heads, s.hidden)),
                t["a_log"]: ParamSpec((s.n_heads,), "vector"), t["dt_bias"]: ParamSpec((s.n_heads,), "vector"),
                t["gate"]: ParamSpec((vw, s.hidden)), t["norm"]: ParamSpec((s.value_dim,), "gain"),
                t["o"]: ParamSpec((s.hidden, vw))}

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        rows = [to_run_dtype(tensors[t[r]], dtype, device) for r in ("q", "k", "v", "gate", "beta", "decay")]
        pad = self.in_width - sum(r.shape[0] for r in rows)
        if pad:
            rows.append(torch.zeros((pad, s.hidden), dtype=dtype, device=device))
        self.w_in = torch.cat(rows).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)
        self.taps = torch.cat([to_float32(tensors[t[r]], device) for r in ("q_conv", "k_conv", "v_conv")]).contiguous()
        # log g = rate * softplus(.) with rate = -exp(A_log), once, in 32-bit
        self.rate = (-torch.exp(to_float32(tensors[t["a_log"]], device))).contiguous()
        self.dt_bias = to_float32(tensors[t["dt_bias"]], device)
        self.norm_weight = to_float32(tensors[t["norm"]], device)

    def mix_weights(self):
        return [self.taps]

    def state_request(self):
        s = self.spec
        return StateRequest(((s.conv_taps - 1) * self.channels + s.n_heads * s.head_dim * s.value_dim,), torch.float32)

    def mix_replay_key(self, step):
        return ()

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        width = ops.delta_rule_work_width(s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim)
        return [BufferRequest("delta_work", (n_tokens, width), torch.float32, 0, 0),
                BufferRequest("delta_o", (n_tokens, self.out_width), torch.float32, 0, 0)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        n = proj.shape[0]
        width = ops.delta_rule_work_width(s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim)
        work = scratch("delta_work", (n, width), torch.float32)
        o = scratch("delta_o", (n, self.out_width), torch.float32)
        if work is None or o is None:
            work = torch.empty((n, width), dtype=torch.float32, device=proj.device)
            o = torch.empty((n, self.out_width), dtype=torch.float32, device=proj.device)
        ops.delta_rule(proj, self.taps, ctx.cache.state_view(entry), ctx.tok_seq, ctx.cu_seqlens, ctx.slot_ids,
                       self.rate, self.dt_bias, s.unit_eps, self.norm_weight, s.eps, work, o, out, s.n_heads,
                       s.n_kv_heads, s.head_dim, s.value_dim)


register_mixer("delta_rule", DeltaRuleMixer)
