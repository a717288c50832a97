"""A state-space recurrence with a scalar decay per head."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import register_mixer, to_float32, to_run_dtype
from .projected import ProjectedMixer


class StateSpaceMixer(ProjectedMixer):
    """Per head a state S [state, value_dim], token by token
        S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T,      y_t = S_t^T C_t + D x_t
    with [z | x | B | C | dt] = W_in h, x, B and C behind one causal convolution per channel (with bias) and
    silu, dt_t = softplus(dt + dt_bias), B and C in groups that serve several heads each; then y silu(z),
    divided by its root mean square in `norm_groups` equal parts, times a weight, before the output product.

    One product (rows padded to a multiple of 8), then ops.state_space (the convolution with its state, the
    step sizes and decays, the scan over each sequence's tokens, the gate and the grouped norm), then the
    output product. Per sequence the cache holds one float32 row: the convolution's last taps - 1 inputs
    [taps - 1, C], then S [heads, value_dim, state]; zeroed when a slot is taken. Everything behind the
    projection is 32-bit in every run."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "state_space")

    def __init__(self, spec):
        s = spec
        if min(s.n_heads, s.value_dim, s.state, s.groups, s.conv_taps, s.norm_groups) < 1 or s.n_heads % s.groups:
            raise FormatError("a state-space mixer needs positive sizes, at least one tap and heads in whole groups")
        if (s.n_heads * s.value_dim) % s.norm_groups:
            raise FormatError(f"{s.n_heads * s.value_dim} channels cannot be normed in {s.norm_groups} equal parts")
        self.spec = spec
        self.taps = self.conv_bias = self.rate = self.dt_bias = self.skip = self.norm_weight = None

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.value_dim

    @property
    def channels(self):
        """The channels that pass the convolution: x, B and C."""
        return self.out_width + 2 * self.spec.groups * self.spec.state

    @property
    def rows(self):
        return self.out_width + self.channels + self.spec.n_heads

    @property
    def in_width(self):
        return (self.rows + 7) // 8 * 8

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        return {t["in"]: ParamSpec((self.rows, s.hidden)),
                t["conv"]: ParamSpec((self.channels, s.conv_taps), "taps"), t["conv_bias"]: ParamSpec((self.channels,), "bias"),
                t["dt_bias"]: ParamSpec((s.n_heads,), "vector"), t["a_log"]: ParamSpec((s.n_heads,), "vector"),
                t["skip"]: ParamSpec((s.n_heads,), "vector"), t["norm"]: ParamSpec((self.out_width,), "gain"),
                t["o"]: ParamSpec((s.hidden, self.out_width))}

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        rows = [to_run_dtype(tensors[t["in"]], dtype, device)]
        if self.in_width > self.rows:
            rows.append(torch.zeros((self.in_width - self.rows, s.hidden), dtype=dtype, device=device))
        self.w_in = torch.cat(rows).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)
        self.taps = to_float32(tensors[t["conv"]], device)
        self.conv_bias = to_float32(tensors[t["conv_bias"]], device)
        # log decay = rate * dt with rate = -exp(A_log), once, in 32-bit
        self.rate = (-torch.exp(to_float32(tensors[t["a_log"]], device))).contiguous()
        self.dt_bias = to_float32(tensors[t["dt_bias"]], device)
        self.skip = to_float32(tensors[t["skip"]], device)
        self.norm_weight = to_float32(tensors[t["norm"]], device)

    def mix_weights(self):
        return [self.taps]

    def state_request(self):
        s = self.spec
        return StateRequest(((s.conv_taps - 1) * self.channels + s.n_heads * s.state * s.value_dim,), torch.float32)

    def mix_replay_key(self, step):
        return ()

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        width = ops.state_space_work_width(s.n_heads, s.groups, s.state, s.value_dim)
        return [BufferRequest("ssm_work", (n_tokens, width), torch.float32, 0, 0),
                BufferRequest("ssm_y", (n_tokens, self.out_width), torch.float32, 0, 0)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        n = proj.shape[0]
        width = ops.state_space_work_width(s.n_heads, s.groups, s.state, s.value_dim)
        work = scratch("ssm_work", (n, width), torch.float32)
        y = scratch("ssm_y", (n, self.out_width), torch.float32)
        if work is None or y is None:
            work = torch.empty((n, width), dtype=torch.float32, device=proj.device)
            y = torch.empty((n, self.out_width), dtype=torch.float32, device=proj.device)
        ops.state_space(proj, self.taps, self.conv_bias, ctx.cache.state_view(entry), ctx.tok_seq, ctx.cu_seqlens,
                        ctx.slot_ids, self.rate, self.dt_bias, self.skip, self.norm_weight, s.eps, s.norm_groups,
                        s.out_scale, work, y, out, s.n_heads, s.groups, s.state, s.value_dim)


register_mixer("state_space", StateSpaceMixer)
