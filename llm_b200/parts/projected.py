"""Mixers of three stages: a product of the input, a mixing stage, a product into the stream."""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer


class ProjectedMixer(Mixer):
    """A mixer whose forward pass is `linear(h, W_in) -> mix -> linear(., W_out)` into the
    residual stream. The three stages are open, so that mixers that read the same input can
    share the first and the last product (SideBySideMixer): a subclass sets `w_in` [in_width,
    hidden], `b_in` (float32 [in_width] or None) and `w_out` [hidden, out_width] at bind, and
    `mix` turns the projection's rows into the rows that `w_out` reads, already multiplied by the
    spec's `out_scale` (in 32-bit, before they are rounded to the run's dtype).

    `proj` and `out` may be column ranges of wider buffers: the kernels behind `mix` take row
    strides. `scratch(name, shape, dtype)` hands out the buffers that `mix_scratch` declared
    (or None where a step has no plan)."""
    graph_safe = True
    emits = True
    #: `forward` takes `fresh=True`: the result is written into `residual` instead of added to it
    overwrites = True
    w_in = b_in = w_out = None

    @property
    def hidden(self) -> int:
        return self.spec.hidden

    @property
    def in_width(self) -> int:
        raise NotImplementedError

    @property
    def out_width(self) -> int:
        raise NotImplementedError

    def mix_scratch(self, n_tokens: int, dtype) -> list:
        """BufferRequests of `mix` for n_tokens tokens, phases counted from 0."""
        return []

    def mix(self, proj, ctx, entry: int, cache_entry: int, out, scratch) -> None:
        raise NotImplementedError

    def mix_replay_key(self, step):
        return ()

    def mix_shapes(self, dtype, token_counts) -> list:
        return []

    # ------------------------------------------------------------------ the Mixer interface

    def fold_input_norm(self, gain):
        """bfloat16 runs: an RMS norm's gain goes into the columns of the first matrix."""
        if self.w_in is None or self.w_in.dtype != torch.bfloat16 or self.w_in.shape[1] % 8:
            return False
        self.w_in = (self.w_in.float() * gain.to(self.w_in.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def replay_key(self, step):
        return self.mix_replay_key(step)

    def weights(self):
        return [t for t in (self.w_in, self.w_out) if t is not None] + self.mix_weights()

    def mix_weights(self) -> list:
        return []

    def scratch_requests(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        inner = self.mix_scratch(n_tokens, dtype)
        end = 1 + max([r.last_use for r in inner] + [0])
        return ([BufferRequest("proj", (n_tokens, self.in_width), dtype, 0, end),
                 BufferRequest("mixed", (n_tokens, self.out_width), dtype, 1, end + 1)]
                + [r.shifted(1) for r in inner])

    def kernel_shapes(self, dtype, token_counts):
        hidden, out = self.hidden, []
        for n in token_counts:
            out.append((f"input product, {n} tokens", "linear",
                        dict(m=n, n=self.in_width, k=hidden, in_dtype=dtype, out_dtype=dtype, lda=hidden, aligned=True)))
            out.append((f"output product, {n} tokens", "linear",
                        dict(m=n, n=hidden, k=self.out_width, in_dtype=dtype, out_dtype=torch.float32,
                             lda=self.out_width, aligned=True)))
        return out + self.mix_shapes(dtype, token_counts)

    def forward(self, h, ctx, entry, cache_entry, residual, emit=None, fresh=False):
        norm = h if isinstance(h, ops.FoldedNorm) else None
        if norm is not None:
            h = norm.rows
        n = h.shape[0]
        proj = ops.linear(h, self.w_in, self.b_in, out=ctx.scratch("proj", (n, self.in_width), h.dtype), norm=norm)
        out = ctx.scratch("mixed", (n, self.out_width), h.dtype)
        if out is None:
            out = torch.empty((n, self.out_width), dtype=h.dtype, device=h.device)
        self.mix(proj, ctx, entry, cache_entry, out, ctx.scratch)
        if fresh:
            ops.linear(out, self.w_out, out_dtype=torch.float32, out=residual)
        else:
            ops.linear(out, self.w_out, residual=residual, emit=emit)
