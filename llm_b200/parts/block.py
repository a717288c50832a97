"""How a layer's parts are arranged."""
from __future__ import annotations

import os

import torch

from .. import ops
from ..errors import Unsupported
from .base import (Block, Part, build_feed_forward, build_mixer, build_norm, register_block)

# LLMB_NO_FUSION=1: every norm stays a kernel of its own (for comparisons)
FOLD_NORMS = os.environ.get("LLMB_NO_FUSION", "0") in ("", "0")


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the norm feeds the part,
    the residual keeps the un-normed stream (apps/engine/src/model.rs:835-864 of
    MythEclipse/llm).

    In bfloat16 runs a norm is folded into the part behind it where that part offers it
    (`Part.fold_input_norm`): the part's first product reads the bfloat16 copy of the residual
    rows and scales by the norm's factor in its epilogue, and the product that last updated
    the residual (the part before, the block before, or the embedding) has left that copy and
    the rows' sums of squares. MythEclipse/llm fuses its norm into the consumer's input in the
    same spirit (apps/engine/kernels/gpu.cu:351-407). The feed-forward (with its norm) may be absent:
    a layer that only mixes."""

    #: `forward` takes `normed=` and `emit_next=` (see there)
    chains_norms = True

    def __init__(self, spec):
        self.spec = spec
        self.mixer_norm = build_norm(spec.mixer_norm)
        self.mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.ffn_norm = build_norm(spec.ffn_norm) if self.feed_forward is not None else None

    @property
    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    @property
    def libraries(self):
        return tuple(lib for p in self.parts for lib in p.libraries)

    def parameters(self):
        out = {}
        for p in self.parts:
            out.update(p.parameters())
        return out

    def bind(self, tensors, dtype, device):
        for p in self.parts:
            p.bind(tensors, dtype, device)
        self.folded_mixer = self._fold(self.mixer_norm, self.mixer, dtype)
        self.folded_ffn = self.feed_forward is not None and self._fold(self.ffn_norm, self.feed_forward, dtype)

    folded_mixer = folded_ffn = False

    @staticmethod
    def _fold(norm, part, dtype) -> bool:
        if not FOLD_NORMS or dtype != torch.bfloat16 or not getattr(norm, "foldable", False):
            return False
        return bool(part.fold_input_norm(norm.gain))

    def replay_key(self, step):
        keys = [p.replay_key(step) for p in self.parts]
        return None if any(k is None for k in keys) else tuple(keys)

    def input_emit(self, ctx, n_tokens: int, device):
        """Where the product that last updates the residual before this block leaves the folded
        mixer norm's input (None: the mixer norm is a kernel of its own)."""
        if not self.folded_mixer:
            return None
        return self._emit(ctx, "mixer", n_tokens, device)

    def _emit(self, ctx, which: str, n_tokens: int, device):
        hidden = self.spec.mixer_norm.size
        rows = ctx.scratch("h_" + which, (n_tokens, hidden), torch.bfloat16)
        sums = ctx.scratch("s_" + which, (n_tokens, ops.SUMSQ_LD), torch.float32)
        if rows is None or sums is None:
            rows = torch.empty((n_tokens, hidden), dtype=torch.bfloat16, device=device)
            sums = torch.empty((n_tokens, ops.SUMSQ_LD), dtype=torch.float32, device=device)
        return ops.Emit(rows, sums)

    def prepare(self, max_positions, device):
        for p in self.parts:
            p.prepare(max_positions, device)

    def weights(self):
        return [w for p in self.parts for w in p.weights()]

    def kernel_shapes(self, dtype, token_counts):
        return [shape for p in self.parts for shape in p.kernel_shapes(dtype, token_counts)]

    def scratch_requests(self, n_tokens, dtype):
        """The normed inputs of both halves plus what the mixer and the feed-forward
        declare, their phases lined up one after the other. A folded norm's input (bfloat16 rows
        and sums of squares) takes the normed input's place; the mixer's is written by the last
        product of the layer before, so it lives through the whole layer."""
        from ..engine.workspace import BufferRequest
        hidden = self.spec.mixer_norm.size
        mixer = self.mixer.scratch_requests(n_tokens, dtype)
        ffn = self.feed_forward.scratch_requests(n_tokens, dtype) if self.feed_forward is not None else []
        mixer_end = 1 + max([r.last_use for r in mixer] + [0])
        ffn_start = mixer_end + 2
        ffn_end = ffn_start + max([r.last_use for r in ffn] + [0])
        sums = (n_tokens, ops.SUMSQ_LD)
        if self.folded_mixer:
            out = [BufferRequest("h_mixer", (n_tokens, hidden), torch.bfloat16, 0, ffn_end + 1),
                   BufferRequest("s_mixer", sums, torch.float32, 0, ffn_end + 1)]
        else:
            out = [BufferRequest("h_mixer", (n_tokens, hidden), dtype, 0, mixer_end)]
        out += [r.shifted(1, "mixer.") for r in mixer]
        if self.folded_ffn:
            out += [BufferRequest("h_ffn", (n_tokens, hidden), torch.bfloat16, 1, ffn_end),
                    BufferRequest("s_ffn", sums, torch.float32, 1, ffn_end)]
        elif self.feed_forward is not None:
            out.append(BufferRequest("h_ffn", (n_tokens, hidden), dtype, mixer_end + 1, ffn_end))
        out += [r.shifted(ffn_start, "ffn.") for r in ffn]
        return out

    def forward(self, x, ctx, entry, cache_entry, normed=None, emit_next=None):
        """`normed` (an ops.Emit that was filled, or None): the folded mixer norm's input, left by
        the product that last updated x. `emit_next` (an ops.Emit, or None): where this block's
        last product leaves the same for the block that runs next."""
        views = ctx.workspace
        n = x.shape[0]

        def prefixed(prefix):
            if views is not None:
                views.prefix = prefix

        # ---- mixer
        if self.folded_mixer:
            if normed is None:
                normed = ops.cast_sumsq(x, self._emit(ctx, "mixer", n, x.device))
            h = ops.FoldedNorm(normed.rows, normed.sumsq, normed.parts, self.spec.mixer_norm.eps,
                               self.spec.mixer_norm.size)
        else:
            h = self.mixer_norm.forward(x, ctx.dtype, out=ctx.scratch("h_mixer", tuple(x.shape), ctx.dtype))
        emit_ffn = self._emit(ctx, "ffn", n, x.device) if self.folded_ffn else None
        if self.feed_forward is None:                  # the mixer is the layer's last part
            emit_ffn = emit_next
        prefixed("mixer.")
        if emit_ffn is not None and self.mixer.emits:
            self.mixer.forward(h, ctx, entry, cache_entry, x, emit=emit_ffn)
        else:
            self.mixer.forward(h, ctx, entry, cache_entry, x)
            if emit_ffn is not None:
                ops.cast_sumsq(x, emit_ffn)
        prefixed("")
        if self.feed_forward is None:
            return
        # ---- feed-forward
        if emit_ffn is not None:
            h = ops.FoldedNorm(emit_ffn.rows, emit_ffn.sumsq, emit_ffn.parts, self.spec.ffn_norm.eps,
                               self.spec.ffn_norm.size)
        else:
            h = self.ffn_norm.forward(x, ctx.dtype, out=ctx.scratch("h_ffn", tuple(x.shape), ctx.dtype))
        prefixed("ffn.")
        if emit_next is not None and self.feed_forward.emits:
            self.feed_forward.forward(h, ctx, x, emit=emit_next)
        else:
            self.feed_forward.forward(h, ctx, x)
            if emit_next is not None:
                prefixed("")
                ops.cast_sumsq(x, emit_next)
        prefixed("")


register_block("pre_norm", PreNormBlock)


class ParallelBlock(Block):
    """x += mixer(norm(x)) + feed_forward(norm(x)): one norm whose output both parts read; both
    add into the 32-bit residual stream. The feed-forward may be absent, or read a second norm of
    the same x (`ffn_norm` of the spec).

    In bfloat16 runs the norm is folded into both parts where both offer it (each multiplies the
    gain into its own first matrix; both products read the same bfloat16 rows and sums of squares
    that the last update of the stream left), and the block's last product leaves the same for
    the block that runs next."""

    chains_norms = True

    def __init__(self, spec):
        self.spec = spec
        self.norm = build_norm(spec.norm)
        self.mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        # a feed-forward with a norm of its own (of the same x): both norms are kernels of their own
        second = getattr(spec, "ffn_norm", None)
        self.ffn_norm = build_norm(second) if second is not None and self.feed_forward is not None else None
        self.folded = False

    @property
    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    @property
    def libraries(self):
        return tuple(lib for p in self.parts for lib in p.libraries)

    def parameters(self):
        out = {}
        for p in self.parts:
            out.update(p.parameters())
        return out

    def bind(self, tensors, dtype, device):
        for p in self.parts:
            p.bind(tensors, dtype, device)
        # all readers of the norm fold it, or none does (a part's weights change when it folds)
        self.folded = False
        if FOLD_NORMS and dtype == torch.bfloat16 and getattr(self.norm, "foldable", False) and self.ffn_norm is None:
            readers = [p for p in (self.mixer, self.feed_forward) if p is not None]
            if all(type(p).fold_input_norm is not Part.fold_input_norm for p in readers) \
                    and self.norm.spec.size % 8 == 0:
                answers = [bool(p.fold_input_norm(self.norm.gain)) for p in readers]
                if not all(answers):
                    if any(answers):
                        raise Unsupported("a parallel block whose parts do not agree on folding their norm")
                else:
                    self.folded = True

    def replay_key(self, step):
        keys = [p.replay_key(step) for p in self.parts]
        return None if any(k is None for k in keys) else tuple(keys)

    def input_emit(self, ctx, n_tokens: int, device):
        if not self.folded:
            return None
        hidden = self.spec.norm.size
        rows = ctx.scratch("h_block", (n_tokens, hidden), torch.bfloat16)
        sums = ctx.scratch("s_block", (n_tokens, ops.SUMSQ_LD), torch.float32)
        if rows is None or sums is None:
            rows = torch.empty((n_tokens, hidden), dtype=torch.bfloat16, device=device)
            sums = torch.empty((n_tokens, ops.SUMSQ_LD), dtype=torch.float32, device=device)
        return ops.Emit(rows, sums)

    def prepare(self, max_positions, device):
        for p in self.parts:
            p.prepare(max_positions, device)

    def weights(self):
        return [w for p in self.parts for w in p.weights()]

    def kernel_shapes(self, dtype, token_counts):
        return [shape for p in self.parts for shape in p.kernel_shapes(dtype, token_counts)]

    def scratch_requests(self, n_tokens, dtype):
        """The norm's output (or, folded, its input: bfloat16 rows and sums of squares, which the
        block before wrote and both parts read) lives through the whole block; this block's last
        product, which reads neither, writes the next block's into the same place."""
        from ..engine.workspace import BufferRequest
        hidden = self.spec.norm.size
        mixer = self.mixer.scratch_requests(n_tokens, dtype)
        ffn = self.feed_forward.scratch_requests(n_tokens, dtype) if self.feed_forward is not None else []
        mixer_end = 1 + max([r.last_use for r in mixer] + [0])
        ffn_start = mixer_end + 1
        ffn_end = ffn_start + max([r.last_use for r in ffn] + [0])
        sums = (n_tokens, ops.SUMSQ_LD)
        if self.folded:
            out = [BufferRequest("h_block", (n_tokens, hidden), torch.bfloat16, 0, ffn_end + 1),
                   BufferRequest("s_block", sums, torch.float32, 0, ffn_end + 1)]
        else:
            out = [BufferRequest("h_block", (n_tokens, hidden), dtype, 0, ffn_end)]
        if self.ffn_norm is not None:
            out.append(BufferRequest("h_ffn", (n_tokens, hidden), dtype, 0, ffn_end))
        out += [r.shifted(1, "mixer.") for r in mixer]
        out += [r.shifted(ffn_start, "ffn.") for r in ffn]
        return out

    def forward(self, x, ctx, entry, cache_entry, normed=None, emit_next=None):
        views = ctx.workspace
        n = x.shape[0]

        def prefixed(prefix):
            if views is not None:
                views.prefix = prefix

        # the feed-forward's own norm reads the same x as the mixer's: before the mixer adds into it
        if self.folded:
            if normed is None:
                normed = ops.cast_sumsq(x, self.input_emit(ctx, n, x.device))
            h = h_ffn = ops.FoldedNorm(normed.rows, normed.sumsq, normed.parts, self.spec.norm.eps, self.spec.norm.size)
        elif self.ffn_norm is not None and type(self.ffn_norm) is type(self.norm) and hasattr(self.norm, "forward_with"):
            h, h_ffn = self.norm.forward_with(self.ffn_norm, x, ctx.dtype,
                                              out=ctx.scratch("h_block", tuple(x.shape), ctx.dtype),
                                              out_other=ctx.scratch("h_ffn", tuple(x.shape), ctx.dtype))
        else:
            h = h_ffn = self.norm.forward(x, ctx.dtype, out=ctx.scratch("h_block", tuple(x.shape), ctx.dtype))
            if self.ffn_norm is not None:
                h_ffn = self.ffn_norm.forward(x, ctx.dtype, out=ctx.scratch("h_ffn", tuple(x.shape), ctx.dtype))
        last = self.feed_forward if self.feed_forward is not None else self.mixer
        prefixed("mixer.")
        if last is self.mixer and emit_next is not None and self.mixer.emits:
            self.mixer.forward(h, ctx, entry, cache_entry, x, emit=emit_next)
        else:
            self.mixer.forward(h, ctx, entry, cache_entry, x)
        if self.feed_forward is not None:
            prefixed("ffn.")
            if emit_next is not None and self.feed_forward.emits:
                self.feed_forward.forward(h_ffn, ctx, x, emit=emit_next)
            else:
                self.feed_forward.forward(h_ffn, ctx, x)
        prefixed("")
        if emit_next is not None and not last.emits:
            ops.cast_sumsq(x, emit_next)


register_block("parallel", ParallelBlock)


class SandwichBlock(Block):
    """x += post(mixer(pre(x))); x += post'(feed_forward(pre'(x))): every part stands between two
    norms, so a part's result is a stream of its own (32-bit, `y`) that is normed before it joins x.

    Launches beside the parts': the first norm of the layer (unless the layer before left it), and
    behind each part ONE kernel that norms the part's result, adds it to x and norms the new x for the
    part that runs next (ops.norm_add_): the mixer's post norm with the feed-forward's pre norm, the
    feed-forward's post norm with the next layer's first norm. A part that can write its result
    instead of adding it (`Part.overwrites`) gets `fresh=True`; for any other part y is zeroed first.
    A part may leave several partial results per token (`result_terms`, e.g. one per chosen expert):
    the kernel adds them in index order."""

    chains_norms = True

    def __init__(self, spec):
        self.spec = spec
        self.mixer_norm = build_norm(spec.mixer_norm)
        self.mixer = build_mixer(spec.mixer)
        self.mixer_post_norm = build_norm(spec.mixer_post_norm)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.ffn_norm = build_norm(spec.ffn_norm) if self.feed_forward is not None else None
        self.ffn_post_norm = build_norm(spec.ffn_post_norm) if self.feed_forward is not None else None
        for norm in (self.mixer_norm, self.mixer_post_norm, self.ffn_norm, self.ffn_post_norm):
            if norm is not None and not getattr(norm, "foldable", False):
                raise Unsupported("a sandwich block needs RMS norms (a gain and an eps) on both sides of its parts")

    @property
    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.feed_forward,
                                 self.ffn_post_norm) if p is not None)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    @property
    def libraries(self):
        return ("post_norm",) + tuple(lib for p in self.parts for lib in p.libraries)

    def parameters(self):
        out = {}
        for p in self.parts:
            out.update(p.parameters())
        return out

    def bind(self, tensors, dtype, device):
        for p in self.parts:
            p.bind(tensors, dtype, device)

    def replay_key(self, step):
        keys = [p.replay_key(step) for p in self.parts]
        return None if any(k is None for k in keys) else tuple(keys)

    def prepare(self, max_positions, device):
        for p in self.parts:
            p.prepare(max_positions, device)

    def weights(self):
        return [w for p in self.parts for w in p.weights()]

    def kernel_shapes(self, dtype, token_counts):
        return [shape for p in self.parts for shape in p.kernel_shapes(dtype, token_counts)]

    class _Normed:
        """What the block before leaves for this one: the first norm's output (run dtype), filled."""
        __slots__ = ("rows", "gain", "eps", "filled")

        def __init__(self, rows, gain, eps):
            self.rows, self.gain, self.eps, self.filled = rows, gain, eps, False

    @staticmethod
    def accepts_emit(emit) -> bool:
        return isinstance(emit, SandwichBlock._Normed)

    def input_emit(self, ctx, n_tokens: int, device):
        """Where the kernel that last updates x before this block leaves this block's first norm."""
        rows = ctx.scratch("h_first", (n_tokens, self.spec.mixer_norm.size), ctx.dtype)
        if rows is None:
            return None
        return SandwichBlock._Normed(rows, self.mixer_norm.gain, self.spec.mixer_norm.eps)

    @staticmethod
    def _terms(part) -> int:
        return int(getattr(part, "result_terms", 1))

    def scratch_requests(self, n_tokens, dtype):
        """h_first lives through the whole layer (this layer's last kernel writes the next layer's into
        it; the mixer has read it by then); y takes the part's result (terms rows a token)."""
        from ..engine.workspace import BufferRequest
        hidden = self.spec.mixer_norm.size
        mixer = self.mixer.scratch_requests(n_tokens, dtype)
        ffn = self.feed_forward.scratch_requests(n_tokens, dtype) if self.feed_forward is not None else []
        mixer_end = 1 + max([r.last_use for r in mixer] + [0])
        ffn_start = mixer_end + 2
        ffn_end = ffn_start + max([r.last_use for r in ffn] + [0])
        terms = max(self._terms(self.mixer), self._terms(self.feed_forward) if self.feed_forward is not None else 1)
        out = [BufferRequest("h_first", (n_tokens, hidden), dtype, 0, ffn_end + 2),
               BufferRequest("y_part", (n_tokens * terms, hidden), torch.float32, 0, ffn_end + 1)]
        out += [r.shifted(1, "mixer.") for r in mixer]
        if self.feed_forward is not None:
            out.append(BufferRequest("h_ffn", (n_tokens, hidden), dtype, mixer_end + 1, ffn_end))
            out += [r.shifted(ffn_start, "ffn.") for r in ffn]
        return out

    def _result(self, ctx, part, n, hidden, device):
        terms = self._terms(part)
        y = ctx.scratch("y_part", (n * terms, hidden), torch.float32)
        if y is None:
            y = torch.empty((n * terms, hidden), dtype=torch.float32, device=device)
        fresh = bool(getattr(part, "overwrites", False))
        if not fresh:
            ops.fill_(y, 0.0)
        return y, terms, fresh

    def forward(self, x, ctx, entry, cache_entry, normed=None, emit_next=None):
        """`normed`: this block's first norm as the block before left it (a filled _Normed), or None.
        `emit_next`: where this block's last kernel leaves the next block's first norm (a _Normed, or
        anything else / None: that block norms for itself)."""
        views = ctx.workspace
        n, hidden = x.shape
        s = self.spec

        def prefixed(prefix):
            if views is not None:
                views.prefix = prefix

        if isinstance(normed, SandwichBlock._Normed) and normed.filled:
            h = normed.rows
        else:
            h = self.mixer_norm.forward(x, ctx.dtype, out=ctx.scratch("h_first", (n, hidden), ctx.dtype))
        following = emit_next if isinstance(emit_next, SandwichBlock._Normed) else None
        y, terms, fresh = self._result(ctx, self.mixer, n, hidden, x.device)
        prefixed("mixer.")
        if fresh:
            self.mixer.forward(h, ctx, entry, cache_entry, y, fresh=True)
        else:
            self.mixer.forward(h, ctx, entry, cache_entry, y)
        prefixed("")
        if self.feed_forward is None:
            self._join(x, y, terms, self.mixer_post_norm, following)
            return
        h = ops.norm_add_(x, y, self.mixer_post_norm.gain, s.mixer_post_norm.eps, terms, self.ffn_norm.gain,
                          s.ffn_norm.eps, out=ctx.scratch("h_ffn", (n, hidden), ctx.dtype), out_dtype=ctx.dtype)
        y, terms, fresh = self._result(ctx, self.feed_forward, n, hidden, x.device)
        prefixed("ffn.")
        if fresh:
            self.feed_forward.forward(h, ctx, y, fresh=True)
        else:
            self.feed_forward.forward(h, ctx, y)
        prefixed("")
        self._join(x, y, terms, self.ffn_post_norm, following)

    @staticmethod
    def _join(x, y, terms, post_norm, following):
        if following is None:
            ops.norm_add_(x, y, post_norm.gain, post_norm.spec.eps, terms)
        else:
            ops.norm_add_(x, y, post_norm.gain, post_norm.spec.eps, terms, following.gain, following.eps,
                          out=following.rows, out_dtype=following.rows.dtype)
            following.filled = True


register_block("sandwich", SandwichBlock)
