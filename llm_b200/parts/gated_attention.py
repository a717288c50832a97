"""Softmax attention with an element-wise output gate and, optionally, values that are the keys."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import build_position, register_mixer, to_run_dtype
from .projected import ProjectedMixer


class GatedAttentionMixer(ProjectedMixer):
    """Grouped-query softmax attention over a sliding window: q = W_q h, k = W_k h, partly rotated;
    v = W_v h, or (spec.values_are_keys) a key head's values are its keys as projected, before the
    rotation; the concatenated heads are multiplied element by element by sigmoid(W_g h)
    (spec.out_gate) before the output projection.

    One product [q; k; (v); gate], one launch that rotates queries and keys and writes keys and
    values into the paged cache (ops.norm_rope_cache_write without norms; for shared values it
    reads the value rows from the key columns), the library's attention kernels (a windowed layer
    keeps a ring of pages), the gate, the output product. Rotated keys and unrotated values are both
    cached: the attention kernels then need nothing new."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "projection_norm", "post_norm",
                 "attention_generic", "attention_decode", "attention_decode_window", "attention_prefill",
                 "attention_prefill_tc")

    def __init__(self, spec):
        s = spec
        if min(s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim) < 1 or s.n_heads % s.n_kv_heads or s.window < 0:
            raise FormatError("a gated attention needs positive sizes, heads in whole groups and a window that is not negative")
        if s.values_are_keys and s.value_dim != s.head_dim:
            raise FormatError(f"values that are the keys have the keys' size {s.head_dim}, not {s.value_dim}")
        if s.value_dim != s.head_dim:
            raise FormatError("the softmax attention kernels take values of the keys' size")
        self.spec = spec
        self.position = build_position(spec.position)

    @property
    def q_width(self):
        return self.spec.n_heads * self.spec.head_dim

    @property
    def k_width(self):
        return self.spec.n_kv_heads * self.spec.head_dim

    @property
    def v_width(self):
        return self.spec.n_kv_heads * self.spec.value_dim

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.value_dim

    @property
    def gate_offset(self):
        return self.q_width + self.k_width + (0 if self.spec.values_are_keys else self.v_width)

    @property
    def in_width(self):
        return self.gate_offset + (self.out_width if self.spec.out_gate else 0)

    def _roles(self):
        s = self.spec
        return ["q", "k"] + ([] if s.values_are_keys else ["v"]) + (["gate"] if s.out_gate else [])

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width, "gate": self.out_width}
        out = {t[r]: ParamSpec((widths[r], s.hidden)) for r in self._roles()}
        out[t["o"]] = ParamSpec((s.hidden, self.out_width))
        return out

    def bind(self, tensors, dtype, device):
        t = self.spec.tensor
        self.w_in = torch.cat([to_run_dtype(tensors[t[r]], dtype, device) for r in self._roles()]).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def kv_request(self):
        s = self.spec
        return KvRequest(s.n_kv_heads, s.head_dim, s.window)

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        # phases: 0 rotation + cache write, 1 attention
        return [BufferRequest("queries", (n_tokens, self.q_width), dtype, 0, 1)]

    def mix_replay_key(self, step):
        return ops.attention_replay_key(step, self.spec.n_heads, self.spec.n_kv_heads, self.spec.window)

    def mix_shapes(self, dtype, token_counts):
        s = self.spec
        return [("decode attention" if decode else "prefill attention", "attention",
                 dict(decode=decode, dtype=dtype, n_heads=s.n_heads, n_kv_heads=s.n_kv_heads, head_dim=s.head_dim,
                      window=s.window, packed=True, aligned=True)) for decode in (True, False)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        group, keys, values = ctx.cache.layer_view(cache_entry)
        table, ring = ctx.block_tables[group], ctx.cache.table_width(group)
        n = proj.shape[0]
        queries = scratch("queries", (n, self.q_width), proj.dtype)
        if queries is None:
            queries = torch.empty((n, self.q_width), dtype=proj.dtype, device=proj.device)
        ops.norm_rope_cache_write(proj, self.q_width, self.k_width, self.v_width, None, None, 0.0,
                                  self.position.table if self.position is not None else None, s.head_dim,
                                  self.position.interleaved if self.position is not None else False,
                                  ctx.tok_pos, ctx.tok_seq, queries, table, ring, keys, values,
                                  write_cache=(entry == cache_entry),
                                  value_source=self.q_width if s.values_are_keys else self.q_width + self.k_width)
        ops.attention(queries, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads, s.n_kv_heads,
                      s.head_dim, s.scale, s.window, out=out, decode=ctx.decode, seq_lens=ctx.seq_lens,
                      max_len=ctx.max_len, cu_seqlens=ctx.cu_seqlens, max_new=max(ctx.new_counts),
                      seq_order=ctx.seq_order)
        if s.out_gate:
            ops.sigmoid_gate_(out, proj[:, self.gate_offset:self.gate_offset + self.out_width])


register_mixer("gated_attention", GatedAttentionMixer)
