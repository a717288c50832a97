"""Softmax attention with an element-wise output gate and, optionally, values that are the keys."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import build_position, register_mixer, to_float32, to_run_dtype
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
    cached: the attention kernels then need nothing new.

    The spec's switches (all off by default) ride in the same launches: `head_norm` in the launch that rotates
    (per-head RMS norms of queries and keys with weights the heads share), `value_mix` there too (the values are
    blended with those the first layer of the same name cached for the same token, before they are cached),
    `head_gate` (one gate per head), `softcap`, `unit_sink` and `out_scale` inside the attention kernels. Values
    may be wider or narrower than keys (the cache keeps a tensor for each; the kernel for any sizes runs)."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "projection_norm", "post_norm",
                 "attention_generic", "attention_decode", "attention_decode_window", "attention_prefill",
                 "attention_prefill_tc")

    def __init__(self, spec):
        s = spec
        if min(s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim) < 1 or s.n_heads % s.n_kv_heads or s.window < 0:
            raise FormatError("a gated attention needs positive sizes, heads in whole groups and a window that is not negative")
        if s.values_are_keys and s.value_dim != s.head_dim:
            raise FormatError(f"values that are the keys have the keys' size {s.head_dim}, not {s.value_dim}")
        if s.out_gate and s.head_gate:
            raise FormatError("a gated attention has a gate per element or a gate per head, not both")
        if s.value_mix is not None and s.values_are_keys:
            raise FormatError("values that are the keys cannot be blended with another layer's")
        self.spec = spec
        self.position = build_position(spec.position)
        self.q_gain = self.k_gain = self.sinks = None
        self.mix_weight = 0.0

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
    def gate_width(self):
        s = self.spec
        return self.out_width if s.out_gate else (s.n_heads if s.head_gate else 0)

    @property
    def in_width(self):
        return (self.gate_offset + self.gate_width + 7) // 8 * 8       # (rows of zeros fill up to a multiple of 8)

    def _roles(self):
        s = self.spec
        return ["q", "k"] + ([] if s.values_are_keys else ["v"]) + (["gate"] if s.out_gate or s.head_gate else [])

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width, "gate": self.gate_width}
        out = {t[r]: ParamSpec((widths[r], s.hidden)) for r in self._roles()}
        out[t["o"]] = ParamSpec((s.hidden, self.out_width))
        if s.head_norm:
            out[t["q_norm"]] = ParamSpec((s.head_dim,), "gain")
            out[t["k_norm"]] = ParamSpec((s.head_dim,), "gain")
        if s.value_mix is not None:
            out[t["value_mix"]] = ParamSpec((), "gate_scalar")         # (stored, but unused, in the first such layer too)
        return out

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        rows = [to_run_dtype(tensors[t[r]], dtype, device) for r in self._roles()]
        pad = self.in_width - sum(r.shape[0] for r in rows)
        if pad:
            rows.append(torch.zeros((pad, s.hidden), dtype=dtype, device=device))
        self.w_in = torch.cat(rows).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)
        if s.head_norm:
            self.q_gain = to_float32(tensors[t["q_norm"]], device)
            self.k_gain = to_float32(tensors[t["k_norm"]], device)
        if s.value_mix is not None:
            self.mix_weight = float(tensors[t["value_mix"]].float())
        if s.unit_sink:
            self.sinks = torch.zeros(s.n_heads, dtype=torch.float32, device=device)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def kv_request(self):
        s = self.spec
        return KvRequest(s.n_kv_heads, s.head_dim, s.window,
                         value_dim=s.value_dim if s.value_dim != s.head_dim else None)

    def mix_weights(self):
        return [t for t in (self.q_gain, self.k_gain) if t is not None]

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
        blend = {}
        if s.value_mix is not None:
            # the first layer of the name leaves where its values are cached; the others blend those in
            key = ("value_mix", s.value_mix)
            if s.value_mix_first:
                ctx.extras[key] = (values, table, ring)
            elif key in ctx.extras:
                first_values, first_table, first_ring = ctx.extras[key]
                blend = dict(mix_cache=first_values, mix_table=first_table, mix_ring=first_ring, mix=self.mix_weight)
            else:
                raise FormatError(f"values are blended with those of the first '{s.value_mix}' layer, which has not run")
        ops.norm_rope_cache_write(proj, self.q_width, self.k_width, self.v_width, self.q_gain, self.k_gain, s.norm_eps,
                                  self.position.table if self.position is not None else None, s.head_dim,
                                  self.position.interleaved if self.position is not None else False,
                                  ctx.tok_pos, ctx.tok_seq, queries, table, ring, keys, values,
                                  write_cache=(entry == cache_entry),
                                  value_source=self.q_width if s.values_are_keys else self.q_width + self.k_width,
                                  norm_unit=s.head_dim if s.head_norm else 0, **blend)
        gate = proj[:, self.gate_offset:self.gate_offset + s.n_heads] if s.head_gate else None
        ops.attention(queries, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads, s.n_kv_heads,
                      s.head_dim, s.scale, s.window, out=out, decode=ctx.decode, seq_lens=ctx.seq_lens,
                      max_len=ctx.max_len, cu_seqlens=ctx.cu_seqlens, max_new=max(ctx.new_counts),
                      seq_order=ctx.seq_order, sinks=self.sinks, gate=gate, out_scale=s.out_scale, softcap=s.softcap,
                      value_dim=s.value_dim)
        if s.out_gate:
            ops.sigmoid_gate_(out, proj[:, self.gate_offset:self.gate_offset + self.out_width])


register_mixer("gated_attention", GatedAttentionMixer)
