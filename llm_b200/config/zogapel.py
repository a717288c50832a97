"""Configuration of the Zogapel decoder, read from its own config.json keys.

A Zogapel model is a list of layers, each with a norm in front of and behind both of its parts:
x += norm1b(mixer(norm1(x))); x += norm2b(feed_forward(norm2(x))), RMS norms whose weights are stored
around zero. A layer's `type` names its mixer: `delta` (the gated delta rule behind short
convolutions) or `attention` (grouped softmax attention over a sliding window whose values are its
keys before rotation, partly rotated heads with band-wise scaled frequencies, an element-wise
sigmoid gate on the result). Its `mlp` is `dense` (two matrices, tanh-form gelu), `moe` (routed
gated experts) or null. The embedding is scaled, and the head is the embedding table itself.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..errors import FormatError, Unsupported
from ..parts.spec import (DeltaRuleSpec, GatedAttentionSpec, MlpSpec, ModelSpec, NormSpec, PositionSpec,
                          RoutedExpertsSpec, SandwichBlockSpec, ScheduleEntry, names)
from .base import ConfigReader

# no key of the configuration bounds a sequence: the engine's context does
MAX_POSITIONS = 1 << 22
# the unit norms of the delta rule divide by sqrt(sum of squares + this)
UNIT_NORM_EPS = 1e-6


@dataclass(frozen=True)
class ZogapelConfig:
    """`layers` keeps the configuration's list as JSON text per layer (hashable); the typed view is `model_spec()`."""
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple

    architecture = "Zogapel"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "ZogapelConfig":
        r = ConfigReader(raw, where)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise FormatError(f"{where}: 'layers' must be a non-empty list")
        norm = ConfigReader(r.mapping("norm"), f"{where}: norm")
        embedding = r.mapping("embedding", None)
        scale = ConfigReader(embedding, f"{where}: embedding").number("scale", 1.0) if embedding is not None else 1.0
        config = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                     eps=norm.number("eps", positive=True), embedding_scale=scale,
                     layers=tuple(json.dumps(layer, sort_keys=True) for layer in layers))
        config.model_spec()            # every layer is read once here, so that a bad key is reported at load
        return config

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                "layers": [json.loads(text) for text in self.layers]}

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"

    # ------------------------------------------------------------------ the model as data

    @staticmethod
    def _heads(m, where):
        heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise FormatError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        return heads, kv_heads

    def _attention(self, p: str, raw: dict, where: str):
        m = ConfigReader(raw, where)
        heads, kv_heads = self._heads(m, where)
        dim = m.integer("dim", minimum=1)
        vdim = m.integer("vdim", dim, minimum=1)
        if vdim != dim:
            raise FormatError(f"{where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
        position = None
        rot = m.mapping("rot", None)
        if rot is not None:
            rr = ConfigReader(rot, f"{where}: rot")
            dims = rr.integer("dims", minimum=2)
            if dims % 2 or dims > dim:
                raise FormatError(f"{where}: rot.dims {dims} must be even and at most dim {dim}")
            scaling = None
            sc = rr.mapping("scaling", None)
            if sc is not None:
                ss = ConfigReader(sc, f"{where}: rot.scaling")
                scaling = tuple(sorted({"type": "ramp", "factor": ss.number("factor", positive=True),
                                        "original": ss.number("original", positive=True),
                                        "fast": ss.number("fast", positive=True),
                                        "slow": ss.number("slow", positive=True)}.items()))
            position = PositionSpec(head_dim=dim, theta=rr.number("base", positive=True), max_positions=MAX_POSITIONS,
                                    scaling=scaling, pairing="half", rotary_dim=dims)
        mask = m.mapping("mask", None)
        window = ConfigReader(mask, f"{where}: mask").integer("size", 0, minimum=0) if mask is not None else 0
        return GatedAttentionSpec(
            hidden=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, value_dim=vdim, scale=m.number("scale"),
            window=window, values_are_keys=True, out_gate=True, position=position,
            names=names(q=p + "q", k=p + "k", gate=p + "g", o=p + "o"))

    def _delta(self, p: str, raw: dict, where: str):
        m = ConfigReader(raw, where)
        heads, kv_heads = self._heads(m, where)
        return DeltaRuleSpec(
            hidden=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=m.integer("dim", minimum=1),
            value_dim=m.integer("vdim", minimum=1), conv_taps=m.integer("conv", minimum=1), eps=self.eps,
            unit_eps=UNIT_NORM_EPS,
            names=names(q=p + "q", k=p + "k", v=p + "v", q_conv=p + "q.conv", k_conv=p + "k.conv", v_conv=p + "v.conv",
                        beta=p + "b", decay=p + "a", a_log=p + "A_log", dt_bias=p + "dt_bias", gate=p + "g",
                        norm=p + "norm", o=p + "o"))

    def _feed_forward(self, p: str, raw: dict, where: str):
        f = ConfigReader(raw, where)
        kind = f.string("kind", "dense")
        if kind == "dense":
            return MlpSpec(hidden=self.width, intermediate=f.integer("ff", minimum=1), activation="gelu_tanh",
                           names=names(up=p + "up", down=p + "down"))
        if kind == "moe":
            router = ConfigReader(f.mapping("router"), f"{where}: router")
            expert = ConfigReader(f.mapping("expert"), f"{where}: expert")
            experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
            if top > experts:
                raise FormatError(f"{where}: top {top} of {experts} experts")
            return RoutedExpertsSpec(
                hidden=self.width, intermediate=expert.integer("ff", minimum=1), n_experts=experts, top=top,
                router_bias=True, names=names(router=p + "router", router_bias=p + "router.b"),
                expert_names=names(gate=p + "e{e}.gate", up=p + "e{e}.up", down=p + "e{e}.down"))
        raise Unsupported(f"{where}: kind '{kind}' (built: 'dense', 'moe')")

    def _norm(self, name: str):
        return NormSpec(self.width, self.eps, name, unit_offset=True)

    def model_spec(self) -> ModelSpec:
        blocks = []
        for i, text in enumerate(self.layers):
            layer = json.loads(text)
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise FormatError(f"{where} is not an object")
            if not isinstance(layer.get("mixer"), dict):
                raise FormatError(f"{where}: 'mixer' must be an object")
            kind, p = layer.get("type"), f"l{i}.mix."
            if kind == "attention":
                mixer = self._attention(p, layer["mixer"], f"{where}.mixer")
            elif kind == "delta":
                mixer = self._delta(p, layer["mixer"], f"{where}.mixer")
            else:
                raise Unsupported(f"{where}: a layer of type '{kind}' (built: 'attention', 'delta')")
            mlp = layer.get("mlp")
            ffn = self._feed_forward(f"l{i}.mlp.", mlp, f"{where}.mlp") if mlp is not None else None
            blocks.append(SandwichBlockSpec(
                mixer_norm=self._norm(f"l{i}.norm1"), mixer=mixer, mixer_post_norm=self._norm(f"l{i}.norm1b"),
                ffn_norm=self._norm(f"l{i}.norm2") if ffn is not None else None, feed_forward=ffn,
                ffn_post_norm=self._norm(f"l{i}.norm2b") if ffn is not None else None))
        return ModelSpec(
            architecture=self.architecture, vocab=self.vocab, hidden=self.width, max_positions=MAX_POSITIONS,
            embedding="embed", blocks=tuple(blocks), schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=self._norm("final.norm"), head=None, embedding_scale=self.embedding_scale)
