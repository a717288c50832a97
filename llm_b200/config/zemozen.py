"""Configuration of the Zemozen decoder, read from its own config.json keys.

A Zemozen model is a list of pre-norm layers with one constant m in front of both parts:
x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x)), RMS norms with plain weights. A layer's `type`
names its mixer: `attention` (grouped softmax attention over a sliding window, every head of queries and
keys normed on its own before a half-split rotation whose positions may be stretched by a factor, values
that may be blended with those of the first such layer, a sigmoid gate per head read from the mixer's
input) or `parallel` (two mixers on the same input, each with a scale: on the left a windowed attention
with interleaved rotation, soft-capped scores and a softmax whose denominator holds a one; on the right a
state-space recurrence with a scalar decay per head behind a short convolution). Its `mlp` is a routed
mixture of gated experts (scores by a softmax over all router outputs, the choice by score plus a stored
correction, some outputs standing for experts that hand their input through) or null. The embedding is
scaled; the head is a matrix of its own.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..errors import FormatError, Unsupported
from ..parts.spec import (BlockSpec, GatedAttentionSpec, ModelSpec, NormSpec, PositionSpec, RoutedExpertsSpec,
                          ScheduleEntry, SideBySideSpec, StateSpaceSpec, names)
from .base import ConfigReader

# no key of the configuration bounds a sequence: the engine's context does
MAX_POSITIONS = 1 << 22
# the layers whose values are blended share this name in their specs
VALUE_MIX = "v_mix"


@dataclass(frozen=True)
class ZemozenConfig:
    """`layers` keeps the configuration's list as JSON text per layer (hashable); the typed view is `model_spec()`."""
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: tuple

    architecture = "Zemozen"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "ZemozenConfig":
        r = ConfigReader(raw, where)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise FormatError(f"{where}: 'layers' must be a non-empty list")
        norm = ConfigReader(r.mapping("norm"), f"{where}: norm")
        embedding = r.mapping("embedding", None)
        scale = ConfigReader(embedding, f"{where}: embedding").number("scale", 1.0) if embedding is not None else 1.0
        config = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                     eps=norm.number("eps", positive=True), embedding_scale=scale,
                     residual_mult=r.number("residual_mult", 1.0),
                     layers=tuple(json.dumps(layer, sort_keys=True) for layer in layers))
        config.model_spec()            # every layer is read once here, so that a bad key is reported at load
        return config

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                "residual_mult": self.residual_mult, "layers": [json.loads(text) for text in self.layers]}

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"

    # ------------------------------------------------------------------ the model as data

    def _attention(self, p: str, raw: dict, where: str, pairing: str, out_scale: float, head_gate: bool,
                   unit_sink: bool, mix_first):
        """`mix_first`: None where the layer's values are not blended, else whether it is the first that says so."""
        m = ConfigReader(raw, where)
        heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise FormatError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        dim = m.integer("dim", minimum=1)
        vdim = m.integer("vdim", dim, minimum=1)
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
                factor = ConfigReader(sc, f"{where}: rot.scaling").number("factor", positive=True)
                scaling = tuple(sorted({"type": "linear", "factor": factor}.items()))
            position = PositionSpec(head_dim=dim, theta=rr.number("base", positive=True), max_positions=MAX_POSITIONS,
                                    scaling=scaling, pairing=pairing, rotary_dim=dims)
        mask = m.mapping("mask", None)
        window = ConfigReader(mask, f"{where}: mask").integer("size", 0, minimum=0) if mask is not None else 0
        roles = dict(q=p + "q", k=p + "k", v=p + "v", o=p + "o", q_norm=p + "q.norm", k_norm=p + "k.norm")
        if head_gate:
            roles["gate"] = p + "g"
        if mix_first is not None:
            roles["value_mix"] = p + "vmix"
        return GatedAttentionSpec(
            hidden=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, value_dim=vdim, scale=m.number("scale"),
            window=window, values_are_keys=False, out_gate=False, position=position, names=names(**roles),
            head_norm=True, norm_eps=self.eps, head_gate=head_gate, softcap=m.number("softcap", 0.0),
            unit_sink=unit_sink, value_mix=VALUE_MIX if mix_first is not None else None,
            value_mix_first=bool(mix_first), out_scale=out_scale)

    def _state_space(self, p: str, raw: dict, where: str, out_scale: float):
        m = ConfigReader(raw, where)
        heads, groups = m.integer("heads", minimum=1), m.integer("groups", minimum=1)
        if heads % groups:
            raise FormatError(f"{where}: {heads} heads are no multiple of {groups} groups")
        vdim, parts = m.integer("vdim", minimum=1), m.integer("norm_groups", 1, minimum=1)
        if (heads * vdim) % parts:
            raise FormatError(f"{where}: {heads * vdim} channels cannot be normed in {parts} equal parts")
        return StateSpaceSpec(
            hidden=self.width, n_heads=heads, value_dim=vdim, state=m.integer("state", minimum=1), groups=groups,
            conv_taps=m.integer("conv", minimum=1), norm_groups=parts, eps=self.eps, out_scale=out_scale,
            names=names(**{"in": p + "in"}, conv=p + "conv", conv_bias=p + "conv.b", dt_bias=p + "dt_bias",
                        a_log=p + "A_log", skip=p + "D", norm=p + "norm", o=p + "o"))

    def _feed_forward(self, p: str, raw: dict, where: str):
        f = ConfigReader(raw, where)
        kind = f.string("kind", "moe")
        if kind != "moe":
            raise Unsupported(f"{where}: kind '{kind}' (built: 'moe')")
        router = ConfigReader(f.mapping("router"), f"{where}: router")
        expert = ConfigReader(f.mapping("expert"), f"{where}: expert")
        outputs, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
        identity = router.integer("identity", 0, minimum=0)
        # `experts` counts the experts with tensors; the router has `identity` more outputs
        if top > outputs + identity:
            raise FormatError(f"{where}: top {top} of {outputs + identity} experts")
        return RoutedExpertsSpec(
            hidden=self.width, intermediate=expert.integer("ff", minimum=1), n_experts=outputs, top=top,
            router_bias=False, names=names(router=p + "router", correction=p + "correction"),
            expert_names=names(gate=p + "e{e}.gate", up=p + "e{e}.up", down=p + "e{e}.down"),
            scoring="all", correction=True, pass_through=identity, out_scale=self.residual_mult)

    def _norm(self, name: str):
        return NormSpec(self.width, self.eps, name)

    def model_spec(self) -> ModelSpec:
        blocks, mixes = [], 0
        for i, text in enumerate(self.layers):
            layer = json.loads(text)
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise FormatError(f"{where} is not an object")
            if not isinstance(layer.get("mixer"), dict):
                raise FormatError(f"{where}: 'mixer' must be an object")
            kind, p, m = layer.get("type"), f"l{i}.mix.", self.residual_mult
            if kind == "attention":
                blended = bool(ConfigReader(layer["mixer"], f"{where}.mixer").boolean("v_mix", False))
                mixer = self._attention(p, layer["mixer"], f"{where}.mixer", "half", m, True, False,
                                        (mixes == 0) if blended else None)
                mixes += blended
            elif kind == "parallel":
                sides = ConfigReader(layer["mixer"], f"{where}.mixer")
                left = self._attention(p + "left.", sides.mapping("left"), f"{where}.mixer.left", "interleaved",
                                       m * sides.number("left_scale", 1.0), False, True, None)
                right = self._state_space(p + "right.", sides.mapping("right"), f"{where}.mixer.right",
                                          m * sides.number("right_scale", 1.0))
                mixer = SideBySideSpec(left=left, right=right)
            else:
                raise Unsupported(f"{where}: a layer of type '{kind}' (built: 'attention', 'parallel')")
            mlp = layer.get("mlp")
            ffn = self._feed_forward(f"l{i}.mlp.", mlp, f"{where}.mlp") if mlp is not None else None
            blocks.append(BlockSpec(mixer_norm=self._norm(f"l{i}.norm1"), mixer=mixer,
                                    ffn_norm=self._norm(f"l{i}.norm2") if ffn is not None else None, feed_forward=ffn))
        return ModelSpec(
            architecture=self.architecture, vocab=self.vocab, hidden=self.width, max_positions=MAX_POSITIONS,
            embedding="embed", blocks=tuple(blocks), schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=self._norm("final.norm"), head="head", embedding_scale=self.embedding_scale)
