"""A feed-forward of routed experts."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import FormatError, Unsupported
from ..weights.loader import ParamSpec
from .base import FeedForward, register_feed_forward, to_float32, to_run_dtype


class RoutedExperts(FeedForward):
    """Every token goes to the `top` experts with the largest router logits (W_r h + bias, 32-bit;
    h is the normed input in the run's dtype) and gets their results weighted by the softmax over
    the chosen logits; an expert is down(silu(gate h) * (up h)).

    One call of ops.routed_experts: the router, a plan made on the device (the tokens of each
    expert, cut into tiles; nothing comes back to the host, so a step can be captured), one grouped
    product for gate and up with the activation in its epilogue, one for down with the routing
    weight (tcgen05 tiles of 128 rows where a step brings many rows an expert, tiles of 32 else).
    Each (token, chosen expert) leaves a 32-bit row of its own; the sum over a token's rows, in the
    order of choice, is taken by whoever reads them (`result_terms` rows a token when written
    fresh; else they are added into the residual here).

    With the spec's `scoring` 'all' the scores are the softmax over every router output, the choice is by score
    plus a stored correction, and the weights are the chosen scores over their sum; with `pass_through` the
    router's last outputs stand for experts without matrices that hand their input through; `out_scale`
    multiplies the weights. All of it is the router kernel's work (and one small launch for the rows handed
    through): the plan and the grouped products see the assignments of experts with matrices only."""
    graph_safe = True
    overwrites = True
    libraries = ("routed_experts", "post_norm")

    def __init__(self, spec):
        s = spec
        if s.activation != "silu":
            raise Unsupported(f"activation '{s.activation}' in routed experts")
        if min(s.hidden, s.intermediate, s.n_experts, s.top) < 1 or s.pass_through < 0 or s.top > s.n_experts + s.pass_through:
            raise FormatError(f"{s.top} of {s.n_experts + max(s.pass_through, 0)} experts cannot be chosen")
        if s.scoring not in ("chosen", "all"):
            raise Unsupported(f"scoring '{s.scoring}' in routed experts (built: 'chosen', 'all')")
        if s.correction and s.scoring != "all":
            raise Unsupported("a correction of the choice needs scores over all experts")
        self.spec = spec
        self.router = self.router_bias = self.correction = self.w_up = self.w_down = None

    @property
    def result_terms(self):
        return self.spec.top

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        outputs = s.n_experts + s.pass_through
        out = {t["router"]: ParamSpec((outputs, s.hidden))}
        if s.router_bias:
            out[t["router_bias"]] = ParamSpec((outputs,), "bias")
        if s.correction:
            out[t["correction"]] = ParamSpec((outputs,), "bias")
        for e in range(s.n_experts):
            names = s.expert_tensor(e)
            out[names["gate"]] = ParamSpec((s.intermediate, s.hidden))
            out[names["up"]] = ParamSpec((s.intermediate, s.hidden))
            out[names["down"]] = ParamSpec((s.hidden, s.intermediate))
        return out

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        self.router = to_float32(tensors[t["router"]], device)          # the router is 32-bit in every run
        self.router_bias = to_float32(tensors[t["router_bias"]], device) if s.router_bias else None
        self.correction = to_float32(tensors[t["correction"]], device) if s.correction else None
        ups, downs = [], []
        for e in range(s.n_experts):
            names = s.expert_tensor(e)
            ups.append(torch.cat([to_run_dtype(tensors[names["gate"]], dtype, device),
                                  to_run_dtype(tensors[names["up"]], dtype, device)]))
            downs.append(to_run_dtype(tensors[names["down"]], dtype, device))
        self.w_up = torch.stack(ups).contiguous()                      # [E, 2 F, hidden]
        self.w_down = torch.stack(downs).contiguous()                  # [E, hidden, F]

    def weights(self):
        """A decode step reads the router and, per token, `top` experts (counted as if all differed)."""
        return [self.router]

    def replay_key(self, step):
        return ()

    def scratch_requests(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        a = n_tokens * s.top
        plan = (s.n_experts + 2 + 3 * ((a + 31) // 32 + s.n_experts),)
        out = [BufferRequest("route_ids", (a,), torch.int32, 0, 0), BufferRequest("route_weights", (a,), torch.float32, 0, 0),
               BufferRequest("route_order", (a,), torch.int32, 0, 0), BufferRequest("route_plan", plan, torch.int32, 0, 0),
               BufferRequest("expert_act", (a, s.intermediate), dtype, 0, 0),
               BufferRequest("expert_rows", (a, s.hidden), torch.float32, 0, 0)]
        if ops.routed_experts_wide(n_tokens, s.top, s.n_experts, s.hidden, s.intermediate, dtype):
            out.append(BufferRequest("expert_in", (a, s.hidden), dtype, 0, 0))       # the rows of h in the plan's order
        return out

    def forward(self, h, ctx, residual, fresh=False):
        s = self.spec
        n, a = h.shape[0], h.shape[0] * s.top
        plan_ints = ops.routed_experts_plan_ints(n, s.top, s.n_experts)

        def buffer(name, shape, dtype):
            t = ctx.scratch(name, shape, dtype)
            return t if t is not None else torch.empty(shape, dtype=dtype, device=h.device)

        ids, weights = buffer("route_ids", (a,), torch.int32), buffer("route_weights", (a,), torch.float32)
        order, plan = buffer("route_order", (a,), torch.int32), buffer("route_plan", (plan_ints,), torch.int32)
        act = buffer("expert_act", (a, s.intermediate), h.dtype)
        rows = residual if fresh else buffer("expert_rows", (a, s.hidden), torch.float32)
        wide = ops.routed_experts_wide(n, s.top, s.n_experts, s.hidden, s.intermediate, h.dtype)
        gathered = buffer("expert_in", (a, s.hidden), h.dtype) if wide else None
        ops.routed_experts(h, self.router, self.router_bias, self.w_up, self.w_down, s.top, ids, weights, order, plan,
                           act, rows, gathered, scoring=1 if s.scoring == "all" else 0, correction=self.correction,
                           pass_through=s.pass_through, weight_scale=s.out_scale)
        if not fresh:
            ops.add_terms_(residual, rows, s.top)


register_feed_forward("routed_experts", RoutedExperts)
