"""A routed feed-forward: a mixture of SwiGLU experts, a few per token, some of them identities.

Per token (all of the router in float32): scores = softmax(W_router x) over every router output; the choice goes by
score + correction among the outputs of the best groups of neighbours; the weights are the chosen outputs' plain
scores over their sum; the result is the weighted sum of the chosen experts' W_down (silu(W_gate x) * (W_up x)),
where a router output past the real experts stands for an expert that returns x. The experts' matrices are stacked
at load ([experts, 2 F, C] with the gate rows first, and [experts, C, F]), so the kernels address an expert by its
number.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, register_ffn, renamed


class RoutedExperts(FeedForward):
    chain_safe = True
    takes_out_dtype = True

    @classmethod
    def kernels(cls, spec):
        return ("moe",)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        outputs = s.num_experts + s.num_identity
        if s.num_experts < 1 or s.num_identity < 0:
            raise ValueError("a mixture needs at least one real expert")
        if s.groups < 1 or outputs % s.groups or not 1 <= s.keep_groups <= s.groups:
            raise ValueError(f"{outputs} router outputs do not form {s.groups} equal groups of which {s.keep_groups} stay")
        if not 1 <= s.top <= s.keep_groups * (outputs // s.groups):
            raise ValueError(f"top {s.top} exceeds what {s.keep_groups} groups of {outputs // s.groups} offer")
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        s = self.spec
        c, f, outputs = s.hidden_size, s.intermediate_size, s.num_experts + s.num_identity
        p = {
            self._n("router"): Param((outputs, c), role="vector"),  # held in float32: the router's own precision
            self._n("correction"): Param((outputs,), role="vector"),
        }
        for e in range(s.num_experts):
            p[self._n(f"e{e}.gate")] = Param((f, c))
            p[self._n(f"e{e}.up")] = Param((f, c))
            p[self._n(f"e{e}.down")] = Param((c, f))
        return p

    def load(self, get):
        s = self.spec
        self.w_router = get(self._n("router"))
        self.correction = get(self._n("correction"))
        self.w_gate_up = torch.stack(
            [torch.cat([get(self._n(f"e{e}.gate")), get(self._n(f"e{e}.up"))], dim=0) for e in range(s.num_experts)]
        ).contiguous()
        self.w_down = torch.stack([get(self._n(f"e{e}.down")) for e in range(s.num_experts)]).contiguous()

    def forward_update(self, x, ctx, h, a, scale_a, scale_b, mult):
        """h += mult * (scale_a * a + scale_b * experts(x)) in place on the float32 residual stream h, by the experts' last
        kernel: what a block whose sublayers' results meet the stream in one sum asks for."""
        s, ops = self.spec, self.rt.ops
        chosen, weights = ops.moe_route(x, self.w_router, self.correction, s.groups, s.keep_groups, s.top)
        return ops.moe_experts(x, self.w_gate_up, self.w_down, chosen, weights, update=(h, a, scale_a, scale_b, mult))

    def forward(self, x, ctx, residual=None, out_dtype=None):
        s, ops = self.spec, self.rt.ops
        chosen, weights = ops.moe_route(x, self.w_router, self.correction, s.groups, s.keep_groups, s.top)
        out = ops.moe_experts(x, self.w_gate_up, self.w_down, chosen, weights)  # float32 [N, C]
        if residual is not None:
            return ops.scaled_add(residual, out, None, None, None, 1.0)
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)


register_ffn("routed_experts", RoutedExperts)
