"""A dense feed-forward with the PolyNorm activation: W_down act(W_up x).

act(z) = a N(z) + b N(z^2) + c N(z^3) + e, where the powers are taken element by element, N divides a token's
row of ``intermediate_size`` values by its root mean square (eps under the root), and a, b, c, e are four
learned numbers (one tensor [4]). The up product's result stays float32 until the activation has normed it (a
bfloat16 z would cost the activation a third of its traffic less and put three times z's rounding into the cubic
term);
the powers, the three root mean squares and the sum of the terms are float32.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Param, project, register_ffn, renamed


class PolyNormMLP(FeedForward):
    takes_normed = True
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.w_up = self.w_down = self.coeffs = None

    def _n(self, local):
        return renamed(self.spec, local)

    def params(self):
        c, f = self.spec.hidden_size, self.spec.intermediate_size
        return {
            self._n("up"): Param((f, c)),
            self._n("down"): Param((c, f)),
            self._n("act"): Param((4,), role="vector", mean=0.5),
        }

    def load(self, get):
        self.w_up, self.w_down, self.coeffs = get(self._n("up")), get(self._n("down")), get(self._n("act"))

    def forward(self, x, ctx, residual=None):
        z = project(self.rt, x, self.w_up, out_dtype=torch.float32)
        act = self.rt.ops.polynorm(z, self.coeffs, self.spec.eps, self.rt.dtype)
        return project(self.rt, act, self.w_down, residual=residual)


register_ffn("polynorm_mlp", PolyNormMLP)
