"""Several mixers side by side on the same input: the result is the sum of ``scale_i * mixer_i(x)``.

Each branch is a mixer of its own kind with a cache of its own kind (pages for one, a state slot for another). What
the branches share is the two ends: their input matrices are stacked into ONE product over the mixer's input, and
their output matrices are laid side by side along the inner size, so that ONE product over the concatenated
activations gives the scaled sum (the scale of a branch rides on its activations, which the branch's last kernel
writes, in float32 before their rounding, into its own columns of the shared row). A branch therefore offers
``w_in`` and ``w_out`` after loading and ``core(proj, ctx, cache, write, out, out_scale)`` for what lies between.
"""

from __future__ import annotations

import torch

from .base import Mixer, build_part, mixer_class, project, register_mixer


class ParallelMixer(Mixer):
    takes_normed = True
    takes_out_dtype = True  # forward(..., out_dtype=) gives the result in that type when no residual is passed

    @classmethod
    def kernels(cls, spec):
        kinds = []
        for _prefix, branch, _scale in spec.branches:
            for kind in getattr(mixer_class(branch), "kernels", lambda s: ())(branch):
                if kind not in kinds:
                    kinds.append(kind)
        return tuple(kinds)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if not spec.branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.branches = [(prefix, build_part("mixer", branch, runtime), float(scale)) for prefix, branch, scale in spec.branches]
        for prefix, part, _ in self.branches:
            if not hasattr(part, "core"):
                raise ValueError(f"branch {prefix!r} ({type(part).__name__}) has no core(): it cannot share the two products")
        self.w_in = self.w_out = None
        self.in_spans, self.out_spans = [], []
        self.padded = False

    def params(self):
        return {prefix + name: p for prefix, part, _ in self.branches for name, p in part.params().items()}

    def load(self, get):
        for prefix, part, _ in self.branches:
            part.load(lambda name, prefix=prefix: get(prefix + name))
        at = 0
        for _, part, _ in self.branches:
            self.in_spans.append((at, at + part.w_in.shape[0]))
            at += part.w_in.shape[0]
        self.w_in = torch.cat([part.w_in for _, part, _ in self.branches], dim=0).contiguous()
        # every branch's columns start on a multiple of 8 elements (16 bytes of bfloat16); the columns added for that
        # are zeros in the matrix, and the activations there are zeroed once per step
        outs, at = [], 0
        for _, part, _ in self.branches:
            w = part.w_out
            width = w.shape[1]
            pad = -width % 8
            self.out_spans.append((at, at + width))
            if pad:
                w = torch.cat([w, torch.zeros((w.shape[0], pad), dtype=w.dtype, device=w.device)], dim=1)
                self.padded = True
            outs.append(w)
            at += width + pad
        self.w_out = torch.cat(outs, dim=1).contiguous()
        for _, part, _ in self.branches:  # the branches' own copies are not read again
            part.w_out = None
            if hasattr(part, "w_qkv"):
                part.w_qkv = None
            else:
                part.w_in = None

    def cache(self):
        return tuple(part.cache() for _, part, _ in self.branches)

    def forward(self, x, ctx, cache=None, residual=None, write=True, out_dtype=None):
        proj = project(self.rt, x, self.w_in)
        make = torch.zeros if self.padded else torch.empty
        acts = make((proj.shape[0], self.w_out.shape[1]), dtype=self.rt.dtype, device=proj.device)
        for (_, part, scale), (a, b), (oa, ob), view in zip(self.branches, self.in_spans, self.out_spans, cache):
            part.core(proj[:, a:b], ctx, view, write, out=acts[:, oa:ob], out_scale=scale)
        return project(self.rt, acts, self.w_out, out_dtype=out_dtype, residual=residual)


register_mixer("parallel_mixer", ParallelMixer)
