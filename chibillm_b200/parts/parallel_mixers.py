"""Two mixers side by side behind one input (ParallelMixersSpec): the result is
left_scale * left + right_scale * right.  Each branch adds into a 32-bit array of its
own, and one kernel adds the weighted two to the residual.  The branches' cache needs
are joined: the part asks for all of them and hands each branch its own views.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Mixer, Runtime, TensorSpec, make_mixer, register_mixer


def _own(names: Dict[str, str], prefix: str) -> Dict[str, str]:
    return {role[len(prefix):]: name for role, name in names.items() if role.startswith(prefix)}


class ParallelMixers(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.left = make_mixer(spec.left, _own(names, "left."), runtime)
        self.right = make_mixer(spec.right, _own(names, "right."), runtime)
        self._needs = []
        for branch in (self.left, self.right):
            need = branch.cache_need()
            self._needs.append(tuple(need) if isinstance(need, (tuple, list)) else (need,))

    def expected_tensors(self) -> List[TensorSpec]:
        return self.left.expected_tensors() + self.right.expected_tensors()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.left.bind(tensors)
        self.right.bind(tensors)

    def cache_need(self):
        return tuple(n for needs in self._needs for n in needs)

    def launch_key(self, ctx):
        keys = (self.left.launch_key(ctx), self.right.launch_key(ctx))
        return None if any(k is None for k in keys) else keys

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache):
        k = self.runtime.kernels
        views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        sums = []
        for tag, branch, needs in (("left", self.left, self._needs[0]), ("right", self.right, self._needs[1])):
            mine, views = views[:len(needs)], views[len(needs):]
            acc = ctx.workspace.get("parallel." + tag, tuple(residual.shape), torch.float32)
            k.zero(acc)
            left_over = branch.forward(x, acc, ctx, mine[0] if len(mine) == 1 else tuple(mine))
            if left_over is not None:
                left_over.add_into(acc)
            sums.append(acc)
        k.add_weighted(residual, sums[0], self.spec.left_scale, sums[1], self.spec.right_scale)
        return None


register_mixer("parallel_mixers", ParallelMixers, replace=True)
