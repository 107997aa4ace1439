"""Two mixers side by side: both read the same rows, each output is divided by its own root mean square over the
model width and multiplied by a weight of its own, and the result is the weighted sum of the two (half the sum:
their mean).  The two keep what they keep independently: the pair's cache need is the list of theirs (at most one
paged cache and one fixed-size state between them), and both get the entry's binding."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import MIXERS, BuildEnv, CacheBinding, Mixer, NormedBranches, StepContext, build_part, split_needs
from .spec import PartSpec, TensorDecl


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """params: ``left`` / ``right`` (PartSpecs of two mixers; their tensor names follow the pair's prefix),
    ``left_out`` / ``right_out`` (tensor names of the per-channel weights behind each branch's norm), ``eps``,
    ``coef`` (0.5: the mean)."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.left: Mixer = build_part(MIXERS, p["left"], env, prefix)
        self.right: Mixer = build_part(MIXERS, p["right"], env, prefix)
        self.eps = float(p["eps"])
        self.coef = float(p.get("coef", 0.5))
        self.names = (prefix + p.get("left_out", "left.out"), prefix + p.get("right_out", "right.out"))
        split_needs(self.cache_need())                     # refuses two of a kind

    @property
    def graph_capturable(self):
        return all(m.cache_need() is None or getattr(m, "graph_capturable", False) or
                   split_needs(m.cache_need())[1] is None for m in (self.left, self.right))

    def declare(self) -> List[TensorDecl]:
        h = self.env.hidden_size
        return (self.left.declare() + self.right.declare()
                + [TensorDecl(self.names[0], (h,), init="ones"), TensorDecl(self.names[1], (h,), init="ones")])

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.left.bind(tensors)
        self.right.bind(tensors)
        self.left_w, self.right_w = (tensors[n].contiguous() for n in self.names)
        if self.left_w.dtype != self.right_w.dtype:
            self.left_w, self.right_w = self.left_w.float(), self.right_w.float()

    def cache_need(self):
        return [n for m in (self.left, self.right) for n in split_needs(m.cache_need()) if n is not None]

    def kernel_libraries(self):
        return ["norm"] + self.left.kernel_libraries() + self.right.kernel_libraries()

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        a = self.left.forward(x, ctx, cache)
        b = self.right.forward(x, ctx, cache)
        return NormedBranches([(a, self.left_w), (b, self.right_w)], self.coef, self.eps)
