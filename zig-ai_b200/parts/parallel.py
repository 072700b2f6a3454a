"""Two mixers side by side: both read the same input, their outputs are summed with two weights,

    out = left_scale * left(h) + right_scale * right(h)

Each keeps its own cache; the pair's needs are the left one's followed by the right one's.  The tensors
of the two are told apart by the prefixes `left_prefix` and `right_prefix` in front of their own names.
"""
from __future__ import annotations

from .base import Mixer, ParamDecl, make_part, needs_of, register_part


class ParallelMixers(Mixer):
    accepts_lazy_input = False    # the normed input is made once and read twice

    def __init__(self, left, right, left_scale: float = 1.0, right_scale: float = 1.0,
                 left_prefix: str = "left.", right_prefix: str = "right."):
        self.left, self.right = make_part("mixer", left), make_part("mixer", right)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.left_prefix, self.right_prefix = left_prefix, right_prefix
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))
        self.kernel_libs = tuple(getattr(self.left, "kernel_libs", ())) + tuple(getattr(self.right, "kernel_libs", ()))

    def params(self):
        p = {self.left_prefix + k: d for k, d in self.left.params().items()}
        p.update({self.right_prefix + k: d for k, d in self.right.params().items()})
        return p

    def cache_need(self):
        needs = needs_of(self.left) + needs_of(self.right)
        return needs if needs else None

    def bind(self, tensors, dtype):
        for part, prefix in ((self.left, self.left_prefix), (self.right, self.right_prefix)):
            part.bind({k: tensors[prefix + k] for k in part.params()}, dtype)

    @staticmethod
    def _share(part, views):
        from ..cache.manager import CacheView
        need = part.cache_need() if hasattr(part, "cache_need") else None
        if need is None:
            return CacheView()
        return tuple(views) if isinstance(need, (tuple, list)) else views[0]

    def forward(self, x, step, cache, write_cache=True):
        views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        n_left = len(needs_of(self.left))
        a = self.left.forward(x, step, self._share(self.left, views[:n_left]), write_cache)
        b = self.right.forward(x, step, self._share(self.right, views[n_left:]), write_cache)
        return step.ops.weighted_sum(a, b, self.left_scale, self.right_scale)


register_part("mixer", "parallel", ParallelMixers)
