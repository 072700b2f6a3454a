"""Minimal gated recurrence (minGRU): gates that read only the current token.

    z = sigmoid(h . W_z^T + b_z)        u = h . W_x^T + b_x        cand = u + 1/2 (u >= 0),  sigmoid(u) (u < 0)
    S_t = (1 - z) S_{t-1} + z cand      (element by element, `width` channels)
    out = (S_t * silu(h . W_g^T)) . W_o^T

Kept per request: S [width] in 32-bit.  Gates, candidate and state are 32-bit in every mode.  The three
input projections run as one product.  `names` gives the tensors' names.
"""
from __future__ import annotations

import torch

from .base import Mixer, ParamDecl, StateNeed, register_part

DEFAULT_NAMES = {"z": "gru_z.weight", "z_bias": "gru_z.bias", "x": "gru_x.weight", "x_bias": "gru_x.bias",
                 "g": "gru_g.weight", "o": "gru_out.weight"}


class MinGru(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("min_gru",)

    def __init__(self, hidden: int, width: int, names=None):
        self.hidden, self.width = int(hidden), int(width)
        self.names = {**DEFAULT_NAMES, **(names or {})}

    def params(self):
        nm, W = self.names, self.width
        return {nm["z"]: ParamDecl((W, self.hidden)), nm["z_bias"]: ParamDecl((W,), "vector", init="conv"),
                nm["x"]: ParamDecl((W, self.hidden)), nm["x_bias"]: ParamDecl((W,), "vector", init="conv"),
                nm["g"]: ParamDecl((W, self.hidden)), nm["o"]: ParamDecl((self.hidden, W))}

    def cache_need(self):
        return StateNeed((self.width,))

    def bind(self, tensors, dtype):
        nm = self.names
        self.w_zxg = torch.cat([tensors[nm["z"]], tensors[nm["x"]], tensors[nm["g"]]], dim=0).contiguous()
        self.b_z, self.b_x, self.w_o = tensors[nm["z_bias"]], tensors[nm["x_bias"]], tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops = step.ops
        zxg = ops.linear(x, self.w_zxg)
        return ops.linear(ops.min_gru(zxg, self.b_z, self.b_x, cache.state, step, write_cache), self.w_o)


register_part("mixer", "min_gru", MinGru)
