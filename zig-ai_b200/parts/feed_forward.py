"""SwiGLU feed-forward: `down( silu(gate(x)) * up(x) )`, no biases
(src/transformer/ffn.zig:7-34; device activation src/cuda/layer_kernels.cu:62-70; tensor names
src/transformer/hybrid_layer.zig:313-321).  The gate and up matrices are stacked into one
[2F, hidden] matrix at load so that one product feeds the activation.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamDecl, register_part


class SwiGlu(FeedForward):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("gemm_tc_pair",)       # gate/up products of many rows with the activation as their epilogue (bfloat16)

    def __init__(self, hidden: int, ff_dim: int):
        self.hidden, self.ff_dim = int(hidden), int(ff_dim)

    def params(self):
        return {
            "ffn_gate.weight": ParamDecl((self.ff_dim, self.hidden)),
            "ffn_up.weight": ParamDecl((self.ff_dim, self.hidden)),
            "ffn_down.weight": ParamDecl((self.hidden, self.ff_dim)),
        }

    def bind(self, tensors, dtype):
        self.w_gate_up = torch.cat([tensors["ffn_gate.weight"], tensors["ffn_up.weight"]], dim=0).contiguous()
        self.w_down = tensors["ffn_down.weight"]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        a = ops.linear_swiglu(x, self.w_gate_up, self.ff_dim)
        return ops.linear(a, self.w_down)


class DenseMlp(FeedForward):
    """`down( act(up(x)) )`, no gate and no biases; `activation` is one of gelu (the exact one, with erf),
    gelu_tanh, silu, relu.  `names` gives the two tensors' names."""
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True

    def __init__(self, hidden: int, ff_dim: int, activation: str = "gelu", names=None):
        self.hidden, self.ff_dim, self.activation = int(hidden), int(ff_dim), str(activation)
        if self.activation not in ("gelu", "gelu_erf", "gelu_tanh", "silu", "relu"):
            raise ValueError(f"unknown activation '{self.activation}'")
        self.names = {"up": "ffn_up.weight", "down": "ffn_down.weight", **(names or {})}

    def params(self):
        return {self.names["up"]: ParamDecl((self.ff_dim, self.hidden)),
                self.names["down"]: ParamDecl((self.hidden, self.ff_dim))}

    def bind(self, tensors, dtype):
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        return ops.linear(ops.linear_activation(x, self.w_up, self.activation), self.w_down)


class ClampedGlu(FeedForward):
    """A gated feed-forward with bounded branches, no biases:

        g = min(gate(x), limit);  u = clamp(up(x), -limit, limit);  out = down( g * sigmoid(alpha * g) * (u + 1) )

    The gate and up matrices are stacked into one [2F, hidden] matrix at load.  `names` gives the tensors' names."""
    accepts_lazy_input = True
    graph_safe = True

    def __init__(self, hidden: int, ff_dim: int, limit: float, alpha: float = 1.702, names=None):
        self.hidden, self.ff_dim, self.limit, self.alpha = int(hidden), int(ff_dim), float(limit), float(alpha)
        self.names = {"gate": "ffn_gate.weight", "up": "ffn_up.weight", "down": "ffn_down.weight", **(names or {})}

    def params(self):
        nm = self.names
        return {nm["gate"]: ParamDecl((self.ff_dim, self.hidden)), nm["up"]: ParamDecl((self.ff_dim, self.hidden)),
                nm["down"]: ParamDecl((self.hidden, self.ff_dim))}

    def bind(self, tensors, dtype):
        nm = self.names
        self.w_gate_up = torch.cat([tensors[nm["gate"]], tensors[nm["up"]]], dim=0).contiguous()
        self.w_down = tensors[nm["down"]]
        self.dtype = dtype

    def forward(self, x, step):
        ops = step.ops
        return ops.linear(ops.linear_clamped_glu(x, self.w_gate_up, self.ff_dim, self.limit, self.alpha), self.w_down)


register_part("feed_forward", "swiglu", SwiGlu)
register_part("feed_forward", "clamped_glu", ClampedGlu)
register_part("feed_forward", "dense", DenseMlp)
