"""Gated delta rule mixer.

    q, k = h . W_q^T, h . W_k^T   [kv_heads x dim]      v = h . W_v^T   [heads x vdim]       (no biases)
    each passes a short causal depthwise convolution over time (no bias) and SiLU
    q, k <- unit vectors per head: x / sqrt(sum(x^2) + 1e-6);  q also times dim^-1/2
    beta = sigmoid(h . W_b^T),   g = exp(-exp(A_log) * softplus(h . W_a^T + dt_bias))        one per head
    per head (head i reads q/k head i // (heads / kv_heads)):
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = ( o / rms(o) * norm weight * silu(h . W_g^T) ) . W_o^T                              rms over vdim

Kept per request: S [heads, dim, vdim] and the convolutions' last taps - 1 inputs, both 32-bit.  Unit
norms, beta, g, the state and the output norm are 32-bit in every mode.  The six input projections run as
one product and the three convolutions as one.  `names` gives the tensors' names.
"""
from __future__ import annotations

import torch

from .base import Mixer, ParamDecl, StateNeed, register_part

DEFAULT_NAMES = {"q": "delta_q.weight", "k": "delta_k.weight", "v": "delta_v.weight", "q_conv": "delta_q_conv.weight",
                 "k_conv": "delta_k_conv.weight", "v_conv": "delta_v_conv.weight", "b": "delta_beta.weight",
                 "a": "delta_a.weight", "a_log": "delta_a_log", "dt_bias": "delta_dt_bias", "g": "delta_gate.weight",
                 "norm": "delta_norm.weight", "o": "delta_out.weight"}
UNIT_EPS = 1e-6


class GatedDelta(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("causal_conv", "gated_delta")

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, names=None):
        self.hidden, self.heads, self.kv_heads = int(hidden), int(heads), int(kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads cannot share {self.kv_heads} query/key heads evenly")
        if self.taps < 1 or self.taps > 16:
            raise ValueError(f"the convolution kernels take 1 to 16 taps, not {self.taps}")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"the delta-rule kernel takes head sizes up to 256, not {self.dim}")
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.qk_cols, self.v_cols = 2 * self.kv_heads * self.dim, self.heads * self.vdim

    def params(self):
        nm, H, G, D, V, L, W = self.names, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.hidden
        conv = lambda c: ParamDecl((c, L), "vector", alt_shapes=((c, 1, L),), init="conv")
        return {nm["q"]: ParamDecl((G * D, W)), nm["k"]: ParamDecl((G * D, W)), nm["v"]: ParamDecl((H * V, W)),
                nm["q_conv"]: conv(G * D), nm["k_conv"]: conv(G * D), nm["v_conv"]: conv(H * V),
                nm["b"]: ParamDecl((H, W)), nm["a"]: ParamDecl((H, W)),
                nm["a_log"]: ParamDecl((H,), "vector", init="conv"), nm["dt_bias"]: ParamDecl((H,), "vector", init="conv"),
                nm["g"]: ParamDecl((H * V, W)), nm["norm"]: ParamDecl((V,), "vector", init="norm_weight"),
                nm["o"]: ParamDecl((W, H * V))}

    def cache_need(self):
        return (StateNeed((self.heads, self.dim, self.vdim)), StateNeed((max(self.taps - 1, 1), self.qk_cols + self.v_cols)))

    def bind(self, tensors, dtype):
        nm = self.names
        # one product for everything that reads h: q | k | v | gate | b | a
        self.w_all = torch.cat([tensors[nm[k]] for k in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous()
        self.conv_w = torch.cat([tensors[nm[k]].reshape(-1, self.taps) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w, self.w_o = tensors[nm["a_log"]], tensors[nm["dt_bias"]], tensors[nm["norm"]], tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops, H = step.ops, self.heads
        matrix_state, conv_state = cache
        y = ops.linear(x, self.w_all)
        c0 = self.qk_cols + self.v_cols
        c1 = c0 + self.v_cols
        qkv = ops.causal_conv(y[:, :c0], self.conv_w, None, conv_state.state, step, True, write_cache)
        o = ops.gated_delta(qkv, y[:, c1:c1 + H], y[:, c1 + H:c1 + 2 * H], y[:, c0:c1], self.a_log, self.dt_bias, self.norm_w,
                            self.eps, matrix_state.state, step, H, self.kv_heads, self.dim, self.vdim, write_cache, UNIT_EPS)
        return ops.linear(o, self.w_o)


register_part("mixer", "gated_delta", GatedDelta)
