"""Selective-scan mixer (the Mamba recurrence).

    [x | z] = h . W_in^T                                   x, z: `inner` channels each
    x       = silu(causal_conv(x) + conv bias)             short depthwise convolution over time
    [dt_in | B | C] = x . W_x^T                            dt_rank, state, state columns
    dt      = softplus(dt_in . W_dt^T + dt bias)           one step size per channel
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n    A = -exp(A_log)
    y_c     = sum_n S[c, n] C_n + D_c x_c
    out     = (y * silu(z)) . W_o^T

Kept per request: the state S [inner, state] and the convolution's last taps - 1 inputs, both 32-bit.
Step sizes, decays, the state and its sums are 32-bit in every mode; the projections and the
convolution's output follow the model's dtype.  `names` gives the tensors' names.
"""
from __future__ import annotations

from .base import Mixer, ParamDecl, StateNeed, register_part

DEFAULT_NAMES = {"in": "ssm_in.weight", "conv": "ssm_conv1d.weight", "conv_bias": "ssm_conv1d.bias", "x": "ssm_x.weight",
                 "dt": "ssm_dt.weight", "dt_bias": "ssm_dt.bias", "a_log": "ssm_a", "d": "ssm_d", "o": "ssm_out.weight"}


class SelectiveScan(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("causal_conv", "selective_scan")

    def __init__(self, hidden: int, inner: int, state: int, dt_rank: int, taps: int, conv_bias: bool = True, names=None):
        self.hidden, self.inner, self.state, self.dt_rank, self.taps = int(hidden), int(inner), int(state), int(dt_rank), int(taps)
        self.conv_bias = bool(conv_bias)
        if self.taps < 1 or self.taps > 16:
            raise ValueError(f"the convolution kernels take 1 to 16 taps, not {self.taps}")
        if not 1 <= self.state <= 256:
            raise ValueError(f"the scan kernel takes 1 to 256 states per channel, not {self.state}")
        self.names = {**DEFAULT_NAMES, **(names or {})}

    def params(self):
        nm, I, S, R = self.names, self.inner, self.state, self.dt_rank
        p = {nm["in"]: ParamDecl((2 * I, self.hidden)),
             nm["conv"]: ParamDecl((I, self.taps), "vector", alt_shapes=((I, 1, self.taps),), init="conv"),
             nm["x"]: ParamDecl((R + 2 * S, I)),
             nm["dt"]: ParamDecl((I, R)),
             nm["dt_bias"]: ParamDecl((I,), "vector", init="conv"),
             nm["a_log"]: ParamDecl((I, S), "vector", init="conv"),
             nm["d"]: ParamDecl((I,), "vector", init="norm_weight"),
             nm["o"]: ParamDecl((self.hidden, I))}
        if self.conv_bias:
            p[nm["conv_bias"]] = ParamDecl((I,), "vector", init="conv")
        return p

    def cache_need(self):
        return (StateNeed((self.inner, self.state)), StateNeed((max(self.taps - 1, 1), self.inner)))

    def bind(self, tensors, dtype):
        nm = self.names
        self.w_in, self.w_x, self.w_dt, self.w_o = tensors[nm["in"]], tensors[nm["x"]], tensors[nm["dt"]], tensors[nm["o"]]
        self.conv_w = tensors[nm["conv"]].reshape(self.inner, self.taps).contiguous()
        self.conv_b = tensors.get(nm["conv_bias"])
        self.dt_b, self.a_log, self.d = tensors[nm["dt_bias"]], tensors[nm["a_log"]], tensors[nm["d"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops, I = step.ops, self.inner
        scan_state, conv_state = cache
        xz = ops.linear(x, self.w_in)
        xc = ops.causal_conv(xz[:, :I], self.conv_w, self.conv_b, conv_state.state, step, True, write_cache)
        proj = ops.linear(xc, self.w_x)
        y = ops.selective_scan(xc, proj, xz[:, I:], self.w_dt, self.dt_b, self.a_log, self.d, scan_state.state, step,
                               self.dt_rank, write_cache)
        return ops.linear(y, self.w_o)


register_part("mixer", "selective_scan", SelectiveScan)
