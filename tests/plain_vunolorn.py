"""A plain, slow implementation of the Vunolorn hybrid: whole sequences, no cache, one function per
mechanism, float64 on the CPU.  It shares no code with the engine: the configuration is read as a
dict and the tensors as a dict of float64 tensors by stored name.

The design in short (T tokens, width W):

    x_0   = table[token] * embedding.scale
    layer:  x += rms(mixer(rms(x, norm1)), norm1b);   x += rms(ff(rms(x, norm2)), norm2b)   (ff optional)
    logits = head . rms(x, final.norm)

with three kinds of mixer: a selective scan (`mamba1`), a gated delta rule (`delta`), and a pair
(`parallel`) of softmax attention beside a minimal gated recurrence, summed with two weights.
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir):
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F64)
    return out


# ----------------------------------------------------------------------------- small pieces
def rms(x, eps, weight=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times a weight if there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def causal_conv(x, taps, bias=None):
    """x [T, C], taps [C, L]: y[t, c] = sum_j taps[c, j] * x[t - (L-1) + j, c], zeros before t = 0."""
    T, C = x.shape
    L = taps.shape[1]
    padded = torch.cat([torch.zeros((L - 1, C), dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(L):
        y = y + padded[j:j + T] * taps[:, j][None, :]
    return y if bias is None else y + bias[None, :]


def rotate_half_split(x, positions, base, dims):
    """x [T, heads, D]: for i < dims/2 the pair (x[i], x[i + dims/2]) turns by position * base^(-2i/dims);
    dimensions from `dims` on are left alone."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- mixers
def selective_scan_mixer(h, W, p, m):
    """Mamba-style scan.  m: inner, state, dt_rank, conv."""
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :I], xz[:, I:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    proj = x @ W[p + "x"].T
    dt_in, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(dt_in @ W[p + "dt"].T + W[p + "dt.b"])              # [T, I]
    A = -torch.exp(W[p + "A_log"])                                   # [I, N]
    S = torch.zeros((I, N), dtype=F64)
    y = torch.zeros_like(x)
    for t in range(h.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def gated_delta_mixer(h, W, p, m, eps):
    """Gated delta rule.  m: heads, kv_heads, dim, vdim, conv."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                        # [T, H]
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))   # [T, H]
    gate = silu(h @ W[p + "g"].T).reshape(T, H, V)
    o = torch.zeros((T, H, V), dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros((D, V), dtype=F64)
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + k[t, kv][:, None] * u[None, :]
            o[t, hd] = S.T @ q[t, kv]
    o = rms(o, eps, W[p + "norm"]) * gate
    return o.reshape(T, H * V) @ W[p + "o"].T


def softmax_attention(h, W, p, m, eps):
    """Causal grouped-query attention with q/k norm, partial rotation and normed values."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms((h @ W[p + "q"].T).reshape(T, H, D), eps, W[p + "q.norm"])
    k = rms((h @ W[p + "k"].T).reshape(T, G, D), eps, W[p + "k.norm"])
    v = rms((h @ W[p + "v"].T).reshape(T, G, V), eps)
    pos = torch.arange(T)
    q = rotate_half_split(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half_split(k, pos, m["rot"]["base"], m["rot"]["dims"])
    out = torch.zeros((T, H, V), dtype=F64)
    mask = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for hd in range(H):
        kv = hd // (H // G)
        s = (q[:, hd] @ k[:, kv].T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, kv]
    return out.reshape(T, H * V) @ W[p + "o"].T


def min_gru_mixer(h, W, p, m):
    """S_t = (1 - z_t) S_{t-1} + z_t c_t with gates that see only the current token."""
    z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(m["width"], dtype=F64)
    out = torch.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    return (out * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    left = softmax_attention(h, W, p + "left.", m["left"], eps)
    right = min_gru_mixer(h, W, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ff(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


# ----------------------------------------------------------------------------- the model
def mixer(kind, h, W, p, m, eps):
    if kind == "mamba1":
        return selective_scan_mixer(h, W, p, m)
    if kind == "delta":
        return gated_delta_mixer(h, W, p, m, eps)
    if kind == "parallel":
        return parallel_mixer(h, W, p, m, eps)
    raise ValueError(kind)


def forward(c, W, tokens, layers_out=None):
    """Logits [T, vocab] for a whole sequence; `layers_out`, a list, receives x after every layer."""
    eps = c["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * c["embedding"]["scale"]
    for i, layer in enumerate(c["layers"]):
        p = f"l{i}."
        y = mixer(layer["type"], rms(x, eps, W[p + "norm1"]), W, p + "mix.", layer["mixer"], eps)
        x = x + rms(y, eps, W[p + "norm1b"])
        if layer.get("mlp") is not None:
            y = dense_ff(rms(x, eps, W[p + "norm2"]), W, p + "mlp.")
            x = x + rms(y, eps, W[p + "norm2b"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms(x, eps, W["final.norm"]) @ W["head"].T
