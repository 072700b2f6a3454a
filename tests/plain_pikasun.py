"""A plain, slow implementation of the Pikasun design: whole sequences, no cache, one function per
mechanism, float64 on the CPU.  It shares no code with the engine: the configuration is read as a
dict and the tensors as a dict of float64 tensors by stored name.

The design in short (T tokens, width W):

    x_0    = table[token]
    layer:   x += mixer(ln(x, norm1));   x += ff(ln(x, norm2))          (ff optional; ln has weight and bias)
    logits = cap * tanh(head . ln(x, final.norm) * logit_scale / cap)

with two kinds of mixer: grouped-query attention inside chunks of positions (`attention`: biased
projections, one RMS norm over the whole q and the whole k projection, pairwise-interleaved rotation,
one sigmoid gate per head) and attention over a shared low-rank latent (`latent_attention`: a normed
latent and one rotated key part per position, expanded per head; frequency-interpolated rotation;
an element-wise sigmoid gate), whose latent a later layer may borrow (`kv_from`).
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
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def layer_norm(x, weight, bias, eps):
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * weight + bias


def base_frequencies(base, dims):
    i = torch.arange(dims // 2, dtype=F64)
    return base ** (-2.0 * i / dims)


def interpolated_frequencies(base, dims, factor, original, fast, slow):
    """Frequencies of a rotation stretched for longer contexts: pairs that turn often within the
    original length keep their frequency, pairs that turn rarely are slowed by `factor`, with a
    linear ramp between.  Returns (frequencies, the factor on cos and sin)."""
    f = base_frequencies(base, dims)
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(fast)), 0)
    hi = min(math.ceil(where(slow)), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn(u, v, angles, magnitude=1.0):
    c, s = torch.cos(angles) * magnitude, torch.sin(angles) * magnitude
    return u * c - v * s, v * c + u * s


def rotate_interleaved(x, positions, freqs, dims):
    """x [T, heads, D]: the pair (x[2i], x[2i+1]), i < dims/2, turns by position * freqs[i]."""
    ang = (positions.to(F64)[:, None] * freqs[None, :])[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    a, b = turn(u, v, ang)
    out = x.clone()
    out[..., 0:dims:2] = a
    out[..., 1:dims:2] = b
    return out


def rotate_halves(x, positions, freqs, dims, magnitude=1.0):
    """x [T, heads, D]: the pair (x[i], x[i + dims/2]), i < dims/2, turns by position * freqs[i]."""
    half = dims // 2
    ang = (positions.to(F64)[:, None] * freqs[None, :])[:, None, :]
    a, b = turn(x[..., :half], x[..., half:dims], ang, magnitude)
    return torch.cat([a, b, x[..., dims:]], dim=-1)


def softmax_rows(scores, visible):
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1)


# ----------------------------------------------------------------------------- mixers
def chunk_attention(h, w, p, m, eps):
    """Grouped-query attention that sees back to the start of the query's chunk of `mask.size` positions."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms(q, eps, w[p + "q.norm"]).reshape(T, H, D)
    k = rms(k, eps, w[p + "k.norm"]).reshape(T, G, D)
    v = v.reshape(T, G, Dv)
    rot = m["rot"]
    if rot["dims"]:
        f = base_frequencies(rot["base"], rot["dims"])
        q = rotate_interleaved(q, pos, f, rot["dims"])
        k = rotate_interleaved(k, pos, f, rot["dims"])
    visible = pos[None, :] <= pos[:, None]
    if m.get("mask") is not None:                                # no mask given: plain causal attention
        size = m["mask"]["size"]
        visible = visible & ((pos[None, :] // size) == (pos[:, None] // size))
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    out = torch.zeros((T, H, Dv), dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        out[:, hd] = softmax_rows(s, visible) @ v[:, g] * gate[:, hd:hd + 1]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def latent_of(h, w, p, m, eps):
    """What a latent layer keeps per position: the normed latent [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    R, Dr = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms(d[:, :R], eps, w[p + "dkv.norm"])
    f, mag = latent_rotation(m)
    kr = rotate_halves(d[:, R:].reshape(T, 1, Dr), torch.arange(T), f, Dr, mag).reshape(T, Dr)
    return c, kr


def latent_rotation(m):
    rot = m["rot"]
    sc = rot.get("scaling")
    if sc is None:
        return base_frequencies(rot["base"], rot["dims"]), 1.0
    return interpolated_frequencies(rot["base"], rot["dims"], sc["factor"], sc["original"], sc["fast"], sc["slow"])


def latent_attention(h, w, p, m, eps, latent):
    """Causal attention whose keys and values are expanded per head from the latent `(c, kr)`."""
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = latent
    q = (h @ w[p + "q"].T).reshape(T, H, D + Dr)
    f, mag = latent_rotation(m)
    q_rot = rotate_halves(q[..., D:], torch.arange(T), f, Dr, mag)
    k_flat = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, Dv)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    out = torch.zeros((T, H, Dv), dtype=F64)
    for hd in range(H):
        s = (q[:, hd, :D] @ k_flat[:, hd].T + q_rot[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = softmax_rows(s, visible) @ v[:, hd]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward and the whole model
def clamped_glu(h, w, p, mlp):
    limit = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and, if asked, the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    latents, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            x = x + chunk_attention(h, w, p + "mix.", m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, p + "mix.", m, eps)
                src = i
            x = x + latent_attention(h, w, p + "mix.", m, eps, latents[src])
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + clamped_glu(h, w, p + "mlp.", layer["mlp"])
        layers.append(x)
    n = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = n @ w["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits
