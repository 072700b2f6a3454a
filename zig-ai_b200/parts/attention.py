"""Grouped-query attention over the paged cache.

    q = x.Wq^T [N,Hq,D]   k = x.Wk^T, v = x.Wv^T [N,Hkv,D]       (no biases)
    q, k = rms(q, q_norm), rms(k, k_norm)  per head over D           (if qk_norm)
    q, k = position(q, k)                                           (v is neither normed nor rotated)
    k, v of the new positions are written into the request's pages
    s = q.k^T * scale over the request's cached positions <= the query's (and inside the window)
    out = softmax(s).v  -> [N, Hq*D] . Wo^T

Options beside that: `scale` (default 1/sqrt(D)); `value_dim`, a value head size Dv other than D; `value_norm`,
values divided by their root mean square over Dv (no weight) before they are cached; `names`, the
tensors' names.  With Dv != D every head is kept at max(D, Dv) with zeros behind its own values (zeros
change neither a score nor a sum), so the same pages and kernels serve; the q/k norm still averages
over D.

Reference: projections src/transformer/hybrid_attn.zig:285-354, per-head norm :371-382 (device
:719,723), scale 1/sqrt(D) :571, causal mask :587, softmax :578-600, query head hq reads kv head
hq // (Hq/Hkv) :553-569 and src/cuda/paged_attention.cu:142, output projection :622-640; tensor
names :250-267.  Softmax and the norms are 32-bit.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedKVNeed, ParamDecl, make_part, register_part, PartSpec


class Attention(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool, eps: float,
                 position: PartSpec, window=None, scale=None, kv_proj: bool = True, value_dim=None,
                 value_norm: bool = False, names=None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot share {self.kv_heads} key/value heads evenly")
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.kv_proj = bool(kv_proj)
        self.position = make_part("position", position)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        self.value_norm = bool(value_norm)
        if (self.value_norm or self.value_dim != self.head_dim) and not self.kv_proj:
            raise ValueError("a value norm or a value head size of its own needs the layer's own k/v projections")
        self.cache_dim = max(self.head_dim, self.value_dim)      # the head size of the pages and the kernels
        self.names = {"q": "attn_q.weight", "k": "attn_k.weight", "v": "attn_v.weight", "o": "attn_output.weight",
                      "q_norm": "attn_q_norm.weight", "k_norm": "attn_k_norm.weight", **(names or {})}

    def params(self):
        q_dim, kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        nm = self.names
        p = {nm["q"]: ParamDecl((q_dim, self.hidden)),
             nm["o"]: ParamDecl((self.hidden, self.heads * self.value_dim))}
        if self.kv_proj:
            p[nm["k"]] = ParamDecl((kv_dim, self.hidden))
            p[nm["v"]] = ParamDecl((self.kv_heads * self.value_dim, self.hidden))
        if self.qk_norm:
            p[nm["q_norm"]] = ParamDecl((self.head_dim,), "vector", init="norm_weight")
            if self.kv_proj:
                p[nm["k_norm"]] = ParamDecl((self.head_dim,), "vector", init="norm_weight")
        return p

    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.cache_dim, self.window)

    def bind(self, tensors, dtype):
        nm = self.names
        mats = [tensors[nm["q"]]]
        if self.kv_proj:
            mats += [tensors[nm["k"]], tensors[nm["v"]]]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[nm["o"]]
        self.q_norm = tensors.get(nm["q_norm"])
        self.k_norm = tensors.get(nm["k_norm"])
        self.norm_eps = self.eps
        D, Dv, Dp = self.head_dim, self.value_dim, self.cache_dim
        if Dp != D and self.qk_norm:
            # the kernels average a head's squares over the Dp values they see, of which Dp - D are zero:
            # mean_D = mean_Dp * Dp / D, so  rsqrt(mean_D + eps) = rsqrt(mean_Dp + eps D / Dp) * sqrt(D / Dp)
            grow = lambda g: None if g is None else torch.cat([g * (D / Dp) ** 0.5, g.new_zeros(Dp - D)]).contiguous()
            self.q_norm, self.k_norm, self.norm_eps = grow(self.q_norm), grow(self.k_norm), self.eps * D / Dp
        if Dp != Dv:
            # the heads come out of attention Dp wide with zeros behind their Dv values: the output
            # projection gets zero columns there
            w = self.w_o.reshape(self.hidden, self.heads, Dv)
            self.w_o = torch.cat([w, w.new_zeros(self.hidden, self.heads, Dp - Dv)], dim=2).reshape(self.hidden, -1).contiguous()
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops = step.ops
        write = write_cache and self.kv_proj
        qkv = ops.linear(x, self.w_qkv)
        if self.value_norm or self.value_dim != self.head_dim:
            qkv = ops.value_norm_pad(qkv, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.eps, self.value_norm)
        rot = self.position.rotary()
        fused = getattr(ops, "fused_decode_attention_available", None)
        if (rot is not None and step.decode_only and self.kv_proj and fused is not None
                and fused(qkv.dtype, self.heads, self.kv_heads, self.cache_dim)):
            # every row is one token: norm, rotation, page write, attention and the combination of
            # the key chunks run as one kernel
            o = ops.decode_attention_fused(qkv, self.q_norm, self.k_norm, self.norm_eps, rot[0], rot[1], step, cache,
                                           self.heads, self.kv_heads, self.cache_dim, self.scale, self.window, write)
            return ops.linear(o, self.w_o)
        if rot is not None:
            q, _ = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.norm_eps, rot[0], rot[1], step, cache,
                                    self.heads, self.kv_heads, self.cache_dim, self.kv_proj, write, False)
        else:
            q, k = ops.qk_norm_rope(qkv, self.q_norm, self.k_norm, self.norm_eps, 0, 1.0, step, cache,
                                    self.heads, self.kv_heads, self.cache_dim, self.kv_proj, False, self.kv_proj)
            q, k = self.position.apply(q, k, step.positions, step)
            if write:
                v = qkv[:, (self.heads + self.kv_heads) * self.cache_dim:]
                ops.kv_write(k, v, step, cache, self.kv_heads, self.cache_dim)
        o = ops.paged_attention(q, step, cache, self.heads, self.kv_heads, self.cache_dim, self.scale, self.window)
        return ops.linear(o, self.w_o)


register_part("mixer", "attention", Attention)
