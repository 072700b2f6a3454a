"""Attention over a shared low-rank latent.

Per position the layer keeps one vector: a latent c of `rank` values and one rotated key part r of `rot_dim`
values that all heads share.

    q      = x . Wq^T                      per head [dim unrotated | rot_dim rotated]
    d      = x . Wdkv^T                    [rank + rot_dim]
    c      = rms(d[:rank]) * norm weight;  r = rotate(d[rank:])             -> the request's pages, [c | r] per position
    per head h:  k_j = Wuk_h c_j,  v_j = Wuv_h c_j
                 s_j = (q_h[:dim] . k_j + rotate(q_h[dim:]) . r_j) * scale   for cached j <= the query's position
                 o_h = sum_j softmax(s)_j v_j
    out    = ( concat_h(o_h) * sigmoid(x . Wg^T) ) . Wo^T                    (`gate="element"`; None: no gate)

The rotation pairs (i, i + rot_dim/2) over the whole rotated part, with the position part's frequencies.

Keys and values are never expanded: q_h[:dim] . (Wuk_h c_j) = (Wuk_h^T q_h[:dim]) . c_j and
sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j), so the attention kernel runs every head against the cached
vectors themselves (query [rank | rot_dim], value = the latent) and two small per-head products sit before and
after it.  Scores, softmax and the weighted sum are 32-bit.

`kv_proj=False`: the layer has no Wdkv and reads the pages another layer wrote (that layer's `rank`, `rot_dim`
and rotation must equal this one's); everything else is its own.
"""
from __future__ import annotations

import torch

from .base import Mixer, PagedRowsNeed, ParamDecl, PartSpec, make_part, register_part

DEFAULT_NAMES = {"q": "attn_q.weight", "dkv": "attn_kv_down.weight", "dkv_norm": "attn_kv_norm.weight",
                 "uk": "attn_k_up.weight", "uv": "attn_v_up.weight", "g": "attn_gate.weight", "o": "attn_output.weight"}


class LatentAttention(Mixer):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True             # forward launches kernels only; nothing is read back to the host
    kernel_libs = ("latent_attention", "qkv_prepare")

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float, eps: float,
                 position: PartSpec, kv_proj: bool = True, gate="element", names=None):
        self.hidden, self.heads, self.dim, self.rot_dim = int(hidden), int(heads), int(dim), int(rot_dim)
        self.vdim, self.rank, self.scale, self.eps = int(vdim), int(rank), float(scale), float(eps)
        self.kv_proj, self.gate = bool(kv_proj), gate
        if gate not in (None, "element"):
            raise ValueError("gate is None or 'element'")
        if self.rot_dim % 2:
            raise ValueError("the rotated part has an even number of dimensions")
        self.position = make_part("position", position)
        if self.position.to_half_split(self.rot_dim) is not None:
            raise ValueError("the shared key part is rotated in the half-split pairing")
        self.names = {**DEFAULT_NAMES, **(names or {})}

    def params(self):
        nm, H, D, Dr, Dv, R, W = self.names, self.heads, self.dim, self.rot_dim, self.vdim, self.rank, self.hidden
        p = {nm["q"]: ParamDecl((H * (D + Dr), W)), nm["uk"]: ParamDecl((H * D, R)), nm["uv"]: ParamDecl((H * Dv, R)),
             nm["o"]: ParamDecl((W, H * Dv))}
        if self.kv_proj:
            p[nm["dkv"]] = ParamDecl((R + Dr, W))
            p[nm["dkv_norm"]] = ParamDecl((R,), "vector", init="norm_weight")
        if self.gate:
            p[nm["g"]] = ParamDecl((H * Dv, W))
        return p

    def cache_need(self):
        return PagedRowsNeed(self.rank + self.rot_dim)

    def bind(self, tensors, dtype):
        nm, H, D, Dr, Dv, R = self.names, self.heads, self.dim, self.rot_dim, self.vdim, self.rank
        mats = [tensors[nm["q"]]] + ([tensors[nm["g"]]] if self.gate else []) + ([tensors[nm["dkv"]]] if self.kv_proj else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()              # q | gate | latent: everything that reads x
        self.gate_at = H * (D + Dr)
        self.dkv_at = self.gate_at + (H * Dv if self.gate else 0)
        self.c_norm = tensors.get(nm["dkv_norm"])
        self.w_uk_t = tensors[nm["uk"]].reshape(H, D, R).transpose(1, 2).contiguous()     # [H, R, D]: q_h[:dim] -> the latent's space
        self.w_uv = tensors[nm["uv"]].reshape(H, Dv, R).contiguous()                      # [H, Dv, R]: the latent's space -> v
        self.w_o = tensors[nm["o"]]
        self.dtype = dtype

    def forward(self, x, step, cache, write_cache=True):
        ops, H, D, Dr, Dv, R = step.ops, self.heads, self.dim, self.rot_dim, self.vdim, self.rank
        y = ops.linear(x, self.w_in)
        N = y.shape[0]
        q = y[:, :self.gate_at].view(N, H, D + Dr)
        _, table = self.position.table(step, y.device)
        own = self.kv_proj and write_cache
        q_rot = ops.latent_prepare(q, y[:, self.dkv_at:self.dkv_at + R + Dr] if own else None, self.c_norm, self.eps, table,
                                   step, cache, H, D, Dr, R)
        q_lat = ops.head_linear(q[:, :, :D], self.w_uk_t)            # [N, H, R]
        o_lat = ops.latent_attention(q_lat, q_rot, step, cache, H, R, Dr, self.scale)
        o = ops.head_linear(o_lat, self.w_uv).view(N, H * Dv)
        if self.gate:
            o = ops.sigmoid_gate(o, y[:, self.gate_at:self.gate_at + H * Dv], H, Dv, False)
        return ops.linear(o, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
