"""Configuration of the Pikasun design, read from its own config.json keys.

    architecture    "Pikasun"
    vocab, width    vocabulary and model width
    norm.eps        eps of every norm (layer norms, q/k norms, the latent's norm), inside the root
    logit_scale     factor on the head's product
    logit_softcap   cap c of the logits, c * tanh(logits / c) (absent or null: none)
    layers          one entry per layer: `type` (which mixer), `mixer` (its sizes and constants), `mlp` (null, or
                    {kind: "dense", ff, limit})

Mixers by `type`:
    attention         heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size}
                      grouped-query attention inside chunks of `mask.size` positions (no `mask`: plain causal)
    latent_attention  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling {factor, original, fast, slow}},
                      kv_from (optional: the layer whose cached latent this layer reads instead of making its own)
Every size and constant comes from the file; nothing is assumed equal to anything else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, read_key

ARCHITECTURE = "Pikasun"
MAX_POSITIONS = 1 << 20      # the design names no limit; block tables and graphs are sized by the cache, not by this
MLP_KINDS = ("dense",)


def _object(d, key, where, required=True):
    v = d.get(key) if isinstance(d, dict) else None
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: required key '{key}' should be an object")
    return v


def _positive(d, names, where):
    for n in names:
        if d[n] < 1:
            raise ConfigError(f"{where}: '{n}' should be at least 1, got {d[n]}")


def _rotation(rot, where, limit):
    out = {"base": read_key(rot, "base", float, where=where), "dims": read_key(rot, "dims", int, where=where)}
    if out["dims"] % 2 or not 0 <= out["dims"] <= limit:
        raise ConfigError(f"{where}: dims should be even and at most {limit}")
    if out["base"] <= 0:
        raise ConfigError(f"{where}: base should be positive")
    sc = _object(rot, "scaling", where, required=False)
    if sc is not None:
        out["scaling"] = {k: read_key(sc, k, float, where=where + ".scaling") for k in ("factor", "original", "fast", "slow")}
        if out["scaling"]["factor"] <= 0 or out["scaling"]["original"] <= 0 or min(out["scaling"]["fast"], out["scaling"]["slow"]) <= 0:
            raise ConfigError(f"{where}.scaling: factor, original, fast and slow should be positive")
    return out


def _attention(m, where):
    out = {k: read_key(m, k, int, where=where) for k in ("heads", "kv_heads", "dim", "vdim")}
    _positive(out, ("heads", "kv_heads", "dim", "vdim"), where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: heads should be a multiple of kv_heads")
    out["scale"] = read_key(m, "scale", float, where=where)
    out["rot"] = _rotation(_object(m, "rot", where), where + ".rot", out["dim"])
    mask = _object(m, "mask", where, required=False)
    if mask is not None:
        out["mask"] = {"size": read_key(mask, "size", int, where=where + ".mask")}
        if out["mask"]["size"] < 1:
            raise ConfigError(f"{where}.mask: size should be at least 1")
    return out


def _latent(m, where):
    out = {k: read_key(m, k, int, where=where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
    _positive(out, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where)
    out["scale"] = read_key(m, "scale", float, where=where)
    out["rot"] = _rotation(_object(m, "rot", where), where + ".rot", out["rot_dim"])
    if out["rot"]["dims"] != out["rot_dim"]:
        raise ConfigError(f"{where}: rot.dims should equal rot_dim (the whole shared key part is rotated)")
    if m.get("kv_from") is not None:
        out["kv_from"] = read_key(m, "kv_from", int, where=where)
    return out


@dataclass
class PikasunConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = MAX_POSITIONS

    # the names the engine and the command line use for every architecture
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PikasunConfig":
        vocab, width = read_key(d, "vocab", int), read_key(d, "width", int)
        if vocab < 1 or width < 1:
            raise ConfigError("vocab and width should be positive")
        norm = _object(d, "norm", "config.json")
        layers_in = read_key(d, "layers", list)
        if not layers_in:
            raise ConfigError("'layers' should list at least one layer")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} should be an object")
            kind = read_key(entry, "type", str, where=where)
            m = _object(entry, "mixer", where)
            if kind == "attention":
                m = _attention(m, where + ".mixer")
            elif kind == "latent_attention":
                src = m.get("kv_from")
                if isinstance(src, int) and 0 <= src < i and layers[src]["type"] == "latent_attention":
                    # what describes the borrowed latent may be left to the layer that makes it
                    m = {**{k: layers[src]["mixer"][k] for k in ("kv_rank", "rot_dim", "rot")}, **m}
                m = _latent(m, where + ".mixer")
            else:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; known: attention, latent_attention")
            mlp = entry.get("mlp")
            if mlp is not None:
                w = where + ".mlp"
                mlp = {"kind": read_key(mlp, "kind", str, where=w), "ff": read_key(mlp, "ff", int, where=w),
                       "limit": read_key(mlp, "limit", float, where=w)}
                if mlp["kind"] not in MLP_KINDS:
                    raise ConfigError(f"{w}: unknown kind '{mlp['kind']}'; known: {', '.join(MLP_KINDS)}")
                if mlp["ff"] < 1 or mlp["limit"] <= 0:
                    raise ConfigError(f"{w}: ff and limit should be positive")
            layers.append({"type": kind, "mixer": m, "mlp": mlp})
        for i, layer in enumerate(layers):
            src = layer["mixer"].get("kv_from")
            if src is None:
                continue
            where = f"layers[{i}].mixer"
            if not 0 <= src < i or layers[src]["type"] != "latent_attention" or "kv_from" in layers[src]["mixer"]:
                raise ConfigError(f"{where}: kv_from should name an earlier latent_attention layer that makes its own latent")
            a, b = layers[src]["mixer"], layer["mixer"]
            if (a["kv_rank"], a["rot_dim"], a["rot"]) != (b["kv_rank"], b["rot_dim"], b["rot"]):
                raise ConfigError(f"{where}: kv_rank, rot_dim and rot should equal those of layer {src}, whose latent it reads")
        cap = read_key(d, "logit_softcap", float, default=None)
        if cap is not None and cap <= 0:
            raise ConfigError("logit_softcap should be positive")
        return cls(ARCHITECTURE, vocab=vocab, width=width, norm_eps=read_key(norm, "eps", float, where="norm"),
                   logit_scale=read_key(d, "logit_scale", float, default=1.0), logit_softcap=cap, layers=layers,
                   max_positions=read_key(d, "max_positions", int, default=MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "layers": copy.deepcopy(self.layers)}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out
