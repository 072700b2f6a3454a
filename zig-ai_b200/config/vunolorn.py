"""Configuration of the Vunolorn hybrid, read from its own config.json keys.

    architecture     "Vunolorn"
    vocab, width     vocabulary and model width
    embedding.scale  factor on the embedding rows
    norm.eps         eps of every RMS norm of the layers (inside the root)
    layers           one entry per layer: `type` (which mixer), `mixer` (its sizes), `mlp` (null, or
                     {kind: "dense", ff})

Mixers by `type`:
    mamba1    inner, state, dt_rank, conv (taps)
    delta     heads, kv_heads, dim, vdim, conv (taps)
    parallel  left  {heads, kv_heads, dim, vdim, scale, rot {base, dims}}   softmax attention
              right {width}                                                 minimal gated recurrence
              left_scale, right_scale                                       weights of the sum
Every size and constant comes from the file; nothing is assumed equal to anything else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import ConfigError, ModelConfig, read_key

ARCHITECTURE = "Vunolorn"
MIXER_KEYS = {
    "mamba1": {"inner": int, "state": int, "dt_rank": int, "conv": int},
    "delta": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int},
    "parallel": {"left": dict, "right": dict, "left_scale": float, "right_scale": float},
}
LEFT_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "rot": dict}
MLP_KINDS = ("dense",)
MAX_POSITIONS = 1 << 20      # the design names no limit; block tables and graphs are sized by the cache, not by this


def _typed(d, keys, where):
    if not isinstance(d, dict):
        raise ConfigError(f"{where} should be an object")
    out = {}
    for k, kind in keys.items():
        if kind is dict:
            if not isinstance(d.get(k), dict):
                raise ConfigError(f"{where}: required key '{k}' should be an object")
            out[k] = d[k]
        else:
            out[k] = read_key(d, k, kind, where=where)
    return out


def _positive(d, names, where):
    for n in names:
        if d[n] < 1:
            raise ConfigError(f"{where}: '{n}' should be at least 1, got {d[n]}")


@dataclass
class VunolornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
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
    def from_dict(cls, d: Dict[str, Any]) -> "VunolornConfig":
        vocab, width = read_key(d, "vocab", int), read_key(d, "width", int)
        if vocab < 1 or width < 1:
            raise ConfigError("vocab and width should be positive")
        emb = d.get("embedding") if isinstance(d.get("embedding"), dict) else {}
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' should be an object with 'eps'")
        layers_in = read_key(d, "layers", list)
        if not layers_in:
            raise ConfigError("'layers' should list at least one layer")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} should be an object")
            kind = read_key(entry, "type", str, where=where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; known: {', '.join(sorted(MIXER_KEYS))}")
            m = _typed(entry.get("mixer"), MIXER_KEYS[kind], where + ".mixer")
            if kind == "mamba1":
                _positive(m, ("inner", "state", "dt_rank", "conv"), where + ".mixer")
            elif kind == "delta":
                _positive(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads should be a multiple of kv_heads")
            else:
                left = _typed(m["left"], LEFT_KEYS, where + ".mixer.left")
                _positive(left, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer.left")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.left: heads should be a multiple of kv_heads")
                rot = _typed(left["rot"], {"base": float, "dims": int}, where + ".mixer.left.rot")
                if rot["dims"] % 2 or not 0 <= rot["dims"] <= left["dim"]:
                    raise ConfigError(f"{where}.mixer.left.rot: dims should be even and at most dim")
                left["rot"] = rot
                right = _typed(m["right"], {"width": int}, where + ".mixer.right")
                _positive(right, ("width",), where + ".mixer.right")
                m = {"left": left, "right": right, "left_scale": m["left_scale"], "right_scale": m["right_scale"]}
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = {"kind": read_key(mlp, "kind", str, where=where + ".mlp"), "ff": read_key(mlp, "ff", int, where=where + ".mlp")}
                if mlp["kind"] not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: unknown kind '{mlp['kind']}'; known: {', '.join(MLP_KINDS)}")
                if mlp["ff"] < 1:
                    raise ConfigError(f"{where}.mlp: ff should be positive")
            layers.append({"type": kind, "mixer": m, "mlp": mlp})
        return cls(ARCHITECTURE, vocab=vocab, width=width,
                   embedding_scale=read_key(emb, "scale", float, default=1.0, where="embedding"),
                   norm_eps=read_key(norm, "eps", float, where="norm"), layers=layers,
                   max_positions=read_key(d, "max_positions", int, default=MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(self.layers),
                **({"max_positions": self.max_positions} if self.max_positions != MAX_POSITIONS else {})}
