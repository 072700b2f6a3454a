"""The Vunolorn hybrid as a list of layers made from parts.

Every layer is a block with a norm before and after each sublayer (`sandwich_residual`); its mixer is
a selective scan, a gated delta rule, or softmax attention beside a minimal gated recurrence
(`parallel`); its feed-forward, where it has one, is a dense two-matrix MLP with the exact GELU.  The
embedding rows are scaled; the head is a plain matrix after the final norm.

Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `norm1b`, `norm2`, `norm2b`,
`l<i>.mix.<tensor>` (a parallel mixer's under `mix.left.` and `mix.right.`) and `l<i>.mlp.up`, `mlp.down`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.vunolorn import ARCHITECTURE, VunolornConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

SCAN_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b", "a_log": "A_log",
              "d": "D", "o": "o"}
DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a",
               "a_log": "A_log", "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o"}
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}
GRU_NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}


def _prefixed(names, prefix):
    return {k: prefix + v for k, v in names.items()}


def mixer_spec(cfg: VunolornConfig, kind: str, m: dict) -> PartSpec:
    W, eps = cfg.width, cfg.norm_eps
    if kind == "mamba1":
        return PartSpec("selective_scan", dict(hidden=W, inner=m["inner"], state=m["state"], dt_rank=m["dt_rank"],
                                               taps=m["conv"], conv_bias=True, names=_prefixed(SCAN_NAMES, "mix.")))
    if kind == "delta":
        return PartSpec("gated_delta", dict(hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                            taps=m["conv"], eps=eps, names=_prefixed(DELTA_NAMES, "mix.")))
    left, right = m["left"], m["right"]
    rot = left["rot"]
    position = (PartSpec("rotary_half_split", dict(head_dim=max(left["dim"], left["vdim"]), theta=rot["base"], rotary_dim=rot["dims"]))
                if rot["dims"] else PartSpec("none", {}))
    attention = PartSpec("attention", dict(
        hidden=W, heads=left["heads"], kv_heads=left["kv_heads"], head_dim=left["dim"], value_dim=left["vdim"], qk_norm=True,
        value_norm=True, eps=eps, scale=left["scale"], position=position, names=ATTENTION_NAMES))
    gru = PartSpec("min_gru", dict(hidden=W, width=right["width"], names=GRU_NAMES))
    return PartSpec("parallel", dict(left=attention, right=gru, left_scale=m["left_scale"], right_scale=m["right_scale"],
                                     left_prefix="mix.left.", right_prefix="mix.right."))


def build_spec(cfg: VunolornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", dict(size=W, eps=eps, weight=name))
    layers = []
    for i, layer in enumerate(cfg.layers):
        block = dict(mixer=mixer_spec(cfg, layer["type"], layer["mixer"]), mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"))
        if layer["mlp"] is not None:
            block.update(feed_forward=PartSpec("dense", dict(hidden=W, ff_dim=layer["mlp"]["ff"], activation="gelu",
                                                             names={"up": "mlp.up", "down": "mlp.down"})),
                         ff_norm=norm("norm2"), ff_post_norm=norm("norm2b"))
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("sandwich_residual", block)))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("embedding", dict(weight="embed", scale=cfg.embedding_scale)),
        layers=layers, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=norm("final.norm"), head=PartSpec("linear_head", dict(weight="head", tied=False)))


register_architecture(ARCHITECTURE, VunolornConfig, build_spec, replace=True)
