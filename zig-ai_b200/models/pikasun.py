"""The Pikasun design as a list of layers made from parts.

Every layer is a pre-norm residual block with layer norms (weight and bias); its mixer is grouped-query
attention inside chunks of positions (biased projections, an RMS norm over the whole q and the whole k
projection, interleaved rotation, a sigmoid gate per head) or attention over a shared low-rank latent (with a
stretched rotation and an element-wise sigmoid gate), whose cached latent a later layer may read instead of
making its own; its feed-forward, where it has one, is a gated one with bounded branches.  The head's logits are
scaled and capped.

Tensor names: `embed`, `head`, `final.norm` (+ `.b`), and per layer i `l<i>.norm1`, `norm2` (+ `.b`),
`l<i>.mix.<tensor>` (biases and norm weights: the tensor's name + `.b` / `.norm`) and `l<i>.mlp.gate`, `up`, `down`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.pikasun import ARCHITECTURE, PikasunConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

ATTENTION_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                   "q_bias": "mix.q.b", "k_bias": "mix.k.b", "v_bias": "mix.v.b", "g": "mix.g"}
LATENT_NAMES = {"q": "mix.q", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "g": "mix.g",
                "o": "mix.o"}
MLP_NAMES = {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}
GATE_SLOPE = 1.702          # the design's constant in g * sigmoid(slope * g)


def mixer_spec(cfg: PikasunConfig, kind: str, m: dict) -> PartSpec:
    W, eps, rot = cfg.width, cfg.norm_eps, m["rot"]
    if kind == "attention":
        position = (PartSpec("rotary_interleaved", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"],
                                                        scaling=rot.get("scaling")))
                    if rot["dims"] else PartSpec("none", {}))
        return PartSpec("attention", dict(
            hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"], qk_norm=True,
            norm_scope="whole", bias=True, gate="head", eps=eps, scale=m["scale"], position=position,
            chunk=m["mask"]["size"] if "mask" in m else None, names=ATTENTION_NAMES))
    position = PartSpec("rotary_half_split", dict(head_dim=m["rot_dim"], theta=rot["base"], rotary_dim=rot["dims"],
                                                  scaling=rot.get("scaling")))
    return PartSpec("latent_attention", dict(
        hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], rank=m["kv_rank"], scale=m["scale"],
        eps=eps, position=position, kv_proj="kv_from" not in m, gate="element", names=LATENT_NAMES))


def build_spec(cfg: PikasunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("layernorm", dict(size=W, eps=eps, weight=name, bias=name + ".b"))
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        block = dict(mixer=mixer_spec(cfg, layer["type"], layer["mixer"]), mixer_norm=norm("norm1"))
        if layer["mlp"] is not None:
            block.update(feed_forward=PartSpec("clamped_glu", dict(hidden=W, ff_dim=layer["mlp"]["ff"], limit=layer["mlp"]["limit"],
                                                                   alpha=GATE_SLOPE, names=MLP_NAMES)),
                         ff_norm=norm("norm2"))
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm_residual", block)))
        order.append(LayerCall(i, cache_of=layer["mixer"].get("kv_from")))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("embedding", dict(weight="embed")),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(weight="head", tied=False, scale=cfg.logit_scale, softcap=cfg.logit_softcap)))


register_architecture(ARCHITECTURE, PikasunConfig, build_spec, replace=True)
