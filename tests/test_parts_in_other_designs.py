"""The parts that came with the Vunolorn hybrid are parts like any other: a fourth toy architecture, defined in
this file, pairs LFM2's ShortConv with the minimal gated recurrence in a `parallel` mixer inside LFM2's pre-norm
block with a dense tanh-GELU feed-forward, and puts a gated delta rule (one q/k head per head, three taps) with a
SwiGLU feed-forward into the block with a norm before and after each sublayer.  Registered, written with random
weights, stepped in portions and single tokens, and compared with plain formulas; nothing under the package changes."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

import plain_lfm2 as PL
import plain_vunolorn as PV
import ref_ops
from zig_ai_b200.config import ModelConfig, register_architecture, unregister_architecture
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec
from zig_ai_b200.weights import write_random_model

T4 = dict(hidden=48, vocab=91, eps=1e-5, taps=3, width=40, ff=72, heads=3, dim=16, vdim=8)


@dataclass
class Toy4Config(ModelConfig):
    @classmethod
    def from_dict(cls, d):
        return cls("Toy4ForTests")

    def to_dict(self):
        return {"architectures": ["Toy4ForTests"]}


def toy4_spec(cfg):
    a, H = T4, T4["hidden"]
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=a["eps"], weight=name))
    pair = PartSpec("parallel", dict(
        left=PartSpec("short_conv", dict(hidden=H, conv_dim=H, taps=a["taps"], bias=True)),
        right=PartSpec("min_gru", dict(hidden=H, width=a["width"])), left_scale=0.6, right_scale=1.4,
        left_prefix="a.", right_prefix="b."))
    delta = PartSpec("gated_delta", dict(hidden=H, heads=a["heads"], kv_heads=a["heads"], dim=a["dim"], vdim=a["vdim"],
                                         taps=a["taps"], eps=a["eps"]))
    layers = [
        LayerSpec("l0.", PartSpec("prenorm_residual", dict(
            mixer=pair, feed_forward=PartSpec("dense", dict(hidden=H, ff_dim=a["ff"], activation="gelu_tanh")),
            mixer_norm=norm("n0.weight"), ff_norm=norm("n1.weight")))),
        LayerSpec("l1.", PartSpec("sandwich_residual", dict(
            mixer=delta, mixer_norm=norm("n0.weight"), mixer_post_norm=norm("n1.weight"),
            feed_forward=PartSpec("swiglu", dict(hidden=H, ff_dim=a["ff"])), ff_norm=norm("n2.weight"), ff_post_norm=norm("n3.weight")))),
    ]
    return ModelSpec("Toy4ForTests", H, a["vocab"], 256, PartSpec("embedding", dict(weight="emb.weight", scale=0.5)),
                     layers, [LayerCall(0), LayerCall(1)], norm("final.weight"), PartSpec("linear_head", dict(weight="head.weight", tied=False)))


def toy4_plain(W, tokens):
    a = T4
    n = lambda x, name: PL.rms_norm(x, W[name], a["eps"])
    h = W["emb.weight"][torch.tensor(tokens)] * 0.5
    r = n(h, "l0.n0.weight")
    conv = PL.short_conv_mixer(r, W, "l0.a.", None)
    # the minimal gated recurrence from its formulas, with this model's tensor names
    z = torch.sigmoid(r @ W["l0.b.gru_z.weight"].T + W["l0.b.gru_z.bias"])
    u = r @ W["l0.b.gru_x.weight"].T + W["l0.b.gru_x.bias"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s, rows = torch.zeros(a["width"], dtype=torch.float64), []
    for t in range(len(tokens)):
        s = (1 - z[t]) * s + z[t] * cand[t]
        rows.append(s)
    gru = (torch.stack(rows) * PV.silu(r @ W["l0.b.gru_g.weight"].T)) @ W["l0.b.gru_out.weight"].T
    h = h + 0.6 * conv + 1.4 * gru
    r = n(h, "l0.n1.weight")
    x = r @ W["l0.ffn_up.weight"].T
    h = h + (0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))) @ W["l0.ffn_down.weight"].T
    names = {"q": "delta_q.weight", "k": "delta_k.weight", "v": "delta_v.weight", "q.conv": "delta_q_conv.weight",
             "k.conv": "delta_k_conv.weight", "v.conv": "delta_v_conv.weight", "b": "delta_beta.weight", "a": "delta_a.weight",
             "A_log": "delta_a_log", "dt_bias": "delta_dt_bias", "g": "delta_gate.weight", "norm": "delta_norm.weight",
             "o": "delta_out.weight"}
    Wd = {"d." + short: W["l1." + stored] for short, stored in names.items()}
    m = {"heads": a["heads"], "kv_heads": a["heads"], "dim": a["dim"], "vdim": a["vdim"], "conv": a["taps"]}
    h = h + n(PV.gated_delta_mixer(n(h, "l1.n0.weight"), Wd, "d.", m, a["eps"]), "l1.n1.weight")
    h = h + n(PL.swiglu(n(h, "l1.n2.weight"), W, "l1."), "l1.n3.weight")
    return n(h, "final.weight") @ W["head.weight"].T


@pytest.fixture
def toy4_registered():
    register_architecture("Toy4ForTests", Toy4Config, toy4_spec)
    yield
    unregister_architecture("Toy4ForTests")


def run_toy4(tmp_path, device):
    d = write_random_model(Toy4Config("Toy4ForTests"), 61, str(tmp_path / "toy4"), matrix_std="fan_in")
    kw = dict(device="cpu", ops=ref_ops) if device == "cpu" else {}
    runner = load_runner(d, "float32", max_tokens=128, max_requests=3, page_size=8, **kw)
    assert runner.cache.paged_groups() == []                    # no layer keeps keys and values: states only
    W = PL.read_weights(d)
    g = random.Random(8)
    reqs = {k: [g.randrange(T4["vocab"]) for _ in range(n)] for k, n in (("x", 33), ("y", 12), ("z", 1))}
    for k, toks in reqs.items():
        want = toy4_plain(W, toks)
        for tag, cuts in (("w", [len(toks)]), ("p", [2, 5, 1, 3] + [1] * (len(toks) - 11) if len(toks) > 11 else [1] * len(toks))):
            runner.add_request(k + tag)
            got, at = [], 0
            for n_ in cuts:
                got.append(runner.step([(k + tag, toks[at:at + n_], list(range(n_)))]).double().cpu())
                at += n_
            runner.end_request(k + tag)
            err = (torch.cat(got) - want).abs().max() / want.abs().max()
            assert err < 5e-5, (k, tag, float(err))


def test_fourth_toy_architecture_on_the_cpu_stand_ins(toy4_registered, tmp_path):
    run_toy4(tmp_path, "cpu")


@pytest.mark.gpu
def test_fourth_toy_architecture_on_the_gpu(toy4_registered, tmp_path):
    run_toy4(tmp_path, "cuda")
