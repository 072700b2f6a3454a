"""The Vunolorn hybrid through the engine's host logic on the CPU: the step function, the cache (pages and
state slots) and the batch description run with the plain PyTorch kernels of tests/ref_ops.py in place of the
CUDA kernels and are compared with the plain whole-sequence implementation (tests/plain_vunolorn.py): each
mechanism alone, whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal
requests in a pool so small that pages and slots are used again, keys far away and at page borders with
attention made sharp, the first tokens of a request, long decoding, and greedy generation through the entry
point."""
import copy
import random

import pytest
import torch

import plain_vunolorn as P
import ref_ops
from vunolorn_configs import ALL, ONLY, PAGE_SIZE
from zig_ai_b200.config import ConfigError, config_from_dict
from zig_ai_b200.engine import Engine
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

ATOL = 3e-4          # float32 on the CPU against float64, logits of size one to ten


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("vunolorn")
    out = {}
    for name, (cfg, seed) in list(ALL.items())[:2] + [(k, (c, 5)) for k, c in ONLY.items()]:
        d = str(root / name)
        write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
        out[name] = d
    return out


def plain(model_dir, tokens):
    return P.forward(P.read_config(model_dir), P.read_weights(model_dir), tokens)


def runner(model_dir, page_size=8, max_tokens=512, max_requests=4):
    return load_runner(model_dir, "float32", max_tokens=max_tokens, max_requests=max_requests, page_size=page_size,
                       device="cpu", ops=ref_ops)


def tokens(vocab, n, seed):
    g = random.Random(seed)
    return [g.randrange(vocab) for _ in range(n)]


def close(got, want, what="", atol=ATOL):
    err = (got.double() - want).abs().max()
    assert err < atol, f"{what}: off by {float(err):.3e}"


def run_cut(r, rid, toks, cuts):
    r.add_request(rid)
    got, at = [], 0
    for n in cuts:
        got.append(r.step([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    assert at == len(toks)
    r.end_request(rid)
    return torch.cat(got)


@pytest.mark.parametrize("name", ["scan", "delta", "pair", "scan_ff"])
def test_each_mechanism_alone(models, name):
    r = runner(models[name])
    toks = tokens(r.model.vocab_size, 45, 1)
    want = plain(models[name], toks)
    close(run_cut(r, "w", toks, [45]), want, "whole")
    close(run_cut(r, "d", toks, [1] * 45), want, "token by token")
    close(run_cut(r, "p", toks, [2, 7, 1, 3, 16, 2, 9, 5]), want, "portions")


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_decode_and_portions(models, name):
    r = runner(models[name], PAGE_SIZE[name])
    toks = tokens(r.model.vocab_size, 75, 2)
    want = plain(models[name], toks)
    close(run_cut(r, "w", toks, [75]), want, "whole")
    close(run_cut(r, "d", toks, [43] + [1] * 32), want, "decoded tail")
    for seed, sizes in ((3, (2, 3, 5)), (4, (2, 11, 17)), (5, (7, 8, 9, 16))):
        g, cuts, left = random.Random(seed), [], 75
        while left:
            n = min(g.choice(sizes), left)
            cuts.append(n)
            left -= n
        close(run_cut(r, f"p{seed}", toks, cuts), want, f"portions {sizes}")
    assert r.cache.stats()["slots_used"] == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_and_tiny_requests(models, name):
    r = runner(models[name], PAGE_SIZE[name])
    for n in (1, 2, 3):
        toks = tokens(r.model.vocab_size, n, 10 + n)
        close(run_cut(r, f"t{n}", toks, [n]), plain(models[name], toks), f"{n} tokens")
    toks = tokens(r.model.vocab_size, 9, 20)
    close(run_cut(r, "s", toks, [1, 2, 1, 2, 3]), plain(models[name], toks), "small portions from the start")


@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_together_in_a_small_pool(models, name):
    """Four state slots and a pool of a few pages: requests wait for room, and the pages and slots of finished
    requests go to the next ones; a request is sometimes left out of a step; every row equals the request alone."""
    ps = PAGE_SIZE[name]
    lengths = [23, 40, 9, 31, 1, 17, 28, 2, 36]
    r = runner(models[name], ps, max_tokens=6 * 16, max_requests=4)
    V = r.model.vocab_size
    reqs = {f"r{i}": tokens(V, n, 100 + i) for i, n in enumerate(lengths)}
    want = {k: plain(models[name], t) for k, t in reqs.items()}
    g = random.Random(9)
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    room = r.cache.num_pages * ps
    slots_seen = set()
    while waiting or live:
        while waiting and len(live) < 4 and sum(-(-len(reqs[x]) // ps) * ps for x in live + [waiting[0]]) <= room:
            k = waiting.pop(0)
            live.append(k)
            at[k] = 0
            r.add_request(k)
            slots_seen.add(r.cache.requests[k].slot)
        entries = []
        for k in live:
            if len(live) > 1 and g.random() < 0.25:
                continue
            left = len(reqs[k]) - at[k]
            n = 1 if left <= len(reqs[k]) // 3 else min(g.choice([2, 3, 5, 8]), left)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        if not entries:
            continue
        out = r.step(entries)
        row = 0
        for k, toks, want_rows in entries:
            got[k].append(out[row:row + len(toks)])
            row += len(toks)
            at[k] += len(toks)
            if at[k] == len(reqs[k]):
                live.remove(k)
                r.end_request(k)
    for k in reqs:
        close(torch.cat(got[k]), want[k], f"request {k}")
    st = r.cache.stats()
    assert st["slots_used"] == 0 and len(slots_seen) <= 4 and st["pages_reused"] > 0
    r.cache.check()


def sharpened(model_dir, out_dir, factor=6.0):
    """The same model with the query and key norm weights of its attention scaled up: the softmax then puts
    nearly all weight on one key, wherever it lies, so a key that is lost, misplaced or seen too early changes
    the logits by far more than rounding."""
    f = SafetensorsFile(f"{model_dir}/model.safetensors")
    tensors = {n: f.read(n) for n in f.names()}
    for n in tensors:
        if n.endswith(".q.norm") or n.endswith(".k.norm"):
            tensors[n] = (tensors[n].float() * factor).to(tensors[n].dtype)
    import os
    import shutil
    os.makedirs(out_dir, exist_ok=True)
    shutil.copy(f"{model_dir}/config.json", f"{out_dir}/config.json")
    write_safetensors(f"{out_dir}/model.safetensors", tensors)
    return out_dir


@pytest.mark.parametrize("name", ["A", "B"])
def test_sharp_attention_over_far_keys_and_page_borders(models, tmp_path, name):
    ps = PAGE_SIZE[name]
    d = sharpened(models[name], str(tmp_path / "sharp"))
    r = runner(d, ps, max_tokens=640)
    toks = tokens(r.model.vocab_size, 4 * ps * 3 + 1, 30)
    want = plain(d, toks)
    sharp = 2e-3      # sharp scores carry the rounding of q and k into the weights: 32-bit is a few 1e-4 off
    close(run_cut(r, "w", toks, [len(toks)]), want, "whole", sharp)
    # portions that end just before, at and just after page borders, then decoding across two more borders
    head = [ps - 1, 1, 1, ps - 2, 2 * ps + 1, ps, 3]
    rest = len(toks) - sum(head) - 2 * ps - 3
    close(run_cut(r, "b", toks, head + [rest] + [1] * (2 * ps + 3)), want, "page borders", sharp)


def echo_model(model_dir, out_dir, factor=3.0):
    """A one-layer model in which the last token of the vocabulary (the asking token) looks for the token before
    it in the vocabulary (the answering token): queries and keys read only the first half of the width, the key
    projection of every key/value head equals the query projection of its group's first head, the q/k norm
    weights are equal, large in the dimensions that are not rotated and small in those that are, and the two tokens' embedding rows agree in the first half and are opposite in
    the second.  The layer's input being the embedding alone, the asking token's score is largest at itself and
    at the answering token's keys, wherever they lie, and the answering token's value differs from its own."""
    import os
    import shutil
    c = P.read_config(model_dir)
    left = c["layers"][0]["mixer"]["left"]
    H, G, D, half = left["heads"], left["kv_heads"], left["dim"], c["width"] // 2
    f = SafetensorsFile(f"{model_dir}/model.safetensors")
    t = {n: f.read(n).float() for n in f.names()}
    t["l0.mix.left.q"][:, half:] = 0
    t["l0.mix.left.k"] = t["l0.mix.left.q"].reshape(H, D, -1)[::H // G].reshape(G * D, -1).contiguous()
    weight = torch.full_like(t["l0.mix.left.q.norm"], factor)
    weight[:left["rot"]["dims"]] = 0.05              # the rotated dimensions hardly count: distance costs a key nothing
    t["l0.mix.left.q.norm"], t["l0.mix.left.k.norm"] = weight, weight.clone()
    t["embed"][-2, :half] = t["embed"][-1, :half]
    t["embed"][-2, half:] = -t["embed"][-1, half:]
    os.makedirs(out_dir, exist_ok=True)
    shutil.copy(f"{model_dir}/config.json", f"{out_dir}/config.json")
    write_safetensors(f"{out_dir}/model.safetensors", {n: v.to(torch.bfloat16) for n, v in t.items()})
    return out_dir


@pytest.mark.parametrize("far_at", [0, 1, 7, 8, 9, 23, 24])
def test_one_far_key_decides(models, tmp_path, far_at):
    """The token that the last token looks for occurs once, far back: in the first tokens, just before, at and just after a page
    border.  Its key there takes a large share of the last row's attention, so the row is wrong if that key is
    lost, and the test first makes sure of that with the plain implementation."""
    ps = 8
    d = echo_model(models["echo"], str(tmp_path / "echo"))
    V = P.read_config(d)["vocab"]
    n = 9 * ps + 5
    toks = tokens(V - 2, n, 50)
    toks[far_at], toks[-1] = V - 2, V - 1
    want = plain(d, toks)
    other = list(toks)
    other[far_at] = 0
    assert (plain(d, other)[-1] - want[-1]).abs().max() > 0.3          # the far key matters
    r = runner(d, ps, max_tokens=128)
    close(run_cut(r, "w", toks, [n]), want, "whole")
    close(run_cut(r, "d", toks, [n - 3, 1, 1, 1]), want, "decoded")
    cuts = ([far_at] if far_at else []) + [1, ps - 1, 2 * ps + 1]
    close(run_cut(r, "p", toks, cuts + [n - sum(cuts) - 2, 2]), want, "portions cut at the far key")


def test_long_decoding(models):
    name = "A"
    r = runner(models[name], PAGE_SIZE[name], max_tokens=256)
    toks = tokens(r.model.vocab_size, 180, 40)
    close(run_cut(r, "l", toks, [5] + [1] * 175), plain(models[name], toks), "175 decoded tokens")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(models, name):
    g = random.Random(3)
    cfg = P.read_config(models[name])
    prompts = [[g.randrange(cfg["vocab"]) for _ in range(n)] for n in (7, 13, 1, 22)]
    eng = Engine(models[name], "float32", max_num_seqs=3, max_batched_tokens=6, max_model_len=64,
                 page_size=PAGE_SIZE[name], device="cpu", ops=ref_ops)
    got = eng.generate(prompts, max_new_tokens=8, temperature=0.0)
    W = P.read_weights(models[name])
    for p, out in zip(prompts, got):
        assert len(out) == 8
        logits = P.forward(cfg, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) < ATOL, f"token {i} is not the plain implementation's choice"
    assert eng.stats()["slots_used"] == 0


def test_configuration_is_read_and_checked():
    cfg = config_from_dict(ALL["B"][0])
    assert cfg.architecture == "Vunolorn" and cfg.vocab_size == 257 and len(cfg.layers) == 5
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    for change, text in ((lambda c: c["layers"][0].update(type="rwkv"), "unknown mixer type"),
                         (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
                         (lambda c: c["layers"][1]["mixer"]["left"].update(heads=4, kv_heads=3), "multiple"),
                         (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "even"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "unknown kind"),
                         (lambda c: c.pop("norm"), "norm"),
                         (lambda c: c.update(layers=[]), "at least one")):
        bad = copy.deepcopy(ALL["B"][0])
        change(bad)
        with pytest.raises(ConfigError, match=text):
            config_from_dict(bad)


def test_tensors_are_named_and_shaped_by_the_configuration(models):
    from zig_ai_b200.models import build_model
    decls = build_model(config_from_dict(ALL["B"][0])).param_decls()
    assert decls["embed"].shape == (257, 64) and decls["head"].shape == (257, 64) and decls["final.norm"].shape == (64,)
    assert decls["l0.mix.A_log"].shape == (96, 16) and decls["l0.mix.x"].shape == (4 + 32, 96) and "l0.norm2" not in decls
    assert decls["l1.mix.left.v"].shape == (48, 64) and decls["l1.mix.left.o"].shape == (64, 3 * 48)
    assert decls["l1.mix.right.z.b"].shape == (50,) and decls["l1.mlp.up"].shape == (100, 64) and "l1.norm2b" in decls
    assert decls["l3.mix.q.conv"].shape == (16, 2) and decls["l3.mix.v"].shape == (32, 64) and decls["l3.mix.norm"].shape == (16,)
    stored = set(SafetensorsFile(f"{models['B']}/model.safetensors").names())
    assert stored == set(decls)
