"""The Pikasun design through the engine's host logic on the CPU: the step function, the cache (pages of keys and
values, pages of latent rows, a layer that reads another layer's pages) and the batch description run with the plain
PyTorch kernels of tests/ref_ops.py in place of the CUDA kernels and are compared with the plain whole-sequence
implementation (tests/plain_pikasun.py): each mechanism alone, whole prompts, token-by-token decoding, portions down
to two tokens, batches of unequal requests in a pool so small that pages and slots are used again, keys just inside
and just outside a chunk and at page borders with attention made sharp, the first tokens of a request, long
decoding, pages given back once a chunk has passed them, and greedy generation through the entry point."""
import copy
import random

import pytest
import torch

import plain_pikasun as P
import ref_ops
from pikasun_configs import ALL, ONLY, PAGE_SIZE
from zig_ai_b200.config import ConfigError, config_from_dict
from zig_ai_b200.engine import Engine
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.safetensors_io import SafetensorsFile

ATOL = 3e-4          # float32 on the CPU against float64, logits of size one to ten


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("pikasun")
    out = {}
    for name, (cfg, seed) in list(ALL.items())[:2] + [(k, (c, 5)) for k, c in ONLY.items()]:
        d = str(root / name)
        write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
        out[name] = d
    return out


def plain(model_dir, tokens, cfg=None):
    return P.forward(cfg or P.read_config(model_dir), P.read_weights(model_dir), tokens)


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


@pytest.mark.parametrize("name", ["chunks", "chunks_ff", "chunk_of_one", "causal", "latent", "latent_pair"])
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
    """Four slots and a pool of a few pages: requests wait for room, and the pages and slots of finished requests go
    to the next ones; a request is sometimes left out of a step; every row equals the request alone."""
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
        for k, toks, _ in entries:
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


def rows_at_chunk_edges(n, size):
    """Positions that are the first and the last of a chunk, and those beside them."""
    out = set()
    for start in range(0, n, size):
        out.update(p for p in (start - 1, start, start + 1, start + size - 2) if 0 <= p < n)
    return sorted(out)


def test_keys_just_inside_and_just_outside_a_chunk(models):
    """With attention made sharp, a query that saw one key too many or too few, in a prompt or when decoding, gives
    other logits: the plain implementation with chunks one position longer or shorter differs by far more than the
    limit at the rows beside the chunks' edges, and the engine agrees with the right one at every row."""
    name, ps = "sharp_chunks", 8
    cfg = P.read_config(models[name])
    size = cfg["layers"][0]["mixer"]["mask"]["size"]
    toks = tokens(cfg["vocab"], 5 * size + 3, 60)
    want = plain(models[name], toks)
    edges = rows_at_chunk_edges(len(toks), size)
    for other in (size - 1, size + 1):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["mask"]["size"] = other
        assert (plain(models[name], toks, wrong)[edges] - want[edges]).abs().max() > 0.2
    sharp = 2e-3
    r = runner(models[name], ps, max_tokens=128)
    close(run_cut(r, "w", toks, [len(toks)]), want, "whole", sharp)
    close(run_cut(r, "d", toks, [size - 1] + [1] * (len(toks) - size + 1)), want, "decoded across four edges", sharp)
    # portions that end just before, at and just after the edges of chunks and of pages
    cuts = [size - 1, 1, 1, size - 2, 2, ps - 3, 2 * size + 1]
    close(run_cut(r, "p", toks, cuts + [len(toks) - sum(cuts) - 2, 2]), want, "portions cut at the edges", sharp)


def test_sharp_latent_attention_over_far_keys_and_page_borders(models):
    """Sharp scores put nearly all weight on one cached row, wherever it lies: the first rows, rows at page borders and
    rows hundreds of positions back; the plain implementation without the first token differs, so a lost row shows."""
    name, ps = "sharp_latent", 8
    V = P.read_config(models[name])["vocab"]
    toks = tokens(V, 12 * ps + 5, 61)
    want = plain(models[name], toks)
    other = [(toks[0] + 1) % V] + toks[1:]
    assert (plain(models[name], other)[len(toks) // 2:] - want[len(toks) // 2:]).abs().max() > 0.05     # the far key counts
    sharp = 2e-3
    r = runner(models[name], ps, max_tokens=128)
    close(run_cut(r, "w", toks, [len(toks)]), want, "whole", sharp)
    head = [ps - 1, 1, 1, ps - 2, 2 * ps + 1, ps, 3]
    rest = len(toks) - sum(head) - 2 * ps - 3
    close(run_cut(r, "b", toks, head + [rest] + [1] * (2 * ps + 3)), want, "page borders", sharp)


def test_long_decoding_and_pages_given_back_behind_a_chunk(models):
    """175 tokens decoded one by one across many chunks and pages; the attention layers' pages that lie wholly before
    the current chunk go back to the pool while the request runs, the latent layers keep all of theirs."""
    name = "A"
    ps = PAGE_SIZE[name]
    r = runner(models[name], ps, max_tokens=256)
    toks = tokens(r.model.vocab_size, 180, 40)
    want = plain(models[name], toks)
    r.add_request("l")
    got = [r.step([("l", toks[:5], list(range(5)))])]
    for i in range(5, 180):
        got.append(r.step([("l", toks[i:i + 1], [0])]))
    close(torch.cat(got), want, "175 decoded tokens")
    used = {type(r.cache.groups[g].need).__name__: r.cache.groups[g].pool.n_used for g in r.cache.paged_groups()}
    size = P.read_config(models[name])["layers"][0]["mixer"]["mask"]["size"]
    assert used["PagedRowsNeed"] == -(-180 // ps)
    assert used["PagedKVNeed"] <= -(-(size + ps) // ps) + 1 < used["PagedRowsNeed"]
    r.end_request("l")
    r.cache.check()


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


def test_stretched_frequencies_and_their_ramp():
    """The stretched rotation's frequencies against the formula written out pair by pair."""
    import math
    dims, base, (factor, original, fast, slow) = 16, 300.0, (4.0, 32.0, 8.0, 1.0)
    got, mag = ref_ops.stretched_frequencies(dims, base, (factor, original, fast, slow))
    where = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(float(got[i]) - (f / factor * ramp + f * (1 - ramp))) < 1e-12
    assert abs(mag - (0.1 * math.log(factor) + 1.0)) < 1e-12 and lo < hi
    mine, mag2 = P.interpolated_frequencies(base, dims, factor, original, fast, slow)
    assert torch.allclose(mine, got, rtol=0, atol=1e-12) and mag2 == mag


def test_configuration_is_read_and_checked():
    cfg = config_from_dict(ALL["B"][0])
    assert cfg.architecture == "Pikasun" and cfg.vocab_size == 257 and len(cfg.layers) == 5 and cfg.logit_softcap is None
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert config_from_dict(ALL["A"][0]).logit_softcap == 9.0
    for change, text in ((lambda c: c["layers"][0].update(type="rwkv"), "unknown mixer type"),
                         (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
                         (lambda c: c["layers"][1]["mixer"].update(heads=4, kv_heads=3), "multiple"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
                         (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "at least 1"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown kind"),
                         (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                         (lambda c: c["layers"][3]["mixer"].update(kv_rank=41), "equal"),
                         (lambda c: c.pop("norm"), "norm"),
                         (lambda c: c.update(layers=[]), "at least one")):
        bad = copy.deepcopy(ALL["B"][0])
        change(bad)
        with pytest.raises(ConfigError, match=text):
            config_from_dict(bad)


def test_tensors_are_named_and_shaped_by_the_configuration(models):
    from zig_ai_b200.models import build_model
    decls = build_model(config_from_dict(ALL["B"][0])).param_decls()
    assert decls["embed"].shape == (257, 66) and decls["head"].shape == (257, 66)
    assert decls["final.norm"].shape == (66,) and decls["final.norm.b"].shape == (66,)
    assert decls["l0.mix.q"].shape == (4 * 32, 66) and decls["l0.mix.dkv"].shape == (56, 66) and decls["l0.mix.dkv.norm"].shape == (40,)
    assert decls["l0.mix.uk"].shape == (64, 40) and decls["l0.mix.uv"].shape == (32, 40) and decls["l0.mix.g"].shape == (32, 66)
    assert decls["l1.mix.q.norm"].shape == (72,) and decls["l1.mix.k.b"].shape == (72,) and decls["l1.mix.v"].shape == (24, 66)
    assert decls["l1.mix.g"].shape == (3, 66) and decls["l1.mix.o"].shape == (66, 24) and "l1.norm2" not in decls
    assert "l3.mix.dkv" not in decls and "l3.mix.dkv.norm" not in decls and decls["l3.mix.uk"].shape == (20, 40)
    assert decls["l2.mlp.gate"].shape == (72, 66) and decls["l2.norm2.b"].shape == (66,)
    stored = set(SafetensorsFile(f"{models['B']}/model.safetensors").names())
    assert stored == set(decls)


def random_configuration(g):
    """A small Pikasun configuration drawn at random: layer kinds and order, head counts, head sizes that differ between
    q/k and v, ranks and rotated parts, chunk sizes from one position to longer than the prompt, plain and stretched
    rotations, layers that borrow an earlier layer's latent, layers without feed-forward, logits with and without a cap."""
    from pikasun_configs import attention, config, latent
    layers, own = [], []
    for i in range(g.randint(2, 6)):
        ff = None if g.random() < 0.25 else g.choice([24, 56, 100])
        limit = g.choice([0.5, 1.0, 3.0])
        if g.random() < 0.4:
            heads = g.choice([1, 2, 3, 4, 6])
            kv = g.choice([k for k in (1, 2, 3, 4, 6) if heads % k == 0])
            dim = g.choice([4, 8, 12, 16, 24])
            rot = g.choice([dim, dim // 4 * 2, 0])
            layers.append(attention(heads, kv, dim, g.choice([dim, 4, 8, 20]), g.choice([dim ** -0.5, 0.2, 0.45]), rot,
                                    g.choice([300.0, 10000.0, 1e6]), mask=g.choice([None, 1, 2, 5, 9, 16, 31, 200]), ff=ff, limit=limit))
        else:
            heads, dim, vdim = g.choice([1, 2, 3, 5]), g.choice([4, 6, 16]), g.choice([4, 10, 16])
            src = g.choice(own) if own and g.random() < 0.4 else None
            if src is None:
                rot_dim, rank, base = g.choice([2, 4, 8, 12]), g.choice([8, 17, 24, 32]), g.choice([300.0, 10000.0])
                scaling = g.choice([None, (4.0, 32.0, 8.0, 1.0), (16.0, 24.0, 4.0, 0.5), (2.0, 1000.0, 2.0, 1.0)])
                own.append(i)
            else:
                m = layers[src]["mixer"]
                rot_dim, rank, base = m["rot_dim"], m["kv_rank"], m["rot"]["base"]
                sc = m["rot"].get("scaling")
                scaling = None if sc is None else tuple(sc[k] for k in ("factor", "original", "fast", "slow"))
            layers.append(latent(heads, dim, rot_dim, vdim, rank, g.choice([0.2, (dim + rot_dim) ** -0.5]), base, scaling=scaling,
                                 kv_from=src, ff=ff, limit=limit))
    return config(g.choice([61, 97, 130]), g.choice([24, 40, 50, 64]), g.choice([1e-5, 1e-6]), g.choice([0.5, 1.0, 1.7]),
                  g.choice([None, 4.0, 30.0]), layers)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    g = random.Random(1000 + seed)
    cfg = random_configuration(g)
    d = str(tmp_path / "m")
    write_random_model(config_from_dict(cfg), seed, d, matrix_std="fan_in")
    toks = tokens(cfg["vocab"], 70, seed)
    want = plain(d, toks)
    r = runner(d, g.choice([4, 8, 16]), max_tokens=128)
    close(run_cut(r, "w", toks, [70]), want, "whole")
    close(run_cut(r, "p", toks, [9, 2, 17, 1, 1, 3, 30, 2, 5]), want, "portions")
    close(run_cut(r, "d", toks, [50] + [1] * 20), want, "decoded tail")
    r.cache.check()
