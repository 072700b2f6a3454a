"""Small configurations of the Pikasun design for the tests.  Between them they differ in every size and option:
layer order and count, a feed-forward behind either kind of mixer and none, value heads smaller than, equal to
and larger than the query/key heads, one and several key/value heads, partly, wholly and not rotated heads,
chunks of one position, of a few and none, latent layers that make their own latent and that borrow one, stretched
and plain rotations, logits with and without a cap, widths that are no multiple of four."""


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, mask=None, ff=None, limit=1.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def latent(heads, dim, rot_dim, vdim, rank, scale, base, scaling=None, kv_from=None, ff=None, limit=1.0):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(vocab, width, eps, logit_scale, softcap, layers):
    c = {"architecture": "Pikasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
         "layers": layers}
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


STRETCH = (4.0, 32.0, 8.0, 1.0)       # factor, original length, fast and slow turns: the ramp lies inside eight pairs

P_A = config(131, 48, 1e-5, 0.7, 9.0, [
    attention(4, 2, 16, 24, 0.3, 8, 10000.0, mask=11, ff=80, limit=1.5),
    latent(3, 12, 8, 20, 24, 0.2, 10000.0, scaling=STRETCH),
    latent(2, 8, 8, 16, 24, 0.35, 10000.0, scaling=STRETCH, kv_from=1, ff=64, limit=0.8),
])

P_B = config(257, 66, 1e-6, 1.0, None, [
    latent(4, 16, 16, 8, 40, 0.25, 500.0, ff=100, limit=2.0),
    attention(3, 3, 24, 8, 0.2, 24, 1000000.0, mask=7),
    attention(2, 1, 8, 8, 0.4, 0, 10000.0, ff=72, limit=0.5),
    latent(5, 4, 16, 12, 40, 0.3, 500.0, kv_from=0),
    latent(2, 20, 6, 20, 17, 0.2, 300.0, scaling=(16.0, 24.0, 4.0, 0.5), ff=50, limit=1.0),
])

# one layer of each kind, alone: a fault shows in the mechanism that has it
ONLY = {
    "chunks": config(97, 40, 1e-5, 1.0, None, [attention(4, 2, 16, 12, 0.3, 8, 300.0, mask=9)]),
    "chunks_ff": config(97, 40, 1e-5, 0.5, 6.0, [attention(2, 2, 12, 20, 0.3, 12, 300.0, mask=9, ff=64, limit=0.7)]),
    "chunk_of_one": config(97, 40, 1e-5, 1.0, None, [attention(2, 1, 16, 16, 0.3, 16, 300.0, mask=1, ff=48)]),
    "causal": config(97, 40, 1e-5, 1.0, None, [attention(4, 1, 8, 8, 0.4, 4, 300.0)]),
    "latent": config(97, 40, 1e-5, 1.0, 20.0, [latent(3, 10, 6, 14, 20, 0.3, 300.0, scaling=STRETCH)]),
    "latent_pair": config(97, 40, 1e-5, 1.0, None, [latent(3, 10, 6, 14, 20, 0.3, 300.0, ff=56),
                                                    latent(2, 6, 6, 10, 20, 0.4, 300.0, kv_from=0)]),
    # attention made sharp by its scale: nearly all weight on one key, so a key lost or seen too early shows
    "sharp_chunks": config(97, 40, 1e-5, 1.0, None, [attention(4, 2, 16, 16, 2.5, 8, 300.0, mask=12)]),
    "sharp_latent": config(97, 40, 1e-5, 1.0, None, [latent(3, 10, 6, 14, 20, 1.2, 300.0, scaling=STRETCH)]),
}

# head sizes and widths that the tensor-core attention kernels and the few-rows product kernels take, for the
# whole-model GPU tests in bfloat16
P_C = config(1000, 320, 1e-6, 0.7, 30.0, [
    attention(4, 2, 64, 64, 0.125, 32, 1000000.0, mask=96, ff=512, limit=1.5),
    latent(4, 48, 32, 64, 160, 0.1, 10000.0, scaling=(4.0, 128.0, 16.0, 1.0), ff=256, limit=2.0),
    attention(8, 1, 128, 64, 0.09, 64, 10000.0, mask=160),
    latent(8, 16, 32, 48, 160, 0.15, 10000.0, scaling=(4.0, 128.0, 16.0, 1.0), kv_from=1, ff=448, limit=1.0),
])

ALL = {"A": (P_A, 31), "B": (P_B, 37), "C": (P_C, 41)}
PAGE_SIZE = {"A": 8, "B": 16, "C": 64}
