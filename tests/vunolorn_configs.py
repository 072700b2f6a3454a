"""Small configurations of the Vunolorn hybrid for the tests.  Between them they differ in every size and
option: layer order and count, a feed-forward behind every kind of mixer and none behind every kind, value
heads smaller than, equal to and larger than the query/key heads, one and several key/value heads, partly and
wholly rotated heads, two to four conv taps, state sizes that are no power of two, scales of 1 and other
values, widths that are no multiple of a warp."""


def mamba(inner, state, dt_rank, conv, ff=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(heads, kv_heads, dim, vdim, rot_dims, base, scale, width, left_scale, right_scale, ff=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                               "rot": {"base": base, "dims": rot_dims}},
                      "right": {"width": width}, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, scale, eps, layers):
    return {"architecture": "Vunolorn", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


V_A = config(131, 48, 3.0, 1e-5, [
    delta(4, 2, 16, 24, 3, ff=80),
    parallel(4, 2, 16, 16, 8, 10000.0, 0.3, 40, 1.1, 0.7),
    mamba(64, 5, 3, 2, ff=96),
])

V_B = config(257, 64, 1.0, 1e-6, [
    mamba(96, 16, 4, 4),
    parallel(3, 1, 32, 48, 32, 500.0, 0.2, 50, 0.5, 1.0, ff=100),
    parallel(2, 2, 24, 8, 12, 1000000.0, 0.25, 70, 1.0, 1.3),
    delta(2, 2, 8, 16, 2),
    mamba(40, 33, 7, 3, ff=72),
])

# one layer of each kind, alone: a fault shows in the mechanism that has it
ONLY = {
    "scan": config(97, 40, 2.0, 1e-5, [mamba(56, 6, 4, 3)]),
    "delta": config(97, 40, 2.0, 1e-5, [delta(4, 2, 12, 20, 4)]),
    "pair": config(97, 40, 2.0, 1e-5, [parallel(4, 2, 16, 24, 16, 300.0, 0.35, 36, 0.8, 0.9)]),
    "scan_ff": config(97, 40, 2.0, 1e-5, [mamba(56, 6, 4, 3, ff=64)]),
    # few rotated dimensions: a key's score depends little on how far back it lies
    "echo": config(97, 40, 2.0, 1e-5, [parallel(4, 2, 16, 24, 4, 1000000.0, 0.35, 36, 0.8, 0.9)]),
}

# head size 64 and bfloat16-friendly sizes: the whole-model GPU tests reach the tensor-core attention kernels
# and the few-rows product kernels through it
V_C = config(1000, 256, 16.0, 1e-6, [
    parallel(4, 2, 64, 64, 64, 1000000.0, 0.125, 192, 0.9, 0.8, ff=384),
    mamba(512, 16, 16, 4),
    delta(4, 2, 64, 128, 4),
    parallel(8, 1, 64, 64, 32, 10000.0, 0.125, 256, 1.0, 1.0),
])

ALL = {"A": (V_A, 31), "B": (V_B, 37), "C": (V_C, 41)}
PAGE_SIZE = {"A": 8, "B": 16, "C": 64}
