"""Small Vepinex configurations for the tests: each differs from the others in every size, in the order of its
layers and in which options it has (a first layer of each kind, one query/key head for several heads, one
head, value columns that do not fill a block of the recurrence kernel, key sizes in each of its register
classes, one to five taps, a router that takes one expert or all of them, experts without a shared one, a
layer without a feed-forward, a latent layer that reads another's cache, sizes that allow no 16-byte pieces)."""


def mlstm(heads, dim, vdim, cap=15.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=6, gate_rank=10):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def model(width, vocab, layers, mlps, eps=1e-5):
    return {"architecture": "Vepinex", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{**layer, "mlp": mlp} for layer, mlp in zip(layers, mlps)]}


CONFIGS = {
    # latent attention first; the last layer reads its cache; a router that takes all of its experts
    "A": model(64, 257,
               [latent(3, 12, 4, 20, 24, base=500.0), delta(4, 2, 16, 8, 3, 5, 7), mlstm(3, 8, 20, cap=10.0), latent(2, 8, 4, 6, 24, base=500.0, kv_from=0)],
               [dense(96), moe(5, 2, 40, 1.5, shared=(24, 0.75)), None, moe(3, 3, 16, 1.0)]),
    # a matrix memory first, one head; one query/key head for six heads; five taps and two; a router that takes one expert
    "B": model(96, 500,
               [mlstm(1, 40, 48), delta(2, 2, 24, 40, 2), latent(4, 16, 8, 16, 32), delta(6, 1, 8, 16, 5, 9, 4), latent(2, 24, 16, 8, 40, base=1e6),
                latent(5, 8, 16, 24, 40, base=1e6, kv_from=4)],
               [moe(8, 1, 32, 2.0, shared=(48, 1.0)), dense(64), None, moe(4, 2, 24, 0.5, shared=(8, 3.0)), dense(200), moe(6, 4, 16, 1.0)],
               eps=1e-6),
    # the delta rule first; key sizes in the recurrence kernel's larger register classes; long heads
    "C": model(128, 300,
               [delta(2, 1, 136, 16, 4), mlstm(2, 72, 32, cap=5.0), latent(8, 32, 16, 32, 64), mlstm(4, 16, 8)],
               [dense(128), moe(16, 2, 64, 1.0, shared=(64, 1.0)), moe(2, 1, 96, 4.0), dense(32)]),
    # sizes that are multiples of two at most: no product on the tensor cores, no 16-byte pieces anywhere
    "D": model(54, 131,
               [delta(3, 3, 6, 10, 4, 3, 5), latent(3, 6, 2, 10, 10, base=100.0), mlstm(2, 6, 18, cap=8.0), latent(1, 10, 2, 14, 10, base=100.0, kv_from=1)],
               [moe(7, 3, 18, 1.0, shared=(10, 1.0)), dense(30), moe(3, 2, 14, 2.0), None]),
    # larger and deeper: two latent layers with latents of their own, each read by a later layer; many small experts
    "E": model(256, 1000,
               [latent(4, 48, 16, 40, 96, base=1e5), mlstm(4, 48, 96, cap=12.0), delta(4, 2, 96, 48, 3, 12, 20), latent(6, 32, 16, 32, 96, base=1e5, kv_from=0),
                delta(8, 8, 32, 32, 4, 8, 8), latent(2, 64, 64, 128, 160, base=3e4), mlstm(2, 128, 64), latent(8, 16, 64, 16, 160, base=3e4, kv_from=5)],
               [moe(32, 4, 64, 1.0, shared=(192, 1.0)), dense(512), moe(32, 4, 64, 1.0, shared=(192, 1.0)), None, moe(12, 3, 96, 6.0), dense(384),
                moe(32, 4, 64, 1.0, shared=(192, 1.0)), moe(5, 2, 200, 2.0, shared=(64, 0.5))]),
}
SEEDS = {"A": 101, "B": 202, "C": 303, "D": 404, "E": 505}
#: the configurations every test of the engine runs on; "E" has tests of its own
SMALL = ("A", "B", "C", "D")
