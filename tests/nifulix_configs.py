"""Small Nifulix configurations for the tests: each differs from the others in every size, in the order of
its layers and in which options it has (grouped or ungrouped heads, one key/value head, values longer or
shorter than keys, a window smaller than a page, no kept first tokens, no cap, a layer without a
feed-forward, rotation of part of a head, blending that starts in a later layer)."""


def attention(heads, kv_heads, dim, vdim, window=None, keep_first=0, softcap=None, v_mix=False, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def retention(heads, dim, vdim, decay, rot_dims=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "retention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def model(width, vocab, layers, ffs, mult=0.5, eps=1e-5):
    out = []
    for layer, ff in zip(layers, ffs):
        out.append({**layer, "mlp": {"kind": "dense", "ff": ff} if ff else None})
    return {"architecture": "Nifulix", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps}, "layers": out}


CONFIGS = {
    # retention first; windows smaller than a page; blending between the two attention layers
    "P": model(48, 211, [retention(3, 16, 24, (0.9, 0.95, 0.99), rot_dims=8, base=500.0),
                         attention(4, 2, 16, 24, window=20, keep_first=3, softcap=5.0, v_mix=True),
                         latent(3, 8, 4, 12, 20, 24, window=37),
                         attention(6, 2, 16, 24, window=9, keep_first=0, v_mix=True, scale=0.4)],
               [64, 80, None, 64], mult=0.7),
    # one key/value head, ungrouped heads, values shorter than keys, no window at all, no rotation in the retention,
    # a window that spans pages, blending that starts at the second attention layer
    "Q": model(80, 300, [attention(2, 1, 32, 16, softcap=20.0),
                         latent(2, 16, 8, 16, 24, 40),
                         attention(3, 3, 16, 32, window=70, keep_first=5, v_mix=True),
                         retention(2, 24, 16, (0.97, 0.999)),
                         attention(3, 3, 16, 32, window=130, keep_first=2, softcap=50.0, v_mix=True),
                         latent(5, 12, 6, 8, 16, 28, window=66, base=77.0)],
               [96, 96, 112, 96, None, 96], mult=0.3, eps=1e-6),
    # one layer of each kind, heads of 64 and more, a state larger than a warp's
    "R": model(128, 128, [latent(4, 32, 16, 32, 48, 64, window=100),
                          retention(2, 64, 64, (0.98, 0.995), rot_dims=64, base=1e6),
                          attention(8, 2, 64, 64, window=64, keep_first=4, softcap=30.0, v_mix=True)],
               [256, 256, 256], mult=1.0),
    # long keys and values (the heavy forms of the kernels: blocks of eight warps, states spread over blocks, the head-wise
    # maps as one product a head), keys and values of different sizes, more kept first tokens than a page
    "T": model(256, 400, [latent(4, 32, 32, 32, 96, 224, window=200, base=5e4),
                          attention(8, 2, 128, 96, window=150, keep_first=70, softcap=25.0, v_mix=True),
                          retention(2, 128, 128, (0.99, 0.999), rot_dims=128, base=1e6),
                          attention(4, 2, 160, 96, v_mix=True)],
               [320, None, 320, 320], mult=0.4),
    # sizes that are multiples of nothing in particular: the products' and the kernels' roads for rows and heads that allow
    # no 16-byte pieces, groups of two heads, a window and kept tokens that end inside a page
    "U": model(100, 333, [attention(6, 3, 20, 28, window=33, keep_first=2, softcap=12.0, v_mix=True, scale=0.3),
                          retention(3, 12, 20, (0.9, 0.97, 0.995), rot_dims=6, base=300.0),
                          latent(5, 12, 6, 10, 36, 50, window=45, base=700.0),
                          attention(3, 3, 20, 28, window=70, keep_first=9, v_mix=True)],
               [130, 130, 70, None], mult=0.6, eps=1e-4),
    # nothing but retention (no paged cache at all), heads whose sizes are no powers of two, one layer without a feed-forward
    "S": model(40, 150, [retention(2, 20, 12, (0.9, 0.99), rot_dims=10, base=100.0), retention(5, 8, 8, (0.5, 0.8, 0.9, 0.95, 0.999))],
               [None, 48], mult=0.9),
}
SEEDS = {"P": 5, "Q": 6, "R": 7, "S": 8, "T": 9, "U": 10}
