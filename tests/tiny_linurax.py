"""Tiny Linurax configurations for the tests.  They differ from one another in every size and option:
order of layers (a recurrent layer first, an attention layer last, layers with and without a feed-forward
behind either mixer), head counts (groups of 2, of 1, a single head, a single key/value head), head sizes
(multiples of 16 and not), rotated share of a head (part, all, none), widths of the recurrent state,
feed-forward sizes (multiples of 8 and not), vocabulary, embedding scale, eps."""


def attention(heads, kv_heads, dim, rot_dims, base, scale, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                      "rot": {"dims": rot_dims, "base": base}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mingru(width, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


LINURAX_A = {
    "architecture": "Linurax", "vocab": 160, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [mingru(80, ff=96), attention(4, 2, 16, 8, 1000.0, 0.3, ff=72), attention(2, 2, 32, 32, 20000.0, 0.2),
               mingru(48)],
}

LINURAX_B = {
    "architecture": "Linurax", "vocab": 97, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [attention(3, 1, 24, 12, 50.0, 0.25), mingru(56, ff=100), attention(1, 1, 40, 0, 10000.0, 0.15, ff=44)],
}

# head sizes the tensor-core kernels take (64), more heads than a warp tile's eight columns in one group
LINURAX_C = {
    "architecture": "Linurax", "vocab": 211, "width": 128, "embedding": {"scale": 6.5}, "norm": {"eps": 1e-6},
    "layers": [attention(12, 1, 64, 32, 300000.0, 0.11, ff=160), mingru(192), attention(8, 4, 64, 64, 7000.0, 0.125, ff=None),
               mingru(64, ff=136)],
}

# sizes no fast path takes: a width that is no multiple of 8, a head size that is no multiple of 8, five heads that
# are their own key/value heads, odd recurrent and feed-forward sizes, an odd vocabulary
LINURAX_D = {
    "architecture": "Linurax", "vocab": 53, "width": 36, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-4},
    "layers": [mingru(30), attention(5, 5, 20, 10, 123.0, 0.2, ff=50), mingru(31, ff=27), attention(2, 1, 12, 12, 9.0, 0.4)],
}

LINURAX_CONFIGS = {"A": LINURAX_A, "B": LINURAX_B, "C": LINURAX_C, "D": LINURAX_D}
LINURAX_PAGE = {"A": 8, "B": 4, "C": 16, "D": 2}
LINURAX_SEEDS = {"A": 5, "B": 6, "C": 7, "D": 8}
LINURAX_STD = {"A": 0.12, "B": 0.2, "C": 0.08, "D": 0.25}
