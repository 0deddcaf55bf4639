"""Tiny Sapatar configurations for the tests.  They differ from one another in every size and option: order of
layers, number of stream copies (several, one, none), layers with and without a feed-forward, layers that run on an
earlier layer's tensors, head counts and groups, key and value sizes (equal, different, multiples of 16 and not),
rotated share of a head (part, all, none), windows (short, longer than a page, none), decays, gate caps, numbers of
experts and of chosen experts (one, some, all), with and without a shared expert, vocabulary, eps."""


def moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def wkv(heads, dim, rank, mlp=None, **more):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp, **more}


def retention(heads, dim, vdim, decay, rot_dims, base, mlp=None, **more):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                           "rot": {"dims": rot_dims, "base": base}}, "mlp": mlp, **more}


def left(heads, kv_heads, dim, vdim, window, rot_dims, base, scale):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if window:
        d["mask"] = {"size": window}
    return d


def right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def parallel(lft, rgt, left_scale, right_scale, mlp=None, **more):
    return {"type": "parallel", "mixer": {"left": lft, "right": rgt, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp, **more}


_A_PAR = parallel(left(4, 2, 16, 32, 9, 8, 1000.0, 0.3), right(3, 16, 24, 6.0), 0.7, 1.4)
_A_WKV = wkv(2, 16, 8, mlp=moe(6, 2, 40, shared=24))
SAPATAR_A = {
    "architecture": "Sapatar", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [_A_WKV, _A_PAR, retention(2, 16, 8, [0.9, 0.99], 16, 5e4, mlp=moe(4, 4, 24)),
               {**_A_PAR, "weights_of": 1}, {**_A_WKV, "weights_of": 0}],
}

# one stream kept the plain way (no copies), equal key and value sizes that no tensor-core kernel takes, no rotation
SAPATAR_B = {
    "architecture": "Sapatar", "vocab": 97, "width": 40, "norm": {"eps": 1e-6},
    "layers": [parallel(left(3, 1, 24, 24, 5, 0, 10.0, 0.25), right(1, 8, 40, 3.0), 1.0, 1.0, mlp=moe(3, 1, 20, shared=12)),
               retention(1, 24, 40, [0.97], 12, 100.0, mlp=moe(5, 2, 16)), wkv(5, 8, 4)],      # the last layer has no feed-forward
}

# sizes the tensor-core attention kernels take (key = value = 64, the whole head rotated, a window longer than a page;
# then 32 with a part rotated and no window), a single copy of the stream
_C_PAR = parallel(left(8, 2, 64, 64, 40, 64, 3e5, 0.11), right(2, 32, 32, 15.0), 1.3, 0.6, mlp=moe(8, 3, 48, shared=64))
SAPATAR_C = {
    "architecture": "Sapatar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [_C_PAR, retention(4, 32, 16, [0.5, 0.9, 0.99, 1.0], 8, 7e3),
               parallel(left(4, 4, 32, 32, None, 16, 2e4, 0.2), right(4, 16, 16, 8.0), 0.5, 0.5),
               wkv(2, 64, 24, mlp=moe(4, 2, 32)), {**_C_PAR, "weights_of": 0}],
}

# sizes no fast path takes: a width that is no multiple of 8, odd head and feed-forward sizes, an odd vocabulary
SAPATAR_D = {
    "architecture": "Sapatar", "vocab": 53, "width": 36, "norm": {"eps": 1e-4}, "streams": 2,
    "layers": [retention(3, 10, 6, [0.8, 0.95, 0.999], 4, 9.0, mlp=moe(5, 2, 50, shared=27)),
               parallel(left(5, 5, 12, 20, 3, 12, 123.0, 0.4), right(3, 5, 7, 2.0), 2.0, 0.25),
               wkv(3, 12, 5, mlp=moe(2, 2, 9))],
}

# equal key and value sizes of 64 and 32 with windows that prompts of hundreds of tokens pass many times (the
# tensor-core prompt kernel, and the decode kernel that is fed by TMA, with pages given back on the way)
SAPATAR_E = {
    "architecture": "Sapatar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "streams": 2,
    "layers": [parallel(left(4, 2, 64, 64, 70, 32, 1e4, 0.125), right(2, 32, 32, 8.0), 1.1, 0.9, mlp=moe(6, 2, 32, shared=48)),
               wkv(3, 32, 8),
               parallel(left(2, 1, 32, 32, 150, 32, 5e5, 0.18), right(3, 16, 48, 5.0), 0.8, 1.2)],
}

SAPATAR_CONFIGS = {"A": SAPATAR_A, "B": SAPATAR_B, "C": SAPATAR_C, "D": SAPATAR_D}
SAPATAR_PAGE = {"A": 8, "B": 4, "C": 16, "D": 2}
SAPATAR_SEEDS = {"A": 15, "B": 16, "C": 17, "D": 18}
SAPATAR_STD = {"A": 0.12, "B": 0.2, "C": 0.08, "D": 0.25}
