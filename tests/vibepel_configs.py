"""Small Vibepel configurations of the tests.  Between them they vary what a configuration may vary: the order of the two
kinds of layers, layers with and without a feed-forward, grouped and ungrouped heads on either side of a parallel layer,
value heads smaller and larger than key heads, windows of one token, of a few and longer than any prompt, no window, a
part of a head rotating, all of it or nothing, frequencies scaled band by band or left alone, convolutions of two to
five taps, branch scales of one and far from it, decay ranks, capped and uncapped logits, and embedding scales of one,
below and above it (the deepest model's is above: a stream that starts small lets every sub-layer's bfloat16 rounding weigh
more in what the next ones read)."""


def _left(heads, kv_heads, dim, vdim, scale, window, dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims, "scaling": scaling} if dims else None
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window} if window else None, "rot": rot}


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _wkv(heads, dim, rank, mlp):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "w_rank": rank}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


BANDS = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}

WKV_ONLY = {
    "architecture": "Vibepel", "vocab": 150, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.6}, "logit_softcap": 0.0,
    "layers": [_wkv(2, 24, 8, None), _wkv(5, 8, 24, _dense(72)), _wkv(1, 72, 4, None)],
}

PARALLEL_ONLY = {
    "architecture": "Vibepel", "vocab": 211, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0}, "logit_softcap": 12.0,
    "layers": [
        _parallel(_left(3, 3, 16, 24, 0.25, 5, 8), _right(3, 3, 8, 16, 2), 1.0, 1.0, None),
        _parallel(_left(6, 2, 8, 8, 0.35, None, 8, base=500.0, scaling=BANDS), _right(4, 2, 24, 8, 5), 0.3, 1.7, _dense(40)),
        _parallel(_left(2, 1, 24, 40, 0.2, 1, None), _right(1, 1, 40, 33, 3), 2.0, 0.25, None),
        _parallel(_left(2, 2, 12, 10, 0.3, 400, 4, base=50.0, scaling=BANDS), _right(6, 1, 16, 8, 4), 0.5, 0.5, _dense(56)),
    ],
}

BOTH_KINDS = {
    "architecture": "Vibepel", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.5}, "logit_softcap": 25.0,
    "layers": [
        _wkv(3, 16, 12, _dense(64)),
        _parallel(_left(4, 2, 16, 16, 0.25, 23, 16, base=1e6, scaling={"factor": 6.0, "low": 1.0, "high": 3.5, "original": 64}),
                  _right(4, 2, 16, 24, 4), 0.62, 0.48, _dense(80)),
        _wkv(6, 16, 20, None),
        _parallel(_left(2, 1, 32, 48, 0.18, 9, 10), _right(2, 2, 32, 16, 3), 0.8, 1.2, None),
        _parallel(_left(4, 2, 16, 16, 0.25, 23, 16, base=1e6), _right(4, 2, 16, 24, 2), 0.58, 0.52, _dense(80)),
    ],
}

# sizes at which the bfloat16 path takes its tensor-core kernels (heads of 64 and 128, widths in 64s)
TENSOR_CORE_SIZES = {
    "architecture": "Vibepel", "vocab": 384, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_softcap": 30.0,
    "layers": [
        _parallel(_left(4, 2, 64, 64, 0.125, 70, 32, base=1e5, scaling={"factor": 5.0, "low": 0.5, "high": 4.0, "original": 128}),
                  _right(4, 2, 64, 64, 4), 0.7, 0.4, _dense(256)),
        _wkv(3, 64, 32, _dense(128)),
        _parallel(_left(2, 1, 128, 128, 0.09, 150, 128, base=1e4), _right(2, 1, 128, 128, 4), 0.5, 0.5, None),
        _parallel(_left(4, 1, 128, 64, 0.09, None, 64), _right(3, 3, 64, 128, 2), 1.0, 1.0, _dense(128)),
    ],
}

# name -> (config.json contents, seed of the random weights)
VIBEPEL = {"wkv_only": (WKV_ONLY, 3), "parallel_only": (PARALLEL_ONLY, 4), "both_kinds": (BOTH_KINDS, 5),
           "tensor_core_sizes": (TENSOR_CORE_SIZES, 6)}
