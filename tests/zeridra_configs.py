"""Small Zeridra configurations of the tests.  Between them they vary what a configuration may vary: the order of the two
kinds of layers, layers with and without a feed-forward, grouped and ungrouped key/value heads, queries with and without
a temperature, windows of one token, of a few and longer than any prompt, no window, a rotating part that turns whole,
in part or not at all, latent layers that read another layer's cache (with a narrower and with a wider window than its
owner), one expert per token, several and all, an embedding scale and a logit scale of one and other than one, capped and
uncapped logits."""


def _attention(heads, kv_heads, dim, scale, temperature=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
            "q_temp": {"coef": temperature[0], "every": temperature[1]} if temperature else None}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, dims, base=10000.0, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
             "mask": {"size": window} if window else None, "rot": {"base": base, "dims": dims} if dims else None}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


# sizes that are a multiple of nothing much: a width of 44, heads of 10 and 14 elements, experts of 18 and 27 rows
ATTENTION_ONLY = {
    "architecture": "Zeridra", "vocab": 211, "width": 44, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "logit_scale": 1.0,
    "layers": [
        {"type": "attention", "mixer": _attention(3, 3, 14, 0.25, (0.5, 7)), "mlp": None},
        {"type": "attention", "mixer": _attention(6, 2, 10, 0.35), "mlp": _moe(5, 2, 18)},
        {"type": "attention", "mixer": _attention(2, 1, 24, 0.2, (0.2, 1)), "mlp": _moe(3, 3, 27)},
    ],
}

LATENT_ONLY = {
    "architecture": "Zeridra", "vocab": 190, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
    "logit_scale": 0.5, "logit_softcap": 12.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 8, 24, 40, 0.25, 5, 8), "mlp": _moe(4, 1, 56)},
        {"type": "latent_attention", "mixer": _latent(5, 8, 12, 24, 72, 16, 0.35, None, 6, base=500.0), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(2, 24, 8, 40, 16, 40, 0.2, 1, 8, kv_from=0), "mlp": _moe(7, 3, 16)},
        {"type": "latent_attention", "mixer": _latent(4, 8, 4, 16, 32, 24, 0.3, 200, None), "mlp": None},
    ],
}

# both kinds; layer 2 reads layer 0's cache through a wider window than layer 0's own, layer 5 reads layer 4's through a
# narrower one, layer 6 reads every key layer 4 cached
ALL_KINDS = {
    "architecture": "Zeridra", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.7},
    "logit_scale": 2.0, "logit_softcap": 25.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 16, 16, 24, 40, 56, 0.18, 23, 16, base=2e5), "mlp": _moe(6, 2, 32)},
        {"type": "attention", "mixer": _attention(4, 2, 24, 0.2, (0.4, 16)), "mlp": _moe(9, 1, 48)},
        {"type": "latent_attention", "mixer": _latent(2, 32, 16, 48, 24, 56, 0.15, 61, 16, base=2e5, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _attention(6, 6, 16, 0.25), "mlp": _moe(4, 4, 24)},
        {"type": "latent_attention", "mixer": _latent(3, 24, 8, 16, 48, 32, 0.2, 40, 4), "mlp": _moe(5, 2, 40)},
        {"type": "latent_attention", "mixer": _latent(5, 8, 8, 32, 16, 32, 0.3, 9, 4, kv_from=4), "mlp": _moe(6, 2, 32)},
        {"type": "latent_attention", "mixer": _latent(2, 16, 8, 8, 32, 32, 0.25, None, 4, kv_from=4), "mlp": None},
    ],
}

# sizes at which the bfloat16 path takes its tensor-core kernels: heads of 64 and 128, cached latent rows of 64 and 128,
# widths and expert sizes in 64s
TENSOR_CORE_SIZES = {
    "architecture": "Zeridra", "vocab": 384, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
    "logit_scale": 0.4, "logit_softcap": 20.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 32, 32, 64, 64, 96, 0.125, 70, 32, base=1e5), "mlp": _moe(8, 2, 128)},
        {"type": "attention", "mixer": _attention(4, 2, 64, 0.125, (0.25, 32)), "mlp": _moe(6, 1, 64)},
        {"type": "latent_attention", "mixer": _latent(8, 64, 16, 32, 128, 48, 0.1, 150, 16), "mlp": None},
        {"type": "attention", "mixer": _attention(2, 1, 128, 0.09), "mlp": _moe(4, 3, 128)},
        {"type": "latent_attention", "mixer": _latent(2, 64, 32, 128, 64, 96, 0.1, 33, 32, base=1e5, kv_from=0), "mlp": _moe(8, 8, 64)},
    ],
}

# name -> (config.json contents, seed of the random weights)
ZERIDRA = {"attention_only": (ATTENTION_ONLY, 3), "latent_only": (LATENT_ONLY, 4), "all_kinds": (ALL_KINDS, 6),
           "tensor_core_sizes": (TENSOR_CORE_SIZES, 7)}
