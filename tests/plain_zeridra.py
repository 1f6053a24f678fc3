"""A plain, slow implementation of the Zeridra design: one function per mechanism, float64 on the CPU.

It shares no code with the engine.  ``weights`` is a dict name -> torch tensor (any float type), ``config`` the dict
form of config.json.  Everything is computed per sequence, whole prompt at once.

    rms_norm(x)       = x / sqrt(mean(x^2) + eps) * w
    layer             h = rms_norm(x);  x += ls1 * mixer(h) + ls2 * ff(h)         (one norm, both sub-layers read it)
    attention         grouped heads whose values are their keys; queries warmed up with the position; a denominator
                      that also holds a one
    latent_attention  queries and keys/values through low-rank latents, one turning key part shared by the heads, a
                      window, a learned term in the denominator; a layer may read an earlier layer's latents
    feed-forward      a sigmoid router picks ``top`` experts; each sees the token times its score
    logits            head(rms_norm(x)) * logit_scale, capped by a tanh
"""
import math

import torch

F = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F)


def turn_pairs(x, positions, rot):
    """x: [T, ..., n]; the first rot.dims elements of the last axis turn, element 2i paired with 2i + 1:
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i / dims)."""
    if not rot:
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def visible(positions, window=None):
    """[T, T] bool: query i (rows) sees key j (columns): 0 <= i - j (< window)."""
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    if window:
        seen = seen & (distance < int(window))
    return seen


def softmax_with_extra(scores, seen, extra):
    """Softmax over the seen keys whose denominator also holds exp(extra) (``extra``: [heads], no key, no value)."""
    scores = scores.masked_fill(~seen, -math.inf)
    extra = extra.to(F).view(-1, 1, 1)
    top = torch.maximum(scores.max(-1, keepdim=True).values, extra)
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(extra - top))


def query_temperature(positions, q_temp):
    """1 + coef * ln(floor((p + 1) / every) + 1), per position."""
    if not q_temp:
        return torch.ones(positions.shape[0], dtype=F)
    steps = torch.div(positions + 1, int(q_temp["every"]), rounding_mode="floor").to(F)
    return 1.0 + float(q_temp["coef"]) * torch.log(steps + 1.0)


def attention_mixer(h, positions, mixer, weights, prefix, one_more=True):
    """Grouped-query attention without rotation and without a value projection: a key is also its value.  ``one_more``
    False leaves the one out of the denominator (a deliberately wrong model)."""
    heads, groups, dim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"])
    T = h.shape[0]
    q = (h @ weights[prefix + "q"].to(F).T).view(T, heads, dim)
    k = (h @ weights[prefix + "k"].to(F).T).view(T, groups, dim)
    q = q * query_temperature(positions, mixer.get("q_temp")).view(T, 1, 1)
    k = k.repeat_interleave(heads // groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(mixer["scale"])
    p = softmax_with_extra(scores, visible(positions), torch.zeros(heads) if one_more else torch.full((heads,), -1e30))
    out = torch.einsum("hij,jhd->ihd", p, k).reshape(T, heads * dim)
    return out @ weights[prefix + "o"].to(F).T


def latent_kv(h, positions, mixer, weights, prefix, eps):
    """What a latent layer leaves per token: the normalised latent and the turned key part."""
    rank = int(mixer["kv_rank"])
    down = h @ weights[prefix + "dkv"].to(F).T
    c = rms_norm(down[:, :rank], weights[prefix + "dkv.norm"], eps)
    return c, turn_pairs(down[:, rank:], positions, mixer.get("rot"))


def latent_mixer(h, positions, mixer, weights, prefix, eps, kv, window_shift=0):
    """``kv`` = (c [T, kv_rank], turned key part [T, rot_dim]): the layer's own, or those of the layer it names."""
    heads, dim, rot_dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer.get("rot_dim") or 0), int(mixer["vdim"])
    T = h.shape[0]
    c, k_turn = kv
    c_q = rms_norm(h @ weights[prefix + "dq"].to(F).T, weights[prefix + "dq.norm"], eps)
    q = (c_q @ weights[prefix + "uq"].to(F).T).view(T, heads, dim + rot_dim)
    q_still, q_turn = q[..., :dim], turn_pairs(q[..., dim:], positions, mixer.get("rot"))
    k_still = (c @ weights[prefix + "uk"].to(F).T).view(T, heads, dim)
    v = (c @ weights[prefix + "uv"].to(F).T).view(T, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_still, k_still) + torch.einsum("ihd,jd->hij", q_turn, k_turn)) * float(mixer["scale"])
    window = (mixer.get("mask") or {}).get("size")
    seen = visible(positions, int(window) + window_shift if window else None)
    p = softmax_with_extra(scores, seen, weights[prefix + "sink"])
    out = torch.einsum("hij,jhd->ihd", p, v).reshape(T, heads * vdim)
    return out @ weights[prefix + "o"].to(F).T


def route(h, mlp, weights, prefix):
    """(chosen [T, top], scores [T, top]): the experts with the largest sigmoid(router h), the lower index on a tie."""
    s = torch.sigmoid(h @ weights[prefix + "router"].to(F).T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :int(mlp["router"]["top"])]
    return order, torch.gather(s, 1, order)


def expert(x, weights, prefix):
    gate, up = x @ weights[prefix + "gate"].to(F).T, x @ weights[prefix + "up"].to(F).T
    return (gate * torch.sigmoid(gate) * up) @ weights[prefix + "down"].to(F).T


def route_margin(h, mlp, weights, prefix):
    """Per token, the gap between the last chosen score and the best one left out (inf when every expert is chosen)."""
    s = torch.sort(torch.sigmoid(h @ weights[prefix + "router"].to(F).T), dim=-1, descending=True).values
    top = int(mlp["router"]["top"])
    return s[:, top - 1] - s[:, top] if top < s.shape[1] else torch.full((h.shape[0],), math.inf, dtype=F)


def feed_forward(h, mlp, weights, prefix):
    """sum over a token's chosen experts e of expert_e(score_e * h): the score multiplies what goes in."""
    chosen, scores = route(h, mlp, weights, prefix)
    out = torch.zeros_like(h)
    for e in range(int(mlp["router"]["experts"])):
        for slot in range(chosen.shape[1]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += expert(scores[rows, slot, None] * h[rows], weights, f"{prefix}e{e}.")
    return out


def forward(config, weights, tokens, keep_layers=False, window_shift=0, drop_sinks=False, margins=None):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the stream behind every layer).  ``window_shift``
    and ``drop_sinks`` make deliberately wrong models for the tests that show a fault would be seen.  ``margins`` (a
    list): gets one tensor [T], the smallest routing margin of each token over all layers."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = weights["embed"].to(F)[tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    left, streams = {}, []
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}.", layer["mixer"]
        h = rms_norm(x, weights[prefix + "norm1"], eps)
        if layer["type"] == "attention":
            mixed = attention_mixer(h, positions, mixer, weights, prefix + "mix.", one_more=not drop_sinks)
        else:
            if mixer.get("kv_from") is None:
                left[index] = latent_kv(h, positions, mixer, weights, prefix + "mix.", eps)
            local = dict(weights)
            if drop_sinks:
                local[prefix + "mix.sink"] = torch.full_like(weights[prefix + "mix.sink"].to(F), -1e30)
            mixed = latent_mixer(h, positions, mixer, local, prefix + "mix.", eps,
                                 left[index if mixer.get("kv_from") is None else int(mixer["kv_from"])], window_shift)
        x = x + mixed * weights[prefix + "ls1"].to(F)
        if layer.get("mlp") is not None:
            if margins is not None:
                margin = route_margin(h, layer["mlp"], weights, prefix + "mlp.")
                margins[:] = [margin if not margins else torch.minimum(margins[0], margin)]
            x = x + feed_forward(h, layer["mlp"], weights, prefix + "mlp.") * weights[prefix + "ls2"].to(F)
        streams.append(x.clone())
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].to(F).T * float(config.get("logit_scale", 1.0))
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return (logits, torch.stack(streams)) if keep_layers else logits
