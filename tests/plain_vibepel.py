"""A plain float64 implementation of the Vibepel decoder, written from the design's equations: one function per
mechanism, token-by-token recurrences, dense score matrices, no cache.  It shares nothing with the engine and serves as
the oracle of the tests.

Notation: T tokens, positions 0 .. T - 1; W x means the stored [out, in] matrix times the vector; a mixer's tensors are
looked up under its prefix.  Every function takes what came before the tokens it is given as explicit state, so the same
code answers "whole prompt" (state absent) and "continued from a state" (for tests of the state itself)."""
import math

import torch

F64 = torch.float64


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The block's norm: weights are stored as their distance from one."""
    return rms_divide(x, eps) * (1.0 + w)


def silu(x):
    return x * torch.sigmoid(x)


def squared_relu(x):
    return torch.relu(x) ** 2


# ------------------------------------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    dims, base = int(rot["dims"]), float(rot["base"])
    table = []
    scaling = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            wavelength = 2.0 * math.pi / f
            original, low, high, factor = (float(scaling[key]) for key in ("original", "low", "high", "factor"))
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        table.append(f)
    return torch.tensor(table, dtype=F64)


def rotate_heads(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims elements of every head turn, element i with element i + dims / 2."""
    dims = int(rot["dims"])
    angle = positions.to(F64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------------------------ windowed attention
def window_attention(h, weights, prefix, m, eps, first_position=0, want_probabilities=False):
    T = h.shape[0]
    H, G, D, DV = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ weights[prefix + "q"].T).view(T, H, D)
    k = (h @ weights[prefix + "k"].T).view(T, G, D)
    v = (h @ weights[prefix + "v"].T).view(T, G, DV)
    q = rms_divide(q, eps) * weights[prefix + "q.norm"]
    k = rms_divide(k, eps) * weights[prefix + "k.norm"]
    positions = torch.arange(first_position, first_position + T)
    if m.get("rot"):
        q, k = rotate_heads(q, positions, m["rot"]), rotate_heads(k, positions, m["rot"])
    distance = positions[:, None] - positions[None, :]
    visible = distance >= 0
    if m.get("mask"):
        visible = visible & (distance < int(m["mask"]["size"]))
    out = torch.zeros((T, H, DV), dtype=F64)
    kept = []
    for head in range(H):
        group = head // (H // G)
        scores = (q[:, head] @ k[:, group].T) * float(m["scale"])
        p = torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)
        kept.append(p)
        out[:, head] = p @ v[:, group]
    y = out.reshape(T, H * DV) @ weights[prefix + "o"].T
    return (y, kept) if want_probabilities else y


# ------------------------------------------------------------------------------------------------ gated delta rule
def short_convolution(x, taps_w, history=None):
    """x [T, C], taps_w [C, taps] (last column: the current token); history [taps - 1, C]: the inputs before x."""
    taps = taps_w.shape[1]
    if history is None:
        history = torch.zeros((taps - 1, x.shape[1]), dtype=F64)
    padded = torch.cat([history, x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + x.shape[0]] * taps_w[:, j]
    return y, padded[padded.shape[0] - (taps - 1):]


def delta_rule_scan(q, k, v, beta, g, S):
    """q, k [T, dim], v [T, vdim], beta, g [T]; S [dim, vdim] is advanced token by token."""
    out = torch.zeros((q.shape[0], v.shape[1]), dtype=F64)
    for t in range(q.shape[0]):
        S = g[t] * S
        d = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], d)
        out[t] = S.T @ q[t]
    return out, S


def gated_delta_rule(h, weights, prefix, m, eps, state=None):
    """state: None or (S [heads, dim, vdim], conv histories {role: [taps - 1, C]}); returns (y, new state)."""
    T = h.shape[0]
    H, G, D, DV = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    S, histories = state if state is not None else (torch.zeros((H, D, DV), dtype=F64), {})
    made, new_histories = {}, {}
    for role in ("q", "k", "v"):
        y, new_histories[role] = short_convolution(h @ weights[prefix + role].T, weights[prefix + role + ".conv"], histories.get(role))
        made[role] = silu(y)
    q = made["q"].view(T, G, D)
    k = made["k"].view(T, G, D)
    v = made["v"].view(T, H, DV)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ weights[prefix + "b"].T)
    g = torch.exp(-torch.exp(weights[prefix + "A_log"]) * torch.nn.functional.softplus(h @ weights[prefix + "a"].T + weights[prefix + "dt_bias"]))
    out = torch.zeros((T, H, DV), dtype=F64)
    new_S = torch.zeros_like(S)
    for head in range(H):
        group = head // (H // G)
        out[:, head], new_S[head] = delta_rule_scan(q[:, group], k[:, group], v[:, head], beta[:, head], g[:, head], S[head])
    gate = silu(h @ weights[prefix + "g"].T).view(T, H, DV)
    y = (rms_divide(out, eps) * weights[prefix + "norm"] * gate).reshape(T, H * DV) @ weights[prefix + "o"].T
    return y, (new_S, new_histories)


# ------------------------------------------------------------------------------------------------ time mixing
def wkv_scan(r, k, v, w, u, S):
    """r, k, v, w [T, dim], u [dim]; the current token reads the state before its own write, plus its bonus."""
    out = torch.zeros_like(v)
    for t in range(r.shape[0]):
        kv = torch.outer(k[t], v[t])
        out[t] = (S + u[:, None] * kv).T @ r[t]
        S = w[t][:, None] * S + kv
    return out, S


def time_mix(h, weights, prefix, m, eps, state=None):
    """state: None or (S [heads, dim, dim], the input row before h [width]); returns (y, new state)."""
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    S, before = state if state is not None else (torch.zeros((H, D, D), dtype=F64), torch.zeros(h.shape[1], dtype=F64))
    previous = torch.cat([before[None, :], h[:-1]], dim=0)

    def mixed(which):
        return h + (previous - h) * weights[prefix + "mu." + which]

    r = (mixed("r") @ weights[prefix + "r"].T).view(T, H, D)
    k = (mixed("k") @ weights[prefix + "k"].T).view(T, H, D)
    v = (mixed("v") @ weights[prefix + "v"].T).view(T, H, D)
    gate = silu(mixed("g") @ weights[prefix + "g"].T)
    log_log = torch.tanh(mixed("w") @ weights[prefix + "w1"].T) @ weights[prefix + "w2"].T + weights[prefix + "w0"]
    w = torch.exp(-torch.exp(log_log)).view(T, H, D)
    out = torch.zeros((T, H, D), dtype=F64)
    new_S = torch.zeros_like(S)
    for head in range(H):
        out[:, head], new_S[head] = wkv_scan(r[:, head], k[:, head], v[:, head], w[:, head], weights[prefix + "u"][head], S[head])
    y = (rms_divide(out, eps).reshape(T, H * D) * weights[prefix + "norm"] * gate) @ weights[prefix + "o"].T
    return y, (new_S, h[-1])


# ------------------------------------------------------------------------------------------------ the model
def feed_forward(h, weights, prefix):
    return squared_relu(h @ weights[prefix + "up"].T) @ weights[prefix + "down"].T


def mixer_output(layer, x, weights, prefix, eps, lose_state_at=None):
    """One layer's mixer over the whole sequence.  ``lose_state_at``: recurrent state and convolution history are dropped
    in front of that token (what a fault in the state manager would do), windows untouched."""
    m = layer["mixer"]

    def recurrent(function, *args):
        if lose_state_at is None:
            return function(x, *args)[0]
        return torch.cat([function(x[:lose_state_at], *args)[0], function(x[lose_state_at:], *args)[0]], dim=0)

    if layer["type"] == "wkv":
        return recurrent(time_mix, weights, prefix, m, eps)
    left = window_attention(x, weights, prefix + "left.", m["left"], eps)
    right = recurrent(gated_delta_rule, weights, prefix + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def forward(config, weights, tokens, lose_state_at=None, streams=None):
    """float64 logits [T, vocab] of the whole sequence."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"][torch.tensor(list(tokens))] * float((config.get("embedding") or {}).get("scale", 1.0))
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        x = x + offset_norm(mixer_output(layer, x, weights, prefix + "mix.", eps, lose_state_at), weights[prefix + "norm1"], eps)
        if layer.get("mlp"):
            x = x + offset_norm(feed_forward(x, weights, prefix + "mlp."), weights[prefix + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    logits = offset_norm(x, weights["final.norm"], eps) @ weights["embed"].T
    cap = float(config.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits
