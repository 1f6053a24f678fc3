"""Latent attention: keys and values are made from one small latent per token, which is all the cache holds."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import KVPagesNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Queries through a latent of ``q_rank``, keys and values from a latent of ``kv_rank`` (the low-rank scheme of
    DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient Mixture-of-Experts Language Model"), with or without
    its rotating part:

        c_q = rmsnorm(W_dq x) * w_dq,   q = W_uq c_q                      [heads, dim + rot_dim]
        d   = W_dkv x                                                     [kv_rank + rot_dim]
        c   = rmsnorm(d[:kv_rank]) * w_dkv,   r = turn(d[kv_rank:])       what is cached: c and r
        k   = W_uk c,  v = W_uv c                                         [heads, dim], [heads, value_dim]
        s_h,j = (q_h[:dim] . k_h,j + turn(q_h[dim:]) . r_j) * scale       r is one key part shared by all heads
        y   = W_o concat_h(softmax_j(s_h,j) v_h,j)                        causal; the last ``window`` keys, if given;
                                                                          exp(sink_h) in the denominator, if given

    The engine never forms k and v: q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j,
    so a cached row [c | r] is read as ONE key/value head of kv_rank + rot_dim that all query heads share, keys and values
    being the same tensor (``KVPagesNeed(keys_only=True)``).  Queries are carried into that space head by head in front of
    the attention kernel (one matrix per head: W_uk,h^T on the still part, the identity on the turned part) and the
    attended rows out of it behind (W_uv,h on the latent part; the columns under r are zero), both with
    ``ops.head_linear``.

    Parameters: ``hidden``, ``heads``, ``dim``, ``value_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``eps``; ``rot_dim``
    (default 0: no rotating part; how it turns comes from the position encoding the layer names); ``window`` (None: every
    earlier key); ``cache_window``: the window the cache has to keep (default ``window``; larger where other layers read
    this layer's cache with wider windows, None where one of them reads everything); ``sinks`` (bool: a learned number
    per head); ``shared_kv`` (bool): the layer has no W_dkv and reads the rows another layer cached; ``names``: pairs
    (role, tensor name behind the prefix) for dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o, sinks."""

    KNOWN_PARAMS = ("hidden", "heads", "dim", "value_dim", "q_rank", "kv_rank", "scale", "eps", "names", "rot_dim", "window",
                    "cache_window", "sinks", "shared_kv")
    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "o": "o", "sinks": "sink"}

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"latent_attention has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, dim, value_dim = int(params["hidden"]), int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        q_rank, kv_rank, rot_dim = int(params["q_rank"]), int(params["kv_rank"]), int(params.get("rot_dim") or 0)
        name = cls.names(params)
        wanted = {name["dq"]: WeightDecl((q_rank, hidden)), name["dq_norm"]: WeightDecl((q_rank,), NORM),
                  name["uq"]: WeightDecl((heads * (dim + rot_dim), q_rank)), name["dkv"]: WeightDecl((kv_rank + rot_dim, hidden)),
                  name["dkv_norm"]: WeightDecl((kv_rank,), NORM), name["uk"]: WeightDecl((heads * dim, kv_rank)),
                  name["uv"]: WeightDecl((heads * value_dim, kv_rank)), name["o"]: WeightDecl((hidden, heads * value_dim))}
        if params.get("shared_kv"):
            del wanted[name["dkv"]], wanted[name["dkv_norm"]]
        if params.get("sinks"):
            wanted[name["sinks"]] = WeightDecl((heads,), WIDE)
        return wanted

    @classmethod
    def cache_need(cls, params):
        window = params["cache_window"] if "cache_window" in params else params.get("window")
        return KVPagesNeed(1, int(params["kv_rank"]) + int(params.get("rot_dim") or 0), int(window) if window else None, None,
                           keys_only=True)

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.dim, self.value_dim = int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        self.q_rank, self.kv_rank, self.rot_dim = int(params["q_rank"]), int(params["kv_rank"]), int(params.get("rot_dim") or 0)
        self.scale, self.eps = float(params["scale"]), float(params["eps"])
        self.window = int(params["window"]) if params.get("window") else 0
        self.shared_kv = bool(params.get("shared_kv"))
        self.row = self.kv_rank + self.rot_dim       # a cached row, and a query once it is carried into that space
        name = self.names(params)
        self.q_norm = weights[name["dq_norm"]].contiguous()
        if self.shared_kv:
            self.down, self.c_norm = weights[name["dq"]].contiguous(), None
        else:
            self.down = torch.cat([weights[name["dq"]], weights[name["dkv"]]], dim=0).contiguous()
            self.c_norm = weights[name["dkv_norm"]].contiguous()
            if self.q_norm.dtype != self.c_norm.dtype:
                self.q_norm, self.c_norm = self.q_norm.to(torch.float32), self.c_norm.to(torch.float32)
        self.up_q = weights[name["uq"]].contiguous()
        # per head: the matrix that carries a query [dim | rot_dim] into the cached rows' space [kv_rank | rot_dim] (the
        # transposed key matrix, and ones that pass the turned part on), and the value matrix [value_dim, kv_rank | 0],
        # which carries an attended row out of it
        up_k = weights[name["uk"]].view(self.heads, self.dim, self.kv_rank)
        up_v = weights[name["uv"]].view(self.heads, self.value_dim, self.kv_rank)
        self.key_in = torch.zeros((self.heads, self.row, self.dim + self.rot_dim), dtype=up_k.dtype, device=up_k.device)
        self.key_in[:, :self.kv_rank, :self.dim] = up_k.transpose(1, 2)
        if self.rot_dim:
            self.key_in[:, self.kv_rank:, self.dim:] = torch.eye(self.rot_dim, dtype=up_k.dtype, device=up_k.device)
        self.value_out = torch.zeros((self.heads, self.value_dim, self.row), dtype=up_v.dtype, device=up_v.device)
        self.value_out[:, :, :self.kv_rank] = up_v
        self.out = weights[name["o"]].contiguous()
        self.sinks = weights[name["sinks"]].to(torch.float32).contiguous() if params.get("sinks") else None
        self.inv_freq, self.rotary_dim, self.interleaved = None, 0, False

    def attach(self, position):
        """``position``: None (nothing turns) or an encoding with ``inv_freq`` (float32 [rotary_dim / 2] on the device) and,
        optionally, ``rotary_dim`` (at most rot_dim) and ``pairing`` ("halves" | "interleaved")."""
        if position is None:
            return
        inv_freq = getattr(position, "inv_freq", None)
        if inv_freq is None or not self.rot_dim:
            raise ValueError("latent_attention turns its rot_dim part by an encoding that gives inv_freq; this layer has "
                             f"rot_dim {self.rot_dim} and the encoding {type(position).__name__}")
        rotary_dim = int(getattr(position, "rotary_dim", 2 * inv_freq.numel()))
        if rotary_dim != 2 * inv_freq.numel() or rotary_dim > self.rot_dim or rotary_dim % 2:
            raise ValueError(f"the position encoding turns {rotary_dim} elements with {inv_freq.numel()} frequencies; "
                             f"latent_attention needs an even number of at most rot_dim {self.rot_dim} and half as many frequencies")
        if float(getattr(position, "attention_factor", 1.0)) != 1.0:
            raise ValueError("latent_attention does not scale the turned values (attention_factor must be 1)")
        pairing = getattr(position, "pairing", "halves")
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"latent_attention pairs turned elements as 'halves' or 'interleaved', not {pairing!r}")
        self.inv_freq, self.rotary_dim, self.interleaved = inv_freq, rotary_dim, pairing == "interleaved"

    def forward(self, x, batch, cache):
        tables = batch.block_tables[cache.group]
        down = ops.linear(x, self.down)
        if self.shared_kv:
            c_q = ops.rmsnorm(down, self.q_norm, self.eps)
        else:
            c_q = torch.empty((x.shape[0], self.q_rank), dtype=x.dtype, device=x.device)
            ops.norm_rope_units(down, batch.positions, batch.seq_of_token, tables, cache.k_pages, None, 1, 1, 1, self.q_rank,
                                self.row, 0, batch.error_flag, q_weight=self.q_norm, k_weight=self.c_norm, eps=self.eps,
                                inv_freq=self.inv_freq, rotary_dim=self.rotary_dim, q_out=c_q, write_cache=cache.writes,
                                k_norm_dim=self.kv_rank if self.rot_dim else 0, q_rot_start=-1, k_rot_start=self.kv_rank,
                                interleaved=self.interleaved)
        q = ops.linear(c_q, self.up_q)
        if self.inv_freq is not None:
            ops.rotate_units(q, batch.positions, self.heads, self.dim + self.rot_dim, self.inv_freq, self.rotary_dim,
                             rot_start=self.dim, interleaved=self.interleaved)
        q = ops.head_linear(q, self.key_in)
        attended = ops.attention(q, batch, tables, cache.k_pages, cache.v_pages, self.heads, 1, self.row, self.scale,
                                 self.window, sinks=self.sinks, precise=True, q_stride=self.heads * self.row)
        return ops.linear(ops.head_linear(attended, self.value_out), self.out)
