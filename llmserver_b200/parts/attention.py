"""Grouped-query attention over the paged cache, with optional per-head Q/K RMSNorm, rotary
positions and a sliding window."""
from __future__ import annotations

import functools

import torch

from .. import ops
from ..cache.manager import KVPagesNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """Q, K, V = x Wq^T, x Wk^T, x Wv^T as one fused product (utils/attention.py:54-66,118-128); each Q
    and K head RMS-normalised with a shared [D] weight before the rotation (utils/attention.py:38-39,
    143-158); K stored after norm and rotation, V raw (utils/attention.py:172-176); softmax(Q K^T *
    scale) V over the request's cached tokens, query head h reading kv head h // group
    (utils/attention.py:186-198); output through Wo (utils/attention.py:299-300).

    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``scale``, ``qk_norm`` (bool),
    ``eps`` (of the Q/K norms), ``window`` (None = all keys; else a query at position p reads keys
    p - window + 1 .. p).  ``bias`` and ``softcap`` are known and must be off: the kernels have neither a bias
    epilogue nor score capping, and say so instead of computing without them.  ``value_dim``: the size of a value
    head where it differs from ``head_dim`` (the output projection then reads heads * value_dim columns).  ``sinks``
    (bool): a learned number per query head joins each softmax's denominator as exp(sink), without a key or a value,
    neither scaled nor masked.  ``precise_weights`` (bool): the design wants its attention weights in 32-bit, so the
    bfloat16 kernels may not round them to 8 bits for the P V product.  ``values_are_keys`` (bool): there is no value
    projection, a head's key as projected (and normalised and rotated, where the layer does that) is also its value; the
    cache then keeps keys alone.  ``unit_sink`` (bool): every softmax denominator holds one more 1 (a sink whose score is
    0, without a learned number).  ``query_temperature`` = (coef, every): the query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1).  ``names``: pairs (role, tensor name behind the prefix) for checkpoints that call the
    tensors otherwise; roles are q, k, v, o, q_norm, k_norm, sinks.

    How positions are encoded comes from the position encoding the layer names (``attach``): its inverse
    frequencies, how many elements of a head rotate (``rotary_dim``, at most head_dim) and how they pair
    ("halves" or "interleaved").  An encoding that scales the rotated values (``attention_factor`` other than 1) is
    goes through the rotation kernel that takes a magnitude, which has no per-head norm: with ``qk_norm`` it is
    refused.  The same kernel serves heads whose values have another size than their keys; with ``qk_norm`` as well,
    such heads go through the kernel for heads made of units (pairing "halves" only)."""

    KNOWN_PARAMS = ("hidden", "heads", "kv_heads", "head_dim", "scale", "qk_norm", "eps", "window", "bias", "softcap",
                    "value_dim", "sinks", "names", "precise_weights", "values_are_keys", "unit_sink", "query_temperature")
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sinks": "sinks"}

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"gqa_attention has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if params.get("bias"):
            raise ValueError("gqa_attention has no biases in its projections (bias must be absent or false)")
        if params.get("softcap"):
            raise ValueError("gqa_attention does not cap attention scores (softcap must be absent or 0)")
        if params.get("values_are_keys") and params.get("value_dim") and int(params["value_dim"]) != int(params["head_dim"]):
            raise ValueError("gqa_attention: values that are the keys have the keys' size")
        if params.get("unit_sink") and params.get("sinks"):
            raise ValueError("gqa_attention: a softmax has learned sinks or the unit sink, not both")
        temperature = params.get("query_temperature")
        if temperature and (len(temperature) != 2 or int(temperature[1]) <= 0):
            raise ValueError("gqa_attention: query_temperature is (coef, every) with a positive period")

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, kv_heads, dim = params["hidden"], params["heads"], params["kv_heads"], params["head_dim"]
        value_dim = params.get("value_dim") or dim
        name = cls.names(params)
        wanted = {name["q"]: WeightDecl((heads * dim, hidden)),
                  name["k"]: WeightDecl((kv_heads * dim, hidden)),
                  name["v"]: WeightDecl((kv_heads * value_dim, hidden)),
                  name["o"]: WeightDecl((hidden, heads * value_dim))}
        if params.get("values_are_keys"):
            del wanted[name["v"]]
        if params.get("qk_norm"):
            wanted[name["q_norm"]] = WeightDecl((dim,), NORM)
            wanted[name["k_norm"]] = WeightDecl((dim,), NORM)
        if params.get("sinks"):
            wanted[name["sinks"]] = WeightDecl((heads,), WIDE)
        return wanted

    @classmethod
    def cache_need(cls, params):
        if params.get("values_are_keys"):
            return KVPagesNeed(int(params["kv_heads"]), int(params["head_dim"]), params.get("window"), None, keys_only=True)
        return KVPagesNeed(int(params["kv_heads"]), int(params["head_dim"]), params.get("window"),
                           int(params["value_dim"]) if params.get("value_dim") else None)

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.kv_heads, self.head_dim = int(params["heads"]), int(params["kv_heads"]), int(params["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else 0
        self.eps = float(params.get("eps", 0.0))
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        # keys and values of different sizes are rotated and cached by the kernel for split sizes
        self.split = self.value_dim != self.head_dim
        name = self.names(params)
        self.values_are_keys = bool(params.get("values_are_keys"))
        self.temperature = tuple(params["query_temperature"]) if params.get("query_temperature") else None
        self.qkv = torch.cat([weights[name["q"]], weights[name["k"]]] + ([] if self.values_are_keys else [weights[name["v"]]]),
                             dim=0).contiguous()
        self.out = weights[name["o"]].contiguous()
        self.q_norm = weights[name["q_norm"]].contiguous() if params.get("qk_norm") else None
        self.k_norm = weights[name["k_norm"]].contiguous() if params.get("qk_norm") else None
        self.sinks = weights[name["sinks"]].to(torch.float32).contiguous() if params.get("sinks") else None
        if params.get("unit_sink"):
            self.sinks = torch.zeros(self.heads, dtype=torch.float32, device=runtime.device)      # exp(0): a one in every denominator
        # keys that are their own values and queries with a temperature go through the kernel for heads made of units
        self.by_units = self.values_are_keys or self.temperature is not None
        self.inv_freq, self.rotary_dim, self.interleaved, self.magnitude = None, self.head_dim, False, 1.0

    def attach(self, position):
        """``position``: None (no rotation) or an encoding with ``inv_freq`` (float32 [rotary_dim / 2] on the device)
        and, optionally, ``rotary_dim``, ``pairing`` ("halves" | "interleaved") and ``attention_factor``."""
        if position is None:
            return
        inv_freq = getattr(position, "inv_freq", None)
        if inv_freq is None:
            raise ValueError(f"gqa_attention rotates queries and keys: the position encoding {type(position).__name__} "
                             "gives no inv_freq (an encoding that acts on the embedding is not named by a layer)")
        rotary_dim = int(getattr(position, "rotary_dim", 2 * inv_freq.numel()))
        if rotary_dim != 2 * inv_freq.numel() or rotary_dim > self.head_dim or rotary_dim % 2:
            raise ValueError(f"the position encoding rotates {rotary_dim} elements with {inv_freq.numel()} frequencies; "
                             f"gqa_attention needs an even rotary_dim of at most head_dim {self.head_dim} and half as many frequencies")
        pairing = getattr(position, "pairing", "halves")
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"gqa_attention pairs rotated elements as 'halves' or 'interleaved', not {pairing!r}")
        self.magnitude = float(getattr(position, "attention_factor", 1.0))
        if self.magnitude != 1.0:
            if self.by_units:
                raise ValueError("gqa_attention: the kernel for heads made of units does not scale the rotated values, and the "
                                 f"position encoding's attention_factor is {self.magnitude}")
            if self.q_norm is not None:
                raise ValueError("gqa_attention: the rotation kernel that applies per-head Q/K norms does not scale the rotated "
                                 f"values, and the position encoding's attention_factor is {self.magnitude}")
            self.split = True
        self.inv_freq, self.rotary_dim, self.interleaved = inv_freq, rotary_dim, pairing == "interleaved"
        if self.interleaved and self.split and self.q_norm is not None and not self.by_units:
            raise ValueError("gqa_attention: per-head Q/K norms with values of another size than the keys rotate in halves only")

    feeds_stream = True

    @functools.cached_property
    def takes_unscaled(self):
        return not self.split and not self.by_units and ops.unscaled_rows_supported(self.qkv)

    def forward(self, x, batch, cache, sink=None):
        tables = batch.block_tables[cache.group]
        if self.by_units:
            # one unit per head: norms, temperature, rotation and the cache write in one kernel; without a value projection
            # the packed row ends behind the keys and the V pages are the K pages
            qkv = ops.linear(x, self.qkv)
            rotating = self.rotary_dim if self.inv_freq is not None else 0
            ops.norm_rope_units(qkv, batch.positions, batch.seq_of_token, tables, cache.k_pages,
                                None if self.values_are_keys else cache.v_pages, self.heads, self.kv_heads, 1, self.head_dim,
                                self.head_dim, 0 if self.values_are_keys else self.value_dim, batch.error_flag,
                                q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, inv_freq=self.inv_freq,
                                rotary_dim=rotating, write_cache=cache.writes, interleaved=self.interleaved,
                                q_temp=self.temperature)
            attended = ops.attention(qkv, batch, tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads, self.head_dim,
                                     self.scale, self.window, value_dim=self.value_dim, sinks=self.sinks,
                                     precise=bool(self.params.get("precise_weights")), q_stride=qkv.shape[1])
            return ops.linear(attended, self.out, sink=sink)
        if self.split and self.q_norm is not None:
            # heads with a norm whose values have another size than their keys: the kernel for heads made of units, one
            # unit per head
            qkv = ops.linear(x, self.qkv)
            ops.norm_rope_units(qkv, batch.positions, batch.seq_of_token, tables, cache.k_pages, cache.v_pages, self.heads,
                                self.kv_heads, 1, self.head_dim, self.head_dim, self.value_dim, batch.error_flag,
                                q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, inv_freq=self.inv_freq,
                                rotary_dim=self.rotary_dim if self.inv_freq is not None else 0, write_cache=cache.writes)
        elif self.split:
            qkv = ops.linear(x, self.qkv)
            ops.rope_kv_write_split(qkv, self.inv_freq, self.magnitude, batch.positions, batch.seq_of_token, tables,
                                    cache.k_pages, cache.v_pages, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                                    cache.writes, batch.error_flag, self.rotary_dim if self.inv_freq is not None else 0,
                                    self.interleaved)
        else:
            qkv = ops.qkv_projection(x, self.qkv, self.q_norm, self.k_norm, self.inv_freq, batch.positions, batch.seq_of_token,
                                     tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads, self.head_dim, self.eps,
                                     cache.writes, batch.error_flag, self.rotary_dim, self.interleaved)
        attended = ops.attention(qkv, batch, tables, cache.k_pages, cache.v_pages, self.heads, self.kv_heads,
                                 self.head_dim, self.scale, self.window, value_dim=self.value_dim, sinks=self.sinks,
                                 precise=bool(self.params.get("precise_weights")))
        return ops.linear(attended, self.out, sink=sink)
