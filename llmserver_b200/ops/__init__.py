"""Tensor-level entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors and launches on PyTorch's current stream; none has a CPU or
library stand-in.  Shapes use N = tokens of the step, H = width of the residual stream.
The residual stream is always float32; "activation type" is the model's dtype (float32 on the
32-bit path, bfloat16 on the serving path).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .library import (KernelError, call, check, declare, dtype_code, launch_count, library, pointer,
                      require_device, stream_handle, wait_error_flag)
from .stream import STREAM_ROWS, RowScaled, StreamSink

__all__ = ["KernelError", "embedding", "add_rmsnorm", "rmsnorm", "silu_mul", "sample", "qk_norm_rope_kv_write",
           "attention_generic", "rope_kv_write_split", "normed_add_rmsnorm", "scaled_add_rmsnorm", "moe_route", "moe_select", "indexed_linear", "moe_combine", "moe_plan", "moe_grouped",
           "moe_grouped_supported", "moe_combine_rows", "ExpertPlan",
           "clamped_glu", "gemm_f32", "linear", "linear_wide", "qkv_projection", "gate_up_silu", "interleave_gate_up", "require_device", "library", "launch_count",
           "RowScaled", "StreamSink", "STREAM_ROWS", "unscaled_rows_supported", "norm_rope_units", "rotate_units", "attention_diff", "gla_supported",
           "gla_recurrent", "head_linear", "relu_squared", "tanh_narrow", "softcap_", "scaled_sum", "token_shift_mix",
           "short_conv_units", "matrix_recurrence_supported", "wkv_recurrent", "delta_rule_recurrent"]


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """residual[n] = table[ids[n]] * scale, widened to float32.  ids: int32 [N]."""
    check(table, "embedding table")
    check(ids, "token ids", torch.int32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    check(out, "embedding output", torch.float32, hidden)
    call("llm_embedding_gather", out.data_ptr(), table.data_ptr(), ids.data_ptr(), tokens, hidden, vocab,
         dtype_code(table.dtype), float(scale), stream_handle())
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                write_residual: bool = True, act_dtype: Optional[torch.dtype] = None, unscaled: bool = False):
    """residual += delta (in place, 32-bit), then out = rmsnorm(residual) * weight in the activation
    type ``act_dtype`` (default: weight's dtype; the weight may be float32 beside bfloat16 activations).

    ``rows`` (int32) selects source rows: output row o comes from row rows[o]; then the residual is
    left untouched and ``delta`` is added on the fly.  ``unscaled``: the division by the root mean square is left to
    the product that consumes the result; returns a ``RowScaled`` (residual * weight and the rows' sums of squares)."""
    check(residual, "residual", torch.float32)
    width = residual.shape[-1]
    check(weight, "norm weight", last_dim=width)
    act = act_dtype or weight.dtype
    if delta is not None:
        check(delta, "delta", act, width)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {tuple(residual.shape)}")
    if rows is not None:
        check(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // width
    if out is None:
        out = torch.empty((n_rows, width), dtype=act, device=residual.device)
    check(out, "norm output", act, width)
    squares = torch.empty((1, max(n_rows, 1)), dtype=torch.float32, device=residual.device) if unscaled else None
    call("llm_add_rmsnorm", residual.data_ptr(), pointer(delta), weight.data_ptr(), out.data_ptr(), pointer(rows),
         n_rows, width, float(eps), int(write_residual), dtype_code(act), dtype_code(weight.dtype), pointer(squares),
         stream_handle())
    return RowScaled(out, squares, eps) if unscaled else out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x) * weight over the last dimension; x in the activation type."""
    width = x.shape[-1]
    check(x, "x")
    check(weight, "norm weight", last_dim=width)
    if out is None:
        out = torch.empty_like(x)
    check(out, "norm output", x.dtype, width)
    call("llm_rmsnorm", x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // width, width, float(eps),
         dtype_code(x.dtype), dtype_code(weight.dtype), stream_handle())
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, group: int = 0) -> torch.Tensor:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]; gate_up is [N, 2 I], gate half first.  With ``group`` > 0
    gate and up columns are interleaved in groups of that many: output i finds its gate value at column
    (i // group) * 2 * group + i % group and its up value ``group`` columns further."""
    check(gate_up, "gate_up")
    rows, doubled = gate_up.shape
    if doubled % 2:
        raise KernelError(f"gate_up's last dimension must be even, got {doubled}")
    if out is None:
        out = torch.empty((rows, doubled // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(out, "silu_mul output", gate_up.dtype, doubled // 2)
    call("llm_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, doubled // 2, int(group), dtype_code(gate_up.dtype),
         stream_handle())
    return out


GATE_UP_GROUP = 64      # rows of gate and of up that share a 128-row tile of the fused weight


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """The fused [2 I, H] weight with gate and up rows interleaved in groups (see ``silu_mul``): a 128-row tile then
    holds 64 gate rows and their 64 up rows, so the product kernel can apply the gate in its epilogue."""
    inter, hidden = gate.shape
    if inter % group:
        raise KernelError(f"the intermediate size {inter} is no multiple of {group}")
    return torch.stack([gate.reshape(inter // group, group, hidden), up.reshape(inter // group, group, hidden)],
                       dim=1).reshape(2 * inter, hidden).contiguous()


def gate_up_silu(x, weight: torch.Tensor, group: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for the fused weight ``weight`` [2 I, H] (halves when ``group`` is 0, else interleaved in
    groups): as one kernel where the product kernel can apply the gate in its epilogue (bfloat16, groups of 64, few
    rows), else as the product followed by ``silu_mul``.  ``x`` may be a ``RowScaled``."""
    if x.dtype == torch.bfloat16 and group == GATE_UP_GROUP:
        from . import gemm_bf16
        fused = gemm_bf16.gate_up_silu_fused(x, weight)
        if fused is not None:
            return fused
    return silu_mul(linear(x, weight), group=group)


def sample(logits: torch.Tensor, temperatures: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
           steps: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: argmax where the temperature is 0, else the
    Gumbel-max draw keyed by (seeds[r], steps[r]).  Returns int32 [R]."""
    check(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperatures is not None:
        check(temperatures, "temperatures", torch.float32)
        if seeds is None or steps is None:
            raise KernelError("temperature sampling needs seeds and steps")
        check(seeds, "seeds", torch.int64)
        check(steps, "steps", torch.int32)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(out, "sampled tokens", torch.int32)
    slices = library().llm_sample_slices(rows, vocab)
    scores = indices = None
    if slices > 1:      # large vocabularies are scanned by several blocks per row, merged by a second kernel
        scores = torch.empty((rows, slices), dtype=torch.float32, device=logits.device)
        indices = torch.empty((rows, slices), dtype=torch.int32, device=logits.device)
    call("llm_sample", logits.data_ptr(), pointer(temperatures), pointer(seeds), pointer(steps), out.data_ptr(), rows,
         vocab, pointer(scores), pointer(indices), stream_handle())
    return out


def qk_norm_rope_kv_write(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                          block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, n_q_heads: int,
                          n_kv_heads: int, head_dim: int, eps: float, write_cache: bool,
                          error_flag: torch.Tensor, rotary_dim: Optional[int] = None, interleaved: bool = False) -> None:
    """In place on qkv [N, (Hq + 2 Hkv) D]: Q heads normalised and rotated where they are; K heads
    normalised, rotated and written to the K pages; V heads copied to the V pages.  Pages are
    [page, Hkv, page_size, D]; block_tables int32 [S, max_blocks].  ``rotary_dim`` (default: all of the head)
    elements of each head are rotated, by the angles position * inv_freq[i], i < rotary_dim / 2, paired as halves
    (i, i + rotary_dim / 2) or, ``interleaved``, as neighbours (2i, 2i + 1)."""
    if rotary_dim is None:
        rotary_dim = head_dim if inv_freq is None else 2 * inv_freq.numel()
    if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
        raise KernelError(f"rotary_dim must be even and at most head_dim {head_dim}, got {rotary_dim}")
    check(qkv, "qkv", last_dim=(n_q_heads + 2 * n_kv_heads) * head_dim)
    tokens = qkv.shape[0]
    weight_dtype = qkv.dtype
    for name, tensor in (("q norm weight", q_weight), ("k norm weight", k_weight)):
        if tensor is not None:
            check(tensor, name, last_dim=head_dim)
            weight_dtype = tensor.dtype
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    if inv_freq is not None:
        check(inv_freq, "inv_freq", torch.float32, rotary_dim // 2)
    check(positions, "positions", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(block_tables, "block_tables", torch.int32)
    check(k_pages, "k pages", qkv.dtype, head_dim)
    check(v_pages, "v pages", qkv.dtype, head_dim)
    if k_pages.shape != v_pages.shape or k_pages.dim() != 4 or k_pages.shape[1] != n_kv_heads:
        raise KernelError(f"pages must be [pages, {n_kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)}")
    if positions.numel() != tokens or seq_of_token.numel() != tokens:
        raise KernelError("positions and seq_of_token need one entry per token")
    check(error_flag, "error flag", torch.int32)
    call("llm_qk_norm_rope_kv_write", qkv.data_ptr(), pointer(q_weight), pointer(k_weight), pointer(inv_freq),
         positions.data_ptr(), seq_of_token.data_ptr(), block_tables.data_ptr(), block_tables.shape[-1],
         k_pages.data_ptr(), v_pages.data_ptr(), tokens, n_q_heads, n_kv_heads, head_dim, k_pages.shape[2],
         k_pages.shape[0], float(eps), int(write_cache), error_flag.data_ptr(), int(rotary_dim), int(bool(interleaved)),
         dtype_code(qkv.dtype), dtype_code(weight_dtype), stream_handle())


def attention_generic(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_tables: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                      n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      out: Optional[torch.Tensor] = None, error_flag: Optional[torch.Tensor] = None,
                      value_dim: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal (optionally windowed) attention of every token over its sequence's pages, 32-bit
    arithmetic.  ``q`` holds head h of token n at q[n * q_stride + h * D]; returns [N, Hq * Dv], Dv = ``value_dim``
    (default D).  ``sinks`` (float32 [Hq]): one more term exp(sinks[h]) in each head's softmax denominator.  A
    block-table entry that names no page of the pool is not followed: page 0 is read instead and ``error_flag``
    (default: the device's shared flag) is set to 5."""
    check(q, "q")
    tokens = positions.numel()
    value_dim = head_dim if value_dim is None else int(value_dim)
    check(k_pages, "k pages", q.dtype, head_dim)
    check(v_pages, "v pages", q.dtype, value_dim)
    if k_pages.shape[:-1] != v_pages.shape[:-1]:
        raise KernelError(f"k pages {tuple(k_pages.shape)} and v pages {tuple(v_pages.shape)} differ in more than the last dimension")
    check(block_tables, "block_tables", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(positions, "positions", torch.int32)
    if sinks is not None:
        check(sinks, "sinks", torch.float32)
        if sinks.numel() != n_q_heads:
            raise KernelError(f"sinks must hold one number per query head ({n_q_heads}), got {sinks.numel()}")
    if out is None:
        out = torch.empty((tokens, n_q_heads * value_dim), dtype=q.dtype, device=q.device)
    check(out, "attention output", q.dtype, n_q_heads * value_dim)
    call("llm_attention_generic", q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
         block_tables.data_ptr(), block_tables.shape[-1], seq_of_token.data_ptr(), positions.data_ptr(),
         out.data_ptr(), tokens, n_q_heads, n_kv_heads, head_dim, value_dim, k_pages.shape[2], k_pages.shape[0],
         float(scale), int(window), pointer(sinks),
         (error_flag if error_flag is not None else wait_error_flag(q.device)).data_ptr(), dtype_code(q.dtype),
         stream_handle())
    return out


def rope_kv_write_split(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], magnitude: float, positions: torch.Tensor,
                        seq_of_token: torch.Tensor, block_tables: torch.Tensor, k_pages: torch.Tensor,
                        v_pages: torch.Tensor, n_q_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                        write_cache: bool, error_flag: torch.Tensor, rotary_dim: Optional[int] = None,
                        interleaved: bool = False) -> None:
    """In place on qkv [N, (Hq + Hkv) D + Hkv Dv]: the first ``rotary_dim`` elements of every Q and K head rotated by
    position * inv_freq[i] with cos and sin multiplied by ``magnitude``; K heads written to the K pages
    [page, Hkv, page_size, D], V heads copied to the V pages [page, Hkv, page_size, Dv]."""
    if rotary_dim is None:
        rotary_dim = 0 if inv_freq is None else 2 * inv_freq.numel()
    check(qkv, "qkv", last_dim=(n_q_heads + n_kv_heads) * key_dim + n_kv_heads * value_dim)
    tokens = qkv.shape[0]
    if inv_freq is not None:
        check(inv_freq, "inv_freq", torch.float32, rotary_dim // 2)
    check(positions, "positions", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(block_tables, "block_tables", torch.int32)
    check(k_pages, "k pages", qkv.dtype, key_dim)
    check(v_pages, "v pages", qkv.dtype, value_dim)
    if k_pages.dim() != 4 or k_pages.shape[1] != n_kv_heads or k_pages.shape[:-1] != v_pages.shape[:-1]:
        raise KernelError(f"pages must be [pages, {n_kv_heads}, page_size, {key_dim} | {value_dim}], got "
                          f"{tuple(k_pages.shape)} and {tuple(v_pages.shape)}")
    if positions.numel() != tokens or seq_of_token.numel() != tokens:
        raise KernelError("positions and seq_of_token need one entry per token")
    check(error_flag, "error flag", torch.int32)
    call("llm_rope_kv_write_split", qkv.data_ptr(), pointer(inv_freq), float(magnitude), positions.data_ptr(),
         seq_of_token.data_ptr(), block_tables.data_ptr(), block_tables.shape[-1], k_pages.data_ptr(), v_pages.data_ptr(),
         tokens, n_q_heads, n_kv_heads, key_dim, value_dim, k_pages.shape[2], k_pages.shape[0], int(write_cache),
         error_flag.data_ptr(), int(rotary_dim), int(bool(interleaved)), dtype_code(qkv.dtype), stream_handle())


def normed_add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], post_weight: Optional[torch.Tensor],
                       post_eps: float, weight: Optional[torch.Tensor], eps: float, extra: Optional[torch.Tensor] = None,
                       rows: Optional[torch.Tensor] = None, act_dtype: Optional[torch.dtype] = None,
                       want_output: bool = True, delta_bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """residual += rmsnorm(delta + delta_bias) * post_weight (+ extra), all 32-bit and in place; then, unless
    ``want_output`` is False, returns rmsnorm(residual) * weight in the activation type, or, without a ``weight``, the
    updated stream itself in the activation type.  ``delta`` (activation type), ``delta_bias`` (float32 [width]: the bias
    of the projection that made delta) and ``extra`` (float32, the stream's shape) may each be absent.  With ``rows``
    (int32) output row o comes from row rows[o] and the stream is left as it was."""
    check(residual, "residual", torch.float32)
    width = residual.shape[-1]
    act = act_dtype or (delta.dtype if delta is not None else weight.dtype)
    if delta_bias is not None:
        check(delta_bias, "delta bias", torch.float32, width)
    weight_dtype = None
    for name, tensor in (("post-norm weight", post_weight), ("norm weight", weight)):
        if tensor is not None:
            check(tensor, name, last_dim=width)
            if weight_dtype is not None and tensor.dtype != weight_dtype:
                raise KernelError("the two norm weights must share a dtype")
            weight_dtype = tensor.dtype
    if delta is not None:
        check(delta, "delta", act, width)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {tuple(residual.shape)}")
    if extra is not None:
        check(extra, "extra stream", torch.float32, width)
        if extra.shape != residual.shape:
            raise KernelError(f"extra {tuple(extra.shape)} does not match residual {tuple(residual.shape)}")
    write_residual = rows is None
    if rows is not None:
        check(rows, "rows", torch.int32)
        n_rows = rows.numel()
    else:
        n_rows = residual.numel() // width
    out = torch.empty((n_rows, width), dtype=act, device=residual.device) if want_output else None
    call("llm_normed_add_rmsnorm", residual.data_ptr(), pointer(delta), pointer(post_weight), float(post_eps), pointer(extra),
         pointer(weight), pointer(out), pointer(rows), n_rows, width, float(eps), int(write_residual), dtype_code(act),
         dtype_code(weight_dtype if weight_dtype is not None else act), pointer(delta_bias), stream_handle())
    return out


def scaled_add_rmsnorm(residual: torch.Tensor, a: torch.Tensor, scale_a: torch.Tensor, b: Optional[torch.Tensor],
                       scale_b: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                       rows: Optional[torch.Tensor] = None, act_dtype: Optional[torch.dtype] = None,
                       want_output: bool = True) -> Optional[torch.Tensor]:
    """residual += a * scale_a (+ b * scale_b), 32-bit and in place, the scales float32 [width] per channel; then, unless
    ``want_output`` is False, returns rmsnorm(residual) * weight in the activation type.  ``a`` and ``b`` are two
    sub-layers' outputs in the activation type.  With ``rows`` (int32) output row o comes from row rows[o] and the stream
    is left as it was."""
    check(residual, "residual", torch.float32)
    width = residual.shape[-1]
    act = act_dtype or a.dtype
    for name, part, scale in (("first output", a, scale_a), ("second output", b, scale_b)):
        if part is None:
            continue
        check(part, name, act, width)
        if part.shape != residual.shape:
            raise KernelError(f"the {name} {tuple(part.shape)} does not match the stream {tuple(residual.shape)}")
        check(scale, name + "'s scale", torch.float32, width)
    if want_output:
        check(weight, "norm weight", last_dim=width)
    if rows is not None:
        check(rows, "rows", torch.int32)
        n_rows = rows.numel()
    else:
        n_rows = residual.numel() // width
    out = torch.empty((n_rows, width), dtype=act, device=residual.device) if want_output else None
    call("llm_scaled_add_rmsnorm", residual.data_ptr(), a.data_ptr(), scale_a.data_ptr(), pointer(b), pointer(scale_b),
         pointer(weight) if want_output else 0, pointer(out), pointer(rows), n_rows, width, float(eps), int(rows is None),
         dtype_code(act), dtype_code(weight.dtype if weight is not None else act), stream_handle())
    return out


def norm_rope_units(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_tables: torch.Tensor,
                    k_pages: torch.Tensor, v_pages: Optional[torch.Tensor], n_q_heads: int, n_kv_heads: int, maps: int,
                    q_dim: int, k_dim: int, value_dim: int, error_flag: torch.Tensor, bias: Optional[torch.Tensor] = None,
                    q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                    inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, q_out: Optional[torch.Tensor] = None,
                    write_cache: bool = True, k_norm_dim: int = 0, q_rot_start: int = 0, k_rot_start: int = 0,
                    interleaved: bool = False, q_temp: Optional[tuple] = None) -> None:
    """On the packed projection ``qkv`` [N, >= (Hq M Dq + Hkv M Dk + Hkv Dv)], whose query and key heads consist of
    ``maps`` units each: per unit the projection's ``bias`` (float32, over the q, k and v columns) is added, the unit
    RMS-normalised with the weight of its kind ([Dq] / [Dk], shared by all units), and its first ``rotary_dim`` elements
    rotated (element i with i + rotary_dim / 2, angle position * inv_freq[i]).  Query units are written back in place,
    or packed into ``q_out`` [N, Hq M Dq]; key units go to the K pages [page, Hkv, slot, M Dk], value heads (bias added)
    to the V pages [page, Hkv, slot, Dv].  ``value_dim`` 0: there are no values.  Everything in 32-bit, one rounding.

    ``k_norm_dim`` > 0: only a key unit's first ``k_norm_dim`` elements are normalised (``k_weight`` [k_norm_dim]), the
    rest stays as projected.  ``q_rot_start`` / ``k_rot_start``: the element of a query / key unit from which the
    ``rotary_dim`` rotating elements lie (negative: units of that kind do not rotate); ``interleaved``: element 2i pairs
    with 2i + 1.  ``q_temp`` = (coef, every): query units are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) at
    position p."""
    check(qkv, "qkv")
    tokens, row_width = qkv.shape
    weight_dtype = qkv.dtype
    for name, tensor, size in (("q norm weight", q_weight, q_dim), ("k norm weight", k_weight, k_norm_dim or k_dim)):
        if tensor is not None:
            check(tensor, name, last_dim=size)
            weight_dtype = tensor.dtype
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    temp_coef, temp_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if q_temp and temp_every <= 0:
        raise KernelError(f"the query temperature's period must be positive, got {temp_every}")
    used = (n_q_heads * q_dim + n_kv_heads * k_dim) * maps + n_kv_heads * value_dim
    if bias is not None:
        check(bias, "projection bias", torch.float32)
        if bias.numel() < used:
            raise KernelError(f"the bias holds {bias.numel()} numbers; the q, k and v columns are {used}")
    if inv_freq is not None:
        check(inv_freq, "inv_freq", torch.float32, rotary_dim // 2)
    check(positions, "positions", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(block_tables, "block_tables", torch.int32)
    check(k_pages, "k pages", qkv.dtype, maps * k_dim)
    if value_dim:
        check(v_pages, "v pages", qkv.dtype, value_dim)
        if k_pages.shape[:-1] != v_pages.shape[:-1]:
            raise KernelError(f"k pages {tuple(k_pages.shape)} and v pages {tuple(v_pages.shape)} differ in more than the last dimension")
    if k_pages.dim() != 4 or k_pages.shape[1] != n_kv_heads:
        raise KernelError(f"pages must be [pages, {n_kv_heads}, page_size, ...], got {tuple(k_pages.shape)}")
    if q_out is not None:
        check(q_out, "packed queries", qkv.dtype, n_q_heads * maps * q_dim)
    if positions.numel() != tokens or seq_of_token.numel() != tokens:
        raise KernelError("positions and seq_of_token need one entry per token")
    check(error_flag, "error flag", torch.int32)
    call("llm_norm_rope_units", qkv.data_ptr(), row_width, pointer(bias), pointer(q_weight), pointer(k_weight), float(eps),
         pointer(inv_freq), positions.data_ptr(), seq_of_token.data_ptr(), block_tables.data_ptr(), block_tables.shape[-1],
         pointer(q_out), k_pages.data_ptr(), pointer(v_pages) if value_dim else 0, tokens, n_q_heads, n_kv_heads, int(maps),
         int(q_dim), int(k_dim), int(value_dim), k_pages.shape[2], k_pages.shape[0], int(write_cache), error_flag.data_ptr(),
         int(rotary_dim) if inv_freq is not None else 0, dtype_code(qkv.dtype), dtype_code(weight_dtype), int(k_norm_dim),
         int(q_rot_start), int(k_rot_start), int(bool(interleaved)), temp_coef, temp_every, stream_handle())


def rotate_units(q: torch.Tensor, positions: torch.Tensor, n_heads: int, dim: int, inv_freq: torch.Tensor, rotary_dim: int,
                 rot_start: int = 0, interleaved: bool = False) -> None:
    """In place on ``q`` [N, >= n_heads * dim]: ``rotary_dim`` elements of every head, from element ``rot_start`` on, are
    rotated by the angles position * inv_freq[i] (``norm_rope_units`` for queries alone: nothing is normalised or cached)."""
    check(q, "q")
    check(positions, "positions", torch.int32)
    check(inv_freq, "inv_freq", torch.float32, rotary_dim // 2)
    tokens, row_width = q.shape
    if positions.numel() != tokens:
        raise KernelError("positions need one entry per token")
    call("llm_norm_rope_units", q.data_ptr(), row_width, 0, 0, 0, 0.0, inv_freq.data_ptr(), positions.data_ptr(), positions.data_ptr(),
         positions.data_ptr(), 1, 0, 0, 0, tokens, int(n_heads), 0, 1, int(dim), 1, 0, 1, 1, 0, wait_error_flag(q.device).data_ptr(),
         int(rotary_dim), dtype_code(q.dtype), dtype_code(q.dtype), 0, int(rot_start), -1, int(bool(interleaved)), 0.0, 0,
         stream_handle())


def attention_diff(qkv: torch.Tensor, gate_column: Optional[int], batch, block_tables: torch.Tensor, k_pages: torch.Tensor,
                   v_pages: torch.Tensor, n_q_heads: int, n_kv_heads: int, dim: int, value_dim: int, scale: float, cap: float,
                   window: int, lam: float, eps: float, out_scale: float) -> torch.Tensor:
    """Differential attention of a step's tokens over the paged cache.  ``qkv`` [N, row] holds each token's query heads
    first, a head as [map 1 | map 2] of ``dim`` elements each, already normalised and rotated; K pages hold key heads
    in the same form, V pages value heads of ``value_dim``.  Per head: a_m = softmax(cap(q_m . k_m * scale)) V over keys
    p - window + 1 .. p (window 0: all), o = a_1 - lam * a_2, out = o / sqrt(mean(o^2) + eps) * out_scale, times
    sigmoid(qkv[n, gate_column + head]) when ``gate_column`` is given.  Returns [N, Hq * value_dim]."""
    check(qkv, "qkv")
    tokens, row_width = qkv.shape
    check(k_pages, "k pages", qkv.dtype, 2 * dim)
    check(v_pages, "v pages", qkv.dtype, value_dim)
    if k_pages.shape[:-1] != v_pages.shape[:-1] or k_pages.shape[1] != n_kv_heads:
        raise KernelError(f"k pages {tuple(k_pages.shape)} and v pages {tuple(v_pages.shape)} do not fit {n_kv_heads} kv heads")
    check(block_tables, "block_tables", torch.int32)
    out = torch.empty((tokens, n_q_heads * value_dim), dtype=qkv.dtype, device=qkv.device)
    if qkv.dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.try_attention_diff(qkv, gate_column, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, dim,
                                             value_dim, scale, cap, window, lam, eps, out_scale, out):
            return out
    gate = 0 if gate_column is None else qkv.data_ptr() + gate_column * qkv.element_size()
    call("llm_attention_diff", qkv.data_ptr(), row_width, gate, row_width, k_pages.data_ptr(), v_pages.data_ptr(),
         block_tables.data_ptr(), block_tables.shape[-1], batch.seq_of_token.data_ptr(), batch.positions.data_ptr(),
         out.data_ptr(), tokens, n_q_heads, n_kv_heads, int(dim), int(value_dim), k_pages.shape[2], k_pages.shape[0],
         float(scale), float(cap or 0.0), int(window or 0), float(lam), float(eps), float(out_scale),
         wait_error_flag(qkv.device).data_ptr(), dtype_code(qkv.dtype), stream_handle())
    return out


def gla_supported(dim: int, value_dim: int) -> bool:
    return bool(library().llm_gla_supports(int(dim), int(value_dim)))


def gla_recurrent(proj: torch.Tensor, q_column: int, k_column: int, v_column: int, g_column: int, z: torch.Tensor,
                  z_bias: Optional[torch.Tensor], weight: torch.Tensor, state: torch.Tensor, batch, heads: int, dim: int,
                  value_dim: int, tau: float, q_scale: float, eps: float, segment: Optional[int] = None) -> torch.Tensor:
    """The gated-linear-attention recurrence over a step's tokens, sequence by sequence, from and into each sequence's
    slot of ``state`` (float32 [slots, heads, dim, value_dim]):

        alpha = sigmoid(z + z_bias) ^ (1 / tau);  S <- diag(alpha) S + k v^T;  o = S^T (q * q_scale)
        out   = o / sqrt(mean(o^2) + eps) * weight * silu(g)          per head, over value_dim

    q, k (heads * dim columns each), v and g (heads * value_dim) start at the given columns of ``proj``; ``z`` is
    float32 [N, heads * dim] in either path.  Returns [N, heads * value_dim] in the activation type; the recurrence itself is 32-bit.

    ``segment``: tokens per segment of the form that walks a long portion's segments in parallel (two passes and a scan
    between them; results equal to rounding).  None: chosen here, for bfloat16 steps whose longest portion spans several
    segments; 0: always the one-pass form, which is also what the 32-bit path runs."""
    check(proj, "packed projection")
    tokens, row_width = proj.shape
    check(z, "decay projection", torch.float32, heads * dim)
    if z_bias is not None:
        check(z_bias, "decay bias", torch.float32, heads * dim)
    check(weight, "norm weight", last_dim=value_dim)
    check(state, "recurrent state", torch.float32, value_dim)
    if state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, value_dim):
        raise KernelError(f"the state must be [slots, {heads}, {dim}, {value_dim}], got {tuple(state.shape)}")
    for column, size in ((q_column, heads * dim), (k_column, heads * dim), (v_column, heads * value_dim), (g_column, heads * value_dim)):
        if column < 0 or column + size > row_width:
            raise KernelError(f"columns {column}..{column + size} lie outside a row of {row_width}")
    out = torch.empty((tokens, heads * value_dim), dtype=proj.dtype, device=proj.device)
    longest = int(batch.max_q_len)
    if segment is None:
        # at most GLA_MAX_SEGMENTS segments per sequence, none shorter than GLA_SEGMENT tokens
        segment = 0 if proj.dtype != torch.bfloat16 or longest < 2 * GLA_SEGMENT else max(GLA_SEGMENT, -(-longest // GLA_MAX_SEGMENTS))
    segments, segment_state, segment_decay = 0, None, None
    if segment:
        segments = -(-longest // segment)
        key = ("gla_segments", batch.n_seqs, segments, heads, dim, value_dim)
        scratch = batch.scratch.get(key)
        if scratch is None:
            scratch = (torch.empty((batch.n_seqs, segments, heads, dim, value_dim), dtype=torch.float32, device=proj.device),
                       torch.empty((batch.n_seqs, segments, heads, dim), dtype=torch.float32, device=proj.device))
            batch.scratch[key] = scratch
        segment_state, segment_decay = scratch
    call("llm_gla_recurrent", proj.data_ptr(), row_width, int(q_column), int(k_column), int(v_column), int(g_column),
         z.data_ptr(), pointer(z_bias), weight.data_ptr(), state.data_ptr(), batch.state_slots.data_ptr(), batch.q_start.data_ptr(),
         out.data_ptr(), batch.n_seqs, int(heads), int(dim), int(value_dim), 1.0 / float(tau), float(q_scale), float(eps),
         dtype_code(proj.dtype), dtype_code(weight.dtype), int(segment), int(segments), pointer(segment_state), pointer(segment_decay),
         stream_handle())
    return out


GLA_SEGMENT = 64          # fewest tokens per segment of the segmented recurrence
GLA_MAX_SEGMENTS = 128    # most segments per sequence (the scratch holds a state per segment)


def _pointwise(kind: int, x: torch.Tensor, y: Optional[torch.Tensor], out: torch.Tensor, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
    check(x, "x")
    check(out, "output")
    if y is not None:
        check(y, "y", x.dtype)
        if y.shape != x.shape:
            raise KernelError(f"y {tuple(y.shape)} does not match x {tuple(x.shape)}")
    if out.shape != x.shape:
        raise KernelError(f"the output {tuple(out.shape)} does not match x {tuple(x.shape)}")
    call("llm_pointwise", int(kind), x.data_ptr(), pointer(y), out.data_ptr(), x.numel(), float(a), float(b), dtype_code(x.dtype),
         dtype_code(out.dtype), stream_handle())
    return out


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, formed in 32-bit and rounded once."""
    return _pointwise(0, x, None, torch.empty_like(x))


def tanh_narrow(x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """tanh of 32-bit values, stored in the activation type."""
    check(x, "x", torch.float32)
    return _pointwise(1, x, None, torch.empty(x.shape, dtype=act_dtype, device=x.device))


def softcap_(logits: torch.Tensor, cap: float, scale: float = 1.0) -> torch.Tensor:
    """logits <- cap * tanh(scale * logits / cap), in place on 32-bit values; without a cap (0), logits <- scale * logits."""
    check(logits, "logits", torch.float32)
    if not cap:
        return _pointwise(3, logits, logits, logits, a=scale, b=0.0)
    return _pointwise(2, logits, None, logits, a=cap, b=scale)


def scaled_sum(x: torch.Tensor, a: float, y: torch.Tensor, b: float) -> torch.Tensor:
    """a * x + b * y in 32-bit, rounded once."""
    return _pointwise(3, x, y, torch.empty_like(x), a=a, b=b)


def token_shift_mix(h: torch.Tensor, shift_state: torch.Tensor, batch, mu: torch.Tensor) -> torch.Tensor:
    """out[s, n] = h[n] + (h'[n] - h[n]) * mu[s] for the M mixing vectors ``mu`` (float32 [M, width]); h'[n] is the row
    of the token before in the same sequence, for a sequence's first token of this step the row kept in its slot of
    ``shift_state`` (float32 [slots, width]; zeros for a new request).  The slot is brought up to date by
    ``wkv_recurrent``.  Returns [M, N, width] in h's type."""
    check(h, "h")
    tokens, width = h.shape
    check(mu, "mixing vectors", torch.float32, width)
    check(shift_state, "shift state", torch.float32, width)
    mixes = mu.shape[0]
    out = torch.empty((mixes, tokens, width), dtype=h.dtype, device=h.device)
    call("llm_token_shift_mix", h.data_ptr(), shift_state.data_ptr(), batch.state_slots.data_ptr(), batch.q_start.data_ptr(),
         batch.seq_of_token.data_ptr(), mu.data_ptr(), out.data_ptr(), tokens, width, mixes, dtype_code(h.dtype), stream_handle())
    return out


def short_conv_units(x: torch.Tensor, column: int, taps_w: torch.Tensor, state: torch.Tensor, batch, n_unit_norm: int,
                     unit_dim: int, n_scaled: int, n_plain: int, plain_dim: int, norm_eps: float, scale: float) -> torch.Tensor:
    """A short causal convolution over time, channel by channel, then SiLU:

        y_t[c] = silu(sum_j taps_w[c, j] * x_(t - taps + 1 + j)[c])        zeros before a sequence's start

    over the channels that start at ``column`` of ``x`` [N, row]; ``taps_w`` is float32 [channels, taps], the last column
    the current token's.  Channels come in units: first ``n_unit_norm`` units of ``unit_dim`` channels, each made a unit
    vector y / sqrt(sum(y^2) + norm_eps), the first ``n_scaled`` of them multiplied by ``scale``; then ``n_plain`` units of
    ``plain_dim`` channels that stay as they are.  A sequence's last taps - 1 inputs live in its slot of ``state``
    (float32 [slots, max(taps - 1, 1), channels]) and are brought up to date.  Returns float32 [N, channels]."""
    check(x, "x")
    tokens, row_width = x.shape
    channels = n_unit_norm * unit_dim + n_plain * plain_dim
    taps = taps_w.shape[1]
    check(taps_w, "convolution weights", torch.float32)
    if taps_w.shape[0] != channels or column < 0 or column + channels > row_width:
        raise KernelError(f"{channels} channels from column {column} do not fit rows of {row_width} or weights {tuple(taps_w.shape)}")
    check(state, "convolution state", torch.float32, channels)
    if state.dim() != 3 or state.shape[1] != max(taps - 1, 1):
        raise KernelError(f"the convolution state must be [slots, {max(taps - 1, 1)}, {channels}], got {tuple(state.shape)}")
    out = torch.empty((tokens, channels), dtype=torch.float32, device=x.device)
    call("llm_short_conv_units", x.data_ptr(), row_width, int(column), taps_w.data_ptr(), int(taps), state.data_ptr(),
         batch.state_slots.data_ptr(), batch.q_start.data_ptr(), out.data_ptr(), batch.n_seqs, int(batch.max_q_len), int(n_unit_norm),
         int(unit_dim), int(n_scaled), int(n_plain), int(plain_dim), float(norm_eps), float(scale), dtype_code(x.dtype), stream_handle())
    return out


def matrix_recurrence_supported(dim: int, value_dim: int) -> bool:
    return bool(library().llm_matrix_recurrence_supports(int(dim), int(value_dim)))


def wkv_recurrent(rkvg: torch.Tensor, z: torch.Tensor, w0: torch.Tensor, bonus: torch.Tensor, weight: torch.Tensor,
                  state: torch.Tensor, batch, heads: int, dim: int, eps: float, h: Optional[torch.Tensor] = None,
                  shift_state: Optional[torch.Tensor] = None, segment: Optional[int] = None) -> torch.Tensor:
    """The recurrence with a per-channel decay and a bonus for the current token, sequence by sequence, from and into each
    sequence's slot of ``state`` (float32 [slots, heads, dim, dim]):

        w = exp(-exp(z + w0));  o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T
        out = o / sqrt(mean(o^2) + eps) * weight * silu(g)           per head, over its dim value channels

    ``rkvg`` is [4, N, heads * dim] (r, k, v and the gate's pre-activation) in the activation type, ``z`` float32
    [N, heads * dim], ``w0`` float32 [heads * dim], ``bonus`` (u) float32 [heads, dim], ``weight`` [heads * dim].  With
    ``h`` and ``shift_state`` the sequence's last row of ``h`` is left in its slot of ``shift_state`` for the next step's
    ``token_shift_mix``.  Returns [N, heads * dim] in the activation type; the recurrence itself is 32-bit.  ``segment`` as
    for ``delta_rule_recurrent``."""
    check(rkvg, "r, k, v and gate", last_dim=heads * dim)
    if rkvg.dim() != 3 or rkvg.shape[0] != 4:
        raise KernelError(f"r, k, v and the gate come as [4, N, {heads * dim}], got {tuple(rkvg.shape)}")
    tokens = rkvg.shape[1]
    plane = tokens * heads * dim
    if 3 * plane >= 2 ** 31:
        raise KernelError(f"{tokens} tokens of {heads * dim} channels are more than one launch of wkv_recurrent takes")
    check(z, "decay projection", torch.float32, heads * dim)
    check(w0, "decay offset", torch.float32)
    check(bonus, "bonus", torch.float32, dim)
    check(weight, "norm weight", last_dim=heads * dim)
    check(state, "recurrent state", torch.float32, dim)
    if state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, dim):
        raise KernelError(f"the state must be [slots, {heads}, {dim}, {dim}], got {tuple(state.shape)}")
    width = 0
    if h is not None:
        check(h, "h", rkvg.dtype)
        width = h.shape[1]
        check(shift_state, "shift state", torch.float32, width)
    out = torch.empty((tokens, heads * dim), dtype=rkvg.dtype, device=rkvg.device)
    segment, segments, segment_state, segment_move = _recurrence_segments(batch, rkvg, segment, heads, dim, dim, dim)
    call("llm_wkv_recurrent", rkvg.data_ptr(), heads * dim, 0, plane, 2 * plane, 3 * plane, z.data_ptr(), w0.data_ptr(),
         bonus.data_ptr(), weight.data_ptr(), state.data_ptr(), batch.state_slots.data_ptr(), batch.q_start.data_ptr(),
         out.data_ptr(), batch.n_seqs, int(heads), int(dim), float(eps), pointer(h), pointer(shift_state) if h is not None else 0,
         int(width), dtype_code(rkvg.dtype), dtype_code(weight.dtype), segment, segments, pointer(segment_state),
         pointer(segment_move), stream_handle())
    return out


REC_SEGMENT = 64                   # fewest tokens per segment of the segmented matrix recurrences
REC_MAX_SEGMENTS = 64              # most segments per sequence
REC_SCRATCH_BYTES = 1 << 30        # most scratch that the segments' states and transitions may take


def _recurrence_segments(batch, activations: torch.Tensor, segment: Optional[int], heads: int, dim: int, value_dim: int,
                         move_columns: int):
    """Segment length, segments per sequence and the scratch of the segmented form of ``wkv_recurrent`` and
    ``delta_rule_recurrent``: a state [dim, value_dim] and a transition (``move_columns`` values per key channel: 1 for a
    diagonal one, dim for a full one) per (sequence, segment, head).  ``segment`` None: chosen here, for bfloat16 steps
    whose longest portion spans several segments and whose scratch stays within REC_SCRATCH_BYTES; 0: the one-pass form."""
    longest = int(batch.max_q_len)
    per_segment = batch.n_seqs * heads * dim * (value_dim + move_columns) * 4
    if segment is None:
        most = min(REC_MAX_SEGMENTS, REC_SCRATCH_BYTES // max(per_segment, 1))
        segment = 0 if activations.dtype != torch.bfloat16 or longest < 2 * REC_SEGMENT or most < 2 else max(REC_SEGMENT, -(-longest // most))
    if not segment:
        return 0, 0, None, None
    segments = -(-longest // int(segment))
    key = ("matrix_recurrence_segments", batch.n_seqs, segments, heads, dim, value_dim, move_columns)
    scratch = batch.scratch.get(key)
    if scratch is None:
        scratch = (torch.empty((batch.n_seqs, segments, heads, dim, value_dim), dtype=torch.float32, device=activations.device),
                   torch.empty((batch.n_seqs, segments, heads, dim, move_columns), dtype=torch.float32, device=activations.device))
        batch.scratch[key] = scratch
    return int(segment), segments, scratch[0], scratch[1]


def delta_rule_recurrent(proj: torch.Tensor, g_column: int, pre: torch.Tensor, wide: torch.Tensor, a_log: torch.Tensor,
                         dt_bias: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, batch, heads: int, qk_heads: int,
                         dim: int, value_dim: int, eps: float, segment: Optional[int] = None) -> torch.Tensor:
    """The gated delta rule, sequence by sequence, from and into each sequence's slot of ``state`` (float32
    [slots, heads, dim, value_dim]):

        g = exp(-exp(A) * softplus(a + dt));  beta = sigmoid(b)
        S <- g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q
        out = o / sqrt(mean(o^2) + eps) * weight * silu(gate)         per head, over value_dim; weight [value_dim]

    ``pre`` is float32 [N, 2 * qk_heads * dim + heads * value_dim] = q | k | v as ``short_conv_units`` leaves them (head h
    reads q/k head h // (heads / qk_heads)); ``wide`` float32 [N, 2 heads] = b | a; ``a_log`` (A) and ``dt_bias`` float32
    [heads]; the gate's pre-activation is heads * value_dim columns of ``proj`` from ``g_column``.  Returns
    [N, heads * value_dim] in the activation type; the recurrence itself is 32-bit.

    ``segment``: tokens per segment of the form that walks a long portion's segments in parallel: every segment from a
    zero state, which also yields its transition; a scan that gives each segment the state it starts from; every segment
    again for the outputs (results equal to rounding).  None: chosen for bfloat16 steps whose longest portion spans several
    segments; 0: always the one-pass form, which is also what the 32-bit path runs."""
    check(proj, "packed projection")
    tokens, row_width = proj.shape
    if g_column < 0 or g_column + heads * value_dim > row_width:
        raise KernelError(f"the gate's columns {g_column}..{g_column + heads * value_dim} lie outside a row of {row_width}")
    check(pre, "convolved q, k, v", torch.float32, 2 * qk_heads * dim + heads * value_dim)
    check(wide, "b and a", torch.float32, 2 * heads)
    check(a_log, "A", torch.float32)
    check(dt_bias, "dt bias", torch.float32)
    check(weight, "norm weight", last_dim=value_dim)
    check(state, "recurrent state", torch.float32, value_dim)
    if state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, value_dim):
        raise KernelError(f"the state must be [slots, {heads}, {dim}, {value_dim}], got {tuple(state.shape)}")
    if pre.shape[0] != tokens or wide.shape[0] != tokens:
        raise KernelError("every input needs one row per token")
    out = torch.empty((tokens, heads * value_dim), dtype=proj.dtype, device=proj.device)
    segment, segments, segment_state, segment_move = _recurrence_segments(batch, proj, segment, heads, dim, value_dim, dim)
    call("llm_delta_rule_recurrent", proj.data_ptr(), row_width, int(g_column), pre.data_ptr(), pre.shape[1], 0, qk_heads * dim,
         2 * qk_heads * dim, wide.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), weight.data_ptr(), state.data_ptr(),
         batch.state_slots.data_ptr(), batch.q_start.data_ptr(), out.data_ptr(), batch.n_seqs, int(heads), int(qk_heads), int(dim),
         int(value_dim), float(eps), dtype_code(proj.dtype), dtype_code(weight.dtype), segment, segments, pointer(segment_state),
         pointer(segment_move), stream_handle())
    return out


def head_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[n, h, :] = weight[h] x[n, h, :] for ``x`` [N, H * K] and ``weight`` [H, R, K]: every head has a matrix of its
    own.  Returns [N, H * R] in the activation type.  Steps of many rows in bfloat16 go to the library's batched product;
    the others, and the 32-bit path, multiply row by row with sums whose order depends on K alone."""
    check(x, "x")
    heads, rows, inner = weight.shape
    check(weight, "per-head matrices", x.dtype, inner)
    tokens = x.shape[0]
    if x.shape[1] != heads * inner:
        raise KernelError(f"x has {x.shape[1]} columns; {heads} heads of {inner} are {heads * inner}")
    if x.dtype == torch.bfloat16 and tokens > HEAD_LINEAR_ROWS:
        out = torch.empty((tokens, heads, rows), dtype=x.dtype, device=x.device)
        torch.bmm(x.view(tokens, heads, inner).transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
        return out.view(tokens, heads * rows)
    return indexed_linear(x.view(tokens * heads, inner), weight, None, tokens * heads, cyclic=True).view(tokens, heads * rows)


HEAD_LINEAR_ROWS = 32     # up to this many tokens a bfloat16 step multiplies row by row


def moe_route(x: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, scale: float,
              counts: Optional[torch.Tensor] = None):
    """Per token the ``top`` experts with the largest sigmoid(router x) + correction (ties: the lower index) and their
    weights sigmoid(router x) * scale: (chosen int32 [N, top], weights float32 [N, top]).  ``router`` [E, H] and
    ``correction`` [E] are float32; with ``counts`` (int32 [E]) each choice also adds one to its expert's count."""
    check(x, "x")
    tokens, width = x.shape
    check(router, "router weight", torch.float32, width)
    experts = router.shape[0]
    if correction is not None:
        check(correction, "router correction", torch.float32, experts)
    if counts is not None:
        check(counts, "expert counts", torch.int32, experts)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    call("llm_moe_route", x.data_ptr(), router.data_ptr(), pointer(correction), chosen.data_ptr(), weights.data_ptr(),
         pointer(counts), tokens, width, experts, int(top), float(scale), dtype_code(x.dtype), stream_handle())
    return chosen, weights


def moe_select(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, scale: float):
    """``moe_route``'s choice from router logits that a product has already made: logits float32 [N, E]."""
    check(logits, "router logits", torch.float32)
    tokens, experts = logits.shape
    if correction is not None:
        check(correction, "router correction", torch.float32, experts)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    call("llm_moe_select", logits.data_ptr(), pointer(correction), chosen.data_ptr(), weights.data_ptr(), tokens, experts,
         int(top), float(scale), stream_handle())
    return chosen, weights


def indexed_linear(x: torch.Tensor, weight: torch.Tensor, index: Optional[torch.Tensor], pairs: int, in_div: int = 1,
                   gated: Optional[tuple] = None, out_dtype: Optional[torch.dtype] = None, cyclic: bool = False,
                   in_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[p] = weight[index[p]] x[p // in_div] for p < ``pairs``; ``weight`` is [E, R, K] (``index`` None: E = 1, or,
    ``cyclic``, pair p uses matrix p mod E).
    ``gated`` = (limit, alpha): the matrices hold R gate rows and then R up rows, [E, 2 R, K], and the result is
    min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + up_shift); ``gated`` may carry
    up_shift as a third number (default 1; (inf, 1, 0) is silu(g) * u).  ``in_scale`` (float32 [pairs]): pair p's input
    row is multiplied by in_scale[p] as it is read."""
    check(x, "x")
    check(weight, "expert weights", x.dtype, x.shape[-1])
    if in_scale is not None:
        check(in_scale, "input scales", torch.float32)
        if in_scale.numel() < pairs:
            raise KernelError(f"{in_scale.numel()} input scales for {pairs} pairs")
    if weight.dim() != 3:
        raise KernelError(f"expert weights must be [experts, rows, inner], got {tuple(weight.shape)}")
    rows = weight.shape[1] // 2 if gated else weight.shape[1]
    if index is not None:
        check(index, "expert index", torch.int32)
        if index.numel() < pairs:
            raise KernelError(f"{index.numel()} expert indices for {pairs} pairs")
    elif weight.shape[0] != 1 and not cyclic:
        raise KernelError("without an index the weights hold one matrix")
    if x.shape[0] * in_div < pairs:
        raise KernelError(f"{x.shape[0]} input rows cannot serve {pairs} pairs, {in_div} per row")
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise KernelError(f"indexed_linear writes the input's type or float32, not {out_dtype}")
    out = torch.empty((pairs, rows), dtype=out_dtype, device=x.device)
    limit, alpha, up_shift = _gate_constants(gated)
    call("llm_indexed_linear", x.data_ptr(), weight.data_ptr(), pointer(index), out.data_ptr(), pairs, rows, x.shape[-1],
         int(in_div), int(bool(gated)), limit, alpha, dtype_code(x.dtype),
         int(out_dtype == torch.float32 and x.dtype != torch.float32), weight.shape[0] if cyclic and index is None else 0,
         pointer(in_scale), up_shift, stream_handle())
    return out


def _gate_constants(gated: Optional[tuple]):
    """(limit, alpha, up_shift) of a gated product's activation; up_shift is 1 unless a third number says otherwise."""
    if not gated:
        return 0.0, 0.0, 1.0
    return float(gated[0]), float(gated[1]), float(gated[2]) if len(gated) > 2 else 1.0


def moe_combine(down: torch.Tensor, weights: torch.Tensor, shared_out: Optional[torch.Tensor], act_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * down[t * top + j] (+ shared_out[t]); ``down`` float32 [N * top, H]."""
    check(down, "expert outputs", torch.float32)
    check(weights, "routing weights", torch.float32)
    tokens, top = weights.shape
    width = down.shape[-1]
    if down.shape[0] != tokens * top:
        raise KernelError(f"{down.shape[0]} expert outputs for {tokens} tokens with {top} experts each")
    if shared_out is not None:
        check(shared_out, "shared expert output", act_dtype, width)
    out = torch.empty((tokens, width), dtype=act_dtype, device=down.device)
    call("llm_moe_combine", down.data_ptr(), weights.data_ptr(), pointer(shared_out), out.data_ptr(), tokens, width, top,
         dtype_code(act_dtype), stream_handle())
    return out


class ExpertPlan:
    """The (token, expert) pairs of a step sorted by expert: ``pair_of_row[r]`` is the pair that row r of the sorted
    order holds, ``row_of_pair`` the inverse, ``offsets[e]`` the first row of expert e, ``tiles`` the row tiles the
    grouped product walks (count first, then (expert, first row, rows) per tile)."""

    def __init__(self, pairs, offsets, pair_of_row, row_of_pair, tiles, max_tiles):
        self.pairs, self.offsets, self.pair_of_row, self.row_of_pair = pairs, offsets, pair_of_row, row_of_pair
        self.tiles, self.max_tiles = tiles, max_tiles


MOE_TILE_ROWS = 128


def moe_plan(chosen: torch.Tensor, experts: int) -> ExpertPlan:
    """Sorts the pairs of ``chosen`` (int32 [N, top]) by expert on the device; nothing comes back to the host."""
    check(chosen, "chosen experts", torch.int32)
    pairs = chosen.numel()
    max_tiles = -(-pairs // MOE_TILE_ROWS) + experts
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=chosen.device)
    pair_of_row = torch.empty((pairs,), dtype=torch.int32, device=chosen.device)
    row_of_pair = torch.empty((pairs,), dtype=torch.int32, device=chosen.device)
    tiles = torch.empty((1 + 3 * max_tiles,), dtype=torch.int32, device=chosen.device)
    call("llm_moe_plan", chosen.data_ptr(), pairs, experts, offsets.data_ptr(), pair_of_row.data_ptr(), row_of_pair.data_ptr(),
         tiles.data_ptr(), max_tiles, stream_handle())
    return ExpertPlan(pairs, offsets, pair_of_row, row_of_pair, tiles, max_tiles)


# "tcgen05" (default): the tiled product with its accumulator in tensor memory; "mma": the mma.sync kernel
MOE_GROUPED_KERNEL = os.environ.get("LLMSERVER_B200_MOE_GROUPED", "tcgen05")


def moe_grouped_supported(weight: torch.Tensor, gated: bool) -> bool:
    """Whether a tiled product over sorted pairs takes these expert matrices ([E, rows, inner], bfloat16)."""
    rows = weight.shape[1] // 2 if gated else weight.shape[1]
    if weight.dtype != torch.bfloat16:
        return False
    return bool(library().llm_moe_grouped_tc_supports(rows, weight.shape[2], int(gated))) or \
        bool(library().llm_moe_grouped_supports(rows, weight.shape[2], int(gated)))


def moe_grouped(x: torch.Tensor, weight: torch.Tensor, plan: ExpertPlan, gather_div: Optional[int] = None,
                gated: Optional[tuple] = None, pair_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One tiled product over all experts: row r of the plan's order gets weight[its expert] times its input row,
    which is x[pair_of_row[r] // gather_div] or, with ``gather_div`` None, x[r].  ``gated`` = (limit, alpha): the
    matrices are [E, 2 R, K], gate rows first, and the result is the experts' activation in bfloat16 [pairs, R];
    otherwise the 32-bit sums [pairs, R].  On tcgen05 where that kernel takes the sizes (it reads its rows by TMA, so
    rows that have to be gathered are copied into the plan's order first), else the mma.sync kernel.  ``pair_scale``
    (float32 [pairs], with ``gather_div``): the gathered row of pair p is multiplied by pair_scale[p] on the way.
    ``gated`` may carry the activation's up_shift as a third number (see ``indexed_linear``)."""
    check(x, "x", torch.bfloat16)
    if pair_scale is not None:
        check(pair_scale, "pair scales", torch.float32)
        if gather_div is None or pair_scale.numel() < plan.pairs:
            raise KernelError("pair scales go with gathered rows, one per pair")
    check(weight, "expert weights", torch.bfloat16, x.shape[-1])
    rows = weight.shape[1] // 2 if gated else weight.shape[1]
    inner = x.shape[-1]
    out = torch.empty((plan.pairs, rows), dtype=torch.bfloat16 if gated else torch.float32, device=x.device)
    limit, alpha, up_shift = _gate_constants(gated)
    tensor_memory = MOE_GROUPED_KERNEL != "mma" and library().llm_moe_grouped_tc_supports(rows, inner, int(bool(gated))) and (gated or rows % 4 == 0)
    if gather_div is not None and (tensor_memory or pair_scale is not None):
        ordered = torch.empty((plan.pairs, inner), dtype=torch.bfloat16, device=x.device)
        call("llm_moe_gather_rows", x.data_ptr(), plan.pair_of_row.data_ptr(), int(gather_div), ordered.data_ptr(), plan.pairs,
             inner, pointer(pair_scale), stream_handle())
        x, gather_div = ordered, None
    if tensor_memory:
        call("llm_moe_grouped_tc", x.data_ptr(), plan.pairs, weight.data_ptr(), weight.shape[0], plan.tiles.data_ptr(), out.data_ptr(),
             rows, inner, plan.max_tiles, int(bool(gated)), limit, alpha, up_shift, wait_error_flag(x.device).data_ptr(),
             stream_handle())
        return out
    call("llm_moe_grouped", x.data_ptr(), weight.data_ptr(), plan.tiles.data_ptr(),
         plan.pair_of_row.data_ptr() if gather_div is not None else 0, int(gather_div or 1), out.data_ptr(), rows,
         inner, plan.max_tiles, int(bool(gated)), limit, alpha, up_shift, stream_handle())
    return out


def moe_combine_rows(down: torch.Tensor, plan: ExpertPlan, weights: torch.Tensor, shared_out: Optional[torch.Tensor],
                     act_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * down[row_of_pair[t * top + j]] (+ shared_out[t]); ``down`` float32 in the plan's order."""
    check(down, "expert outputs", torch.float32)
    check(weights, "routing weights", torch.float32)
    tokens, top = weights.shape
    width = down.shape[-1]
    if shared_out is not None:
        check(shared_out, "shared expert output", act_dtype, width)
    out = torch.empty((tokens, width), dtype=act_dtype, device=down.device)
    call("llm_moe_combine_rows", down.data_ptr(), plan.row_of_pair.data_ptr(), weights.data_ptr(), pointer(shared_out),
         out.data_ptr(), tokens, width, top, dtype_code(act_dtype), stream_handle())
    return out


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out[n, i] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate_up[n, i], limit) and u = gate_up[n, I + i] clamped
    to [-limit, limit]; gate columns first."""
    check(gate_up, "gate_up")
    rows, doubled = gate_up.shape
    if doubled % 2:
        raise KernelError(f"gate_up's last dimension must be even, got {doubled}")
    out = torch.empty((rows, doubled // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("llm_clamped_glu", gate_up.data_ptr(), out.data_ptr(), rows, doubled // 2, float(limit), float(alpha),
         dtype_code(gate_up.dtype), stream_handle())
    return out


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, all float32, FMA only (no tensor cores, no TF32)."""
    check(x, "x", torch.float32)
    check(weight, "weight", torch.float32, x.shape[-1])
    rows, inner = x.shape
    cols = weight.shape[0]
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float32, device=x.device)
    check(out, "gemm output", torch.float32, cols)
    call("llm_gemm_f32", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, inner, inner, inner, cols,
         stream_handle())
    return out


def linear(x, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, sink: Optional[StreamSink] = None) -> Optional[torch.Tensor]:
    """y = x W^T for W stored [out, in] (utils/attention.py:119-124 uses nn.Linear for the same).

    float32: this package's FMA kernel.  bfloat16: the library matrix product (cuBLAS through
    PyTorch) where the reference's engine uses a library too, or this package's own kernels where
    they apply (see ``gemm_bf16``).  ``x`` may be a ``RowScaled``.  With a ``sink`` the product is added to the sink's
    residual stream by the product kernel itself where that kernel takes the case (``sink.added`` then says so and
    nothing is returned); otherwise the sink is left alone and the product is returned as usual."""
    if x.device.type != "cuda":
        raise KernelError("linear: there is no CPU path")
    if x.dtype == torch.float32:
        result = gemm_f32(x, weight, out)
        return result
    from . import gemm_bf16
    if sink is not None and out is None and not isinstance(x, RowScaled) and gemm_bf16.linear_into_stream(x, weight, sink):
        return None
    return gemm_bf16.linear_bf16(x, weight, out=out, out_dtype=out_dtype)


def linear_wide(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x W^T with bfloat16 operands and a float32 result taken straight from the 32-bit sums (never a rounded result
    widened): a product with few output columns whose values decide something, a router's logits for instance.  Up
    to 64 rows: this package's kernel; more: the library's product with a 32-bit result in one launch."""
    if x.dtype == torch.float32:
        return gemm_f32(x, weight)
    from . import gemm_bf16
    if x.shape[0] <= gemm_bf16.SMALL_M:
        return gemm_bf16.linear_bf16(x, weight, out_dtype=torch.float32)
    return gemm_bf16._float32_by_library(x, weight, None)


def unscaled_rows_supported(weight: torch.Tensor) -> bool:
    """Whether products with ``weight`` take ``RowScaled`` rows."""
    from . import gemm_bf16
    return gemm_bf16.unscaled_rows_supported(weight)


def qkv_projection(x, weight: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                   inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                   block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, n_q_heads: int, n_kv_heads: int,
                   head_dim: int, eps: float, write_cache: bool, error_flag: torch.Tensor, rotary_dim: Optional[int] = None,
                   interleaved: bool = False) -> torch.Tensor:
    """qkv = x W^T followed by ``qk_norm_rope_kv_write``: as one kernel where the product kernel can finish heads in its
    epilogue (bfloat16, heads of 128, up to 64 tokens, the whole head rotating in halves; from 17 tokens on only where
    that is measured to be faster), else as two.  ``x`` may be a ``RowScaled``."""
    whole_head = rotary_dim is None or rotary_dim == head_dim
    if x.dtype == torch.bfloat16 and whole_head and not interleaved and x.shape[0] <= 64:
        from . import gemm_bf16
        fused = gemm_bf16.qkv_rope_fused(x, weight, q_weight, k_weight, inv_freq, positions, seq_of_token, block_tables,
                                         k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, eps, write_cache, error_flag)
        if fused is not None:
            return fused
    qkv = linear(x, weight)
    qk_norm_rope_kv_write(qkv, q_weight, k_weight, inv_freq, positions, seq_of_token, block_tables, k_pages, v_pages,
                          n_q_heads, n_kv_heads, head_dim, eps, write_cache, error_flag, rotary_dim, interleaved)
    return qkv


def attention(qkv: torch.Tensor, batch, block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
              value_dim: Optional[int] = None, sinks: Optional[torch.Tensor] = None, precise: bool = False,
              q_stride: Optional[int] = None) -> torch.Tensor:
    """Attention of a step's tokens over the paged cache; ``qkv`` is the packed projection whose Q
    heads have been normalised and rotated in place (``q_stride``: elements from one token's queries to the next's,
    where they are not such a packed row).  Chooses the kernel by dtype, head size and the
    shape of the batch; every choice computes the same function.  ``value_dim`` (default: head_dim) and ``sinks`` as
    in ``attention_generic``.  ``precise``: the attention weights may not be rounded to bfloat16 on their way into the
    P V product (the tensor-core kernels then carry each as two bfloat16 numbers)."""
    value_dim = head_dim if value_dim is None else int(value_dim)
    if q_stride is None:
        q_stride = (n_q_heads + n_kv_heads) * head_dim + n_kv_heads * value_dim
    if qkv.dtype == torch.bfloat16:
        from . import attention_bf16
        if value_dim == head_dim and sinks is None and not precise:
            result = attention_bf16.try_attention(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads,
                                                  n_kv_heads, head_dim, scale, window)
        else:
            result = attention_bf16.try_attention_precise(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads,
                                                          n_kv_heads, head_dim, value_dim, scale, window, sinks)
        if result is not None:
            return result
    return attention_generic(qkv, q_stride, k_pages, v_pages, block_tables, batch.seq_of_token, batch.positions,
                             n_q_heads, n_kv_heads, head_dim, scale, window, value_dim=value_dim, sinks=sinks)
