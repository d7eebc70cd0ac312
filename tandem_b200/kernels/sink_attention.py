"""Entry points of ``csrc/sink_attention.cu``: windowed attention with kept first tokens, capped
scores, a bias by distance and a softmax sink, for keys and values of different sizes.

``prepare_rows`` is the step between projection and attention for mixers whose queries and keys are convolved, normed with a
weight and rotated (bias, causal convolution with per-request state, three norms, partial rotation, cache write; values of
their own or the keys as projected); every ``attend*`` takes an optional gate per (token, head).

``prepare`` + ``attend`` serve both storage types (the 32-bit path and bfloat16 caches) and any
step: a request's portion of a prompt and a single decoded token are rows of the same launch, one
warp per (token, head) on the CUDA cores.  In bfloat16, steps that bring prompt portions run
``attend_tiles`` instead (``csrc/sink_attention_tile.cu``, compiled per key and value size): query
tiles that the host cuts (``plan_tiles``), mma.sync tensor-core products, the same float32 score
arithmetic.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library


def _gate_stride(gate: Optional[torch.Tensor], tokens: int, num_heads: int) -> int:
    if gate is None:
        return 0
    ops._need(gate, "gate", torch.float32, contiguous=False)
    if tuple(gate.shape) != (tokens, num_heads) or gate.stride(1) != 1:
        raise ops.KernelError(f"the heads' gate has shape {tuple(gate.shape)}, expected {(tokens, num_heads)} with contiguous rows")
    return gate.stride(0)


QK_NORMS = {"none": 0, "unit": 1, "head": 2, "whole": 3}


def prepare_rows(proj: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, *,
                 bias: Optional[torch.Tensor] = None, taps: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None,
                 qk_norm: str = "none", q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                 eps: float = 1e-6, freq: Optional[torch.Tensor] = None, has_kv: bool = True,
                 values_from_keys: bool = False) -> torch.Tensor:
    """Queries float32 [T, nh dk] from the float32 projection ``proj`` (rows any stride apart, columns [q | k | v]; no k
    and v columns without ``has_kv``, no v columns with ``values_from_keys``), and the tokens' keys and values into
    their cache slots: bias [columns]; causal convolution over time with ``taps`` [K, columns] (tap j of every column side by
    side, the oldest input's first; the inputs in front of
    the step from ``state`` [slots, >= (K - 1) columns], a request's last K - 1 rows, oldest first); ``qk_norm`` of q and
    k ("unit", "head" with weights [dk], "whole" with weights [nh dk] and [nkv dk]); rotation of the first 2 len(freq)
    numbers of every head by position * freq.  The cached values are the v columns (or, with ``values_from_keys``, the k
    columns) after bias and convolution.  The caller moves the state on afterwards (``post_norm.short_conv_state``)."""
    ops._need(proj, "projection", torch.float32, contiguous=False)
    T = proj.shape[0]
    cols = num_heads * head_dim
    if has_kv:
        cols += num_kv_heads * head_dim + (0 if values_from_keys else num_kv_heads * value_dim)
    if proj.stride(1) != 1 or proj.shape[1] < cols:
        raise ops.KernelError(f"the projection has rows of {proj.shape[1]} numbers, {cols} are needed")
    if qk_norm not in QK_NORMS:
        raise ops.KernelError(f"no norm {qk_norm!r} of queries and keys (have {sorted(QK_NORMS)})")
    for t, name, n in ((bias, "bias", cols), (q_weight, "q norm weight", None), (k_weight, "k norm weight", None), (freq, "freq", None)):
        if t is not None:
            ops._need(t, name, torch.float32)
            if n is not None and t.numel() != n:
                raise ops.KernelError(f"{name} has {t.numel()} numbers, {n} are needed")
    if qk_norm in ("head", "whole"):
        want_q = head_dim if qk_norm == "head" else num_heads * head_dim
        want_k = head_dim if qk_norm == "head" else num_kv_heads * head_dim
        if q_weight is None or q_weight.numel() != want_q or (has_kv and (k_weight is None or k_weight.numel() != want_k)):
            raise ops.KernelError(f"the {qk_norm!r} norm needs weights of {want_q} and {want_k} numbers")
    K, state_stride = 0, 0
    if taps is not None:
        ops._need(taps, "taps", torch.float32)
        if taps.dim() != 2 or taps.shape[1] != cols:
            raise ops.KernelError(f"taps {tuple(taps.shape)} do not fit {cols} columns")
        K = taps.shape[0]
        if K > 1:
            ops._need(state, "state", torch.float32)
            state_stride = state[0].numel()
    rot = 0 if freq is None else 2 * freq.numel()
    if has_kv and kv.writable:
        ops._need(kv.slots, "slots", torch.int32)
        if tuple(kv.k.shape[1:]) != (num_kv_heads, kv.page_size, head_dim) or \
                tuple(kv.v.shape[1:]) != (num_kv_heads, kv.page_size, value_dim):
            raise ops.KernelError(f"caches {tuple(kv.k.shape)} / {tuple(kv.v.shape)} do not fit {num_kv_heads} kv heads of "
                                  f"{head_dim} / {value_dim}")
    q = torch.empty((T, num_heads * head_dim), dtype=torch.float32, device=proj.device)
    write = bool(has_kv and kv.writable)
    lib = load_library("sink_attention")
    ops._check(lib.tb_attention_prepare(
        ops._stream(), ops._ptr(proj), ctypes.c_longlong(proj.stride(0)), ops._ptr(bias), ops._ptr(taps), K,
        ops._ptr(state if K > 1 else None), ctypes.c_longlong(state_stride), ops._ptr(q_weight), ops._ptr(k_weight), QK_NORMS[qk_norm],
        ctypes.c_float(eps), ops._ptr(freq), rot, ops._ptr(ctx.positions), ops._ptr(ctx.seq_of_token), ops._ptr(ctx.seq_starts),
        ops._ptr(ctx.state_slots), ops._ptr(kv.slots if write else None), ops._ptr(q), ops._ptr(kv.k if write else None),
        ops._ptr(kv.v if write else None), T, num_heads, num_kv_heads, head_dim, value_dim, kv.page_size, int(bool(has_kv)),
        int(bool(values_from_keys)), int(write), ops._code(kv.k.dtype)), "attention_prepare")
    return q


TILE_ROWS = 64  # rows (token x query head of the group) of a query tile of the tensor-core kernel
TILE_INTS = 4  # first token row, request, first position, number of tokens


def tiles_apply(dtype: torch.dtype, head_dim: int, value_dim: int, groups: int, row_floats: int) -> bool:
    """Whether the tensor-core kernel takes this shape: bfloat16 caches, key and value sizes that are
    multiples of 16 up to 128, at most 64 query heads per kv head, query rows that start on 16 bytes."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= head_dim <= 128
            and 16 <= value_dim <= 128 and 1 <= groups <= TILE_ROWS and row_floats % 4 == 0
            and ops.env("TANDEM_SINK_ATTENTION", "tiles") != "simt")


def plan_tiles(host_starts, host_lens, groups: int) -> list:
    """Query tiles for a step: every request's new tokens in runs of 64 // groups, those with the most
    keys first; flat [first token row, request, first position, number of tokens] * n."""
    per_tile = TILE_ROWS // groups
    tiles, row = [], 0
    for b, (start, n) in enumerate(zip(host_starts, host_lens)):
        tiles.extend([row + off, b, start + off, min(per_tile, n - off)] for off in range(0, n, per_tile))
        row += n
    tiles.sort(key=lambda t: -(t[2] + t[3]))
    return [x for t in tiles for x in t]


def attend_tiles(q: torch.Tensor, kv, tiles: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 window: Optional[int], keep_first: int, scale: float, softcap: Optional[float],
                 bias_by_distance: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                 gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attend`` for the tokens that ``tiles`` (int32 on the device, as ``plan_tiles`` cut them) name, on the tensor cores."""
    ops._need(q, "q", torch.float32, contiguous=False)
    ops._need(tiles, "tiles", torch.int32)
    ops._need(kv.k, "k cache", torch.bfloat16)
    T = q.shape[0]
    max_dist = 0 if bias_by_distance is None else bias_by_distance.shape[0] - 1
    out = torch.empty((T, num_heads * value_dim), dtype=torch.bfloat16, device=q.device)
    lib = load_library("sink_attention_tile", (f"TB_DK={head_dim}", f"TB_DV={value_dim}"))
    ops._check(lib.tb_sink_attention_tile(
        ops._stream(), ops._ptr(q), q.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(tiles), tiles.numel() // TILE_INTS, ops._ptr(out), num_heads, num_kv_heads,
        kv.page_size, int(window or 0), int(keep_first if window else 0), ctypes.c_float(scale), ctypes.c_float(softcap or 0.0),
        ops._ptr(bias_by_distance), max_dist, ops._ptr(sink), ops._ptr(gate), _gate_stride(gate, T, num_heads)), "sink_attention_tile")
    return out


SPLIT_CHUNK = 128  # keys per chunk of the split kernel
MAX_SPLITS = 16


def split_applies(dtype: torch.dtype, head_dim: int, value_dim: int, groups: int, row_floats: int) -> bool:
    """Whether steps of single tokens run the kernel that cuts a token's keys over several blocks:
    bfloat16 caches (the 32-bit path keeps the kernel whose sums never depend on the cut), values of up
    to 256 (more than eight query heads per kv head are served eight to a block)."""
    held = min(8, max(1, groups))
    smem = (held * head_dim + 4 * held * (2 + value_dim)) * 4
    return (dtype == torch.bfloat16 and groups >= 1 and value_dim <= 256 and head_dim % 4 == 0 and row_floats % 4 == 0
            and smem <= 48 * 1024 and ops.env("TANDEM_SINK_ATTENTION", "tiles") != "simt")


def num_splits(window: Optional[int], keep_first: int) -> int:
    """Blocks per (token, kv head): the chunks a window (with its kept first tokens) can touch, sixteen at most."""
    if not window:
        return MAX_SPLITS
    return max(1, min(MAX_SPLITS, -(-(window + keep_first) // SPLIT_CHUNK) + 1))


def attend_split(q: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 window: Optional[int], keep_first: int, scale: float, softcap: Optional[float],
                 bias_by_distance: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                 gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attend`` for steps of single tokens, each token's keys cut over several blocks and merged in a fixed order."""
    ops._need(q, "q", torch.float32, contiguous=False)
    T = q.shape[0]
    max_dist = 0 if bias_by_distance is None else bias_by_distance.shape[0] - 1
    splits = num_splits(window, keep_first)
    out = torch.empty((T, num_heads * value_dim), dtype=kv.k.dtype, device=q.device)
    part_o = torch.empty((T * num_heads * splits, value_dim), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((T * num_heads * splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("sink_attention")
    ops._check(lib.tb_sink_attention_split(
        ops._stream(), ops._ptr(q), q.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(ctx.seq_of_token), ops._ptr(ctx.positions), ops._ptr(out), ops._ptr(part_o),
        ops._ptr(part_ml), splits, T, num_heads, num_kv_heads, head_dim, value_dim, kv.page_size, int(window or 0),
        int(keep_first if window else 0), ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), ops._ptr(bias_by_distance),
        max_dist, ops._ptr(sink), ops._code(kv.k.dtype), ops._ptr(gate), _gate_stride(gate, T, num_heads)), "sink_attention_split")
    ops.launches += 1  # two kernels
    return out


def expand_distance_bias(table: torch.Tensor, bucket_of, max_distance: int) -> torch.Tensor:
    """[buckets, heads] -> float32 [max_distance + 1, heads], one row per distance; the kernel clamps
    larger distances to the last row, so ``bucket_of`` must be constant from ``max_distance`` on.
    The buckets are computed on the host in double precision."""
    index = torch.tensor([bucket_of(n) for n in range(max_distance + 1)], dtype=torch.int64, device=table.device)
    return table.to(torch.float32)[index].contiguous()


def prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], v_other: Optional[torch.Tensor], mix: Optional[torch.Tensor],
            kv, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, unit_norm: bool, eps: float) -> None:
    """In place on the float32 projection ``qkv`` [T, nh dk + nkv dk + nkv dv]: biases added, q and k
    heads divided by their root mean square (``unit_norm``); k and v stored at the tokens' cache slots,
    v first mixed as (1 - mix) v + mix v_other where ``v_other`` (float32 rows of nkv dv values, any
    row stride) is given.  Afterwards the q columns hold the queries and the v columns the layer's own
    (unmixed) values."""
    ops._need(qkv, "qkv", torch.float32)
    T, cols = qkv.shape
    if cols != (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim:
        raise ops.KernelError(f"qkv has {cols} columns, expected {(num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim}")
    if bias is not None:
        ops._need(bias, "bias", torch.float32)
        if bias.numel() != cols:
            raise ops.KernelError(f"bias has {bias.numel()} elements, qkv rows have {cols}")
    stride_other = 0
    if v_other is not None:
        ops._need(v_other, "v_other", torch.float32, contiguous=False)
        ops._need(mix, "mix", torch.float32)
        if v_other.shape != (T, num_kv_heads * value_dim) or v_other.stride(1) != 1:
            raise ops.KernelError(f"values to mix in have shape {tuple(v_other.shape)}, expected {(T, num_kv_heads * value_dim)}")
        stride_other = v_other.stride(0)
    if kv.writable:
        ops._need(kv.slots, "slots", torch.int32)
        if tuple(kv.k.shape[1:]) != (num_kv_heads, kv.page_size, head_dim) or \
                tuple(kv.v.shape[1:]) != (num_kv_heads, kv.page_size, value_dim):
            raise ops.KernelError(f"caches {tuple(kv.k.shape)} / {tuple(kv.v.shape)} do not fit {num_kv_heads} kv heads of "
                                  f"{head_dim} / {value_dim}")
    lib = load_library("sink_attention")
    ops._check(lib.tb_sink_attention_prep(
        ops._stream(), ops._ptr(qkv), qkv.stride(0), ops._ptr(bias), ops._ptr(v_other), stride_other, ops._ptr(mix),
        ops._ptr(kv.slots), ops._ptr(kv.k), ops._ptr(kv.v), T, num_heads, num_kv_heads, head_dim, value_dim, kv.page_size,
        int(bool(unit_norm)), ctypes.c_float(eps), int(bool(kv.writable)), ops._code(kv.k.dtype)), "sink_attention_prep")


def attend(q: torch.Tensor, kv, ctx, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
           window: Optional[int], keep_first: int, scale: float, softcap: Optional[float],
           bias_by_distance: Optional[torch.Tensor], sink: Optional[torch.Tensor],
           gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention output [T, nh dv] in the cache's type for the float32 queries in the first nh dk
    columns of ``q``.  ``bias_by_distance`` float32 [distances, nh]; ``sink`` float32 [nh]; ``gate`` float32 [T, nh]
    (rows any stride apart): every head's output is multiplied by the sigmoid of its number."""
    ops._need(q, "q", torch.float32, contiguous=False)
    if q.stride(1) != 1 or q.shape[1] < num_heads * head_dim:
        raise ops.KernelError("queries must be rows of at least nh dk contiguous float32 values")
    if value_dim > 512:
        raise ops.KernelError(f"value size {value_dim} is larger than the 512 this kernel takes")
    T = q.shape[0]
    max_dist = 0
    if bias_by_distance is not None:
        ops._need(bias_by_distance, "bias_by_distance", torch.float32)
        if bias_by_distance.dim() != 2 or bias_by_distance.shape[1] != num_heads:
            raise ops.KernelError(f"the distance bias has shape {tuple(bias_by_distance.shape)}, expected [distances, {num_heads}]")
        max_dist = bias_by_distance.shape[0] - 1
    if sink is not None:
        ops._need(sink, "sink", torch.float32)
        if sink.numel() != num_heads:
            raise ops.KernelError(f"{sink.numel()} sinks for {num_heads} heads")
    out = torch.empty((T, num_heads * value_dim), dtype=kv.k.dtype, device=q.device)
    lib = load_library("sink_attention")
    ops._check(lib.tb_sink_attention(
        ops._stream(), ops._ptr(q), q.stride(0), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(kv.block_table),
        kv.block_table.stride(0), ops._ptr(ctx.seq_of_token), ops._ptr(ctx.positions), ops._ptr(out), T, num_heads,
        num_kv_heads, head_dim, value_dim, kv.page_size, int(window or 0), int(keep_first if window else 0),
        ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), ops._ptr(bias_by_distance), max_dist, ops._ptr(sink),
        ops._code(kv.k.dtype), ops._ptr(gate), _gate_stride(gate, T, num_heads)), "sink_attention")
    return out
