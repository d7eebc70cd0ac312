"""Entry points of ``csrc/moe.cu``: routing by score, and the chosen experts' feed-forwards (gated with SiLU,
or plain with the exact GELU; router outputs beyond the real experts may stand for identity experts).

``route`` turns float32 router logits into (expert, weight) pairs.  ``experts`` runs the chosen
experts of every token over stacked weights: one warp per output element for steps of few tokens
and for the 32-bit path; slots sorted by expert on the device and 64 x 64 tiles on the tensor
cores (mma.sync) for bfloat16 steps of more tokens; tiles of 128 sorted rows through the package's
grouped tcgen05 product for steps of many tokens.  Nothing goes through the host, so the step can be
captured in a CUDA graph.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

_SCORES = {"sigmoid": 0, "softmax": 1}
TILE_MIN_TOKENS = 33  # from here on the sorted tiles run (bfloat16): below, an expert's rows are read once per slot anyway
WIDE_MIN_TOKENS = 256  # from here on the grouped tcgen05 product runs: tiles of 128 sorted rows
WIDE_TILE = 128
_MAX_SLOTS = 65535  # slots per launch of the one-warp-per-output kernels


def route(logits: torch.Tensor, top_k: int, score: str, normalize: bool, scale: float,
          choice_bias: Optional[torch.Tensor] = None) -> tuple:
    """logits float32 [T, E] -> (experts int32 [T, top_k], weights float32 [T, top_k]): scores sigmoid(z) or
    softmax(z), the ``top_k`` largest chosen (the lower index wins a tie), their scores divided by their sum
    (+ 1e-20) where ``normalize``, times ``scale``.  ``choice_bias`` float32 [E]: the choice is made on score + bias;
    the weights are the scores without it."""
    ops._need(logits, "logits", torch.float32)
    if choice_bias is not None:
        ops._need(choice_bias, "choice_bias", torch.float32)
        if choice_bias.numel() != logits.shape[1]:
            raise ops.KernelError(f"a choice bias of {choice_bias.numel()} entries for {logits.shape[1]} router outputs")
    if score not in _SCORES:
        raise ops.KernelError(f"no score {score!r} (have {sorted(_SCORES)})")
    T, E = logits.shape
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    lib = load_library("moe")
    ops._check(lib.tb_moe_route(ops._stream(), ops._ptr(logits), ops._ptr(choice_bias), ops._ptr(ids), ops._ptr(weights), T, E, top_k,
                                _SCORES[score], int(bool(normalize)), ctypes.c_float(scale)), "moe_route")
    return ids, weights


def route_table(token_ids: torch.Tensor, table: torch.Tensor, num_experts: int) -> tuple:
    """Routing without a router: token ids int32 [T] and a table int32 [vocab, top] -> (experts int32 [T, top] =
    table[token], weights float32 [T, top], each 1 / top)."""
    ops._need(token_ids, "token_ids", torch.int32)
    ops._need(table, "table", torch.int32)
    if table.dim() != 2:
        raise ops.KernelError(f"the experts' table has shape {tuple(table.shape)}, expected [vocab, top]")
    T, (vocab, top) = token_ids.numel(), table.shape
    ids = torch.empty((T, top), dtype=torch.int32, device=table.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=table.device)
    lib = load_library("moe")
    ops._check(lib.tb_moe_route_table(ops._stream(), ops._ptr(token_ids), ops._ptr(table), ops._ptr(ids), ops._ptr(weights), T, top,
                                      vocab, int(num_experts)), "moe_route_table")
    return ids, weights


_PLAIN_ACTIVATIONS = {"gelu": 0, "relu2": -1}  # how the kernels are told which activation an expert without a gate has


def _gate_code(gated: bool, activation: str) -> int:
    if gated:
        return 1
    if activation not in _PLAIN_ACTIVATIONS:
        raise ops.KernelError(f"experts without a gate have no activation {activation!r} (have {sorted(_PLAIN_ACTIVATIONS)})")
    return _PLAIN_ACTIVATIONS[activation]


def tiles_apply(x: torch.Tensor, hidden: int, inner: int) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] >= TILE_MIN_TOKENS and hidden % 8 == 0 and inner % 8 == 0
            and ops.env("TANDEM_MOE", "wide") != "simt")


def wide_applies(x: torch.Tensor, hidden: int, inner: int, top: int, num_experts: int) -> bool:
    """Whether the grouped tcgen05 product runs the experts: bfloat16, enough slots per expert to fill tiles of 128
    rows, sizes its 16-byte pieces take."""
    T = x.shape[0]
    return (x.dtype == torch.bfloat16 and T >= WIDE_MIN_TOKENS and T * top >= 64 * num_experts and hidden % 8 == 0 and inner % 8 == 0
            and ops.env("TANDEM_MOE", "wide") not in ("simt", "tiles"))


def _experts_wide(x, gate_up, down, ids, weights, gated: bool, E: int, activation: str = "gelu") -> torch.Tensor:
    from tandem_b200.kernels import gemm_bf16

    T, K = x.shape
    real, F, top = gate_up.shape[0], down.shape[2], ids.shape[1]
    capacity = -(-(T * top + E * (WIDE_TILE - 1)) // WIDE_TILE) * WIDE_TILE
    dev = x.device
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    order = torch.empty(capacity, dtype=torch.int32, device=dev)
    tile_group = torch.empty(capacity // WIDE_TILE, dtype=torch.int32, device=dev)
    position = torch.empty(T * top, dtype=torch.int32, device=dev)
    xs = torch.empty((capacity, K), dtype=torch.bfloat16, device=dev)
    lib = load_library("moe")
    ops._check(lib.tb_moe_sort_gather(ops._stream(), ops._ptr(x), ops._ptr(ids), ops._ptr(offsets), ops._ptr(order), ops._ptr(tile_group),
                                      ops._ptr(position), ops._ptr(xs), T, top, E, K, capacity, WIDE_TILE, real), "moe_sort_gather")
    ops.launches += 1  # two kernels
    if gated:
        act = gemm_bf16.wide_grouped(xs, gate_up.view(real * 2 * F, K), tile_group, real, torch.bfloat16, gated=True)
    else:
        act = gemm_bf16.wide_grouped(xs, gate_up.view(real * F, K), tile_group, real, torch.bfloat16, activation=activation)
    part = gemm_bf16.wide_grouped(act, down.view(real * K, F), tile_group, real, torch.float32, gated=False)
    y = torch.empty((T, K), dtype=torch.float32, device=dev)
    _combine(lib, part, weights, position, y, T, top, K, ids, real, E, x)
    return y


def _combine(lib, part, weights, position, y, T: int, top: int, N: int, ids, real: int, E: int, x) -> None:
    """y[t] = the weighted sum of a token's slots; slots of identity experts (``real`` <= expert < ``E``) add weight * x[t]."""
    identity = real < E
    ops._check(lib.tb_moe_combine(ops._stream(), ops._ptr(part), ops._ptr(weights), ops._ptr(position), ops._ptr(y), T, top, N,
                                  ops._ptr(ids if identity else None), real, ops._ptr(x if identity else None), ops._code(x.dtype)),
               "moe_combine")


def experts(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
            gated: bool = True, num_router_outputs: Optional[int] = None, activation: str = "gelu") -> torch.Tensor:
    """sum_k weights[t, k] * down[e] (SiLU(gate[e] x_t) * (up[e] x_t)) with e = ids[t, k]: float32 [T, hidden].
    x [T, hidden]; gate_up [E, 2 F, hidden] (an expert's gate rows, then its up rows); down [E, hidden, F].
    Without a gate (``gated`` False): ``gate_up`` is up [E, F, hidden] and an expert is down[e] act(up[e] x_t), ``activation``
    "gelu" (the exact one) or "relu2" (the square of max(z, 0)).  ``num_router_outputs`` > E: experts E and above are identity experts, whose slots add weights[t, k] * x_t."""
    ops._need(x, "x")
    ops._need(gate_up, "gate_up", x.dtype)
    ops._need(down, "down", x.dtype)
    ops._need(ids, "ids", torch.int32)
    ops._need(weights, "weights", torch.float32)
    T, K = x.shape
    real, F2, K2 = gate_up.shape
    F, top = (F2 // 2 if gated else F2), ids.shape[1]
    E = real if num_router_outputs is None else int(num_router_outputs)
    if K2 != K or tuple(down.shape) != (real, K, F) or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top) or E < real:
        raise ops.KernelError(f"x {tuple(x.shape)}, gate_up {tuple(gate_up.shape)}, down {tuple(down.shape)}, ids "
                              f"{tuple(ids.shape)} do not fit together")
    code = _gate_code(gated, activation)
    if wide_applies(x, K, F, top, E):
        return _experts_wide(x, gate_up, down, ids, weights, gated, E, activation)
    y = torch.empty((T, K), dtype=torch.float32, device=x.device)
    lib = load_library("moe")
    if tiles_apply(x, K, F):
        rows = lib.tb_moe_tile_rows()
        capacity = -(-(T * top + E * (rows - 1)) // rows) * rows
        offsets = torch.empty(E + 1, dtype=torch.int32, device=x.device)
        order = torch.empty(capacity, dtype=torch.int32, device=x.device)
        act = torch.empty((capacity, F), dtype=torch.bfloat16, device=x.device)
        part = torch.empty((T * top, K), dtype=torch.float32, device=x.device)
        ops._check(lib.tb_moe_tiles(ops._stream(), ops._ptr(x), ops._ptr(gate_up), ops._ptr(down), ops._ptr(ids), ops._ptr(weights),
                                    ops._ptr(offsets), ops._ptr(order), ops._ptr(act), ops._ptr(part), ops._ptr(y), T, top, E, K, F, K,
                                    capacity, real, code), "moe_tiles")
        ops.launches += 3  # four kernels
        return y
    step = max(1, _MAX_SLOTS // top)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=x.device)
    for t0 in range(0, T, step):
        n = min(step, T - t0)
        order = torch.empty(n * top, dtype=torch.int32, device=x.device)
        act = torch.empty((n * top, F), dtype=x.dtype, device=x.device)
        part = torch.empty((n * top, K), dtype=torch.float32, device=x.device)
        ops._check(lib.tb_moe_order(ops._stream(), ops._ptr(ids[t0:]), ops._ptr(offsets), ops._ptr(order), n, top, E), "moe_order")
        ops._check(lib.tb_moe_gate_up(ops._stream(), ops._ptr(x[t0:]), ops._ptr(gate_up), ops._ptr(ids[t0:]), ops._ptr(order),
                                      ops._ptr(act), n, top, F, K, real, code, ops._code(x.dtype)), "moe_gate_up")
        ops._check(lib.tb_moe_down(ops._stream(), ops._ptr(act), ops._ptr(down), ops._ptr(ids[t0:]), ops._ptr(order), ops._ptr(part),
                                   n, top, K, F, real, ops._code(x.dtype)), "moe_down")
        _combine(lib, part, weights[t0:], None, y[t0:], n, top, K, ids[t0:], real, E, x[t0:])
    return y
