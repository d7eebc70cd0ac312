"""Entry points of ``csrc/post_norm.cu``: what stands between the sublayers of a layer whose norms sit on the
sublayers' OUTPUT, all on one float32 stream: the RMS norm in equal groups of a row, the add of a normed output
into the stream, the short causal convolution in front of a sublayer with its per-request state, the weighted
average over the layers' results, and ``link``, which does all of them for one boundary: the rows' scales in one
launch, the rest in one pass over the rows."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library

MAX_TAPS = 8  # taps the walking kernel takes (its registers hold the inputs in front of a token)


def _fits(weight: torch.Tensor, W: int, groups: int) -> None:
    ops._need(weight, "norm weight", torch.float32)
    if weight.numel() != W or groups <= 0 or W % groups:
        raise ops.KernelError(f"a norm weight of {weight.numel()} numbers in {groups} groups does not fit rows of {W}")


def group_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype,
               rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x float32 [T, W] (rows any stride apart): every row (or the rows ``rows`` int32 names) in ``groups`` equal runs,
    each divided by sqrt(mean(run^2) + eps), times ``weight``; -> [R, W] of ``out_dtype``.  ``out`` may be x itself."""
    ops._need(x, "x", torch.float32, contiguous=False)
    T, W = x.shape
    _fits(weight, W, groups)
    if x.stride(1) != 1:
        raise ops.KernelError("rows must be contiguous")
    R = T
    if rows is not None:
        ops._need(rows, "rows", torch.int32)
        R = rows.numel()
    if out is None:
        out = torch.empty((R, W), dtype=out_dtype, device=x.device)
    lib = load_library("post_norm")
    ops._check(lib.tb_group_norm(ops._stream(), ops._ptr(x), ctypes.c_longlong(x.stride(0)), ops._ptr(rows), ops._ptr(weight),
                                 ops._ptr(out), R, W, groups, ctypes.c_float(eps), ops._code(out.dtype)), "group_norm")
    return out


def group_norm_add(y: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, residual: torch.Tensor,
                   keep: Optional[torch.Tensor] = None) -> None:
    """residual += group_norm(y) * weight in place (float32 [T, W]); ``keep``: the new rows are written there too."""
    ops._need(y, "y", torch.float32)
    ops._need(residual, "residual", torch.float32)
    T, W = y.shape
    _fits(weight, W, groups)
    if tuple(residual.shape) != (T, W) or (keep is not None and (tuple(keep.shape) != (T, W) or keep.dtype != torch.float32
                                                                 or not keep.is_contiguous())):
        raise ops.KernelError(f"y {tuple(y.shape)} and the stream {tuple(residual.shape)} do not fit")
    lib = load_library("post_norm")
    ops._check(lib.tb_group_norm_add(ops._stream(), ops._ptr(y), ops._ptr(weight), ops._ptr(residual), ops._ptr(keep), T, W, groups,
                                     ctypes.c_float(eps)), "group_norm_add")


def depth_average(planes: torch.Tensor, coeff: torch.Tensor, n: int, out: torch.Tensor) -> None:
    """out = sum_(j < n) coeff[j] * planes[j] for float32 planes [>= n, T, W]."""
    ops._need(planes, "planes", torch.float32)
    ops._need(coeff, "coefficients", torch.float32)
    ops._need(out, "out", torch.float32)
    if planes.shape[0] < n or coeff.numel() < n or out.numel() != planes[0].numel():
        raise ops.KernelError(f"{n} coefficients over planes {tuple(planes.shape)} into {tuple(out.shape)} do not fit")
    lib = load_library("post_norm")
    ops._check(lib.tb_depth_average(ops._stream(), ops._ptr(planes), ctypes.c_longlong(planes[0].numel()), ops._ptr(coeff), n,
                                    ops._ptr(out), ctypes.c_longlong(out.numel())), "depth_average")


def short_conv(x: torch.Tensor, taps: Optional[torch.Tensor], state: Optional[torch.Tensor], ctx, out_dtype: torch.dtype) -> torch.Tensor:
    """h_t = x_t + sum_j taps[c, j] x_(t - K + 1 + j) for float32 x [T, W] and taps [W, K]; inputs in front of a request's
    rows of this step come from ``state`` [slots, (K - 1) * W] (the request's last K - 1 inputs, oldest first), zeros in
    front of the request's start.  -> [T, W] of ``out_dtype``.  ``taps`` None: h = x, rounded to ``out_dtype``."""
    ops._need(x, "x", torch.float32)
    T, W = x.shape
    K, stride = 0, 0
    if taps is not None:
        ops._need(taps, "taps", torch.float32)
        K = taps.shape[1]
        if taps.shape[0] != W:
            raise ops.KernelError(f"taps {tuple(taps.shape)} do not fit rows of {W}")
    if K > 1:
        ops._need(state, "state", torch.float32)
        stride = state[0].numel()
        if stride < (K - 1) * W:
            raise ops.KernelError(f"state rows of {stride} numbers do not hold {K - 1} inputs of {W}")
    out = torch.empty((T, W), dtype=out_dtype, device=x.device)
    lib = load_library("post_norm")
    ops._check(lib.tb_short_conv(ops._stream(), ops._ptr(x), ops._ptr(taps), K, ops._ptr(state if K > 1 else None),
                                 ctypes.c_longlong(stride), ops._ptr(ctx.seq_of_token), ops._ptr(ctx.positions), ops._ptr(ctx.seq_starts),
                                 ops._ptr(ctx.state_slots), ops._ptr(out), T, W, ops._code(out_dtype)), "short_conv")
    return out


def short_conv_state(x: torch.Tensor, state: Optional[torch.Tensor], ctx, K: int, width: Optional[int] = None) -> None:
    """Leaves every request's newest K - 1 rows of x (older ones from the state itself) in its state row.  ``width``: only
    the first so many columns of x are the convolution's inputs (x may then be rows of a wider tensor)."""
    if K <= 1:
        return
    ops._need(x, "x", torch.float32, contiguous=width is None)
    ops._need(state, "state", torch.float32)
    W = x.shape[1] if width is None else int(width)
    if x.stride(1) != 1 or W > x.shape[1] or state[0].numel() < (K - 1) * W:
        raise ops.KernelError(f"rows of {tuple(x.shape)} / state rows of {state[0].numel()} numbers do not hold {K - 1} inputs of {W}")
    lib = load_library("post_norm")
    ops._check(lib.tb_short_conv_state_rows(ops._stream(), ops._ptr(x), ctypes.c_longlong(x.stride(0)), W, ops._ptr(state),
                                            ctypes.c_longlong(state[0].numel()), ops._ptr(ctx.cu_seqlens), ops._ptr(ctx.state_slots),
                                            ctx.num_seqs, K), "short_conv_state")


def row_scales(y: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """1 / sqrt(mean(run^2) + eps) of the ``groups`` equal runs of every row of y (float32 or bfloat16 [T, W]) -> float32 [T, groups]."""
    if y.dim() != 2 or not y.is_contiguous() or not y.is_cuda:
        raise ops.KernelError("y must be a contiguous [T, W] tensor on the GPU")
    T, W = y.shape
    if groups <= 0 or W % groups:
        raise ops.KernelError(f"rows of {W} numbers do not split into {groups} equal runs")
    inv = torch.empty((T, groups), dtype=torch.float32, device=y.device)
    lib = load_library("post_norm")
    ops._check(lib.tb_row_scales(ops._stream(), ops._ptr(y), ops._code(y.dtype), T, W, groups, ctypes.c_float(eps), ops._ptr(inv)), "row_scales")
    return inv


def link(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, x_out: torch.Tensor,
         planes: Optional[torch.Tensor] = None, coeff: Optional[torch.Tensor] = None, n_planes: int = 0,
         taps: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, ctx=None,
         out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """The boundary between two sublayers: x_out = x + group_norm(y) * weight for the float32 stream x and a sublayer's
    output y (float32 or bfloat16); with ``planes`` (float32 [>= n_planes + 1, T, W]) that sum is kept as planes[n_planes]
    and x_out becomes sum_(j <= n_planes) coeff[j] planes[j]; with ``taps`` the next sublayer's input
    h = x_out + conv(x_out) is returned in ``out_dtype`` (the convolution's earlier inputs as in ``short_conv``; x_out must
    then be another tensor than x: a token's block reads the rows in front of it).  Two launches: the rows' scales, then
    everything else in one pass."""
    ops._need(x, "x", torch.float32)
    ops._need(x_out, "x_out", torch.float32)
    T, W = x.shape
    _fits(weight, W, groups)
    if tuple(y.shape) != (T, W) or tuple(x_out.shape) != (T, W) or (taps is not None and x_out.data_ptr() == x.data_ptr()):
        raise ops.KernelError("x, y and x_out must be of one shape, and with a convolution x_out another tensor than x")
    inv = row_scales(y, groups, eps)
    plane, kept = 0, None
    if planes is not None:
        ops._need(planes, "planes", torch.float32)
        ops._need(coeff, "coefficients", torch.float32)
        if planes.shape[0] <= n_planes or coeff.numel() != n_planes + 1 or planes[0].numel() != T * W:
            raise ops.KernelError(f"planes {tuple(planes.shape)} / {coeff.numel()} coefficients do not fit {n_planes} earlier results")
        plane, kept = T * W, planes[n_planes]
    K, stride, h = 0, 0, None
    if taps is not None:
        ops._need(taps, "taps", torch.float32)
        K = taps.shape[1]
        if taps.shape[0] != W or K > MAX_TAPS:
            raise ops.KernelError(f"taps {tuple(taps.shape)}: the kernel takes [{W}, up to {MAX_TAPS}]")
        if K > 1:
            ops._need(state, "state", torch.float32)
            stride = state[0].numel()
            if stride < (K - 1) * W:
                raise ops.KernelError(f"state rows of {stride} numbers do not hold {K - 1} inputs of {W}")
        h = torch.empty((T, W), dtype=out_dtype, device=x.device)
    lib = load_library("post_norm")
    ops._check(lib.tb_link(ops._stream(), ops._ptr(x), ops._ptr(y), ops._code(y.dtype), ops._ptr(inv), ops._ptr(weight), groups,
                           ops._ptr(planes), ctypes.c_longlong(plane), ops._ptr(coeff), n_planes, ops._ptr(kept), ops._ptr(x_out),
                           ops._ptr(taps), K, ops._ptr(state if K > 1 else None), ctypes.c_longlong(stride),
                           ops._ptr(ctx.seq_of_token) if ctx is not None else None, ops._ptr(ctx.positions) if ctx is not None else None,
                           ops._ptr(ctx.seq_starts) if ctx is not None else None, ops._ptr(ctx.state_slots) if ctx is not None else None,
                           ops._ptr(h), T, W, ops._code(out_dtype or torch.float32)), "link")
    return h
