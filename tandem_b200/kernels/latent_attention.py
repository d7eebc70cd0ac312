"""Entry points of ``csrc/latent_attention.cu``: what surrounds the attention kernel when keys and
values are expanded from a cached latent (cache entry and query rotation; the small product per
head that folds the key expansion into the queries and applies the value expansion; the gate)."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.kernels.build import load_library


def prepare(proj: torch.Tensor, kv_col: int, norm_weight: torch.Tensor, freq: Optional[torch.Tensor], positions: torch.Tensor, kv,
            num_heads: int, head_dim: int, rotary_dim: int, latent_dim: int, eps: float, queries: Optional[torch.Tensor] = None,
            interleaved: bool = False, magnitude: float = 1.0) -> torch.Tensor:
    """proj float32 [T, cols]: ``num_heads`` query heads of head_dim + rotary_dim numbers from column 0 (or the rows
    of ``queries`` where the queries come from a product of their own) and the down-projection (latent_dim +
    rotary_dim numbers) from ``kv_col``.  Writes the token's cache entry (key row [RMSNorm(latent) * weight |
    rotated key part], value row the normed latent) and returns the queries' room float32 [T, H, latent_dim +
    rotary_dim] with the rotated part of every head filled in.  ``freq`` float32 [pairs]: the angle of pair n is
    position * freq[n]; ``interleaved``: pair n is (2 n, 2 n + 1) instead of (n, n + pairs); ``magnitude``: a factor
    on cos and sin."""
    ops._need(proj, "proj", torch.float32)
    ops._need(norm_weight, "norm weight", torch.float32)
    ops._need(positions, "positions", torch.int32)
    T, R, r = proj.shape[0], latent_dim, rotary_dim
    rd = 0
    if freq is not None:
        ops._need(freq, "freq", torch.float32)
        rd = 2 * freq.numel()
    q_in = proj if queries is None else queries
    if queries is not None:
        ops._need(queries, "queries", torch.float32, contiguous=False)
        if queries.shape[0] != T or queries.stride(1) != 1:
            raise ops.KernelError(f"queries {tuple(queries.shape)} do not fit {T} tokens")
    if norm_weight.numel() != R or kv_col + R + r > proj.shape[1] or num_heads * (head_dim + r) > q_in.shape[1]:
        raise ops.KernelError(f"projection of {proj.shape[1]} columns / queries of {q_in.shape[1]} / norm weight of "
                              f"{norm_weight.numel()} do not fit {num_heads} heads of {head_dim} + {r} and a latent of {R} + {r} "
                              f"at column {kv_col}")
    if kv.writable:
        ops._need(kv.slots, "slots", torch.int32)
        if tuple(kv.k.shape[1:]) != (1, kv.page_size, R + r) or tuple(kv.v.shape[1:]) != (1, kv.page_size, R):
            raise ops.KernelError(f"caches {tuple(kv.k.shape)} / {tuple(kv.v.shape)} do not fit a latent of {R} + {r}")
    q = torch.empty((T, num_heads, R + r), dtype=torch.float32, device=proj.device)
    lib = load_library("latent_attention")
    kv_in = ctypes.c_void_p(proj.data_ptr() + 4 * kv_col)
    ops._check(lib.tb_latent_prep(ops._stream(), ops._ptr(q_in), ctypes.c_longlong(q_in.stride(0)), kv_in,
                                  ctypes.c_longlong(proj.stride(0)), ops._ptr(norm_weight), ops._ptr(freq),
                                  ops._ptr(positions), ops._ptr(kv.slots), ops._ptr(kv.k), ops._ptr(kv.v), ops._ptr(q), T, num_heads,
                                  head_dim, r, rd, R, kv.page_size, ctypes.c_float(eps), int(bool(kv.writable)),
                                  int(bool(interleaved)), ctypes.c_float(magnitude), ops._code(kv.k.dtype)), "latent_prep")
    return q


def head_linear(x: torch.Tensor, x_head: int, weight: torch.Tensor, out: torch.Tensor, out_head: int, num_heads: int, n: int, k: int,
                transposed: bool) -> None:
    """out[t, h, :n] = W[h] x[t, h, :k] for every token and head: x rows of any stride with head h at column
    h * x_head, likewise ``out`` (float32); ``weight`` holds W[h] as [n, k] (or [k, n] with ``transposed``),
    head after head.  x float32 or bfloat16, weight of the model's type; sums in float32."""
    ops._need(x, "x", contiguous=False)
    ops._need(weight, "weight")
    ops._need(out, "out", torch.float32, contiguous=False)
    if weight.numel() != num_heads * n * k or x.stride(-1) != 1 or out.stride(-1) != 1:
        raise ops.KernelError(f"weight of {weight.numel()} elements does not hold {num_heads} matrices of {n} x {k}")
    T = x.shape[0]
    lib = load_library("latent_attention")
    ops._check(lib.tb_head_linear(ops._stream(), ops._ptr(x), ops._code(x.dtype), ctypes.c_longlong(x.stride(0)), x_head,
                                  ops._ptr(weight), ops._code(weight.dtype), ops._ptr(out), ops._code(out.dtype),
                                  ctypes.c_longlong(out.stride(0)), out_head, T, num_heads, n, k, int(bool(transposed))),
               "head_linear")


def sigmoid_gate(o: torch.Tensor, gate: Optional[torch.Tensor], out_dtype: torch.dtype, per: int = 1) -> torch.Tensor:
    """o * sigmoid(gate) for float32 o [T, N] and float32 gate rows of N / ``per`` values (any row stride; None: no gate),
    rounded to ``out_dtype``: every run of ``per`` outputs shares one gate value (the value size: a gate per head)."""
    ops._need(o, "o", torch.float32)
    T, N = o.shape
    stride = 0
    if gate is not None:
        ops._need(gate, "gate", torch.float32, contiguous=False)
        if per <= 0 or N % per or tuple(gate.shape) != (T, N // per) or gate.stride(1) != 1:
            raise ops.KernelError(f"gate {tuple(gate.shape)} does not fit o {tuple(o.shape)} with a value per {per} outputs")
        stride = gate.stride(0)
    y = torch.empty((T, N), dtype=out_dtype, device=o.device)
    lib = load_library("latent_attention")
    ops._check(lib.tb_sigmoid_gate(ops._stream(), ops._ptr(o), ops._ptr(gate), stride, ops._ptr(y), T, N, max(1, per),
                                   ops._code(out_dtype)), "sigmoid_gate")
    return y
