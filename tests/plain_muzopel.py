"""A plain, slow implementation of the Muzopel design in PyTorch on the CPU (float64 by default),
written from the design's equations: one function per mechanism, whole sequences at once, no
cache, no batching, no kernels.  It shares no code with ``tandem_b200``; the tests compare the
engine with it.

Notation: a sequence has T tokens at positions 0 .. T-1; x [T, W] is the residual stream; a
weight ``w[name]`` is stored [out, in] and applied as x @ w.T.  Y_0 is the normed embedding and
Y_(i+1) what layer i makes of its input; the input of layer i + 1 is a learned weighted sum of
Y_0 .. Y_(i+1).
"""

from __future__ import annotations

import json
import math
import os

import torch


def read_folder(folder: str, dtype=torch.float64):
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name).to(dtype)
    return cfg, w


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, groups: int, eps):
    """The last axis in ``groups`` equal runs, each divided by its own root mean square; then times ``weight``."""
    n = x.shape[-1]
    parts = x.reshape(*x.shape[:-1], groups, n // groups)
    return unit_rms(parts, eps).reshape(x.shape) * weight


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotary_frequencies(rot: dict) -> tuple:
    """(frequencies [dims / 2], factor on cos and sin).  Plain: base^(-2 i / dims), factor 1.  With
    ``scaling`` (factor s, original length L, fast, slow): the pair index at which a wave makes t turns
    within L is n(t) = dims ln(L / (2 pi t)) / (2 ln base); pairs below lo = max(floor(n(fast)), 0) keep
    their frequency, pairs above hi = min(ceil(n(slow)), dims - 1) have it divided by s, those between
    are blended linearly; cos and sin are multiplied by 0.1 ln(s) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, L = float(sc["factor"]), float(sc["original"])

    def n(turns: float) -> float:
        return dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(n(float(sc["fast"]))), 0)
    hi = min(math.ceil(n(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s * ramp + f * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate_pairs(x, positions, rot: dict):
    """x [..., T, n] with the token axis second to last: numbers 2i and 2i + 1 of the first ``dims`` form a
    pair (u, v) that becomes (u cos a - v sin a, v cos a + u sin a), a = position * frequency_i; cos and sin
    carry the scaling's factor.  Numbers beyond ``dims`` pass unchanged."""
    dims = rot["dims"]
    f, mag = rotary_frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = (a.cos() * mag).to(x.dtype), (a.sin() * mag).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mechanisms
def short_convolution(u, taps):
    """u [T, C] -> u + conv(u); taps [C, K], column K - 1 weighs the current token, zeros in front of the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = u.clone()
    for j in range(K):
        out = out + padded[j: j + T] * taps[:, j][None, :]
    return out


def latent_attention(h, w, p, m, eps, positions=None, hide=None):
    """h [T, W] -> [T, W].  Keys and values of a head are expansions of a normed latent of ``kv_rank``
    numbers a token; a rotated key part of ``rot_dim`` numbers is shared by the heads.  With ``q_rank``
    the queries come through a normed latent of their own; with a tensor ``.g`` each head's output is
    multiplied by a sigmoid gate (one number per token and head).  ``hide``: a key position that no
    query sees (for tests that show that a key matters)."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T) if positions is None else positions
    if f"{p}.dq" in w:
        cq = unit_rms(h @ w[f"{p}.dq"].T, eps) * w[f"{p}.dq.norm"][None, :]
        q = cq @ w[f"{p}.uq"].T
    else:
        q = h @ w[f"{p}.q"].T
    q = q.reshape(T, H, d + r)
    q_flat = q[..., :d]
    q_rot = rotate_pairs(q[..., d:].transpose(0, 1), positions, m["rot"]).transpose(0, 1)
    dkv = h @ w[f"{p}.dkv"].T
    c = unit_rms(dkv[:, :R], eps) * w[f"{p}.dkv.norm"][None, :]
    k_rot = rotate_pairs(dkv[:, R:], positions, m["rot"])
    k_flat = (c @ w[f"{p}.uk"].T).reshape(T, H, d)
    v = (c @ w[f"{p}.uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_flat, k_flat) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = j > i
    if hide is not None:
        mask = mask | ((j == hide) & (i != hide))
    scores = scores.masked_fill(mask[None], -math.inf)
    o = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v)
    if f"{p}.g" in w:
        o = o * torch.sigmoid(h @ w[f"{p}.g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[f"{p}.o"].T


def route(h, w, p, router):
    """(chosen [T, top], weights [T, top]): softmax over all router outputs; the choice is made on score +
    correction, the weight is the score itself, not renormalised."""
    s = torch.softmax(h @ w[f"{p}.router"].T, dim=-1)
    _, idx = torch.topk(s + w[f"{p}.correction"][None, :], router["top"], dim=-1)
    return idx, torch.gather(s, 1, idx)


def routed_ff(h, w, p, mlp):
    """The router has ``experts`` + ``identity`` outputs; the last ``identity`` of them stand for experts that
    return their input.  A real expert is down(gelu(up h))."""
    r = mlp["router"]
    E = r["experts"]
    idx, weight = route(h, w, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(r["top"]):
            e = int(idx[t, k])
            y = h[t] if e >= E else gelu_erf(h[t] @ w[f"{p}.e{e}.up"].T) @ w[f"{p}.e{e}.down"].T
            out[t] += weight[t, k] * y
    return out


def layer(cfg, w, i, x, positions=None):
    """Y_(i+1) from the layer's input x: each sublayer reads the stream through a short convolution and its
    output enters the stream through a norm."""
    L, p = cfg["layers"][i], f"l{i}"
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    y = latent_attention(short_convolution(x, w[f"{p}.canon1"]), w, f"{p}.mix", L["mixer"], eps, positions)
    x = x + group_norm(y, w[f"{p}.norm1"], groups, eps)
    if L.get("mlp") is not None:
        y = routed_ff(short_convolution(x, w[f"{p}.canon2"]), w, f"{p}.mlp", L["mlp"])
        x = x + group_norm(y, w[f"{p}.norm2"], groups, eps)
    return x


def forward(cfg, w, tokens, keep_layers: bool = False):
    """Logits [T, vocab] for one sequence (and, with ``keep_layers``, the stream after every layer, depth
    average included)."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = group_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], groups, eps)
    made, after = [x], []
    for i in range(len(cfg["layers"])):
        made.append(layer(cfg, w, i, x))
        x = sum(w[f"l{i}.dwa"][j] * made[j] for j in range(i + 2))
        after.append(x)
    logits = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if keep_layers else logits
