"""A plain, slow implementation of the Deletar design, written from its equations: one function per
mechanism, whole sequences only (no cache, no batching), float64 unless asked otherwise.  It shares no
code with the package and is what the package's kernels are compared with.

The model is a dict of the configuration file's keys and a dict of tensors by checkpoint name.

Notation: x [T, W] is the residual stream of one sequence, positions count from 0, a linear weight is
stored [out, in] and applied as x @ W^T.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms: the weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def frequencies(dims: int, base: float, scaling=None) -> list:
    """f_i = base^(-2 i / dims), i < dims / 2; with ``scaling`` (factor, low, high, original) waves longer than
    original / low are slowed by ``factor``, waves shorter than original / high are kept, those between blend."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > original / low:
                f = f / factor
            elif wave >= original / high:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, freqs: list, dims: int) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` numbers of each head turned, number i paired with i + dims / 2."""
    T = x.shape[0]
    half = dims // 2
    angle = torch.arange(T, dtype=x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]  # [T, half]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def causal_convolution(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, K]: y_t = sum_j w[:, j] u_(t - K + 1 + j), zeros in front of the sequence."""
    T, C = u.shape
    K = w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + w[:, j][None, :] * padded[j:j + T]
    return y


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window, softcap, sink: bool) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query head h reads key head h // (H / G); position i
    sees j with 0 <= i - j < window; capped scores; softmax, with one more in the denominator where ``sink``."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


def mixer(kind: str, m: dict, w: dict, p: str, h: torch.Tensor, eps: float, memo: dict, index: int) -> torch.Tensor:
    """One of the three attention mixers on its input h [T, W].  ``memo[layer]`` keeps the (keys, values) a layer
    used, for the layers that borrow them."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    freqs = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    borrowed = m.get("kv_from")

    q = h @ w[f"{p}.q"].T
    if kind == "attention_2":
        q = q + w[f"{p}.q.b"]
    if borrowed is None:
        k = h @ w[f"{p}.k"].T
        if kind == "attention_2":
            k = k + w[f"{p}.k.b"]
            v = k.clone()  # the values are the keys as projected
        else:
            v = h @ w[f"{p}.v"].T
    if kind == "attention" and m.get("conv"):
        q = causal_convolution(q, w[f"{p}.q.conv"])
        k = causal_convolution(k, w[f"{p}.k.conv"])
        v = causal_convolution(v, w[f"{p}.v.conv"])
    if kind == "attention_2":  # one norm over the whole projection
        q = norm_plain(q, w[f"{p}.q.norm"], eps)
        if borrowed is None:
            k = norm_plain(k, w[f"{p}.k.norm"], eps)
    q = q.view(T, H, d)
    if kind == "attention_3":  # a norm per head, one weight for all heads
        q = norm_plain(q, w[f"{p}.q.norm"], eps)
    q = rotate(q, freqs, rot["dims"])
    if borrowed is None:
        k = k.view(T, G, d)
        if kind == "attention_3":
            k = norm_plain(k, w[f"{p}.k.norm"], eps)
        k = rotate(k, freqs, rot["dims"])
        v = v.view(T, G, dv)
        memo[index] = (k, v)
    else:
        k, v = memo[borrowed]
    window = (m.get("mask") or {}).get("size")
    o = attend(q, k, v, m["scale"], window, m.get("softcap"), sink=kind == "attention_3")
    if kind in ("attention_2", "attention_3"):
        o = o * torch.sigmoid(h @ w[f"{p}.g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[f"{p}.o"].T


def expert(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return relu_squared(h @ w[f"{p}.up"].T) @ w[f"{p}.down"].T


def feed_forward(mlp: dict, w: dict, p: str, h: torch.Tensor, tokens: list) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return expert(h, w, p)
    top = mlp["router"]["top"]
    table = w[f"{p}.table"]
    y = torch.zeros_like(h)
    for t, token in enumerate(tokens):
        for e in table[token].tolist():
            y[t] = y[t] + expert(h[t:t + 1], w, f"{p}.e{e}")[0] / top
    if mlp.get("shared"):
        y = y + expert(h, w, f"{p}.shared")
    return y


def forward(config: dict, weights: dict, tokens: list, dtype=torch.float64):
    """-> (logits [T, vocab], the stream after every layer [layers, T, W])."""
    w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    memo: dict = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        a = mixer(layer["type"], layer["mixer"], w, f"{p}.mix", norm_one_plus(x, w[f"{p}.norm1"], eps), eps, memo, i)
        x = x + norm_one_plus(a, w[f"{p}.norm1b"], eps)
        if layer.get("mlp") is not None:
            f = feed_forward(layer["mlp"], w, f"{p}.mlp", norm_one_plus(x, w[f"{p}.norm2"], eps), tokens)
            x = x + norm_one_plus(f, w[f"{p}.norm2b"], eps)
        after.append(x)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(after)


def read_folder(folder: str):
    """(configuration dict, tensors by name) of a model folder."""
    import json
    import os

    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        config = json.load(f)
    return config, load_file(os.path.join(folder, "model.safetensors"))


def greedy(config: dict, weights: dict, prompt: list, steps: int) -> list:
    """``steps`` tokens after ``prompt``, each the argmax of the last position's logits."""
    tokens, out = list(prompt), []
    for _ in range(steps):
        logits, _ = forward(config, weights, tokens)
        out.append(int(logits[-1].argmax()))
        tokens.append(out[-1])
    return out
