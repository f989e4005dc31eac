"""Plain restatement of the Vonedra design: one function per mechanism, token by token where the design is a recurrence.

Slow on purpose and independent of the engine: it shares no code with the package, takes the config dictionary and the
tensors by their checkpoint names, and computes in one floating type (float64 by default) from the bf16 weight values.
The reference service names models by tag and has no model code (app/utils/config.py:86), so nothing here restates it.

Notation: x the stream [T, W]; h what a sublayer reads; S a matrix state [key dim, value dim] per head; X_j the stream
as layer j - 1 left it (X_0: the scaled embedding).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def time_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """y[t, c] = sum_j taps[c, j] u[t - K + 1 + j, c]: the last column weighs the current token, zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            y[back:] += u[:T - back] * taps[:, j]
    return y


def input_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: the stream plus its short convolution over time."""
    return x + time_conv(x, taps)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance-bias table for distance n: one row per distance below rows / 2, logarithmic steps up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(table: torch.Tensor, T: int, far: float) -> torch.Tensor:
    """[T, T, heads]: entry (i, j) is the table row of distance i - j (row 0 where j > i; masked anyway)."""
    rows = table.shape[0]
    by_dist = torch.stack([table[distance_bucket(n, rows, far)] for n in range(T)])
    i = torch.arange(T)
    return by_dist[(i[:, None] - i[None, :]).clamp(min=0)]


def visible(T: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & ((d < size) | (i[None, :] < keep_first))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Coordinates (2i, 2i+1), i < dims / 2, of the last axis turned by pos * base^(-2i / dims); x is [T, ..., d]."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    ang = pos.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float,
                    v_first: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Grouped-query attention with unit-RMS queries and keys, a distance bias, a window that keeps the first tokens, a
    sink in the softmax and values mixed with those of the first such layer.  Returns (output, the values it used)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D), eps)
    k = rms_unit((h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D), eps)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, V)
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->ijh", q, kk) * float(m["scale"]) + distance_bias(w[p + "rel"], T, float(m["bias_max"]))
    mask = visible(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)))
    s = s.masked_fill(~mask[:, :, None], -math.inf)
    sink = w[p + "sink"]
    top = torch.maximum(s.max(1).values, sink)                       # [T, H]
    e = torch.exp(s - top[:, None, :])
    den = e.sum(1) + torch.exp(sink - top)
    o = torch.einsum("ijh,jhv->ihv", e, vv) / den[:, :, None]
    return o.reshape(T, H * V) @ w[p + "o"].T + w[p + "o.b"], v


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are linear images of one normed latent per token, plus one rotated key part that all
    heads share; the queries come through a normed latent of their own; a plain window."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    dkv = h @ w[p + "dkv"].T
    c = rms_unit(dkv[:, :C], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(dkv[:, C:], pos, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    s = (torch.einsum("ihd,jhd->ijh", q_plain, k_plain) + torch.einsum("ihr,jr->ijh", q_rot, k_rot)) * float(m["scale"])
    s = s.masked_fill(~visible(T, int(m["mask"]["size"]))[:, :, None], -math.inf)
    a = torch.softmax(s, 1)
    return torch.einsum("ijh,jhv->ihv", a, v).reshape(T, H * V) @ w[p + "o"].T


def delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Gated delta rule with one decay per head and token."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(time_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, D)
    k = silu(time_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, D)
    v = silu(time_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            qt, kt = q[t, a // (H // G)], k[t, a // (H // G)]
            S = g[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, a] = S.T @ qt
    out = rms_unit(out, eps) * w[p + "norm"]
    return (out.reshape(T, H * V) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            trail: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start.  `trail` (a list) receives the stream after every layer."""
    w = {k: v.to("cpu").to(dtype) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    made = [x]                                   # X_0 .. X_i
    v_first = None
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        h = input_conv(x, w[p + "canon1"])
        if l["type"] == "attention":
            y, v = attention_mixer(h, w, p + "mix.", m, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif l["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, p + "mix.", m, eps)
        elif l["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {l['type']!r}")
        x = x + rms_unit(y, eps) * w[p + "norm1"]
        if l.get("mlp"):
            if l["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward {l['mlp']['kind']!r}")
            x = x + rms_unit(dense_ff(input_conv(x, w[p + "canon2"]), w, p + "mlp."), eps) * w[p + "norm2"]
        made.append(x)
        x = sum(w[p + "dwa"][j] * made[j] for j in range(len(made)))
        if trail is not None:
            trail.append(x)
    return (rms_unit(x, eps) * w["final.norm"]) @ w["head"].T


def greedy(cfg: Dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """n_new tokens of argmax decoding after `prompt` (the whole sequence is recomputed for every token)."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
