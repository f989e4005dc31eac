"""Plain restatement of the Lotinex design: one function per mechanism, token by token where the design is a recurrence.

Slow on purpose and independent of the engine: it shares no code with the package, takes the config dictionary and the
tensors by their checkpoint names, and computes in one floating type (float64 by default) from the bf16 weight values.
The reference service names models by tag and has no model code (app/utils/config.py:86), so nothing here restates it.

Notation: X the streams [T, s, W] (s copies of the residual, mixed by small per-sublayer matrices); h what a sublayer reads;
S a recurrent state; p the position of a token in its sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, gain: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * gain + bias over the last axis."""
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gain + bias


def time_conv(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, c] = sum_j taps[c, j] u[t - K + 1 + j, c] (+ bias): the last column weighs the current token, zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            y[back:] += u[:T - back] * taps[:, j]
    return y if bias is None else y + bias


def rotary_frequencies(rot: Dict, dtype) -> (torch.Tensor, float):
    """Angle per position of every pair (i, i + dims / 2) and the factor on cos and sin.  With `scaling` the slow pairs are
    slowed by `factor`, the fast ones kept, with a linear ramp between the pair indices at which `original` positions hold
    `fast` and `slow` turns."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    at = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(at(float(sc["fast"]))), 0)
    hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, pos: torch.Tensor, rot: Optional[Dict]) -> torch.Tensor:
    """Coordinates (i, i + dims / 2), i < dims / 2, of the last axis turned by pos * f_i; x is [T, heads, d]."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    ang = pos.to(x.dtype)[:, None] * f
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out[..., :dims // 2] = u * c - v * s
    out[..., dims // 2:dims] = v * c + u * s
    return out


def visible_chunk(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: j <= i and both in the same run of `size` positions counted from 0."""
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[:, None] // size) == (i[None, :] // size))


def visible_window(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: 0 <= i - j < size."""
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, scale: float, softcap: float = 0.0,
           zero_sink: bool = False) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H * V]; query head a reads key head a // (H / G).  With zero_sink the
    denominator holds one more term exp(0) that has no value."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->ijh", q, kk) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask[:, :, None], -math.inf)
    top = s.max(1).values
    if zero_sink:
        top = torch.clamp(top, min=0.0)
    e = torch.exp(s - top[:, None, :])
    den = e.sum(1) + (torch.exp(-top) if zero_sink else 0.0)
    return (torch.einsum("ijh,jhv->ihv", e, vv) / den[:, :, None]).reshape(T, -1)


# ------------------------------------------------------------------------------------------------ mixers
def attention_keys(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float):
    """Keys (normed per head with a gain shared by the heads, rotated) and values of an attention layer, as its cache holds them."""
    T, G, D, V = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = rms_unit((h @ w[p + "k"].T).reshape(T, G, D), eps) * w[p + "k.norm"]
    return rotate_halves(k, torch.arange(T), m.get("rot")), (h @ w[p + "v"].T).reshape(T, G, V)


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float, kv) -> torch.Tensor:
    """Grouped-query attention inside runs of mask.size positions (no mask: every earlier position); `kv` = (keys, values) of
    this or of the lending layer."""
    T, H, D = h.shape[0], m["heads"], m["dim"]
    q = rms_unit((h @ w[p + "q"].T).reshape(T, H, D), eps) * w[p + "q.norm"]
    q = rotate_halves(q, torch.arange(T), m.get("rot"))
    o = attend(q, kv[0], kv[1], visible_chunk(T, int((m.get("mask") or {}).get("size") or max(T, 1))), float(m["scale"]))
    return o @ w[p + "o"].T


def delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Gated delta rule with one decay per head and token; the read-out sees the token's own write."""
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


def conv_window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Sliding-window attention whose q, k, v pass a short convolution over time, q and k an RMS norm over all their heads
    together, rotation with stretched frequencies, capped scores and a softmax with a zero-score sink."""
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (time_conv(h @ w[p + n].T, w[p + n + ".conv"]) if m.get("conv") else h @ w[p + n].T for n in "qkv")
    q = (rms_unit(q, eps) * w[p + "q.norm"]).reshape(T, H, D)
    k = (rms_unit(k, eps) * w[p + "k.norm"]).reshape(T, G, D)
    pos = torch.arange(T)
    q, k = rotate_halves(q, pos, m.get("rot")), rotate_halves(k, pos, m.get("rot"))
    o = attend(q, k, v.reshape(T, G, V), visible_window(T, int((m.get("mask") or {}).get("size") or max(T, 1))), float(m["scale"]),
               float(m.get("softcap") or 0.0), zero_sink=True)
    return o @ w[p + "o"].T


def selective_scan(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict) -> torch.Tensor:
    """State space with input-dependent step, input and read-out vectors: per channel c a state S[c, :] of m.state numbers."""
    T, C, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = silu(time_conv(xz[:, :C], w[p + "conv"], w[p + "conv.b"])), xz[:, C:]
    low = x @ w[p + "x"].T
    dt = softplus(low[:, :R] @ w[p + "dt"].T + w[p + "dt.b"])
    Bv, Cv = low[:, R:R + N], low[:, R + N:]
    A = -torch.exp(w[p + "A_log"])
    S = torch.zeros(C, N, dtype=h.dtype)
    y = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bv[t][None, :]
        y[t] = S @ Cv[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Half the sum of the two sides, each RMS-normed over the model width with its own gain."""
    left = conv_window_attention(h, w, p + "left.", m["left"], eps)
    right = selective_scan(h, w, p + "right.", m["right"])
    return 0.5 * (rms_unit(left, eps) * w[p + "left.out"] + rms_unit(right, eps) * w[p + "right.out"])


# ------------------------------------------------------------------------------------------------ feed-forward
def gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: Dict) -> torch.Tensor:
    """Sigmoid scores, the `top` largest; a chosen expert reads score * h (the score scales its INPUT)."""
    r = mlp["router"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], int(r["top"])).indices.tolist():
            out[t] += gated_ff((s[t, e] * h[t])[None], w, f"{p}e{e}.")[0]
    return out


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: Dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_ff(h, w, p)
    if mlp["kind"] == "moe":
        return expert_ff(h, w, p, mlp)
    raise ValueError(f"unknown feed-forward {mlp['kind']!r}")


# ------------------------------------------------------------------------------------------------ the model
def hyper_step(X: torch.Tensor, w: Dict[str, torch.Tensor], p: str, sub) -> torch.Tensor:
    """One sublayer on the streams X [T, s, W]: it reads sum_s in[s] X_s, and every new stream t is
    sum_s mix[s, t] X_s + out[t] * result.  Without the three tensors: one stream, plain residual."""
    if p + "in" not in w:
        return X + sub(X.sum(1))[:, None, :]
    y = sub(torch.einsum("s,tsw->tw", w[p + "in"], X))
    return torch.einsum("sr,tsw->trw", w[p + "mix"], X) + w[p + "out"][None, :, None] * y[:, None, :]


def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            trail: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start.  `trail` (a list) receives the summed streams after every layer."""
    w = {k: v.to("cpu").to(dtype) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    X = x[:, None, :].repeat(1, int(cfg.get("streams", 1)), 1)
    lent = {}                                     # keys and values of attention layers, for the layers that borrow them
    for i, l in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", l["mixer"], l["type"]
        norm1 = lambda u: layer_norm(u, w[p + "norm1"], w[p + "norm1.b"], eps)
        if kind == "attention":
            def mixer(u):
                h = norm1(u)
                src = m.get("kv_from")
                if src is None:
                    lent[i] = attention_keys(h, w, p + "mix.", m, eps)
                return attention_mixer(h, w, p + "mix.", m, eps, lent[i if src is None else int(src)])
        elif kind == "delta":
            mixer = lambda u: delta_mixer(norm1(u), w, p + "mix.", m, eps)
        elif kind == "parallel":
            mixer = lambda u: parallel_mixer(norm1(u), w, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {kind!r}")
        X = hyper_step(X, w, p + "hc1.", mixer)
        if l.get("mlp"):
            X = hyper_step(X, w, p + "hc2.", lambda u: feed_forward(
                layer_norm(u, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", l["mlp"]))
        if trail is not None:
            trail.append(X.sum(1))
    return layer_norm(X.sum(1), w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T


def greedy(cfg: Dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """n_new tokens of argmax decoding after `prompt` (the whole sequence is recomputed for every token)."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
