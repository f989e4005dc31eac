"""Layered models: decoders that config.json describes layer by layer (ft_layer_desc in include/fasttalk_b200.h).

The first design of this family is Gitozen: parallel layers (mixer and feed-forward read one scalar-gain RMS norm and are
added through element-wise sigmoid gates), two token mixers — latent attention without positions, whose cache holds one
normed latent per token, and a gated delta rule with one decay per head and key channel, whose state lives in a
per-session slot — a mixture of experts with group-limited routing, and tanh-capped logits.

The second design is Gedelorn: sandwich layers (an RMS norm with a gain per coordinate before and after each sublayer, the
weight stored as gain - 1), branch mixers — a gated matrix memory ("mlstm"), a selective state space ("mamba2"), and a
"parallel" mixer that adds a sliding-window softmax attention (rotary pairs, capped scores, keys reused as values) to a
linear attention with a constant decay per head — and a feed-forward that is either a dense SwiGLU or a mixture of
squared-ReLU experts with sigmoid scores and a shared expert.  Its mixers are ft_branch_desc entries of the native engine.

The third design is Vonedra: post-norm layers (the sublayers read the stream itself through a short causal convolution over
time, only their results are RMS-normed, and the stream that goes on is a learned weighted sum of what every earlier layer
left), three mixers — grouped-query attention with unit-RMS queries and keys, a bias by bucketed distance, a window that
keeps the first tokens, a sink in the softmax and values mixed with those of the first such layer; latent attention with a
query latent, a shared rotated key part and a window (one shared key head in the engine: FT_BRANCH_LATENT_WINDOW); a gated
delta rule with one decay per head and token and a SiLU gate (the channel-delta kernels with the decay written to all of a
head's channels) — and a dense SwiGLU feed-forward.

The fourth design is Lotinex: pre-norm layers (layer norms with gain and bias) over several copies of the stream that small
per-sublayer matrices mix ("hyper-connections"), three mixers — grouped-query attention inside fixed runs of positions, with
per-head RMS-normed queries and keys, half-split rotary pairs and, optionally, the keys and values of an earlier layer; the
gated delta rule with one decay per head; and a "parallel" mixer that averages a sliding-window attention (short
convolutions on q, k, v, one RMS norm over all heads, stretched rotary frequencies, capped scores, a zero-score sink) with a
selective state-space scan, each side RMS-normed over the width — and a feed-forward that is a dense SwiGLU or a mixture of
experts whose sigmoid scores multiply the experts' inputs.  Its logits come from the embedding table itself.

The reference names models by tag only and owns no model code (app/utils/config.py:86, docker-compose.vllm.yml:39); this
module is the model side of what its engine container would load: config.json -> LayeredSpec, model.safetensors -> the
tensors by their names in the file, pack() -> the device arrays and descriptors the native engine reads.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

MIXER_LATENT_ATTENTION, MIXER_CHANNEL_DELTA, MIXER_BRANCHES = 1, 2, 3
FF_NONE, FF_MOE, FF_DENSE = 0, 1, 2
LAYER_GATED, LAYER_SANDWICH, LAYER_POSTNORM, LAYER_HYPER = 0, 1, 2, 3
ACT_SWIGLU, ACT_RELU2 = 0, 1
ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1
BRANCH_WINDOW_ATTENTION, BRANCH_DECAY_ATTENTION, BRANCH_MATRIX_MEMORY, BRANCH_STATE_SPACE, BRANCH_LATENT_WINDOW = 1, 2, 3, 4, 5
BRANCH_SELECTIVE_SCAN = 6
MIXERS = {"latent_attention": MIXER_LATENT_ATTENTION, "channel_delta": MIXER_CHANNEL_DELTA,
          "mlstm": MIXER_BRANCHES, "mamba2": MIXER_BRANCHES, "parallel": MIXER_BRANCHES}
BRANCHES = {"window_attention": BRANCH_WINDOW_ATTENTION, "decay_attention": BRANCH_DECAY_ATTENTION,
            "matrix_memory": BRANCH_MATRIX_MEMORY, "state_space": BRANCH_STATE_SPACE, "latent_window": BRANCH_LATENT_WINDOW,
            "selective_scan": BRANCH_SELECTIVE_SCAN}
POSTNORM_MIXERS = ("attention", "latent_attention", "delta")      # Vonedra's names for its mixers
SANDWICH_MIXERS = ("mlstm", "mamba2", "parallel")
HYPER_MIXERS = ("attention", "delta", "parallel")                 # Lotinex's names for its mixers


@dataclass(frozen=True)
class BranchSpec:
    """One token mixer of a branch layer (ft_branch_desc).  `prefix` is where its tensors live below '<layer>.mix.'."""
    kind: str                       # key of BRANCHES
    heads: int
    dim: int                        # query / key size per head (state space: the state size)
    vdim: int
    kv_heads: int = 0               # window attention: key heads; state space: groups; otherwise = heads
    prefix: str = ""
    out_scale: float = 1.0
    scale: float = 1.0              # window attention
    softcap: float = 0.0
    window: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    decay: Tuple[float, ...] = ()   # decay attention
    gate_cap: float = 0.0           # matrix memory
    conv: int = 0                   # state space
    norm_groups: int = 1
    # window attention options (Vonedra's attention)
    qk_norm: bool = False
    keep_first: int = 0
    rel_rows: int = 0               # rows of the distance-bias table (0 = none)
    rel_far: float = 0.0            # distance from which the last row applies
    sink: bool = False
    biases: bool = False            # q, k, v and output biases
    v_mix: bool = False
    # latent window attention: dim = plain query/key size per head, rot_dims = rotated size
    kv_rank: int = 0
    q_rank: int = 0
    # window attention options (Lotinex's attention and the left side of its parallel mixer); conv above = taps on q, k, v
    qk_gain: str = ""               # "" | "head" (gain [dim] shared by the heads) | "all" (one norm and gains over all heads)
    rot_half: bool = False          # rotated pairs (i, i + rot_dims / 2)
    rot_scaling: Tuple[float, ...] = ()      # (factor, original, fast, slow): slow pairs slowed by factor, cos / sin magnified
    chunked: bool = False           # runs of `window` positions instead of a sliding window
    zero_sink: bool = False         # one more term exp(0) in the softmax denominator
    kv_from: int = -1               # layer whose keys and values this one reads
    out_norm_width: bool = False    # the projected output is RMS-normed over the width (gain '<side>out')
    dt_rank: int = 0                # selective scan (heads = channels, dim = states per channel)


@dataclass(frozen=True)
class LayerSpec:
    mixer: str                      # "latent_attention" | "channel_delta" | "mlstm" | "mamba2" | "parallel"
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    kv_heads: int = 0               # channel_delta
    conv: int = 0                   # channel_delta: taps
    rank_a: int = 0                 # channel_delta: inner size of the decay projection (from the tensor's shape)
    rank_g: int = 0                 # channel_delta: inner size of the gate projection
    kv_rank: int = 0                # latent_attention
    scale: float = 0.0              # latent_attention
    ff: int = 0                     # 0 = the layer has no feed-forward
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    # sandwich layers (Gedelorn)
    form: str = "gated"             # "gated" | "sandwich" | "postnorm" | "hyper"
    branches: Tuple[BranchSpec, ...] = ()
    ff_kind: str = ""               # sandwich: "" (none) | "dense" | "moe"
    route_scale: float = 1.0
    shared_ff: int = 0


@dataclass(frozen=True)
class LayeredSpec:
    name: str
    architecture: str
    width: int
    vocab: int
    eps: float
    logit_softcap: float
    layers: Tuple[LayerSpec, ...] = field(default_factory=tuple)
    embed_scale: float = 1.0        # post-norm and hyper-connected models
    canon_taps: int = 0             # post-norm models: taps of the input convolutions
    streams: int = 0                # hyper-connected models: copies of the stream (0: one, and no mixing tensors)

    # the attributes the serving code reads from any model spec
    @property
    def hidden(self) -> int:
        return self.width

    def config(self) -> Dict:
        """The config.json of this spec."""
        out = []
        if self.layers and self.layers[0].form == "hyper":
            cfg = {"architecture": self.architecture, "embedding": {"scale": self.embed_scale},
                   "layers": [_hyper_layer_config(l) for l in self.layers], "norm": {"eps": self.eps}, "vocab": self.vocab,
                   "width": self.width}
            if self.streams:
                cfg["streams"] = self.streams
            return cfg
        for l in self.layers:
            if l.form == "sandwich":
                out.append(_sandwich_layer_config(l))
                continue
            if l.form == "postnorm":
                out.append(_postnorm_layer_config(l))
                continue
            if l.mixer == "latent_attention":
                mixer = {"dim": l.dim, "heads": l.heads, "kv_rank": l.kv_rank, "scale": l.scale, "vdim": l.vdim}
            else:
                mixer = {"conv": l.conv, "dim": l.dim, "heads": l.heads, "kv_heads": l.kv_heads, "vdim": l.vdim}
            mlp = None
            if l.ff:
                mlp = {"expert": {"ff": l.ff}, "kind": "moe",
                       "router": {"experts": l.experts, "groups": {"count": l.groups, "keep": l.keep}, "top": l.top}}
            out.append({"mixer": mixer, "mlp": mlp, "type": l.mixer})
        cfg = {"architecture": self.architecture, "layers": out, "norm": {"eps": self.eps}, "vocab": self.vocab,
               "width": self.width}
        if self.logit_softcap or self.architecture == "Gitozen":
            cfg["logit_softcap"] = self.logit_softcap
        if self.layers and self.layers[0].form == "postnorm":
            cfg["canon"] = {"taps": self.canon_taps}
            cfg["embedding"] = {"scale": self.embed_scale}
        return cfg


def _hyper_attention_config(b: BranchSpec) -> Dict:
    m = {"dim": b.dim, "heads": b.heads, "kv_heads": b.kv_heads, "scale": b.scale, "vdim": b.vdim}
    if b.window:
        m["mask"] = {"size": b.window}
    if b.rot_dims:
        m["rot"] = {"base": b.rot_base, "dims": b.rot_dims}
        if b.rot_scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), b.rot_scaling))
    if b.softcap:
        m["softcap"] = b.softcap
    if b.conv:
        m["conv"] = b.conv
    if b.kv_from >= 0:
        m["kv_from"] = b.kv_from
    return m


def _hyper_layer_config(l: LayerSpec) -> Dict:
    if l.mixer == "delta":
        mixer = {"conv": l.conv, "dim": l.dim, "heads": l.heads, "kv_heads": l.kv_heads, "vdim": l.vdim}
    elif l.mixer == "attention":
        mixer = _hyper_attention_config(l.branches[0])
    else:
        left, right = l.branches
        mixer = {"left": _hyper_attention_config(left),
                 "right": {"conv": right.conv, "dt_rank": right.dt_rank, "inner": right.heads, "state": right.dim}}
    mlp = None
    if l.ff_kind == "dense":
        mlp = {"ff": l.ff, "kind": "dense"}
    elif l.ff_kind == "moe":
        mlp = {"expert": {"ff": l.ff}, "kind": "moe", "router": {"experts": l.experts, "top": l.top}}
    return {"mixer": mixer, "mlp": mlp, "type": l.mixer}


def _hyper_attention_from_config(m: Dict, **kw) -> BranchSpec:
    rot = m.get("rot") or {}
    sc = rot.get("scaling") or {}
    return BranchSpec(
        kind="window_attention", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
        vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
        window=int((m.get("mask") or {}).get("size", 0)), rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
        rot_half=True, rot_scaling=tuple(float(sc[k]) for k in ("factor", "original", "fast", "slow")) if sc else (),
        qk_norm=True, conv=int(m.get("conv") or 0), kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else -1, **kw)


def _hyper_layer_from_config(i: int, l: Dict) -> LayerSpec:
    kind, m = l["type"], l["mixer"]
    kw = dict(mixer=kind, form="hyper")
    if kind == "attention":
        kw["branches"] = (_hyper_attention_from_config(m, qk_gain="head", chunked=bool((m.get("mask") or {}).get("size"))),)
    elif kind == "delta":
        kw.update(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                  conv=int(m["conv"]))
    elif kind == "parallel":
        r = m["right"]
        kw["branches"] = (
            _hyper_attention_from_config(m["left"], prefix="left.", qk_gain="all", zero_sink=True, out_norm_width=True, out_scale=0.5),
            BranchSpec(kind="selective_scan", heads=int(r["inner"]), kv_heads=1, dim=int(r["state"]), vdim=1, prefix="right.",
                       conv=int(r["conv"]), dt_rank=int(r["dt_rank"]), out_norm_width=True, out_scale=0.5))
    else:
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
    mlp = l.get("mlp")
    if mlp:
        if mlp.get("kind") == "dense":
            kw.update(ff_kind="dense", ff=int(mlp["ff"]))
        elif mlp.get("kind") == "moe":
            kw.update(ff_kind="moe", ff=int(mlp["expert"]["ff"]), experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]))
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    return LayerSpec(**kw)


def rotary_frequencies(b: BranchSpec) -> Tuple[List[float], float]:
    """Angle per position of every rotated pair and the factor on cos and sin.  With rot_scaling = (factor, original, fast,
    slow): pair i turns `original * f_i / 2 pi` times over the original context; pairs that turn more than `fast` times keep
    f_i, pairs that turn fewer than `slow` times get f_i / factor, with a linear ramp over the pair index between."""
    import math
    half = b.rot_dims // 2
    f = [b.rot_base ** (-2.0 * i / b.rot_dims) for i in range(half)]
    if not b.rot_scaling:
        return f, 1.0
    factor, orig, fast, slow = b.rot_scaling
    at = lambda turns: b.rot_dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(b.rot_base))
    lo, hi = max(math.floor(at(fast)), 0), min(math.ceil(at(slow)), b.rot_dims - 1)
    ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)]
    return [f[i] / factor * ramp[i] + f[i] * (1.0 - ramp[i]) for i in range(half)], 0.1 * math.log(factor) + 1.0


def _postnorm_layer_config(l: LayerSpec) -> Dict:
    if l.mixer == "delta":
        mixer = {"conv": l.conv, "dim": l.dim, "heads": l.heads, "kv_heads": l.kv_heads, "vdim": l.vdim}
    else:
        b = l.branches[0]
        if l.mixer == "attention":
            mixer = {"bias_max": b.rel_far, "dim": b.dim, "heads": b.heads, "kv_heads": b.kv_heads,
                     "mask": {"keep_first": b.keep_first, "size": b.window}, "scale": b.scale, "v_mix": b.v_mix, "vdim": b.vdim}
        else:
            mixer = {"dim": b.dim, "heads": b.heads, "kv_rank": b.kv_rank, "mask": {"size": b.window}, "q_rank": b.q_rank,
                     "rot": {"base": b.rot_base, "dims": b.rot_dims}, "rot_dim": b.rot_dims, "scale": b.scale, "vdim": b.vdim}
    return {"mixer": mixer, "mlp": {"ff": l.ff, "kind": "dense"} if l.ff_kind == "dense" else None, "type": l.mixer}


def _postnorm_layer_from_config(i: int, l: Dict, shapes: Optional[Dict[str, Tuple[int, ...]]]) -> LayerSpec:
    kind, m = l["type"], l["mixer"]
    kw = dict(mixer=kind, form="postnorm")
    if kind == "attention":
        mask = m.get("mask") or {}
        rows = int(shapes[f"l{i}.mix.rel"][0]) if shapes is not None else int(m.get("bias_rows", 0))
        kw["branches"] = (BranchSpec(
            kind="window_attention", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
            vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), window=int(mask.get("size", 0)),
            keep_first=int(mask.get("keep_first", 0)), qk_norm=True, rel_rows=rows, rel_far=float(m.get("bias_max", 0.0)),
            sink=True, biases=True, v_mix=bool(m.get("v_mix", False))),)
    elif kind == "latent_attention":
        rot = m.get("rot") or {}
        rd = int(m.get("rot_dim", rot.get("dims", 0)))
        if rd and int(rot.get("dims", rd)) != rd:
            raise ValueError(f"layer {i}: the rotated key part has {rd} coordinates, the rotation covers {rot.get('dims')}")
        kw["branches"] = (BranchSpec(
            kind="latent_window", heads=int(m["heads"]), kv_heads=1, dim=int(m["dim"]), vdim=int(m["vdim"]),
            scale=float(m["scale"]), window=int((m.get("mask") or {}).get("size", 0)), rot_dims=rd,
            rot_base=float(rot.get("base", 10000.0)), kv_rank=int(m["kv_rank"]),
            q_rank=int(shapes[f"l{i}.mix.dq"][0]) if shapes is not None else int(m["q_rank"])),)
    elif kind == "delta":
        kw.update(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                  conv=int(m["conv"]))
    else:
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
    mlp = l.get("mlp")
    if mlp:
        if mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        kw.update(ff_kind="dense", ff=int(mlp["ff"]))
    return LayerSpec(**kw)


def distance_rows(rows: int, far: float) -> List[int]:
    """Row of a distance-bias table with `rows` rows for every distance 0 .. ceil(far): one row per distance below rows // 2,
    then equal steps of log(distance) up to `far`, from where the last row applies."""
    import math
    half = rows // 2
    if not far > half >= 1:
        raise ValueError(f"a distance-bias table of {rows} rows needs a far distance above {half} (got {far})")
    out = []
    for n in range(int(math.ceil(far)) + 1):
        out.append(n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


def _branch_config(b: BranchSpec) -> Dict:
    if b.kind == "window_attention":
        m = {"dim": b.dim, "heads": b.heads, "kv_heads": b.kv_heads, "mask": {"size": b.window}, "scale": b.scale,
             "vdim": b.vdim}
        if b.rot_dims:
            m["rot"] = {"base": b.rot_base, "dims": b.rot_dims}
        if b.softcap:
            m["softcap"] = b.softcap
        return m
    if b.kind == "decay_attention":
        return {"decay": list(b.decay), "dim": b.dim, "heads": b.heads, "vdim": b.vdim}
    if b.kind == "matrix_memory":
        return {"dim": b.dim, "gate_cap": b.gate_cap, "heads": b.heads, "vdim": b.vdim}
    return {"conv": b.conv, "groups": b.kv_heads, "heads": b.heads, "norm_groups": b.norm_groups, "state": b.dim,
            "vdim": b.vdim}


def _sandwich_layer_config(l: LayerSpec) -> Dict:
    if l.mixer == "parallel":
        left, right = l.branches
        mixer = {"left": _branch_config(left), "left_scale": left.out_scale, "right": _branch_config(right),
                 "right_scale": right.out_scale}
    else:
        mixer = _branch_config(l.branches[0])
    mlp = None
    if l.ff_kind == "dense":
        mlp = {"ff": l.ff, "kind": "dense"}
    elif l.ff_kind == "moe":
        mlp = {"expert": {"ff": l.ff}, "kind": "moe",
               "router": {"experts": l.experts, "scale": l.route_scale, "top": l.top}}
        if l.shared_ff:
            mlp["shared"] = {"ff": l.shared_ff}
    return {"mixer": mixer, "mlp": mlp, "type": l.mixer}


def _branch_from_config(kind: str, m: Dict, prefix: str = "", out_scale: float = 1.0) -> BranchSpec:
    if kind == "window_attention":
        rot = m.get("rot") or {}
        return BranchSpec(kind=kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                          vdim=int(m.get("vdim", m["dim"])), prefix=prefix, out_scale=out_scale, scale=float(m["scale"]),
                          softcap=float(m.get("softcap") or 0.0), window=int((m.get("mask") or {}).get("size", 0)),
                          rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)))
    if kind == "decay_attention":
        decay = tuple(float(x) for x in m["decay"])
        if len(decay) != int(m["heads"]):
            raise ValueError(f"{len(decay)} decays for {m['heads']} heads")
        return BranchSpec(kind=kind, heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                          prefix=prefix, out_scale=out_scale, decay=decay)
    if kind == "matrix_memory":
        return BranchSpec(kind=kind, heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                          prefix=prefix, out_scale=out_scale, gate_cap=float(m["gate_cap"]))
    if kind == "state_space":
        return BranchSpec(kind=kind, heads=int(m["heads"]), kv_heads=int(m.get("groups", 1)), dim=int(m["state"]),
                          vdim=int(m["vdim"]), prefix=prefix, out_scale=out_scale, conv=int(m["conv"]),
                          norm_groups=int(m.get("norm_groups", 1)))
    raise ValueError(f"unknown branch kind {kind!r}")


def _sandwich_layer_from_config(i: int, l: Dict) -> LayerSpec:
    kind, m = l["type"], l["mixer"]
    if kind == "mlstm":
        branches = (_branch_from_config("matrix_memory", m),)
    elif kind == "mamba2":
        branches = (_branch_from_config("state_space", m),)
    else:
        branches = (_branch_from_config("window_attention", m["left"], "left.", float(m.get("left_scale", 1.0))),
                    _branch_from_config("decay_attention", m["right"], "right.", float(m.get("right_scale", 1.0))))
    kw = dict(mixer=kind, form="sandwich", branches=branches)
    mlp = l.get("mlp")
    if mlp:
        if mlp["kind"] == "dense":
            kw.update(ff_kind="dense", ff=int(mlp["ff"]))
        elif mlp["kind"] == "moe":
            r = mlp["router"]
            kw.update(ff_kind="moe", ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]),
                      route_scale=float(r.get("scale", 1.0)), shared_ff=int((mlp.get("shared") or {}).get("ff", 0)))
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    return LayerSpec(**kw)


def spec_from_config(cfg: Dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None, name: str = "checkpoint") -> LayeredSpec:
    """config.json (+ tensor shapes, for the sizes only a shape gives) -> LayeredSpec."""
    layers = []
    postnorm = cfg.get("architecture") == "Vonedra"
    hyper = cfg.get("architecture") == "Lotinex"
    for i, l in enumerate(cfg["layers"]):
        kind, m = l["type"], l["mixer"]
        if hyper:
            layers.append(_hyper_layer_from_config(i, l))
            continue
        if postnorm:
            layers.append(_postnorm_layer_from_config(i, l, shapes))
            continue
        if kind not in MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        if kind in SANDWICH_MIXERS:
            layers.append(_sandwich_layer_from_config(i, l))
            continue
        kw = dict(mixer=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
        if kind == "latent_attention":
            kw.update(kv_rank=int(m["kv_rank"]), scale=float(m["scale"]))
        else:
            kw.update(kv_heads=int(m.get("kv_heads", m["heads"])), conv=int(m["conv"]))
            if shapes is not None:
                kw.update(rank_a=int(shapes[f"l{i}.mix.a1"][0]), rank_g=int(shapes[f"l{i}.mix.g1"][0]))
            else:
                kw.update(rank_a=int(m.get("rank_a", 0)), rank_g=int(m.get("rank_g", 0)))
        mlp = l.get("mlp")
        if mlp:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            r = mlp["router"]
            g = r.get("groups") or {}
            kw.update(ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]),
                      groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))))
        layers.append(LayerSpec(**kw))
    cap = cfg.get("logit_softcap")
    return LayeredSpec(name=name, architecture=str(cfg.get("architecture", "Gitozen")), width=int(cfg["width"]),
                       vocab=int(cfg["vocab"]), eps=float(cfg["norm"]["eps"]), logit_softcap=float(cap) if cap else 0.0,
                       layers=tuple(layers), embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                       canon_taps=int((cfg.get("canon") or {}).get("taps", 0)), streams=int(cfg.get("streams") or 0) if hyper else 0)


def tensor_shapes(spec: LayeredSpec) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes of a checkpoint of this spec."""
    W = spec.width
    out: Dict[str, Tuple[int, ...]] = {"embed": (spec.vocab, W)}
    if spec.layers and spec.layers[0].form == "hyper":
        for i, l in enumerate(spec.layers):
            out.update(_hyper_shapes(f"l{i}.", l, W, spec.streams))
        out.update({"final.norm": (W,), "final.norm.b": (W,)})      # no head: the logits come from the embedding table
        return out
    for i, l in enumerate(spec.layers):
        p = f"l{i}."
        if l.form == "sandwich":
            out.update(_sandwich_shapes(p, l, W))
            continue
        if l.form == "postnorm":
            out.update(_postnorm_shapes(p, i, l, W, spec.canon_taps))
            continue
        out[p + "norm1"] = ()
        if l.mixer == "latent_attention":
            out.update({p + "mix.q": (l.heads * l.dim, W), p + "mix.dkv": (l.kv_rank, W), p + "mix.dkv.norm": (l.kv_rank,),
                        p + "mix.uk": (l.heads * l.dim, l.kv_rank), p + "mix.uv": (l.heads * l.vdim, l.kv_rank),
                        p + "mix.g": (l.heads, W), p + "mix.o": (W, l.heads * l.vdim)})
        else:
            qk, hv = l.kv_heads * l.dim, l.heads * l.vdim
            out.update({p + "mix.q": (qk, W), p + "mix.q.conv": (qk, l.conv), p + "mix.k": (qk, W),
                        p + "mix.k.conv": (qk, l.conv), p + "mix.v": (hv, W), p + "mix.v.conv": (hv, l.conv),
                        p + "mix.b": (l.heads, W), p + "mix.A_log": (l.heads,), p + "mix.norm": (l.vdim,),
                        p + "mix.a1": (l.rank_a, W), p + "mix.a2": (l.heads * l.dim, l.rank_a),
                        p + "mix.dt_bias": (l.heads * l.dim,), p + "mix.g1": (l.rank_g, W),
                        p + "mix.g2": (hv, l.rank_g), p + "mix.o": (W, hv)})
        if l.ff:
            for e in range(l.experts):
                out.update({f"{p}mlp.e{e}.gate": (l.ff, W), f"{p}mlp.e{e}.up": (l.ff, W), f"{p}mlp.e{e}.down": (W, l.ff)})
            out[p + "mlp.router"] = (l.experts, W)
            out.update({p + "rg2": (W, W), p + "rg2.b": (W,)})
        out.update({p + "rg1": (W, W), p + "rg1.b": (W,)})
    out["final.norm"] = (W,) if spec.layers and spec.layers[-1].form in ("sandwich", "postnorm") else ()
    out["head"] = (spec.vocab, W)
    return out


def _hyper_shapes(p: str, l: LayerSpec, W: int, streams: int) -> Dict[str, Tuple[int, ...]]:
    out: Dict[str, Tuple[int, ...]] = {p + "norm1": (W,), p + "norm1.b": (W,)}
    m = p + "mix."
    if l.mixer == "delta":
        qk, hv = l.kv_heads * l.dim, l.heads * l.vdim
        out.update({m + "q": (qk, W), m + "q.conv": (qk, l.conv), m + "k": (qk, W), m + "k.conv": (qk, l.conv),
                    m + "v": (hv, W), m + "v.conv": (hv, l.conv), m + "b": (l.heads, W), m + "A_log": (l.heads,),
                    m + "norm": (l.vdim,), m + "a": (l.heads, W), m + "dt_bias": (l.heads,), m + "g": (hv, W), m + "o": (W, hv)})
    for b in l.branches:
        q = m + b.prefix
        if b.kind == "window_attention":
            nq, nk, nv = b.heads * b.dim, b.kv_heads * b.dim, b.kv_heads * b.vdim
            wide = b.qk_gain == "all"
            out.update({q + "q": (nq, W), q + "q.norm": (nq if wide else b.dim,), q + "o": (W, b.heads * b.vdim)})
            if b.kv_from < 0:
                out.update({q + "k": (nk, W), q + "v": (nv, W), q + "k.norm": (nk if wide else b.dim,)})
            if b.conv:
                out[q + "q.conv"] = (nq, b.conv)
                if b.kv_from < 0:
                    out.update({q + "k.conv": (nk, b.conv), q + "v.conv": (nv, b.conv)})
        else:
            C, N, R = b.heads, b.dim, b.dt_rank
            out.update({q + "in": (2 * C, W), q + "conv": (C, b.conv), q + "conv.b": (C,), q + "x": (R + 2 * N, C),
                        q + "dt": (C, R), q + "dt.b": (C,), q + "A_log": (C, N), q + "D": (C,), q + "o": (W, C)})
        if b.out_norm_width:
            out[q + "out"] = (W,)
    subs = ["hc1"]
    if l.ff_kind:
        out.update({p + "norm2": (W,), p + "norm2.b": (W,)})
        subs.append("hc2")
    if l.ff_kind == "dense":
        out.update({p + "mlp.gate": (l.ff, W), p + "mlp.up": (l.ff, W), p + "mlp.down": (W, l.ff)})
    elif l.ff_kind == "moe":
        for e in range(l.experts):
            out.update({f"{p}mlp.e{e}.gate": (l.ff, W), f"{p}mlp.e{e}.up": (l.ff, W), f"{p}mlp.e{e}.down": (W, l.ff)})
        out[p + "mlp.router"] = (l.experts, W)
    if streams:
        for h in subs:
            out.update({f"{p}{h}.in": (streams,), f"{p}{h}.out": (streams,), f"{p}{h}.mix": (streams, streams)})
    return out


def _postnorm_shapes(p: str, i: int, l: LayerSpec, W: int, taps: int) -> Dict[str, Tuple[int, ...]]:
    out: Dict[str, Tuple[int, ...]] = {p + "norm1": (W,), p + "canon1": (W, taps), p + "dwa": (i + 2,)}
    m = p + "mix."
    if l.mixer == "delta":
        qk, hv = l.kv_heads * l.dim, l.heads * l.vdim
        out.update({m + "q": (qk, W), m + "q.conv": (qk, l.conv), m + "k": (qk, W), m + "k.conv": (qk, l.conv),
                    m + "v": (hv, W), m + "v.conv": (hv, l.conv), m + "b": (l.heads, W), m + "A_log": (l.heads,),
                    m + "norm": (l.vdim,), m + "a": (l.heads, W), m + "dt_bias": (l.heads,), m + "g": (hv, W), m + "o": (W, hv)})
    else:
        b = l.branches[0]
        hv = b.heads * b.vdim
        if b.kind == "window_attention":
            out.update({m + "q": (b.heads * b.dim, W), m + "q.b": (b.heads * b.dim,), m + "k": (b.kv_heads * b.dim, W),
                        m + "k.b": (b.kv_heads * b.dim,), m + "v": (b.kv_heads * b.vdim, W), m + "v.b": (b.kv_heads * b.vdim,),
                        m + "rel": (b.rel_rows, b.heads), m + "vmix": (), m + "sink": (b.heads,), m + "o": (W, hv),
                        m + "o.b": (W,)})
        else:
            out.update({m + "dq": (b.q_rank, W), m + "dq.norm": (b.q_rank,), m + "uq": (b.heads * (b.dim + b.rot_dims), b.q_rank),
                        m + "dkv": (b.kv_rank + b.rot_dims, W), m + "dkv.norm": (b.kv_rank,), m + "uk": (b.heads * b.dim, b.kv_rank),
                        m + "uv": (hv, b.kv_rank), m + "o": (W, hv)})
    if l.ff_kind == "dense":
        out.update({p + "norm2": (W,), p + "canon2": (W, taps), p + "mlp.gate": (l.ff, W), p + "mlp.up": (l.ff, W),
                    p + "mlp.down": (W, l.ff)})
    return out


def _sandwich_shapes(p: str, l: LayerSpec, W: int) -> Dict[str, Tuple[int, ...]]:
    out: Dict[str, Tuple[int, ...]] = {p + "norm1": (W,), p + "norm1b": (W,)}
    for b in l.branches:
        m = p + "mix." + b.prefix
        hv = b.heads * b.vdim
        if b.kind == "window_attention":
            out.update({m + "q": (b.heads * b.dim, W), m + "q.b": (b.heads * b.dim,), m + "k": (b.kv_heads * b.dim, W),
                        m + "k.b": (b.kv_heads * b.dim,), m + "o": (W, hv)})
        elif b.kind == "decay_attention":
            out.update({m + "q": (b.heads * b.dim, W), m + "k": (b.heads * b.dim, W), m + "v": (hv, W), m + "g": (hv, W),
                        m + "o": (W, hv), m + "norm": (hv,)})
        elif b.kind == "matrix_memory":
            out.update({m + "q": (b.heads * b.dim, W), m + "k": (b.heads * b.dim, W), m + "v": (hv, W), m + "g": (hv, W),
                        m + "o": (W, hv), m + "norm": (hv,), m + "i": (b.heads, W), m + "i.b": (b.heads,),
                        m + "f": (b.heads, W), m + "f.b": (b.heads,)})
        else:
            ch = hv + 2 * b.kv_heads * b.dim
            out.update({m + "in": (hv + ch + b.heads, W), m + "conv": (ch, b.conv), m + "conv.b": (ch,),
                        m + "dt_bias": (b.heads,), m + "A_log": (b.heads,), m + "D": (b.heads,), m + "norm": (hv,),
                        m + "o": (W, hv)})
    if l.ff_kind:
        out.update({p + "norm2": (W,), p + "norm2b": (W,)})
    if l.ff_kind == "dense":
        out.update({p + "mlp.gate": (l.ff, W), p + "mlp.up": (l.ff, W), p + "mlp.down": (W, l.ff)})
    elif l.ff_kind == "moe":
        for e in range(l.experts):
            out.update({f"{p}mlp.e{e}.up": (l.ff, W), f"{p}mlp.e{e}.down": (W, l.ff)})
        out[p + "mlp.router"] = (l.experts, W)
        if l.shared_ff:
            out.update({p + "mlp.shared.up": (l.shared_ff, W), p + "mlp.shared.down": (W, l.shared_ff)})
    return out


def init_weights(spec: LayeredSpec, seed: int = 0, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Deterministic random bf16 tensors under the checkpoint's names: projections ~ N(0, 1/fan_in), gains near 1, decay
    parameters in the range where the recurrence neither forgets at once nor never."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    w = {}
    sandwich = bool(spec.layers) and spec.layers[-1].form == "sandwich"
    postnorm = bool(spec.layers) and spec.layers[-1].form == "postnorm"
    hyper = bool(spec.layers) and spec.layers[-1].form == "hyper"
    for name, shape in tensor_shapes(spec).items():
        leaf = name.split(".")[-1]
        part = name.split(".")[-2] if "." in name else ""
        if hyper and part in ("hc1", "hc2"):
            n = shape[0]
            if leaf == "mix":                                    # mostly each stream to itself
                t = torch.eye(n) * 0.8 + 0.2 / n + 0.1 * torch.randn(shape, generator=g)
            elif leaf == "in":
                t = 1.0 / n + 0.2 * torch.randn(shape, generator=g)
            else:
                t = 0.7 + 0.3 * torch.randn(shape, generator=g)
        elif hyper and leaf == "b" and part in ("norm1", "norm2", "norm", "conv", "dt"):
            t = 0.1 * torch.randn(shape, generator=g) - (2.0 if part == "dt" else 0.0)
        elif hyper and (leaf in ("norm1", "norm2", "out") or (leaf == "norm" and part in ("final", "q", "k"))):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif hyper and leaf == "D":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif postnorm and leaf in ("canon1", "canon2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif postnorm and leaf == "dwa":
            t = 0.15 * torch.randn(shape, generator=g)
            t[-1] += 1.0                                         # mostly the layer's own result
        elif postnorm and leaf in ("rel", "sink"):
            t = torch.randn(shape, generator=g)
        elif postnorm and leaf == "vmix":
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
        elif postnorm and leaf == "b" and name.split(".")[-2] in ("q", "k", "v", "o"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif sandwich and (leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm"):
            t = 0.2 * torch.randn(shape, generator=g)          # stored as gain - 1
        elif sandwich and leaf == "b":
            t = 0.5 * torch.randn(shape, generator=g)
            if name.endswith("f.b"):
                t = t + 3.0                                      # forget gates that mostly keep
        elif sandwich and leaf == "D":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("norm1") or name == "final.norm" or name.endswith(".norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.5 + 2.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) - 2.0
        elif leaf == "b" and name.split(".")[-2] in ("rg1", "rg2"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(device)
    return w


def read_safetensors_header(path: str) -> Dict:
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        return json.loads(f.read(n))


def is_layered_config(cfg: Dict) -> bool:
    return isinstance(cfg.get("layers"), list) and "width" in cfg


def load_checkpoint(path: str, device: str = "cpu", name: Optional[str] = None) -> Tuple[LayeredSpec, Dict[str, torch.Tensor]]:
    """A folder with config.json and model.safetensors -> (spec, tensors by name)."""
    from safetensors.torch import load_file
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    st = os.path.join(path, "model.safetensors")
    shapes = {k: tuple(v["shape"]) for k, v in read_safetensors_header(st).items() if k != "__metadata__"}
    spec = spec_from_config(cfg, shapes, name or os.path.basename(os.path.normpath(path)))
    w = load_file(st, device=device)
    want = tensor_shapes(spec)
    for k, shape in want.items():
        if k not in w:
            raise KeyError(f"checkpoint has no tensor {k!r}")
        if tuple(w[k].shape) != tuple(shape):
            raise ValueError(f"{k}: shape {tuple(w[k].shape)} does not match config ({tuple(shape)})")
    return spec, w


def save_checkpoint(spec: LayeredSpec, w: Dict[str, torch.Tensor], path: str) -> None:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(spec.config(), f, indent=1)
    save_file({k: v.detach().cpu().contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))


# ------------------------------------------------------------------ native side
class BranchDesc(C.Structure):
    """ft_branch_desc (include/fasttalk_b200.h)."""
    _fields_ = [
        ("kind", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int),
        ("out_scale", C.c_float),
        ("o_q", C.c_int), ("o_k", C.c_int), ("o_v", C.c_int), ("o_g", C.c_int), ("o_z", C.c_int), ("o_dt", C.c_int),
        ("o_i", C.c_int), ("o_f", C.c_int),
        ("w_o", C.c_void_p), ("out_norm", C.c_void_p),
        ("scale", C.c_float), ("softcap", C.c_float), ("window", C.c_int), ("rot_dims", C.c_int),
        ("rot_freq", C.c_void_p), ("q_bias", C.c_void_p), ("k_bias", C.c_void_p),
        ("decay", C.c_void_p),
        ("gate_cap", C.c_float), ("gate_bias", C.c_void_p),
        ("conv", C.c_int), ("norm_groups", C.c_int),
        ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("dt_bias", C.c_void_p), ("a_log", C.c_void_p), ("skip", C.c_void_p),
        ("qk_norm", C.c_int), ("keep_first", C.c_int), ("rel_n", C.c_int), ("v_role", C.c_int),
        ("sink", C.c_void_p), ("rel", C.c_void_p), ("v_bias", C.c_void_p), ("o_bias", C.c_void_p), ("v_mix", C.c_void_p),
        ("kv_rank", C.c_int), ("q_rank", C.c_int),
        ("w_uq", C.c_void_p), ("w_uk_t", C.c_void_p), ("w_uv", C.c_void_p), ("q_norm", C.c_void_p), ("kv_norm", C.c_void_p),
        ("rot_half", C.c_int), ("chunked", C.c_int), ("kv_lender", C.c_int), ("rot_mag", C.c_float),
        ("q_gain", C.c_void_p), ("k_gain", C.c_void_p), ("out_gain", C.c_void_p),
        ("dt_rank", C.c_int), ("w_x", C.c_void_p), ("w_dt", C.c_void_p), ("x_rows", C.c_int),
    ]


class LayerDesc(C.Structure):
    """ft_layer_desc (include/fasttalk_b200.h)."""
    _fields_ = [
        ("mixer", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int),
        ("kv_rank", C.c_int), ("scale", C.c_float), ("conv", C.c_int), ("rank_a", C.c_int), ("rank_g", C.c_int),
        ("ff_kind", C.c_int), ("experts", C.c_int), ("top", C.c_int), ("groups", C.c_int), ("keep", C.c_int),
        ("ff", C.c_int), ("n_in", C.c_int),
        ("o_q", C.c_int), ("o_k", C.c_int), ("o_v", C.c_int), ("o_dkv", C.c_int), ("o_gate", C.c_int),
        ("o_beta", C.c_int), ("o_a1", C.c_int), ("o_g1", C.c_int), ("o_rg1", C.c_int), ("o_rg2", C.c_int),
        ("o_router", C.c_int), ("norm_gain", C.c_float),
        ("w_in", C.c_void_p), ("w_o", C.c_void_p), ("rg_bias", C.c_void_p),
        ("w_uk_t", C.c_void_p), ("w_uv", C.c_void_p), ("dkv_norm", C.c_void_p),
        ("conv_w", C.c_void_p), ("w_a2", C.c_void_p), ("w_g2", C.c_void_p), ("dt_bias", C.c_void_p),
        ("a_log", C.c_void_p), ("out_norm", C.c_void_p),
        ("w_gu", C.c_void_p), ("w_down", C.c_void_p),
        ("form", C.c_int), ("n_branches", C.c_int), ("branch", BranchDesc * 2),
        ("norm_pre1", C.c_void_p), ("norm_post1", C.c_void_p), ("norm_pre2", C.c_void_p), ("norm_post2", C.c_void_p),
        ("ff_act", C.c_int), ("route_kind", C.c_int), ("route_norm", C.c_int), ("route_scale", C.c_float),
        ("w_router", C.c_void_p), ("router_rows", C.c_int), ("shared_ff", C.c_int), ("w_shared_up", C.c_void_p), ("w_shared_down", C.c_void_p),
        ("canon_taps", C.c_int), ("canon1", C.c_void_p), ("canon2", C.c_void_p), ("depth_w", C.c_void_p), ("gate_act", C.c_int),
        ("norm_pre1_b", C.c_void_p), ("norm_pre2_b", C.c_void_p),
        ("hc_in", C.c_void_p * 2), ("hc_out", C.c_void_p * 2), ("hc_mix", C.c_void_p * 2), ("route_input", C.c_int),
    ]


class LayeredModel(C.Structure):
    """ft_layered_model (include/fasttalk_b200.h)."""
    _fields_ = [
        ("width", C.c_int), ("vocab", C.c_int), ("n_layers", C.c_int),
        ("eps", C.c_float), ("logit_softcap", C.c_float), ("final_norm_gain", C.c_float),
        ("embed", C.c_void_p), ("head", C.c_void_p), ("layers", C.POINTER(LayerDesc)), ("exact_f32", C.c_int),
        ("final_norm_w", C.c_void_p), ("embed_scale", C.c_float), ("final_norm_b", C.c_void_p), ("streams", C.c_int),
    ]


def _stack_inputs(parts: List[Tuple[str, torch.Tensor]], width: int, device) -> Tuple[torch.Tensor, Dict[str, int]]:
    """Projections that read the same input, one under the other; every part starts on a multiple of four rows (the
    kernels read its output columns four at a time) and the whole is a multiple of 128 rows (the tensor-core GEMM's
    tile); the gaps are zero rows."""
    offs, rows = {}, 0
    for name, t in parts:
        rows = (rows + 3) & ~3
        offs[name] = rows
        rows += t.shape[0]
    rows = (rows + 127) & ~127
    out = torch.zeros(rows, width, dtype=torch.bfloat16, device=device)
    for name, t in parts:
        out[offs[name]:offs[name] + t.shape[0]] = t
    return out, offs


def _interleave(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Rows (2j, 2j+1) = (a_j, b_j): the paired layout the SwiGLU epilogue reads."""
    out = torch.empty(2 * a.shape[0], a.shape[1], dtype=a.dtype, device=a.device)
    out[0::2], out[1::2] = a, b
    return out


def _pack_sandwich_layer(l: LayerSpec, w: Dict[str, torch.Tensor], p: str, d, W: int, device, dev, keep: list) -> None:
    """Descriptor of a sandwich layer: its branches' projections stacked into w_in, norm gains as 1 + stored weight."""
    f32 = torch.float32
    d.form, d.mixer, d.n_branches = LAYER_SANDWICH, MIXER_BRANCHES, len(l.branches)
    for f_ in ("o_q", "o_k", "o_v", "o_dkv", "o_gate", "o_beta", "o_a1", "o_g1", "o_rg1", "o_rg2", "o_router"):
        setattr(d, f_, -1)
    d.norm_gain = 1.0
    gain = lambda name: dev(1.0 + w[name].float(), f32).data_ptr()
    d.norm_pre1, d.norm_post1 = gain(p + "norm1"), gain(p + "norm1b")
    parts: List[Tuple[str, torch.Tensor]] = []
    for k, b in enumerate(l.branches):
        m = p + "mix." + b.prefix
        if b.kind == "window_attention":
            parts += [(f"{k}q", w[m + "q"]), (f"{k}k", w[m + "k"])]
        elif b.kind == "decay_attention":      # q | k | v adjacent: one SiLU pass covers them
            parts += [(f"{k}q", torch.cat([w[m + "q"], w[m + "k"], w[m + "v"]], 0)), (f"{k}g", w[m + "g"])]
        elif b.kind == "matrix_memory":
            parts += [(f"{k}q", w[m + "q"]), (f"{k}k", w[m + "k"]), (f"{k}v", w[m + "v"]), (f"{k}g", w[m + "g"]),
                      (f"{k}i", w[m + "i"]), (f"{k}f", w[m + "f"])]
        else:                                   # z | x | B | C | dt as the checkpoint stores them
            parts += [(f"{k}z", w[m + "in"])]
    w_in, offs = _stack_inputs([(n, t.to(device)) for n, t in parts], W, device)
    keep.append(w_in)
    d.w_in, d.n_in = w_in.data_ptr(), w_in.shape[0]
    for k, b in enumerate(l.branches):
        m = p + "mix." + b.prefix
        c = d.branch[k]
        c.kind, c.heads, c.kv_heads, c.dim, c.vdim = BRANCHES[b.kind], b.heads, b.kv_heads or b.heads, b.dim, b.vdim
        c.out_scale = b.out_scale
        for f_ in ("o_q", "o_k", "o_v", "o_g", "o_z", "o_dt", "o_i", "o_f"):
            setattr(c, f_, -1)
        c.w_o = dev(w[m + "o"]).data_ptr()
        hv = b.heads * b.vdim
        if b.kind == "window_attention":
            c.o_q, c.o_k = offs[f"{k}q"], offs[f"{k}k"]
            c.scale, c.softcap, c.window, c.rot_dims = b.scale, b.softcap, b.window, b.rot_dims
            if b.rot_dims:
                i2 = torch.arange(b.rot_dims // 2, dtype=torch.float64)
                c.rot_freq = dev(torch.tensor(b.rot_base, dtype=torch.float64) ** (-2.0 * i2 / b.rot_dims), f32).data_ptr()
            if m + "q.b" in w:
                c.q_bias, c.k_bias = dev(w[m + "q.b"], f32).data_ptr(), dev(w[m + "k.b"], f32).data_ptr()
        elif b.kind == "decay_attention":
            c.o_q = offs[f"{k}q"]
            c.o_k = c.o_q + b.heads * b.dim
            c.o_v = c.o_k + b.heads * b.dim
            c.o_g = offs[f"{k}g"]
            c.decay = dev(torch.tensor(b.decay, dtype=torch.float64), f32).data_ptr()
            c.out_norm = dev(w[m + "norm"], f32).data_ptr()
        elif b.kind == "matrix_memory":
            c.o_q, c.o_k, c.o_v, c.o_g, c.o_i, c.o_f = (offs[f"{k}{x}"] for x in "qkvgif")
            c.gate_cap = b.gate_cap
            c.gate_bias = dev(torch.cat([w[m + "i.b"].float().cpu(), w[m + "f.b"].float().cpu()]), f32).data_ptr()
            c.out_norm = dev(w[m + "norm"], f32).data_ptr()
        else:
            gn = c.kv_heads * b.dim
            c.o_z = offs[f"{k}z"]
            c.o_v = c.o_z + hv
            c.o_k = c.o_v + hv
            c.o_q = c.o_k + gn
            c.o_dt = c.o_q + gn
            c.conv, c.norm_groups = b.conv, b.norm_groups
            c.conv_w = dev(w[m + "conv"], f32).data_ptr()
            c.conv_b = dev(w[m + "conv.b"], f32).data_ptr()
            c.dt_bias = dev(w[m + "dt_bias"], f32).data_ptr()
            c.a_log = dev(w[m + "A_log"], f32).data_ptr()
            c.skip = dev(w[m + "D"], f32).data_ptr()
            c.out_norm = dev(w[m + "norm"], f32).data_ptr()
    d.ff_kind = FF_NONE
    if l.ff_kind:
        d.norm_pre2, d.norm_post2 = gain(p + "norm2"), gain(p + "norm2b")
        d.ff = l.ff
    if l.ff_kind == "dense":
        d.ff_kind, d.ff_act = FF_DENSE, ACT_SWIGLU
        d.w_gu = dev(_interleave(w[p + "mlp.gate"].to(device), w[p + "mlp.up"].to(device))).data_ptr()
        d.w_down = dev(w[p + "mlp.down"]).data_ptr()
    elif l.ff_kind == "moe":
        d.ff_kind, d.ff_act, d.experts, d.top, d.groups, d.keep = FF_MOE, ACT_RELU2, l.experts, l.top, 1, 1
        d.route_kind, d.route_norm, d.route_scale = ROUTE_SIGMOID, 1, l.route_scale
        router = torch.zeros((l.experts + 127) // 128 * 128, W, dtype=torch.bfloat16, device=device)
        router[:l.experts] = w[p + "mlp.router"].to(device)
        d.w_router, d.router_rows = dev(router).data_ptr(), router.shape[0]
        d.w_gu = dev(torch.stack([w[f"{p}mlp.e{e}.up"].to(device) for e in range(l.experts)])).data_ptr()
        d.w_down = dev(torch.stack([w[f"{p}mlp.e{e}.down"].to(device) for e in range(l.experts)])).data_ptr()
        if l.shared_ff:
            d.shared_ff = l.shared_ff
            d.w_shared_up = dev(w[p + "mlp.shared.up"]).data_ptr()
            d.w_shared_down = dev(w[p + "mlp.shared.down"]).data_ptr()


def _pack_hyper_layer(spec: LayeredSpec, i: int, l: LayerSpec, w: Dict[str, torch.Tensor], p: str, d, W: int, device, dev,
                      keep: list) -> None:
    """Descriptor of a hyper-connected layer: layer-norm gains and biases, the stream-mixing tensors, the mixer's projections
    stacked into w_in (q | k | v of an attention side adjacent: their convolution addresses them as one run of channels)."""
    f32 = torch.float32
    m = p + "mix."
    d.form = LAYER_HYPER
    for f_ in ("o_q", "o_k", "o_v", "o_dkv", "o_gate", "o_beta", "o_a1", "o_g1", "o_rg1", "o_rg2", "o_router"):
        setattr(d, f_, -1)
    d.norm_gain = 1.0
    vec = lambda name: dev(w[name], f32).data_ptr()
    d.norm_pre1, d.norm_pre1_b = vec(p + "norm1"), vec(p + "norm1.b")
    for k, h in enumerate(("hc1", "hc2")):
        if spec.streams and (k == 0 or l.ff_kind):
            d.hc_in[k], d.hc_out[k], d.hc_mix[k] = vec(f"{p}{h}.in"), vec(f"{p}{h}.out"), vec(f"{p}{h}.mix")
    if l.mixer == "delta":
        d.mixer, d.heads, d.kv_heads, d.dim, d.vdim, d.conv = MIXER_CHANNEL_DELTA, l.heads, l.kv_heads, l.dim, l.vdim, l.conv
        d.rank_a = d.rank_g = 0
        d.gate_act = 1
        parts = [("q", torch.cat([w[m + "q"], w[m + "k"], w[m + "v"]], 0)), ("beta", w[m + "b"]), ("a1", w[m + "a"]), ("g1", w[m + "g"])]
    else:
        d.mixer, d.n_branches = MIXER_BRANCHES, len(l.branches)
        parts = []
        for k, b in enumerate(l.branches):
            q = m + b.prefix
            if b.kind == "window_attention":
                parts.append((f"{k}q", torch.cat([w[q + "q"]] + ([w[q + "k"], w[q + "v"]] if b.kv_from < 0 else []), 0)))
            else:
                parts.append((f"{k}x", w[q + "in"]))
    w_in, offs = _stack_inputs([(n, t.to(device)) for n, t in parts], W, device)
    keep.append(w_in)
    d.w_in, d.n_in = w_in.data_ptr(), w_in.shape[0]
    if l.mixer == "delta":
        for n, o in offs.items():
            setattr(d, "o_" + n, o)
        d.o_k = d.o_q + l.kv_heads * l.dim
        d.o_v = d.o_k + l.kv_heads * l.dim
        d.w_o = dev(w[m + "o"]).data_ptr()
        d.conv_w = dev(torch.cat([w[m + "q.conv"], w[m + "k.conv"], w[m + "v.conv"]], 0), f32).data_ptr()
        d.dt_bias, d.a_log, d.out_norm = vec(m + "dt_bias"), vec(m + "A_log"), vec(m + "norm")
    for k, b in enumerate(l.branches):
        q, c = m + b.prefix, d.branch[k]
        c.kind, c.heads, c.kv_heads, c.dim, c.vdim = BRANCHES[b.kind], b.heads, b.kv_heads or b.heads, b.dim, b.vdim
        c.out_scale = b.out_scale
        for f_ in ("o_q", "o_k", "o_v", "o_g", "o_z", "o_dt", "o_i", "o_f"):
            setattr(c, f_, -1)
        c.w_o = dev(w[q + "o"]).data_ptr()
        if b.out_norm_width:
            c.out_gain = vec(q + "out")
        if b.kind == "window_attention":
            own = b.kv_from < 0
            c.o_q = offs[f"{k}q"]
            if own:
                c.o_k = c.o_q + b.heads * b.dim
                c.o_v = c.o_k + c.kv_heads * b.dim
            else:
                c.kv_lender = b.kv_from + 1
            c.scale, c.softcap, c.window, c.rot_dims, c.chunked = b.scale, b.softcap, b.window, b.rot_dims, int(b.chunked)
            c.rot_half = int(b.rot_half)
            if b.rot_dims:
                freq, mag = rotary_frequencies(b)
                c.rot_freq, c.rot_mag = dev(torch.tensor(freq, dtype=torch.float64), f32).data_ptr(), mag
            c.qk_norm = (2 if b.qk_gain == "all" else 1) if b.qk_norm else 0
            if b.qk_gain:
                c.q_gain = vec(q + "q.norm")
                if own:
                    c.k_gain = vec(q + "k.norm")
            if b.zero_sink:
                c.sink = dev(torch.zeros(b.heads), f32).data_ptr()
            if b.conv:
                c.conv = b.conv
                c.conv_w = dev(torch.cat([w[q + n + ".conv"] for n in ("qkv" if own else "q")], 0), f32).data_ptr()
        else:
            C_ = b.heads
            c.o_v = offs[f"{k}x"]
            c.o_z = c.o_v + C_
            c.conv, c.dt_rank = b.conv, b.dt_rank
            c.conv_w, c.conv_b = vec(q + "conv"), vec(q + "conv.b")
            # the low-rank projection padded with zero rows to whole tensor-core tiles; the step-size projection reads the whole
            # padded row, its columns beyond dt_rank are zero
            rows = (b.dt_rank + 2 * b.dim + 127) // 128 * 128
            w_x = torch.zeros(rows, C_, dtype=torch.bfloat16, device=device)
            w_x[:b.dt_rank + 2 * b.dim] = w[q + "x"].to(device)
            w_dt = torch.zeros(C_, rows, dtype=torch.bfloat16, device=device)
            w_dt[:, :b.dt_rank] = w[q + "dt"].to(device)
            c.w_x, c.w_dt, c.x_rows = dev(w_x).data_ptr(), dev(w_dt).data_ptr(), rows
            c.dt_bias, c.a_log, c.skip = vec(q + "dt.b"), vec(q + "A_log"), vec(q + "D")
    d.ff_kind = FF_NONE
    if l.ff_kind:
        d.norm_pre2, d.norm_pre2_b = vec(p + "norm2"), vec(p + "norm2.b")
        d.ff, d.ff_act = l.ff, ACT_SWIGLU
    if l.ff_kind == "dense":
        d.ff_kind = FF_DENSE
        d.w_gu = dev(_interleave(w[p + "mlp.gate"].to(device), w[p + "mlp.up"].to(device))).data_ptr()
        d.w_down = dev(w[p + "mlp.down"]).data_ptr()
    elif l.ff_kind == "moe":
        d.ff_kind, d.experts, d.top, d.groups, d.keep = FF_MOE, l.experts, l.top, 1, 1
        d.route_kind, d.route_norm, d.route_scale, d.route_input = ROUTE_SIGMOID, 0, 1.0, 1
        router = torch.zeros((l.experts + 127) // 128 * 128, W, dtype=torch.bfloat16, device=device)
        router[:l.experts] = w[p + "mlp.router"].to(device)
        d.w_router, d.router_rows = dev(router).data_ptr(), router.shape[0]
        gu = torch.stack([_interleave(w[f"{p}mlp.e{e}.gate"].to(device), w[f"{p}mlp.e{e}.up"].to(device)) for e in range(l.experts)])
        d.w_gu = dev(gu).data_ptr()
        d.w_down = dev(torch.stack([w[f"{p}mlp.e{e}.down"].to(device) for e in range(l.experts)])).data_ptr()


def _pack_postnorm_layer(spec: LayeredSpec, i: int, l: LayerSpec, w: Dict[str, torch.Tensor], p: str, d, W: int, device, dev,
                         keep: list, first_mix: int) -> None:
    """Descriptor of a post-norm layer: gains as stored, input convolutions, depth weights, the mixer's projections stacked
    into w_in; the distance-bias table expanded to one row per distance."""
    f32 = torch.float32
    m = p + "mix."
    d.form = LAYER_POSTNORM
    for f_ in ("o_q", "o_k", "o_v", "o_dkv", "o_gate", "o_beta", "o_a1", "o_g1", "o_rg1", "o_rg2", "o_router"):
        setattr(d, f_, -1)
    d.norm_gain = 1.0
    d.norm_post1 = dev(w[p + "norm1"], f32).data_ptr()
    d.canon_taps = spec.canon_taps
    if spec.canon_taps >= 1:
        d.canon1 = dev(w[p + "canon1"], f32).data_ptr()
    d.depth_w = dev(w[p + "dwa"], f32).data_ptr()
    if l.mixer == "delta":
        d.mixer, d.heads, d.kv_heads, d.dim, d.vdim, d.conv = MIXER_CHANNEL_DELTA, l.heads, l.kv_heads, l.dim, l.vdim, l.conv
        d.rank_a = d.rank_g = 0
        d.gate_act = 1
        qkv = torch.cat([w[m + "q"], w[m + "k"], w[m + "v"]], 0)      # adjacent: one run of convolution channels
        parts = [("q", qkv), ("beta", w[m + "b"]), ("a1", w[m + "a"]), ("g1", w[m + "g"])]
    else:
        b = l.branches[0]
        d.mixer, d.n_branches = MIXER_BRANCHES, 1
        parts = [("q", w[m + "q"]), ("k", w[m + "k"]), ("v", w[m + "v"])] if b.kind == "window_attention" else \
                [("q", w[m + "dq"]), ("k", w[m + "dkv"])]
    w_in, offs = _stack_inputs([(n, t.to(device)) for n, t in parts], W, device)
    keep.append(w_in)
    d.w_in, d.n_in = w_in.data_ptr(), w_in.shape[0]
    if l.mixer == "delta":
        for n, o in offs.items():
            setattr(d, "o_" + n, o)
        d.o_k = d.o_q + l.kv_heads * l.dim
        d.o_v = d.o_k + l.kv_heads * l.dim
        d.w_o = dev(w[m + "o"]).data_ptr()
        d.conv_w = dev(torch.cat([w[m + "q.conv"], w[m + "k.conv"], w[m + "v.conv"]], 0), f32).data_ptr()
        d.dt_bias = dev(w[m + "dt_bias"], f32).data_ptr()
        d.a_log = dev(w[m + "A_log"], f32).data_ptr()
        d.out_norm = dev(w[m + "norm"], f32).data_ptr()
    else:
        b, c = l.branches[0], d.branch[0]
        c.kind, c.heads, c.kv_heads, c.dim, c.vdim = BRANCHES[b.kind], b.heads, b.kv_heads or b.heads, b.dim, b.vdim
        c.out_scale = 1.0
        for f_ in ("o_q", "o_k", "o_v", "o_g", "o_z", "o_dt", "o_i", "o_f"):
            setattr(c, f_, -1)
        c.o_q, c.o_k = offs["q"], offs["k"]
        c.w_o = dev(w[m + "o"]).data_ptr()
        c.scale, c.window, c.rot_dims = b.scale, b.window, b.rot_dims
        if b.rot_dims:
            i2 = torch.arange(b.rot_dims // 2, dtype=torch.float64)
            c.rot_freq = dev(torch.tensor(b.rot_base, dtype=torch.float64) ** (-2.0 * i2 / b.rot_dims), f32).data_ptr()
        if b.kind == "window_attention":
            c.o_v = offs["v"]
            c.qk_norm, c.keep_first = int(b.qk_norm), b.keep_first
            if b.biases:
                c.q_bias, c.k_bias = dev(w[m + "q.b"], f32).data_ptr(), dev(w[m + "k.b"], f32).data_ptr()
                c.v_bias, c.o_bias = dev(w[m + "v.b"], f32).data_ptr(), dev(w[m + "o.b"], f32).data_ptr()
            if b.sink:
                c.sink = dev(w[m + "sink"], f32).data_ptr()
            if b.rel_rows:
                rows = distance_rows(b.rel_rows, b.rel_far)
                table = w[m + "rel"].float().cpu()[torch.tensor(rows)]          # [distance][head]
                c.rel, c.rel_n = dev(table, f32).data_ptr(), len(rows)
            if b.v_mix:
                c.v_role = 1 if i == first_mix else 2
                c.v_mix = dev(w[m + "vmix"].reshape(1), f32).data_ptr()
        else:
            c.kv_rank, c.q_rank = b.kv_rank, b.q_rank
            c.w_uq = dev(w[m + "uq"]).data_ptr()
            c.w_uk_t = dev(w[m + "uk"].reshape(b.heads, b.dim, b.kv_rank).transpose(1, 2)).data_ptr()      # [heads][kv_rank][dim]
            c.w_uv = dev(w[m + "uv"]).data_ptr()
            c.q_norm = dev(w[m + "dq.norm"], f32).data_ptr()
            c.kv_norm = dev(w[m + "dkv.norm"], f32).data_ptr()
    d.ff_kind = FF_NONE
    if l.ff_kind == "dense":
        d.ff_kind, d.ff_act, d.ff = FF_DENSE, ACT_SWIGLU, l.ff
        d.norm_post2 = dev(w[p + "norm2"], f32).data_ptr()
        if spec.canon_taps >= 1:
            d.canon2 = dev(w[p + "canon2"], f32).data_ptr()
        d.w_gu = dev(_interleave(w[p + "mlp.gate"].to(device), w[p + "mlp.up"].to(device))).data_ptr()
        d.w_down = dev(w[p + "mlp.down"]).data_ptr()


def pack(spec: LayeredSpec, w: Dict[str, torch.Tensor], device, exact_f32: bool = False) -> Tuple[LayeredModel, list]:
    """Device arrays in the engine's layout + the descriptor structs.  Returns (model, keepalive): the engine borrows
    the pointers, so `keepalive` has to live as long as the engine."""
    keep: list = []
    bf = torch.bfloat16

    def dev(t: torch.Tensor, dtype=bf) -> torch.Tensor:
        t = t.to(device=device, dtype=dtype).contiguous()
        keep.append(t)
        return t

    descs = (LayerDesc * len(spec.layers))()
    W = spec.width
    for i, l in enumerate(spec.layers):
        p, d = f"l{i}.", descs[i]
        m = p + "mix."
        if l.form == "sandwich":
            _pack_sandwich_layer(l, w, p, d, W, device, dev, keep)
            continue
        if l.form == "hyper":
            _pack_hyper_layer(spec, i, l, w, p, d, W, device, dev, keep)
            continue
        if l.form == "postnorm":
            first_mix = next((j for j, x in enumerate(spec.layers) if x.branches and x.branches[0].v_mix), -1)
            _pack_postnorm_layer(spec, i, l, w, p, d, W, device, dev, keep, first_mix)
            continue
        d.mixer, d.heads, d.dim, d.vdim = MIXERS[l.mixer], l.heads, l.dim, l.vdim
        d.norm_gain = float(w[p + "norm1"].float().item())
        for f_ in ("o_q", "o_k", "o_v", "o_dkv", "o_gate", "o_beta", "o_a1", "o_g1", "o_rg1", "o_rg2", "o_router"):
            setattr(d, f_, -1)
        if l.mixer == "latent_attention":
            parts = [("q", w[m + "q"]), ("dkv", w[m + "dkv"]), ("gate", w[m + "g"])]
        else:
            # q | k | v stay adjacent: the convolution kernel addresses them as one run of channels
            qkv = torch.cat([w[m + "q"], w[m + "k"], w[m + "v"]], 0)
            parts = [("q", qkv), ("beta", w[m + "b"]), ("a1", w[m + "a1"]), ("g1", w[m + "g1"])]
        parts.append(("rg1", w[p + "rg1"]))
        if l.ff:
            parts += [("rg2", w[p + "rg2"]), ("router", w[p + "mlp.router"])]
        w_in, offs = _stack_inputs([(n, t.to(device)) for n, t in parts], W, device)
        keep.append(w_in)
        d.w_in, d.n_in = w_in.data_ptr(), w_in.shape[0]
        for n, o in offs.items():
            setattr(d, "o_" + n, o)
        d.w_o = dev(w[m + "o"]).data_ptr()
        bias = [w[p + "rg1.b"].float(), w[p + "rg2.b"].float() if l.ff else torch.zeros(W)]
        d.rg_bias = dev(torch.cat([b.to("cpu") for b in bias]), torch.float32).data_ptr()
        if l.mixer == "latent_attention":
            d.kv_rank, d.scale = l.kv_rank, l.scale
            uk = w[m + "uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2)      # [heads][kv_rank][dim]
            d.w_uk_t = dev(uk).data_ptr()
            d.w_uv = dev(w[m + "uv"]).data_ptr()
            d.dkv_norm = dev(w[m + "dkv.norm"], torch.float32).data_ptr()
        else:
            d.kv_heads, d.conv, d.rank_a, d.rank_g = l.kv_heads, l.conv, l.rank_a, l.rank_g
            d.o_k = d.o_q + l.kv_heads * l.dim
            d.o_v = d.o_k + l.kv_heads * l.dim
            conv = torch.cat([w[m + "q.conv"], w[m + "k.conv"], w[m + "v.conv"]], 0)
            d.conv_w = dev(conv, torch.float32).data_ptr()
            d.w_a2 = dev(w[m + "a2"]).data_ptr()
            d.w_g2 = dev(w[m + "g2"]).data_ptr()
            d.dt_bias = dev(w[m + "dt_bias"], torch.float32).data_ptr()
            d.a_log = dev(w[m + "A_log"], torch.float32).data_ptr()
            d.out_norm = dev(w[m + "norm"], torch.float32).data_ptr()
        if l.ff:
            d.ff_kind, d.experts, d.top, d.groups, d.keep, d.ff = FF_MOE, l.experts, l.top, l.groups, l.keep, l.ff
            gu = torch.empty(l.experts, 2 * l.ff, W, dtype=bf, device=device)
            dn = torch.empty(l.experts, W, l.ff, dtype=bf, device=device)
            for e in range(l.experts):
                gu[e, 0::2] = w[f"{p}mlp.e{e}.gate"].to(device)
                gu[e, 1::2] = w[f"{p}mlp.e{e}.up"].to(device)
                dn[e] = w[f"{p}mlp.e{e}.down"].to(device)
            keep += [gu, dn]
            d.w_gu, d.w_down = gu.data_ptr(), dn.data_ptr()
        else:
            d.ff_kind = FF_NONE
    model = LayeredModel()
    model.width, model.vocab, model.n_layers = W, spec.vocab, len(spec.layers)
    model.eps, model.logit_softcap = spec.eps, spec.logit_softcap
    postnorm = bool(spec.layers) and spec.layers[0].form == "postnorm"
    hyper = bool(spec.layers) and spec.layers[0].form == "hyper"
    if hyper:                                # a layer norm with gain and bias; the logits come from the embedding table
        model.final_norm_gain = 1.0
        model.final_norm_w = dev(w["final.norm"], torch.float32).data_ptr()
        model.final_norm_b = dev(w["final.norm.b"], torch.float32).data_ptr()
        model.streams = max(spec.streams, 1)
    elif w["final.norm"].dim() == 0:
        model.final_norm_gain = float(w["final.norm"].float().item())
    else:
        model.final_norm_gain = 1.0          # sandwich models store gain - 1, post-norm models the gain itself
        model.final_norm_w = dev(w["final.norm"].float() + (0.0 if postnorm else 1.0), torch.float32).data_ptr()
    model.embed_scale = spec.embed_scale if postnorm or hyper else 1.0
    model.embed = dev(w["embed"]).data_ptr()
    model.head = model.embed if hyper else dev(w["head"]).data_ptr()
    model.layers = C.cast(descs, C.POINTER(LayerDesc))
    model.exact_f32 = int(exact_f32)
    keep.append(descs)
    return model, keep
