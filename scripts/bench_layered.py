"""Prefill and decode throughput of the layered family beside its closest relatives of equal size, random weights.

    python bench.py --design gitozen  [--sizes s,m] [--arms gitozen,llama] [--steps K] [--warmup W]
    python bench.py --design gedelorn [--sizes s,m] [--arms gedelorn,gitozen,llama] [--steps K] [--warmup W]
    python bench.py --design vonedra  [--sizes s,m] [--arms vonedra,gedelorn,gitozen,llama] [--steps K] [--warmup W]
    python bench.py --design lotinex  [--sizes s,m] [--arms lotinex,vonedra,gedelorn,llama] [--steps K] [--warmup W]

For every size all arms get the same width, depth, heads x head size, active feed-forward width (top x expert ff =
Llama's ffn) and vocabulary.  Gedelorn's closest relative in the framework is Gitozen (the same engine path: stacked
input projection, a mixer with paged cache or state slot, experts, one residual-and-norm kernel per joint).  Each arm is driven through Engine.feed (ft_engine_feed: the engine's own batch builder and
forward pass, nothing sampled), timed with CUDA events on the engine's stream; a 512 MB write between timed steps
flushes L2.
  prefill  one fresh session, PREFILL tokens in one step
  decode   DECODE_SESSIONS sessions at context DECODE_CTX, one token each per step
One JSON line: per size and arm tok/s and ms per step; the Llama arm is the comparator, not a baseline of the reference.
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PREFILL = 2048
DECODE_SESSIONS = 16
DECODE_CTX = 1024

# name -> width, layers (mixer order), heads, head size, latent size, experts, top, expert ff, vocab
SIZES = {
    "s": dict(width=1024, order="ladl", heads=8, dim=128, kv_rank=128, experts=8, top=2, ff=512, vocab=16384),
    "m": dict(width=2048, order="ladl", heads=16, dim=128, kv_rank=256, experts=16, top=2, ff=1024, vocab=32768),
}


def gitozen_spec(name, c):
    from fasttalk_llm_microservice_b200.layered import LayeredSpec, LayerSpec
    moe = dict(ff=c["ff"], experts=c["experts"], top=c["top"], groups=4, keep=2)
    layers = []
    for k in c["order"]:
        if k == "l":
            layers.append(LayerSpec(mixer="latent_attention", heads=c["heads"], dim=c["dim"], vdim=c["dim"],
                                    kv_rank=c["kv_rank"], scale=c["dim"] ** -0.5, **moe))
        else:
            layers.append(LayerSpec(mixer="channel_delta", heads=c["heads"], kv_heads=c["heads"], dim=c["dim"], vdim=c["dim"],
                                    conv=4, rank_a=64, rank_g=64, **moe))
    return LayeredSpec(name=f"gitozen-{name}", architecture="Gitozen", width=c["width"], vocab=c["vocab"], eps=1e-6,
                       logit_softcap=30.0, layers=tuple(layers))


def gedelorn_spec(name, c):
    """Four layers: state space + dense, parallel (window attention 512 | decay attention) + experts, matrix memory + dense,
    state space + experts.  Heads x head size as in the other arms; the state space has the usual expansion of two."""
    from fasttalk_llm_microservice_b200.layered import spec_from_config
    W, H, D = c["width"], c["heads"], c["dim"]
    space = {"type": "mamba2", "mixer": {"conv": 4, "groups": 1, "heads": 2 * W // 64, "norm_groups": 1, "state": 128, "vdim": 64}}
    par = {"type": "parallel", "mixer": {
        "left": {"dim": D, "heads": H, "kv_heads": max(1, H // 4), "mask": {"size": 512}, "rot": {"base": 1e6, "dims": D},
                 "scale": D ** -0.5, "softcap": 50.0, "vdim": D},
        "left_scale": 1.0, "right": {"decay": [1.0 - 2.0 ** -(3 + 7 * h / max(1, H - 1)) for h in range(H)], "dim": D, "heads": H,
                                     "vdim": D}, "right_scale": 1.0}}
    mem = {"type": "mlstm", "mixer": {"dim": D, "gate_cap": 15.0, "heads": max(1, H // 2), "vdim": 2 * D}}
    dense = {"ff": c["top"] * c["ff"], "kind": "dense"}
    moe = {"expert": {"ff": c["ff"]}, "kind": "moe", "router": {"experts": c["experts"], "scale": 1.0, "top": c["top"]},
           "shared": {"ff": c["ff"]}}
    layers = [{**space, "mlp": dense}, {**par, "mlp": moe}, {**mem, "mlp": dense}, {**space, "mlp": moe}]
    cfg = {"architecture": "Gedelorn", "layers": layers, "norm": {"eps": 1e-6}, "vocab": c["vocab"], "width": W}
    return spec_from_config(cfg, name=f"gedelorn-{name}")


def vonedra_spec(name, c):
    """Four post-norm layers with a dense feed-forward each: attention (window 512 that keeps the first 4 tokens, a quarter as
    many key heads, 32 distance rows), delta rule, attention, latent window attention (64 rotated coordinates, window 512).
    Heads x head size as in the other arms; input convolutions of 4 taps."""
    from fasttalk_llm_microservice_b200.layered import spec_from_config
    W, H, D = c["width"], c["heads"], c["dim"]
    att = {"type": "attention", "mixer": {"bias_max": 512, "dim": D, "heads": H, "kv_heads": max(1, H // 4),
                                          "mask": {"keep_first": 4, "size": 512}, "scale": D ** -0.5, "v_mix": True, "vdim": D}}
    dlt = {"type": "delta", "mixer": {"conv": 4, "dim": D, "heads": H, "kv_heads": H, "vdim": D}}
    lat = {"type": "latent_attention", "mixer": {"dim": D, "heads": H, "kv_rank": c["kv_rank"], "mask": {"size": 512},
                                                 "q_rank": 2 * c["kv_rank"], "rot": {"base": 1e4, "dims": 64}, "rot_dim": 64,
                                                 "scale": (D + 64) ** -0.5, "vdim": D}}
    dense = {"ff": c["top"] * c["ff"], "kind": "dense"}
    layers = [{**att, "mlp": dense}, {**dlt, "mlp": dense}, {**att, "mlp": dense}, {**lat, "mlp": dense}]
    cfg = {"architecture": "Vonedra", "canon": {"taps": 4}, "embedding": {"scale": 1.0}, "layers": layers, "norm": {"eps": 1e-6},
           "vocab": c["vocab"], "width": W}
    shapes = {"l0.mix.rel": (32, H), "l2.mix.rel": (32, H), "l3.mix.dq": (2 * c["kv_rank"], W)}
    return spec_from_config(cfg, shapes, name=f"vonedra-{name}")


def lotinex_spec(name, c):
    """Four hyper-connected layers over four streams: attention inside runs of 512 positions (a quarter as many key heads, half
    of every head rotated) + dense, delta rule + experts, attention over the first layer's keys and values + dense, parallel
    (window 512 attention with 3-tap convolutions on q, k, v | selective scan of twice the width, 16 states per channel,
    4 taps) + experts.  Heads x head size and the active feed-forward width as in the other arms."""
    from fasttalk_llm_microservice_b200.layered import spec_from_config
    W, H, D = c["width"], c["heads"], c["dim"]
    G = max(1, H // 4)
    att = {"dim": D, "heads": H, "kv_heads": G, "mask": {"size": 512}, "rot": {"base": 1e4, "dims": D // 2}, "scale": D ** -0.5, "vdim": D}
    dlt = {"type": "delta", "mixer": {"conv": 4, "dim": D, "heads": H, "kv_heads": H, "vdim": D}}
    par = {"type": "parallel", "mixer": {
        "left": {"conv": 3, "dim": D, "heads": H, "kv_heads": G, "mask": {"size": 512},
                 "rot": {"base": 1e4, "dims": D // 2, "scaling": {"factor": 8.0, "fast": 32.0, "original": 2048.0, "slow": 1.0}},
                 "scale": D ** -0.5, "softcap": 50.0, "vdim": D},
        "right": {"conv": 4, "dt_rank": W // 16, "inner": 2 * W, "state": 16}}}
    dense = {"ff": c["top"] * c["ff"], "kind": "dense"}
    moe = {"expert": {"ff": c["ff"]}, "kind": "moe", "router": {"experts": c["experts"], "top": c["top"]}}
    layers = [{"type": "attention", "mixer": dict(att), "mlp": dense}, {**dlt, "mlp": moe},
              {"type": "attention", "mixer": {**att, "kv_from": 0}, "mlp": dense}, {**par, "mlp": moe}]
    cfg = {"architecture": "Lotinex", "embedding": {"scale": W ** 0.5}, "layers": layers, "norm": {"eps": 1e-6}, "streams": 4,
           "vocab": c["vocab"], "width": W}
    return spec_from_config(cfg, name=f"lotinex-{name}")


def llama_spec(name, c):
    from fasttalk_llm_microservice_b200.model_spec import ModelSpec
    return ModelSpec(name=f"llama-{name}", hidden=c["width"], ffn=c["top"] * c["ff"], layers=len(c["order"]),
                     n_q_heads=c["heads"], n_kv_heads=max(1, c["heads"] // 4), head_dim=c["dim"], vocab=c["vocab"],
                     tied_embeddings=False)


def measure(eng, vocab, steps, warmup):
    import numpy as np
    import torch
    rng = np.random.default_rng(0)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        flush.zero_()
        torch.cuda.synchronize()
        eng.timer_start()
        fn()
        return eng.timer_stop_ms()

    out = {}
    ms = []
    for i in range(warmup + steps):
        toks = rng.integers(0, vocab, PREFILL).tolist()
        t = timed(lambda: eng.feed([("p", toks, [PREFILL - 1])]))
        eng.close_session("p")
        if i >= warmup:
            ms.append(t)
    out["prefill"] = {"tokens": PREFILL, "ms_per_step": sum(ms) / len(ms), "tok_s": PREFILL * len(ms) / (sum(ms) / 1e3)}
    names = [f"d{i}" for i in range(DECODE_SESSIONS)]
    for n in names:
        eng.feed([(n, rng.integers(0, vocab, DECODE_CTX).tolist(), [])])
    ms = []
    for i in range(warmup + steps):
        entries = [(n, [int(rng.integers(0, vocab))], [0]) for n in names]
        t = timed(lambda: eng.feed(entries))
        if i >= warmup:
            ms.append(t)
    for n in names:
        eng.close_session(n)
    out["decode"] = {"sessions": DECODE_SESSIONS, "context": DECODE_CTX, "ms_per_step": sum(ms) / len(ms),
                     "tok_s": DECODE_SESSIONS * len(ms) / (sum(ms) / 1e3)}
    return out


def run(args) -> None:
    import torch
    from fasttalk_llm_microservice_b200 import build
    from fasttalk_llm_microservice_b200.engine import Engine, EngineLimits
    from fasttalk_llm_microservice_b200.layered import init_weights as init_layered
    from fasttalk_llm_microservice_b200.weights import init_weights as init_llama
    build.build()
    torch.cuda.set_device(0)
    steps, warmup = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))
    lim = dict(max_batch=DECODE_SESSIONS, max_batched_tokens=PREFILL, max_context=PREFILL + 64, max_sessions=DECODE_SESSIONS + 1,
               num_pages=(DECODE_SESSIONS + 2) * (PREFILL // 64 + 1), debug_logit_rows=DECODE_SESSIONS)
    sizes = {}
    only = [s for s in (getattr(args, "sizes", "") or "s,m").split(",") if s]
    for name in only:
        c = SIZES[name]
        row = {"config": c}
        design = getattr(args, "design", "") or "gitozen"
        default_arms = {"lotinex": "lotinex,vonedra,gedelorn,llama", "vonedra": "vonedra,gedelorn,gitozen,llama",
                        "gedelorn": "gedelorn,gitozen,llama"}.get(design, "gitozen,llama")
        for arm in (getattr(args, "arms", "") or default_arms).split(","):
            if arm in ("gitozen", "gedelorn", "vonedra", "lotinex"):
                spec = {"gitozen": gitozen_spec, "gedelorn": gedelorn_spec, "vonedra": vonedra_spec, "lotinex": lotinex_spec}[arm](name, c)
                w = init_layered(spec, seed=0, device="cuda")
            else:
                spec = llama_spec(name, c)
                w = init_llama(spec, seed=0, device="cuda")
            eng = Engine(spec, w, EngineLimits(**lim), eos_ids=())
            row[arm] = measure(eng, c["vocab"], steps, warmup)
            row[arm]["kernel_launches"] = eng.stats()["kernel_launches"]
            eng.close()
            del eng, w
            torch.cuda.empty_cache()
        sizes[name] = row
    print(json.dumps({"metric": "prefill / decode tok/s of a layered design beside its closest relatives of equal size",
                      "design": getattr(args, "design", "") or "gitozen",
                      "dtype": "bf16 weights; layered family: fp32 activations, bf16 hi+lo planes on the tensor-core projections",
                      "data": "synthetic (random-init weights, random tokens)", "steps": steps, "warmup": warmup,
                      "l2": "512 MB write between timed steps", "sizes": sizes}), flush=True)
