"""The Vonedra design on the GPU against the plain restatement in oracle/vonedra_oracle.py.

Every test builds its own small configuration and random weights (none of them a published model's sizes).  Logits are
compared at EVERY position; the engine keeps this family in fp32 on bf16 weights, so the bound is rounding: 1e-4 of the
largest logit in the exact form, a few times that when projections run on the tensor cores from bf16 hi + lo planes.
"""
import copy
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import vonedra_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4


# ------------------------------------------------------------------------------------------------ configurations
def attention(heads=6, kv_heads=2, dim=16, vdim=12, size=19, keep_first=3, scale=0.3, bias_max=40, v_mix=True, rows=10):
    return {"type": "attention", "_rows": rows,
            "mixer": {"bias_max": bias_max, "dim": dim, "heads": heads, "kv_heads": kv_heads,
                      "mask": {"keep_first": keep_first, "size": size}, "scale": scale, "v_mix": v_mix, "vdim": vdim}}


def latent(heads=3, dim=12, rot=8, vdim=20, kv_rank=24, q_rank=28, size=23, base=5000.0, scale=0.2):
    return {"type": "latent_attention",
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": size}, "q_rank": q_rank,
                      "rot": {"base": base, "dims": rot}, "rot_dim": rot, "scale": scale, "vdim": vdim}}


def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=4):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}}


def dense(ff=72):
    return {"ff": ff, "kind": "dense"}


def layer(mixer, mlp=None):
    return {**copy.deepcopy(mixer), "mlp": mlp}


def make(layers, width=80, vocab=150, eps=1e-5, seed=0, taps=3, embed_scale=0.7, tweak=None):
    from fasttalk_llm_microservice_b200.layered import init_weights, spec_from_config, tensor_shapes
    layers = copy.deepcopy(layers)
    shapes = {}
    for i, l in enumerate(layers):
        rows = l.pop("_rows", None)
        if rows:
            shapes[f"l{i}.mix.rel"] = (rows, l["mixer"]["heads"])
        if l["type"] == "latent_attention":
            shapes[f"l{i}.mix.dq"] = (l["mixer"]["q_rank"], width)
    cfg = {"architecture": "Vonedra", "canon": {"taps": taps}, "embedding": {"scale": embed_scale}, "layers": layers,
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    spec = spec_from_config(cfg, shapes, name="test")
    assert spec.config() == cfg
    assert spec_from_config(spec.config(), tensor_shapes(spec), name="test") == spec
    w = init_weights(spec, seed=seed)
    if tweak:
        tweak(w)
    return spec, w


def engine(spec, w, **kw):
    from fasttalk_llm_microservice_b200 import build
    from fasttalk_llm_microservice_b200.engine import Engine, EngineLimits
    build.build()
    lim = EngineLimits(**{"max_batch": 4, "max_batched_tokens": 512, "max_context": 512, "num_pages": 16,
                          "max_sessions": 4, "debug_logit_rows": 512, "exact_f32": True, **kw})
    return Engine(spec, w, lim, eos_ids=())


def oracle_logits(spec, w, tokens, cfg=None):
    with torch.no_grad():
        return O.forward(cfg or spec.config(), w, list(tokens)).numpy()


def rel(got, ref):
    return float(np.abs(got - ref).max() / np.abs(ref).max())


def tokens_of(spec, n, seed):
    return np.random.default_rng(seed).integers(0, spec.vocab, n).tolist()


def feed_cut(eng, sid, toks, cuts):
    """Feed `toks` to session `sid` in portions of the given sizes (the last size repeats); logits of every position."""
    out, pos, k = [], 0, 0
    while pos < len(toks):
        n = min(cuts[min(k, len(cuts) - 1)], len(toks) - pos)
        out.append(eng.feed([(sid, toks[pos:pos + n], list(range(n)))]))
        pos, k = pos + n, k + 1
    return np.concatenate(out)


MIXED = [layer(attention(), dense()), layer(delta(), dense(ff=40)), layer(attention(size=30, keep_first=0, rows=7, bias_max=25)),
         layer(latent(), dense(ff=33)), layer(delta(heads=2, kv_heads=2, dim=20, vdim=16, conv=2), dense()),
         layer(attention(v_mix=False, heads=4, kv_heads=4, dim=8, vdim=8, size=9, keep_first=11))]


# ------------------------------------------------------------------------------------------------ every mechanism alone
@pytest.mark.parametrize("layers", [
    [layer(attention())],
    [layer(attention(heads=4, kv_heads=4, dim=10, vdim=6, size=1, keep_first=0, rows=4, bias_max=3))],      # sees itself only
    [layer(attention(heads=3, kv_heads=1, dim=36, vdim=8, size=400, keep_first=5))],      # a window longer than the sequence
    [layer(attention(heads=2, kv_heads=1, dim=7, vdim=9, size=12, keep_first=40, rows=5))],      # kept tokens beyond the window, odd head sizes
    [layer(attention(heads=1, kv_heads=1, dim=160, vdim=264, size=50, scale=0.08, rows=31, bias_max=200))],
    [layer(attention(v_mix=False), dense()), layer(attention(size=7)), layer(attention(size=40, keep_first=1))],      # the second layer is the first that mixes
    [layer(latent())],
    [layer(latent(heads=1, dim=6, rot=2, vdim=5, kv_rank=9, q_rank=3, size=4))],                 # nothing a multiple of four
    [layer(latent(heads=5, dim=20, rot=16, vdim=12, kv_rank=64, q_rank=64, size=300, base=1e6, scale=0.1))],
    [layer(latent(heads=2, dim=8, rot=4, vdim=8, kv_rank=300, q_rank=16, size=33))],             # a latent wider than the tiled kernel takes
    [layer(delta())],
    [layer(delta(heads=1, kv_heads=1, dim=40, vdim=8, conv=1))],
    [layer(delta(heads=6, kv_heads=2, dim=72, vdim=33, conv=7))],
    [layer(delta(), dense())],
    MIXED,
], ids=["attention", "attention-self", "attention-long-window", "attention-kept-far", "attention-wide-head", "attention-late-mix",
        "latent", "latent-odd", "latent-wide", "latent-widest", "delta", "delta-1head-1tap", "delta-wide", "dense", "mixed"])
def test_whole_prompt_matches_oracle(layers):
    spec, w = make(layers, seed=3)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 150, 1)
        got = eng.feed([("s", toks, list(range(len(toks))))])
        assert rel(got, oracle_logits(spec, w, toks)) < TOL
    finally:
        eng.close()


@pytest.mark.parametrize("taps", [1, 2, 6])
def test_other_sizes_and_taps(taps):
    layers = [layer(attention(heads=10, kv_heads=5, dim=12, vdim=14, size=33, keep_first=2, scale=0.5, rows=12, bias_max=17.5), dense(ff=50)),
              layer(latent(heads=7, dim=4, rot=6, vdim=6, kv_rank=10, q_rank=5, size=8, base=77.0)),
              layer(delta(heads=9, kv_heads=3, dim=6, vdim=14, conv=5), dense(ff=10))]
    spec, w = make(layers, width=70, vocab=333, eps=1e-6, seed=9, taps=taps, embed_scale=1.0)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 90, 2)
        ref = oracle_logits(spec, w, toks)
        assert rel(eng.feed([("s", toks, list(range(len(toks))))]), ref) < TOL
        assert rel(feed_cut(eng, "c", toks, [1, 2, 1, 7, 1]), ref) < TOL
    finally:
        eng.close()


def test_residual_after_every_layer():
    spec, w = make(MIXED, seed=4)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 70, 5)
        eng.debug_trail(True)
        eng.feed([("s", toks, [])])
        got = eng.read_trail(len(toks))
        trail = []
        with torch.no_grad():
            O.forward(spec.config(), w, toks, trail=trail)
        for i, t in enumerate(trail):
            assert rel(got[i], t.numpy()) < TOL, i
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ portions, decoding
@pytest.mark.parametrize("cuts", [[1], [2], [3, 2, 29, 1, 1, 17, 2], [64], [63, 1, 1, 64, 2], [65, 2]],
                         ids=["token-by-token", "twos", "ragged", "pages", "around-pages", "over-a-page"])
def test_portions_and_decoding_match_the_whole_prompt(cuts):
    spec, w = make(MIXED, seed=7)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 200, 8)
        ref = oracle_logits(spec, w, toks)
        whole = eng.feed([("w", toks, list(range(len(toks))))])
        got = feed_cut(eng, "c", toks, cuts)
        assert rel(whole, ref) < TOL and rel(got, ref) < TOL
        assert rel(got, whole) < 2e-5
    finally:
        eng.close()


EDGE_CUTS = [130] + [1] * 30 + [60, 1]


@pytest.mark.parametrize("size", [2, 5, 63, 64, 65, 129, 1000])
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_window_edges_with_sharp_attention(kind, size):
    """Windows shorter than, equal to and longer than a page, and longer than the sequence; prompt portions and single
    decoded tokens both cross every edge.  A large score scale rests the softmax on one or two keys, so a key that is wrongly
    seen or wrongly hidden moves the result by far more than rounding."""
    if kind == "attention":
        layers = [layer(attention(heads=4, kv_heads=2, dim=16, vdim=16, size=size, keep_first=0, scale=4.0))]
    else:
        layers = [layer(latent(heads=4, dim=16, rot=8, vdim=12, kv_rank=20, q_rank=16, size=size, scale=2.5))]
    spec, w = make(layers, width=64, seed=11)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 260, 12)
        ref = oracle_logits(spec, w, toks)
        assert rel(feed_cut(eng, "a", toks, EDGE_CUTS), ref) < TOL
        cfg = spec.config()                    # the test has teeth: a window one longer gives another result
        cfg["layers"][0]["mixer"]["mask"]["size"] = size + 1
        if size < 260:
            assert rel(oracle_logits(spec, w, toks, cfg), ref) > 50 * TOL
    finally:
        eng.close()


@pytest.mark.parametrize("keep", [1, 2, 63, 64, 65, 130])
def test_kept_first_tokens_with_sharp_attention(keep):
    """The first `keep` positions stay visible from anywhere, across pages, at their true distances; the next one does not."""
    layers = [layer(attention(heads=4, kv_heads=1, dim=16, vdim=16, size=6, keep_first=keep, scale=4.0, rows=16, bias_max=100))]
    spec, w = make(layers, width=64, seed=15)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 260, 16)
        ref = oracle_logits(spec, w, toks)
        assert rel(feed_cut(eng, "a", toks, EDGE_CUTS), ref) < TOL
        assert rel(feed_cut(eng, "b", toks, [keep + 3, 2, 1, 64, 1]), ref) < TOL
        for other in (keep + 1, keep - 1):
            cfg = spec.config()
            cfg["layers"][0]["mixer"]["mask"]["keep_first"] = other
            assert rel(oracle_logits(spec, w, toks, cfg)[200:], ref[200:]) > 50 * TOL
    finally:
        eng.close()


def test_one_far_key_among_hundreds_and_the_edge_of_the_window():
    """One marked token in a run of equal tokens whose key every query prefers: while it is visible it takes all the weight.
    Inside the kept first tokens it is seen from hundreds of positions away; elsewhere the logits change exactly when it
    leaves the window, in a prompt and in decoding."""
    size, keep = 37, 4

    def tweak(w):
        # queries and keys of equal tokens are equal unit vectors; the marked token's key is the same direction on one more
        # coordinate pair, so after the unit-RMS norm its score differs; the scale makes that difference decide
        for n in ("l0.canon1", "l0.mix.rel", "l0.mix.sink", "l0.mix.q.b", "l0.mix.k.b"):
            w[n][:] = 0
        w["l0.mix.sink"][:] = -30.0
        w["embed"][:] = 0
        w["embed"][0, 0], w["embed"][1, 1], w["embed"][0, 2], w["embed"][1, 3] = 1.0, 1.0, 0.5, -0.5
        for n in ("l0.mix.q", "l0.mix.k"):
            w[n][:] = 0
        w["l0.mix.q"][0, 0] = w["l0.mix.q"][8, 0] = 1.0          # both heads' queries of token 0: channel 0 and, weaker, 1
        w["l0.mix.q"][1, 0] = w["l0.mix.q"][9, 0] = 3.0
        w["l0.mix.k"][0, 0] = 1.0                                  # token 0's key: channel 0; token 1's: channel 1
        w["l0.mix.k"][1, 1] = 1.0
    layers = [layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, size=size, keep_first=keep, scale=30.0, v_mix=False))]
    spec, w = make(layers, width=32, vocab=40, seed=2, tweak=tweak, embed_scale=1.0)
    eng = engine(spec, w)
    try:
        for mark in (70, 2):
            toks = [0] * 300
            toks[mark] = 1
            ref = oracle_logits(spec, w, toks)
            plain = oracle_logits(spec, w, [0] * 300)
            if mark >= keep:
                assert np.abs(ref[mark + size - 1] - plain[mark + size - 1]).max() > 1e-2 * np.abs(ref).max()      # still seen
                assert np.abs(ref[mark + size] - plain[mark + size]).max() < 1e-9                                # gone
            else:
                assert np.abs(ref[299] - plain[299]).max() > 1e-2 * np.abs(ref).max()                              # seen from afar
            for cuts in ([300], [mark + size - 1, 1, 1, 1, 150, 1], [mark + 3, 1], [64, 2, 2]):
                got = feed_cut(eng, "s", toks, cuts)
                eng.close_session("s")
                assert rel(got, ref) < TOL, (mark, cuts)
    finally:
        eng.close()


def test_sink_and_distance_bias_matter():
    """Large sinks and a steep distance bias: leaving either out changes the logits by far more than the bound."""
    def tweak(w):
        w["l0.mix.sink"] = (w["l0.mix.sink"].float() + 3.0).to(torch.bfloat16)
        w["l0.mix.rel"] = (w["l0.mix.rel"].float() * 3.0).to(torch.bfloat16)
    layers = [layer(attention(size=90, keep_first=2, rows=14, bias_max=60))]
    spec, w = make(layers, seed=5, tweak=tweak)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 200, 6)
        ref = oracle_logits(spec, w, toks)
        assert rel(feed_cut(eng, "a", toks, [100, 1, 1, 1, 50, 1]), ref) < TOL
        no_sink = dict(w)
        no_sink["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)
        flat = dict(w)
        flat["l0.mix.rel"] = torch.zeros_like(w["l0.mix.rel"])
        assert rel(oracle_logits(spec, no_sink, toks), ref) > 50 * TOL and rel(oracle_logits(spec, flat, toks), ref) > 50 * TOL
        shifted = spec.config()                 # every bucket border matters: another far distance moves them
        shifted["layers"][0]["mixer"]["bias_max"] = 61
        assert rel(oracle_logits(spec, w, toks, shifted), ref) > 50 * TOL
    finally:
        eng.close()


def test_delta_rule_remembers_a_far_write():
    """Slow decays (small step sizes): one marked token early in the sequence still shows 300 tokens later, across portions
    and decoded tokens; the attention layer beside it cannot see that far."""
    def tweak(w):
        for k in list(w):
            if k.endswith("dt_bias"):
                w[k] = (w[k].float() - 6.0).to(torch.bfloat16)
    layers = [layer(attention(size=4, keep_first=0)), layer(delta(), dense())]
    spec, w = make(layers, seed=29, tweak=tweak)
    eng = engine(spec, w)
    try:
        toks = [3] * 340
        toks[5] = 77
        ref = oracle_logits(spec, w, toks)
        other = list(toks)
        other[5] = 78
        assert rel(oracle_logits(spec, w, other)[330:], ref[330:]) > 20 * TOL      # the write is still felt at the end
        got = feed_cut(eng, "a", toks, [40, 2, 100, 1, 1, 1, 150, 1])
        assert rel(got, ref) < TOL and rel(got[330:], ref[330:]) < TOL
    finally:
        eng.close()


def test_first_tokens_and_long_decoding():
    spec, w = make(MIXED, seed=19)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 300, 21)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [1, 1, 1, 2, 1, 30, 1])      # a sequence that starts with single tokens, then 264 decoded
        assert rel(got[:8], ref[:8]) < TOL
        assert rel(got, ref) < TOL
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ batches, pools
def test_unequal_requests_in_one_batch_match_each_alone():
    spec, w = make(MIXED, seed=13)
    eng = engine(spec, w)
    try:
        seqs = {n: tokens_of(spec, ln, 20 + i) for i, (n, ln) in enumerate([("a", 140), ("b", 33), ("c", 70), ("d", 9)])}
        ref = {n: oracle_logits(spec, w, t) for n, t in seqs.items()}
        alone = {}
        for n, t in seqs.items():
            alone[n] = eng.feed([(n + "-alone", t, list(range(len(t))))])
            eng.close_session(n + "-alone")
        # a schedule of mixed steps: portions of some beside single tokens of others, one request pausing for a step
        plan = [{"a": 64, "b": 1}, {"a": 2, "b": 1, "c": 29}, {"b": 16, "c": 1, "d": 3}, {"a": 1, "c": 1, "d": 1},
                {"a": 70, "b": 15, "c": 39, "d": 5}, {"a": 3}]
        at = {n: 0 for n in seqs}
        got = {n: [] for n in seqs}
        for step in plan:
            entries, names = [], []
            for n, cnt in step.items():
                cnt = min(cnt, len(seqs[n]) - at[n])
                if cnt:
                    entries.append((n, seqs[n][at[n]:at[n] + cnt], list(range(cnt))))
                    names.append((n, cnt))
            out = eng.feed(entries)
            o = 0
            for n, cnt in names:
                got[n].append(out[o:o + cnt])
                o += cnt
                at[n] += cnt
        for n in seqs:
            assert at[n] == len(seqs[n])
            g = np.concatenate(got[n])
            assert rel(g, ref[n]) < TOL, n
            assert rel(g, alone[n]) < 2e-5, n
    finally:
        eng.close()


def test_pages_and_state_slots_are_used_again():
    """A pool of 6 pages and 2 slots serves 6 sequences one after the other and two at a time: what an ended session
    left in its pages and its slot (states, convolution tails of the mixers and of every sublayer's input) must not reach
    the next one."""
    spec, w = make(MIXED, seed=17)
    eng = engine(spec, w, max_batch=2, max_sessions=2, num_pages=6, max_context=384, max_batched_tokens=384,
                 debug_logit_rows=384)
    try:
        seqs = [tokens_of(spec, ln, 40 + i) for i, ln in enumerate([190, 100, 130, 64, 65, 180])]
        ref = [oracle_logits(spec, w, t) for t in seqs]
        for i in (0, 1):                                       # alone, the whole pool in turn
            assert rel(feed_cut(eng, f"s{i}", seqs[i], [50, 1, 1, 90]), ref[i]) < TOL
            eng.close_session(f"s{i}")
            assert eng.stats()["free_pages"] == 6
        for a, b in ((2, 3), (4, 5)):                          # two at a time, the shorter one ends first
            la, lb = len(seqs[a]), len(seqs[b])
            ga, gb, pa, pb = [], [], 0, 0
            while pa < la or pb < lb:
                entries = []
                na, nb = min(37, la - pa), min(1 if pb else 20, lb - pb)
                if na:
                    entries.append((f"s{a}", seqs[a][pa:pa + na], list(range(na))))
                if nb:
                    entries.append((f"s{b}", seqs[b][pb:pb + nb], list(range(nb))))
                out = eng.feed(entries)
                ga.append(out[:na]); gb.append(out[na:na + nb])
                pa, pb = pa + na, pb + nb
                if pa == la and na:
                    eng.close_session(f"s{a}")
                if pb == lb and nb:
                    eng.close_session(f"s{b}")
            assert rel(np.concatenate(ga), ref[a]) < TOL and rel(np.concatenate(gb), ref[b]) < TOL
        st = eng.stats()
        assert st["free_pages"] == 6 and st["live_sessions"] == 0
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ tensor cores
TILING = [layer(attention(heads=8, kv_heads=2, dim=16, vdim=16, size=50, keep_first=4), dense(ff=64)),
          layer(latent(heads=4, dim=16, rot=16, vdim=32, kv_rank=64, q_rank=64, size=40), dense(ff=128)),
          layer(delta(heads=2, kv_heads=1, dim=16, vdim=64, conv=3), dense(ff=100))]


@pytest.mark.parametrize("exact", [False, True], ids=["tensor-cores", "exact-fp32"])
def test_projections_on_tensor_cores_and_in_exact_fp32(exact):
    """Shapes that tile (width, heads * vdim, the latent sizes and the feed-forward sizes multiples of 64 or 128): with enough
    rows the input and output projections, the query expansion and the dense feed-forward run on the tensor cores from bf16
    hi + lo planes unless the engine was made exact; single tokens and short portions take the CUDA-core kernels either way, so
    the two forms must agree along one sequence.  The last layer's feed-forward (100) does not tile."""
    spec, w = make(TILING, width=128, vocab=256, seed=37)
    eng = engine(spec, w, exact_f32=exact)
    try:
        toks = tokens_of(spec, 200, 38)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [150, 1, 1, 12, 3, 10, 1])
        assert rel(got, ref) < (TOL if exact else 4e-4)
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ the serving path
def test_greedy_generation_through_the_scheduler():
    """Engine.generate: submit -> the scheduler's own chunked prefill and decode steps -> argmax sampling; three requests
    of unequal length run together, prompts longer than a step's token budget are cut by the scheduler itself."""
    spec, w = make(MIXED, seed=23)
    eng = engine(spec, w, max_batched_tokens=48, decode_prefill_cap=16)
    try:
        prompts = [tokens_of(spec, ln, 60 + i) for i, ln in enumerate([100, 7, 51])]
        n_new = 12
        got = eng.generate(prompts, n_new, temperature=0.0, ignore_eos=True)
        with torch.no_grad():
            for p, g in zip(prompts, got):
                assert g == O.greedy(spec.config(), w, p, n_new)
        # a conversation that continues keeps its state; one that diverges is rebuilt from its start
        eng.close()
        eng = engine(spec, w, max_batched_tokens=48, decode_prefill_cap=16)
        first = eng.generate([prompts[1]], 5, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0]
        more = prompts[1] + first + tokens_of(spec, 6, 99)
        with torch.no_grad():
            assert eng.generate([more], 4, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0] == O.greedy(spec.config(), w, more, 4)
            other = tokens_of(spec, 11, 98)
            assert eng.generate([other], 3, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0] == O.greedy(spec.config(), w, other, 3)
    finally:
        eng.close()


def test_sampling_with_temperature_runs():
    spec, w = make(MIXED, seed=25)
    eng = engine(spec, w)
    try:
        out = eng.generate([tokens_of(spec, 20, 1), tokens_of(spec, 5, 2)], 8, temperature=0.8, top_k=20, top_p=0.9,
                           ignore_eos=True)
        assert [len(o) for o in out] == [8, 8] and all(0 <= t < spec.vocab for o in out for t in o)
    finally:
        eng.close()


def test_trace_runner_replays_a_schedule(tmp_path):
    """bin/trace_run on a saved checkpoint: three steps, a session pausing and two ending, in both number formats."""
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make(MIXED, seed=31)
    save_checkpoint(spec, w, str(tmp_path / "model"))
    toks = tokens_of(spec, 40, 3)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[31:], "want": [8]}, {"id": "y", "tokens": toks[:5], "want": [4]}],
              "end": ["x", "y"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / ("out-" + dtype)
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        ref = oracle_logits(spec, w, toks)
        a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, spec.vocab)
        c = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, spec.vocab)
        assert not (out / "1.f32").exists()
        tol = TOL if dtype == "float32" else 4e-4
        assert rel(a, ref[[0, 29]]) < tol and rel(c[0], ref[39]) < tol and rel(c[1], ref[4]) < tol


def test_served_through_the_handler(tmp_path, monkeypatch):
    """A Vonedra checkpoint behind the serving path: FASTTALK_CHECKPOINT -> registry -> engine -> NativeHandler streams text."""
    from fasttalk_llm_microservice_b200.handler import NativeHandler, build_runner
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make([layer(attention(), dense()), layer(delta(), dense()), layer(latent())], width=64, vocab=600, seed=41)
    save_checkpoint(spec, w, str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_CHECKPOINT", str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_ALLOW_BYTE_TOKENIZER", "1")
    monkeypatch.setenv("FASTTALK_MAX_SESSIONS", "4")
    monkeypatch.setenv("FASTTALK_MAX_CONTEXT", "512")
    monkeypatch.setenv("FASTTALK_MAX_BATCHED_TOKENS", "256")
    runner = build_runner("vonedra-test")
    h = NativeHandler(model="vonedra-test", runner=runner)
    try:
        assert h.check_connection()
        chunks = list(h.generate_stream([{"role": "user", "content": "hello there"}], temperature=0.0, max_tokens=12,
                                        request_id="conv-1"))
        assert 1 <= len(chunks) <= 12
        st = h.runner.engine.stats()
        assert st["prefill_tokens"] > 0 and st["decode_tokens"] > 0
    finally:
        h.close()
        runner.shutdown()
        runner.engine.close()
