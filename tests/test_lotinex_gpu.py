"""The Lotinex design on the GPU against the plain restatement in oracle/lotinex_oracle.py.

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

from oracle import lotinex_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4


# ------------------------------------------------------------------------------------------------ configurations
def attention(heads=6, kv_heads=2, dim=16, vdim=12, size=19, scale=0.3, rot=8, base=3000.0, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def left_side(heads=4, kv_heads=2, dim=12, vdim=20, size=23, scale=0.25, rot=6, base=700.0, conv=3, softcap=15.0,
              scaling=(6.0, 48.0, 8.0, 1.5)):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": size}, "scale": scale, "vdim": vdim}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if softcap:
        m["softcap"] = softcap
    if conv:
        m["conv"] = conv
    return m


def parallel(left=None, inner=48, state=10, dt_rank=7, conv=3):
    return {"type": "parallel", "mixer": {"left": left or left_side(),
                                          "right": {"conv": conv, "dt_rank": dt_rank, "inner": inner, "state": state}}}


def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=3):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}}


def dense(ff=72):
    return {"ff": ff, "kind": "dense"}


def moe(ff=24, experts=6, top=2):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def layer(mixer, mlp=None):
    return {**copy.deepcopy(mixer), "mlp": mlp}


def make(layers, width=80, vocab=150, eps=1e-5, seed=0, streams=3, embed_scale=4.0, tweak=None):
    from fasttalk_llm_microservice_b200.layered import init_weights, spec_from_config, tensor_shapes
    cfg = {"architecture": "Lotinex", "embedding": {"scale": embed_scale}, "layers": copy.deepcopy(layers), "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if streams:
        cfg["streams"] = streams
    spec = spec_from_config(cfg, None, name="test")
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


MIXED = [layer(delta(), moe()), layer(attention(), dense()), layer(parallel(), moe(ff=16, experts=4, top=3)),
         layer(attention(size=30, kv_from=1)), layer(delta(heads=2, kv_heads=2, dim=20, vdim=16, conv=2), dense(ff=40)),
         layer(attention(heads=4, kv_heads=4, dim=8, vdim=8, size=9, rot=8), moe(top=1)),
         layer(attention(heads=4, kv_heads=4, dim=8, vdim=8, size=64, rot=8, kv_from=5), dense(ff=33))]


# ------------------------------------------------------------------------------------------------ every mechanism alone
@pytest.mark.parametrize("layers", [
    [layer(attention())],
    [layer(attention(heads=4, kv_heads=4, dim=10, vdim=6, size=1, rot=10))],                 # every position sees itself only
    [layer(attention(heads=3, kv_heads=1, dim=36, vdim=8, size=400, rot=0))],                # a run longer than the sequence, no rotation
    [layer(attention(heads=2, kv_heads=1, dim=7, vdim=9, size=12, rot=2))],                  # odd head sizes
    [layer(attention(heads=1, kv_heads=1, dim=160, vdim=264, size=50, scale=0.08, rot=96))],
    [layer(attention(size=0))],                                                              # no mask: every earlier position
    [layer(attention(), dense()), layer(delta()), layer(attention(size=7, kv_from=0)), layer(attention(size=40, kv_from=0))],
    [layer(parallel())],
    [layer(parallel(left_side(heads=2, kv_heads=2, dim=6, vdim=5, size=4, rot=2, conv=2, softcap=0, scaling=None), inner=9, state=3,
                    dt_rank=2, conv=2))],                                                    # nothing a multiple of four
    [layer(parallel(left_side(heads=8, kv_heads=1, dim=32, vdim=16, size=300, rot=32, conv=5, base=1e5, scaling=(16.0, 20.0, 4.0, 0.25)),
                    inner=130, state=40, dt_rank=16, conv=1))],
    [layer(parallel(left_side(conv=0, rot=0), inner=24, state=70, dt_rank=1, conv=6))],      # no convolution, no rotation on the left
    [layer(parallel(left_side(conv=1)))],                                                    # one tap: a gain per channel
    [layer(delta())],
    [layer(delta(heads=1, kv_heads=1, dim=40, vdim=8, conv=1))],
    [layer(delta(heads=6, kv_heads=2, dim=72, vdim=33, conv=7))],
    [layer(delta(), dense())],
    [layer(delta(), moe())],
    [layer(delta(), moe(ff=7, experts=3, top=3))],                                            # every expert is chosen
    [layer(delta(), moe(ff=20, experts=40, top=1))],
    MIXED,
], ids=["attention", "attention-self", "attention-long-run", "attention-odd", "attention-wide-head", "attention-unmasked",
        "attention-lent-twice", "parallel", "parallel-odd", "parallel-wide", "parallel-no-conv", "parallel-one-tap", "delta",
        "delta-1head-1tap", "delta-wide", "dense", "experts", "experts-all", "experts-many", "mixed"])
def test_whole_prompt_matches_oracle(layers):
    spec, w = make(layers, seed=3)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 150, 1)
        got = eng.feed([("s", toks, list(range(len(toks))))])
        assert rel(got, oracle_logits(spec, w, toks)) < TOL
    finally:
        eng.close()


@pytest.mark.parametrize("streams,width", [(0, 70), (1, 70), (2, 70), (7, 70), (7, 72), (9, 72)])
def test_other_sizes_and_stream_counts(streams, width):
    layers = [layer(attention(heads=10, kv_heads=5, dim=12, vdim=14, size=33, scale=0.5, rot=4, base=77.0), moe(ff=10, experts=7, top=4)),
              layer(parallel(left_side(heads=3, kv_heads=3, dim=10, vdim=6, size=8, rot=10, conv=4), inner=33, state=5, dt_rank=3, conv=5)),
              layer(delta(heads=9, kv_heads=3, dim=6, vdim=14, conv=5), dense(ff=50)),
              layer(attention(heads=10, kv_heads=5, dim=12, vdim=14, size=5, scale=0.5, rot=4, base=77.0, kv_from=0))]
    spec, w = make(layers, width=width, vocab=333, eps=1e-6, seed=9, streams=streams, embed_scale=1.0)
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
@pytest.mark.parametrize("kind", ["runs", "runs-lent", "window"])
def test_mask_edges_with_sharp_attention(kind, size):
    """Runs and windows shorter than, equal to and longer than a page, and longer than the sequence; prompt portions and
    single decoded tokens both cross every edge.  A large score scale rests the softmax on one or two keys, so a key that is
    wrongly seen or wrongly hidden moves the result by far more than rounding."""
    if kind == "runs":
        layers = [layer(attention(heads=4, kv_heads=2, dim=16, vdim=16, size=size, scale=4.0))]
    elif kind == "runs-lent":
        layers = [layer(attention(heads=4, kv_heads=2, dim=16, vdim=16, size=3, scale=1.0)),
                  layer(attention(heads=4, kv_heads=2, dim=16, vdim=16, size=size, scale=4.0, kv_from=0))]
    else:
        layers = [layer(parallel(left_side(heads=4, kv_heads=2, dim=16, vdim=12, size=size, scale=4.0, softcap=50.0), inner=16, state=4))]
    spec, w = make(layers, width=64, seed=11)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 260, 12)
        ref = oracle_logits(spec, w, toks)
        assert rel(feed_cut(eng, "a", toks, EDGE_CUTS), ref) < TOL
        assert rel(feed_cut(eng, "b", toks, [size + 1, 2, 1, 64, 1]), ref) < TOL
        cfg = spec.config()                    # the test has teeth: a mask one longer gives another result
        m = cfg["layers"][-1]["mixer"]
        (m["left"] if kind == "window" else m)["mask"]["size"] = size + 1
        if size < 260:
            assert rel(oracle_logits(spec, w, toks, cfg), ref) > 50 * TOL
    finally:
        eng.close()


def test_one_far_key_among_hundreds_and_the_end_of_its_run():
    """One marked token in a sequence of equal tokens whose key every query prefers: while it is visible it takes all the
    weight.  Marked at the start of a run of 300 positions it is seen from 299 positions away and by nobody in the next run;
    marked just before a run's start it is seen by nobody after it — in a prompt and in decoding."""
    size = 300

    def tweak(w):
        # token 0 lives on coordinates (0, 1) of the stream, token 1 on (2, 3); the layer norm keeps that.  Every query
        # points along channel 0 of its head; token 0's key along channel 1, token 1's along channel 0: only the marked
        # token's key meets the queries, and the scale lets it decide.
        w["embed"][:] = 0
        w["embed"][0, 0], w["embed"][0, 1], w["embed"][1, 2], w["embed"][1, 3] = 1.0, -1.0, 1.0, -1.0
        w["l0.norm1"][:] = 1.0
        w["l0.norm1.b"][:] = 0
        for n in ("l0.mix.q", "l0.mix.k"):
            w[n][:] = 0
        w["l0.mix.q.norm"][:] = 1.0
        w["l0.mix.k.norm"][:] = 1.0
        for h in (0, 8):
            w["l0.mix.q"][h, 0] = w["l0.mix.q"][h, 2] = 1.0
        w["l0.mix.k"][1, 0] = 1.0
        w["l0.mix.k"][0, 2] = 1.0
    layers = [layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, size=size, scale=4.0, rot=0))]
    spec, w = make(layers, width=32, vocab=40, seed=2, tweak=tweak, streams=0, embed_scale=1.0)
    eng = engine(spec, w, max_batched_tokens=704, max_context=704, debug_logit_rows=704)
    try:
        n = 700
        plain = oracle_logits(spec, w, [0] * n)
        for mark in (300, 299, 2):
            toks = [0] * n
            toks[mark] = 1
            ref = oracle_logits(spec, w, toks)
            end = (mark // size + 1) * size                         # first position of the next run
            assert np.abs(ref[end - 1] - plain[end - 1]).max() > 1e-2 * np.abs(ref).max()       # still seen at the run's end
            assert np.abs(ref[end:] - plain[end:]).max() < 1e-9                               # gone in the next run
            for cuts in ([n], [end - 1, 1, 1, 1, 150, 1], [mark + 3, 1], [64, 2, 2]):
                got = feed_cut(eng, "s", toks, cuts)
                eng.close_session("s")
                assert rel(got, ref) < TOL, (mark, cuts)
                assert np.abs(got[end - 1] - plain[end - 1]).max() > 1e-2 * np.abs(ref).max()
    finally:
        eng.close()


def test_sink_cap_stretch_and_lent_keys_matter():
    """Leaving out the zero-score sink, the score cap, the stretched frequencies or the borrowing of keys changes the logits by
    far more than the bound, so the agreement with the restatement says that each of them is computed."""
    layers = [layer(attention(size=40), dense()), layer(parallel(left_side(scale=1.5, softcap=4.0, size=90))),
              layer(attention(size=25, kv_from=0))]
    spec, w = make(layers, seed=5)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 200, 6)
        ref = oracle_logits(spec, w, toks)
        assert rel(feed_cut(eng, "a", toks, [100, 1, 1, 1, 50, 1]), ref) < TOL
        cfg = spec.config()
        cfg["layers"][1]["mixer"]["left"]["softcap"] = 400.0
        assert rel(oracle_logits(spec, w, toks, cfg), ref) > 50 * TOL
        cfg = spec.config()
        del cfg["layers"][1]["mixer"]["left"]["rot"]["scaling"]
        assert rel(oracle_logits(spec, w, toks, cfg), ref) > 50 * TOL
        with torch.no_grad():
            wd = {k: v.double() for k, v in w.items()}
            h = torch.randn(50, spec.width, dtype=torch.float64)
            m = spec.config()["layers"][1]["mixer"]["left"]
            q, k, v = (O.time_conv(h @ wd[f"l1.mix.left.{n}"].T, wd[f"l1.mix.left.{n}.conv"]) for n in "qkv")
            args = (q.reshape(50, 4, 12), k.reshape(50, 2, 12), v.reshape(50, 2, 20), O.visible_window(50, 90), 1.5, 4.0)
            assert (O.attend(*args, zero_sink=True) - O.attend(*args)).abs().max() > 1e-2
        # own keys instead of layer 0's: give layer 2 projections of its own
        own = spec.config()
        del own["layers"][2]["mixer"]["kv_from"]
        from fasttalk_llm_microservice_b200.layered import init_weights, spec_from_config
        w2 = {**init_weights(spec_from_config(own), seed=5), **w}
        assert rel(oracle_logits(spec, w2, toks, own), ref) > 50 * TOL
    finally:
        eng.close()


def test_recurrent_layers_remember_a_far_write():
    """Slow decays (small step sizes): one marked token early in the sequence still shows 300 tokens later, across portions
    and decoded tokens, through the delta rule and through the selective scan; the attention beside them cannot see that far."""
    def tweak(w):
        for k in list(w):
            if k.endswith("dt_bias") or k.endswith("right.A_log"):
                w[k] = (w[k].float() - 5.0).to(torch.bfloat16)
    for layers in ([layer(attention(size=4)), layer(delta(), dense())],
                   [layer(parallel(left_side(size=4), inner=32, state=12, dt_rank=4), dense())]):
        spec, w = make(layers, seed=29, tweak=tweak)
        eng = engine(spec, w)
        try:
            toks = [3] * 340
            toks[5] = 77
            ref = oracle_logits(spec, w, toks)
            other = list(toks)
            other[5] = 78
            assert rel(oracle_logits(spec, w, other)[330:], ref[330:]) > 10 * TOL      # the write is still felt at the end
            got = feed_cut(eng, "a", toks, [40, 2, 100, 1, 1, 1, 150, 1])
            assert rel(got, ref) < TOL and rel(got[330:], ref[330:]) < TOL
        finally:
            eng.close()


@pytest.mark.parametrize("slow", [False, True], ids=["fast-decay", "slow-decay"])
def test_selective_scan_of_long_portions_runs_in_segments(slow):
    """The scan kernel cuts a portion of more than 128 tokens into segments that run side by side and are joined through the
    decay of whole segments.  Portions of two to six segments, from a zero state and from a carried one, beside a second
    request whose rows start off a segment's multiple; state counts that are no power of two and that exceed a warp's lanes."""
    def tweak(w):
        for k in list(w):
            if k.endswith("right.dt.b") or k.endswith("right.A_log"):
                w[k] = (w[k].float() - 4.0).to(torch.bfloat16)
    for inner, state in ((40, 9), (24, 37)):
        spec, w = make([layer(parallel(left_side(size=4), inner=inner, state=state, dt_rank=5), dense(ff=24))], width=48, seed=41,
                       tweak=tweak if slow else None)
        eng = engine(spec, w, max_batched_tokens=1024, max_context=1024, num_pages=32, debug_logit_rows=1024)
        try:
            a, b = tokens_of(spec, 800, 42), tokens_of(spec, 300, 43)
            ra, rb = oracle_logits(spec, w, a), oracle_logits(spec, w, b)
            g1 = eng.feed([("a", a[:130], list(range(130)))])
            g2 = eng.feed([("a", a[130:643], list(range(513))), ("b", b[:140], list(range(140)))])
            g3 = eng.feed([("b", b[140:], list(range(160))), ("a", a[643:], list(range(157)))])
            ga = np.concatenate([g1, g2[:513], g3[160:]])
            gb = np.concatenate([g2[513:], g3[:160]])
            assert rel(ga, ra) < TOL and rel(gb, rb) < TOL
            eng.close_session("a")
            whole = eng.feed([("w", a, list(range(len(a))))])
            assert rel(whole, ra) < TOL and rel(whole, ga) < 2e-5
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
    """A pool of 6 pages and 2 slots serves 6 sequences one after the other and two at a time: what an ended session left in
    its pages and its slot (matrix and scan states, the convolution tails of q, k, v and of the scan's input) must not reach
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
TILING = [layer(attention(heads=8, kv_heads=2, dim=16, vdim=16, size=50), dense(ff=64)),
          layer(parallel(left_side(heads=4, kv_heads=2, dim=16, vdim=32, size=40), inner=128, state=16, dt_rank=8), moe(ff=64, experts=4, top=2)),
          layer(delta(heads=2, kv_heads=1, dim=16, vdim=64, conv=3), dense(ff=100)),
          layer(attention(heads=8, kv_heads=2, dim=16, vdim=16, size=70, kv_from=0), moe(ff=128, experts=2, top=1))]


@pytest.mark.parametrize("exact", [False, True], ids=["tensor-cores", "exact-fp32"])
def test_projections_on_tensor_cores_and_in_exact_fp32(exact):
    """Shapes that tile (width, heads * vdim, the scan's channels and the feed-forward sizes multiples of 64 or 128): with
    enough rows the input and output projections, the dense feed-forward and — from 256 (token, choice) pairs — the experts
    run on the tensor cores from bf16 hi + lo planes unless the engine was made exact; single tokens and short portions take
    the CUDA-core kernels either way, so the two forms must agree along one sequence."""
    spec, w = make(TILING, width=128, vocab=256, seed=37)
    eng = engine(spec, w, exact_f32=exact)
    try:
        toks = tokens_of(spec, 400, 38)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [300, 1, 1, 12, 3, 10, 1, 60, 1])
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
    """A Lotinex checkpoint behind the serving path: FASTTALK_CHECKPOINT -> registry -> engine -> NativeHandler streams text."""
    from fasttalk_llm_microservice_b200.handler import NativeHandler, build_runner
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make([layer(attention(), dense()), layer(delta(), moe()), layer(parallel())], width=64, vocab=600, seed=41)
    save_checkpoint(spec, w, str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_CHECKPOINT", str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_ALLOW_BYTE_TOKENIZER", "1")
    monkeypatch.setenv("FASTTALK_MAX_SESSIONS", "4")
    monkeypatch.setenv("FASTTALK_MAX_CONTEXT", "512")
    monkeypatch.setenv("FASTTALK_MAX_BATCHED_TOKENS", "256")
    runner = build_runner("lotinex-test")
    h = NativeHandler(model="lotinex-test", runner=runner)
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
