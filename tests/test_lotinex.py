"""CPU side of the Lotinex design: config <-> spec, checkpoint files, the family registry, the packed descriptors, and
properties of the plain restatement (oracle/lotinex_oracle.py) that the GPU tests lean on."""
import json
import math

import pytest
import torch

from fasttalk_llm_microservice_b200 import layered as LY
from fasttalk_llm_microservice_b200.registry import family_of, load_model
from oracle import lotinex_oracle as O


def small_config():
    att = {"dim": 8, "heads": 6, "kv_heads": 3, "mask": {"size": 11}, "rot": {"base": 500.0, "dims": 4}, "scale": 0.3, "vdim": 10}
    return {"architecture": "Lotinex", "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "streams": 3, "vocab": 60, "width": 28,
            "layers": [
        {"type": "delta", "mixer": {"conv": 3, "dim": 6, "heads": 4, "kv_heads": 2, "vdim": 5}, "mlp": {"ff": 20, "kind": "dense"}},
        {"type": "attention", "mixer": dict(att), "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"conv": 2, "dim": 8, "heads": 4, "kv_heads": 1, "mask": {"size": 7},
                     "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "fast": 16.0, "original": 64.0, "slow": 2.0}},
                     "scale": 0.25, "softcap": 20.0, "vdim": 6},
            "right": {"conv": 3, "dt_rank": 5, "inner": 40, "state": 6}},
         "mlp": {"expert": {"ff": 12}, "kind": "moe", "router": {"experts": 5, "top": 2}}},
        {"type": "attention", "mixer": {**att, "kv_from": 1}, "mlp": {"ff": 16, "kind": "dense"}}]}


def small_spec():
    cfg = small_config()
    return cfg, LY.spec_from_config(cfg, None, name="t")


def test_config_roundtrip_and_shapes():
    cfg, spec = small_spec()
    assert spec.config() == cfg and spec.streams == 3 and abs(spec.embed_scale - 3.0) < 1e-12
    assert [l.form for l in spec.layers] == ["hyper"] * 4
    assert [b.kind for l in spec.layers for b in l.branches] == ["window_attention", "window_attention", "selective_scan", "window_attention"]
    shapes = LY.tensor_shapes(spec)
    assert LY.spec_from_config(cfg, shapes, name="t") == spec
    assert "head" not in shapes and shapes["final.norm.b"] == (28,) and shapes["l0.norm1.b"] == (28,)
    assert shapes["l0.mix.a"] == (4, 28) and shapes["l0.mix.dt_bias"] == (4,) and shapes["l0.mix.q.conv"] == (12, 3)
    assert shapes["l0.hc2.mix"] == (3, 3) and shapes["l1.hc1.in"] == (3,) and "l1.hc2.in" not in shapes and "l1.norm2" not in shapes
    assert shapes["l1.mix.q.norm"] == (8,) and shapes["l1.mix.k.norm"] == (8,) and shapes["l1.mix.v"] == (30, 28)
    assert shapes["l2.mix.left.q.norm"] == (32,) and shapes["l2.mix.left.k.norm"] == (8,) and shapes["l2.mix.left.v.conv"] == (6, 2)
    assert shapes["l2.mix.left.out"] == (28,) and shapes["l2.mix.right.out"] == (28,)
    assert shapes["l2.mix.right.in"] == (80, 28) and shapes["l2.mix.right.x"] == (17, 40) and shapes["l2.mix.right.dt"] == (40, 5)
    assert shapes["l2.mix.right.A_log"] == (40, 6) and shapes["l2.mix.right.conv.b"] == (40,) and shapes["l2.mlp.router"] == (5, 28)
    assert shapes["l2.mlp.e4.down"] == (28, 12)
    assert "l3.mix.k" not in shapes and "l3.mix.v" not in shapes and "l3.mix.k.norm" not in shapes and shapes["l3.mix.q"] == (48, 28)
    plain = small_config()
    del plain["streams"]
    s1 = LY.spec_from_config(plain)
    assert s1.streams == 0 and not any(".hc" in k for k in LY.tensor_shapes(s1)) and s1.config() == plain
    bad = small_config()
    bad["layers"][0]["type"] = "mamba2"
    with pytest.raises(ValueError):
        LY.spec_from_config(bad)
    bad = small_config()
    bad["layers"][0]["mlp"] = {"kind": "sparse"}
    with pytest.raises(ValueError):
        LY.spec_from_config(bad)


def test_checkpoint_files_and_registry(tmp_path):
    _, spec = small_spec()
    w = LY.init_weights(spec, seed=1)
    LY.save_checkpoint(spec, w, str(tmp_path))
    with open(tmp_path / "config.json") as f:
        assert family_of(json.load(f)) == "layered"
    spec2, w2 = load_model(str(tmp_path), name="t")
    assert spec2 == spec and all(torch.equal(w[k], w2[k]) for k in w)
    bad = dict(w)
    del bad["l2.mix.right.dt.b"]
    LY.save_checkpoint(spec, bad, str(tmp_path / "bad"))
    with pytest.raises(KeyError):
        LY.load_checkpoint(str(tmp_path / "bad"))


def test_packed_descriptors():
    _, spec = small_spec()
    w = LY.init_weights(spec, seed=2)
    model, keep = LY.pack(spec, w, "cpu")
    by_ptr = {t.data_ptr(): t for t in keep if isinstance(t, torch.Tensor)}
    assert model.n_layers == 4 and model.streams == 3 and abs(model.embed_scale - 3.0) < 1e-6 and model.head == model.embed
    assert torch.equal(by_ptr[model.final_norm_b], w["final.norm.b"].float())
    d0, d1, d2, d3 = (model.layers[i] for i in range(4))
    assert all(d.form == LY.LAYER_HYPER for d in (d0, d1, d2, d3))
    assert torch.equal(by_ptr[d0.norm_pre1_b], w["l0.norm1.b"].float()) and torch.equal(by_ptr[d0.hc_mix[1]], w["l0.hc2.mix"].float())
    assert torch.equal(by_ptr[d2.hc_out[0]], w["l2.hc1.out"].float()) and not d1.hc_in[1] and not d1.norm_pre2
    # delta: one decay column per head, a full-width SiLU gate, q | k | v adjacent
    assert (d0.mixer, d0.rank_a, d0.rank_g, d0.gate_act, d0.kv_heads) == (LY.MIXER_CHANNEL_DELTA, 0, 0, 1, 2)
    assert d0.o_k == d0.o_q + 12 and d0.o_v == d0.o_k + 12 and d0.n_in % 128 == 0 and d0.ff_kind == LY.FF_DENSE
    # attention inside runs of positions; the last layer reads layer 1's keys and values
    a, b = d1.branch[0], d3.branch[0]
    assert (a.kind, a.qk_norm, a.chunked, a.window, a.rot_dims, a.rot_half, a.kv_lender) == (LY.BRANCH_WINDOW_ATTENTION, 1, 1, 11, 4, 1, 0)
    assert a.o_k == a.o_q + 48 and a.o_v == a.o_k + 24 and not a.sink and not a.out_gain and a.conv == 0
    assert (b.kv_lender, b.o_k, b.o_v) == (2, -1, -1) and not b.k_gain and torch.equal(by_ptr[b.q_gain], w["l3.mix.q.norm"].float())
    assert torch.allclose(by_ptr[a.rot_freq], torch.tensor([1.0, 500.0 ** -0.5])) and abs(a.rot_mag - 1.0) < 1e-7
    # the parallel mixer: both sides normed over the width and halved
    l, r = d2.branch[0], d2.branch[1]
    assert (d2.n_branches, l.qk_norm, l.chunked, l.conv, l.window, abs(l.softcap - 20.0) < 1e-6) == (2, 2, 0, 2, 7, True)
    assert l.sink and by_ptr[l.sink].abs().max() == 0 and by_ptr[l.q_gain].shape == (32,) and by_ptr[l.conv_w].shape == (46, 2)
    assert abs(l.out_scale - 0.5) < 1e-7 and abs(r.out_scale - 0.5) < 1e-7 and torch.equal(by_ptr[r.out_gain], w["l2.mix.right.out"].float())
    assert abs(l.rot_mag - (0.1 * math.log(8.0) + 1.0)) < 1e-6
    assert (r.kind, r.heads, r.dim, r.vdim, r.dt_rank, r.conv, r.o_z - r.o_v) == (LY.BRANCH_SELECTIVE_SCAN, 40, 6, 1, 5, 3, 40)
    assert torch.equal(by_ptr[d2.w_in][r.o_v:r.o_v + 80], w["l2.mix.right.in"]) and by_ptr[r.a_log].shape == (40, 6)
    # experts: sigmoid scores as they are, on the experts' inputs
    assert (d2.ff_kind, d2.route_kind, d2.route_norm, d2.route_input, d2.top, d2.experts) == (LY.FF_MOE, LY.ROUTE_SIGMOID, 0, 1, 2, 5)
    assert torch.equal(by_ptr[d2.w_gu][3][0::2], w["l2.mlp.e3.gate"]) and d2.router_rows == 128


def test_stretched_frequencies_of_the_loader_follow_the_restatement():
    for dims, base, sc in ((8, 100.0, (8.0, 64.0, 16.0, 2.0)), (32, 10000.0, (4.0, 512.0, 32.0, 1.0)), (6, 50.0, (2.0, 30.0, 4.0, 0.5)),
                           (16, 1e6, ())):
        b = LY.BranchSpec(kind="window_attention", heads=1, dim=dims, vdim=4, rot_dims=dims, rot_base=base, rot_scaling=sc)
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        f, mag = LY.rotary_frequencies(b)
        g, mag2 = O.rotary_frequencies(rot, torch.float64)
        assert torch.allclose(torch.tensor(f, dtype=torch.float64), g, rtol=1e-12) and abs(mag - mag2) < 1e-12
        plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        if sc:          # the fastest pair keeps its frequency, the slowest is slowed by the factor, nothing leaves that range
            assert abs(f[0] - plain[0]) < 1e-12 and abs(f[-1] - plain[-1] / sc[0]) < 1e-12 * plain[-1] + 1e-15
            assert all(p / sc[0] - 1e-15 <= x <= p + 1e-15 for x, p in zip(f, plain))
        else:
            assert f == plain and mag == 1.0


def test_oracle_masks_sink_streams_and_experts():
    assert O.visible_chunk(10, 4)[6].tolist() == [False] * 4 + [True] * 3 + [False] * 3
    assert O.visible_chunk(10, 4)[8].tolist() == [False] * 8 + [True, False]
    assert O.visible_window(10, 4)[6].tolist() == [False] * 3 + [True] * 4 + [False] * 3
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 2, 4, dtype=torch.float64), torch.randn(5, 1, 4, dtype=torch.float64), torch.randn(5, 1, 3, dtype=torch.float64)
    m = O.visible_window(5, 5)
    a, b = O.attend(q, k, v, m, 0.5), O.attend(q, k, v, m, 0.5, zero_sink=True)
    s0 = (q[0, 0] @ k[0, 0]) * 0.5          # the first position sees itself only: weight 1, or e^s / (1 + e^s) with the sink
    assert torch.allclose(a[0, :3], v[0, 0]) and torch.allclose(b[0, :3], v[0, 0] * torch.exp(s0) / (1 + torch.exp(s0)))
    # one stream without mixing tensors is the plain residual
    X = torch.randn(4, 1, 6, dtype=torch.float64)
    assert torch.allclose(O.hyper_step(X, {}, "l0.hc1.", lambda u: 2 * u), 3 * X)
    w = {"h.in": torch.tensor([1.0, 0.0], dtype=torch.float64), "h.out": torch.tensor([0.0, 1.0], dtype=torch.float64),
         "h.mix": torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)}
    X = torch.randn(3, 2, 5, dtype=torch.float64)
    Y = O.hyper_step(X, w, "h.", lambda u: u)          # streams swap ([from, to]); stream 1 also gets the result (= old stream 0)
    assert torch.allclose(Y[:, 0], X[:, 1]) and torch.allclose(Y[:, 1], 2 * X[:, 0])


def test_oracle_is_causal_and_scores_scale_expert_inputs():
    cfg, spec = small_spec()
    w = LY.init_weights(spec, seed=3)
    toks = torch.randint(0, spec.vocab, (30,)).tolist()
    with torch.no_grad():
        full = O.forward(cfg, w, toks)
        assert torch.allclose(full[:17], O.forward(cfg, w, toks[:17]), atol=1e-9)
        changed = O.forward(cfg, w, [(toks[0] + 1) % spec.vocab] + toks[1:])
        assert (full[-1] - changed[-1]).abs().max() > 1e-6          # the recurrent layers carry the first token to the end
        h = torch.randn(4, 28, dtype=torch.float64)
        wd = {k: v.double() for k, v in w.items()}
        mlp = cfg["layers"][2]["mlp"]
        got = O.expert_ff(h, wd, "l2.mlp.", mlp)
        s = torch.sigmoid(h @ wd["l2.mlp.router"].T)
        t = 1
        top = torch.topk(s[t], 2).indices.tolist()
        on_input = sum(O.gated_ff((s[t, e] * h[t])[None], wd, f"l2.mlp.e{e}.")[0] for e in top)
        on_output = sum(s[t, e] * O.gated_ff(h[t][None], wd, f"l2.mlp.e{e}.")[0] for e in top)
        assert torch.allclose(got[t], on_input) and (on_input - on_output).abs().max() > 1e-4
