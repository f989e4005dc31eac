"""CPU side of the Vonedra design: config <-> spec, checkpoint files, the family registry, the packed descriptors, and
properties of the plain restatement (oracle/vonedra_oracle.py) that the GPU tests lean on."""
import json
import math

import pytest
import torch

from fasttalk_llm_microservice_b200 import layered as LY
from fasttalk_llm_microservice_b200.registry import family_of, load_model
from oracle import vonedra_oracle as O


def small_config():
    return {"architecture": "Vonedra", "canon": {"taps": 4}, "embedding": {"scale": 0.8}, "norm": {"eps": 1e-5}, "vocab": 50,
            "width": 24, "layers": [
        {"type": "delta", "mixer": {"conv": 3, "dim": 6, "heads": 4, "kv_heads": 2, "vdim": 5}, "mlp": {"ff": 20, "kind": "dense"}},
        {"type": "attention", "mixer": {"bias_max": 30.0, "dim": 6, "heads": 4, "kv_heads": 2, "mask": {"keep_first": 2, "size": 7},
                                        "scale": 0.4, "v_mix": True, "vdim": 10}, "mlp": None},
        {"type": "latent_attention", "mixer": {"dim": 6, "heads": 3, "kv_rank": 8, "mask": {"size": 5}, "q_rank": 10,
                                               "rot": {"base": 100.0, "dims": 4}, "rot_dim": 4, "scale": 0.3, "vdim": 7},
         "mlp": {"ff": 9, "kind": "dense"}},
        {"type": "attention", "mixer": {"bias_max": 30.0, "dim": 6, "heads": 4, "kv_heads": 2, "mask": {"keep_first": 0, "size": 9},
                                        "scale": 0.4, "v_mix": True, "vdim": 10}, "mlp": {"ff": 12, "kind": "dense"}}]}


def small_spec():
    cfg = small_config()
    shapes = {"l1.mix.rel": (8, 4), "l3.mix.rel": (6, 4), "l2.mix.dq": (10, 24)}
    return cfg, LY.spec_from_config(cfg, shapes, name="t")


def test_config_roundtrip_and_shapes():
    cfg, spec = small_spec()
    assert spec.config() == cfg and spec.canon_taps == 4 and abs(spec.embed_scale - 0.8) < 1e-12
    assert [l.form for l in spec.layers] == ["postnorm"] * 4
    assert [b.kind for l in spec.layers for b in l.branches] == ["window_attention", "latent_window", "window_attention"]
    shapes = LY.tensor_shapes(spec)
    assert LY.spec_from_config(cfg, shapes, name="t") == spec
    assert shapes["l0.mix.q.conv"] == (12, 3) and shapes["l0.mix.a"] == (4, 24) and shapes["l0.mix.dt_bias"] == (4,)
    assert shapes["l0.mix.g"] == (20, 24) and shapes["l0.canon2"] == (24, 4) and shapes["l0.dwa"] == (2,)
    assert shapes["l1.mix.rel"] == (8, 4) and shapes["l1.mix.vmix"] == () and shapes["l1.mix.v.b"] == (20,) and shapes["l1.mix.o.b"] == (24,)
    assert "l1.norm2" not in shapes and "l1.canon2" not in shapes and shapes["l1.dwa"] == (3,)
    assert shapes["l2.mix.dkv"] == (12, 24) and shapes["l2.mix.uq"] == (30, 10) and shapes["l2.mix.uk"] == (18, 8) and shapes["l2.mix.uv"] == (21, 8)
    assert shapes["l3.dwa"] == (5,) and shapes["final.norm"] == (24,)
    bad = small_config()
    bad["layers"][2]["mixer"]["rot"]["dims"] = 2
    with pytest.raises(ValueError):
        LY.spec_from_config(bad, shapes)
    bad = small_config()
    bad["layers"][0]["mlp"] = {"kind": "moe"}
    with pytest.raises(ValueError):
        LY.spec_from_config(bad, shapes)


def test_checkpoint_files_and_registry(tmp_path):
    _, spec = small_spec()
    w = LY.init_weights(spec, seed=1)
    LY.save_checkpoint(spec, w, str(tmp_path))
    with open(tmp_path / "config.json") as f:
        assert family_of(json.load(f)) == "layered"
    spec2, w2 = load_model(str(tmp_path), name="t")
    assert spec2 == spec and all(torch.equal(w[k], w2[k]) for k in w)
    bad = dict(w)
    del bad["l1.mix.sink"]
    LY.save_checkpoint(spec, bad, str(tmp_path / "bad"))
    with pytest.raises(KeyError):
        LY.load_checkpoint(str(tmp_path / "bad"))


def test_packed_descriptors():
    _, spec = small_spec()
    w = LY.init_weights(spec, seed=2)
    model, keep = LY.pack(spec, w, "cpu")
    by_ptr = {t.data_ptr(): t for t in keep if isinstance(t, torch.Tensor)}
    assert model.n_layers == 4 and abs(model.embed_scale - 0.8) < 1e-6
    assert torch.equal(by_ptr[model.final_norm_w], w["final.norm"].float())          # the gain as stored
    d0, d1, d2, d3 = (model.layers[i] for i in range(4))
    assert all(d.form == LY.LAYER_POSTNORM and d.canon_taps == 4 for d in (d0, d1, d2, d3))
    assert torch.equal(by_ptr[d0.norm_post1], w["l0.norm1"].float()) and torch.equal(by_ptr[d2.canon2], w["l2.canon2"].float())
    assert torch.equal(by_ptr[d3.depth_w], w["l3.dwa"].float()) and not d1.canon2 and not d1.norm_post2
    # delta: one decay column per head, a full-width SiLU gate, q | k | v adjacent
    assert (d0.mixer, d0.rank_a, d0.rank_g, d0.gate_act, d0.kv_heads) == (LY.MIXER_CHANNEL_DELTA, 0, 0, 1, 2)
    assert d0.o_k == d0.o_q + 12 and d0.o_v == d0.o_k + 12 and d0.o_a1 % 4 == 0 and d0.n_in % 128 == 0
    assert torch.equal(by_ptr[d0.w_in][d0.o_a1:d0.o_a1 + 4], w["l0.mix.a"]) and torch.equal(by_ptr[d0.w_in][d0.o_g1:d0.o_g1 + 20], w["l0.mix.g"])
    assert by_ptr[d0.dt_bias].shape == (4,) and d0.ff_kind == LY.FF_DENSE and torch.equal(by_ptr[d0.w_gu][1::2], w["l0.mlp.up"])
    # attention: options, the bias table expanded to one row per distance, the first mixing layer keeps its values
    a, b = d1.branch[0], d3.branch[0]
    assert (d1.mixer, d1.n_branches, a.kind, a.qk_norm, a.keep_first, a.window, a.rot_dims) == (LY.MIXER_BRANCHES, 1, LY.BRANCH_WINDOW_ATTENTION, 1, 2, 7, 0)
    assert (a.v_role, b.v_role, b.keep_first) == (1, 2, 0) and a.sink and a.o_bias and a.v_bias and a.o_v >= 0
    table = by_ptr[a.rel]
    assert a.rel_n == 31 and table.shape == (31, 4)
    rows = [O.distance_bucket(n, 8, 30.0) for n in range(31)]
    assert rows[:4] == [0, 1, 2, 3] and rows[4] == 4 and rows[30] == 7 and rows == sorted(rows)
    assert torch.equal(table, w["l1.mix.rel"].float()[torch.tensor(rows)])
    assert by_ptr[b.v_mix].item() == w["l3.mix.vmix"].float().item()
    # latent window attention: one shared key head, W_uk transposed per head
    c = d2.branch[0]
    assert (c.kind, c.kv_heads, c.dim, c.vdim, c.kv_rank, c.q_rank, c.rot_dims, c.window) == (LY.BRANCH_LATENT_WINDOW, 1, 6, 7, 8, 10, 4, 5)
    assert torch.equal(by_ptr[c.w_uk_t][1], w["l2.mix.uk"][6:12].T) and torch.allclose(by_ptr[c.rot_freq], torch.tensor([1.0, 0.1]))
    assert torch.equal(by_ptr[d2.w_in][c.o_k:c.o_k + 12], w["l2.mix.dkv"])


def test_distance_rows_of_the_loader_follow_the_formula():
    for rows, far in ((8, 30.0), (16, 100.0), (6, 7.5), (32, 1000.0), (9, 50.0)):
        got = LY.distance_rows(rows, far)
        half = rows // 2
        assert len(got) == math.ceil(far) + 1 and got[-1] == rows - 1
        for n, r in enumerate(got):
            want = n if n < half else min(rows - 1, half + math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))
            assert r == want
    with pytest.raises(ValueError):
        LY.distance_rows(8, 3.0)


def test_oracle_is_causal_and_its_masks_hide_what_they_should():
    cfg, spec = small_spec()
    w = LY.init_weights(spec, seed=3)
    toks = torch.randint(0, spec.vocab, (30,)).tolist()
    with torch.no_grad():
        full = O.forward(cfg, w, toks)
        assert torch.allclose(full[:17], O.forward(cfg, w, toks[:17]), atol=1e-9)
        changed = O.forward(cfg, w, [(toks[0] + 1) % spec.vocab] + toks[1:])
        assert (full[-1] - changed[-1]).abs().max() > 1e-6          # the delta layer carries the first token to the end
    vis = O.visible(12, 4, 2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4 and not vis[3, 4] and vis[5, 2]
    # the attention alone, without input convolution: token 2 (beyond the kept ones) is seen up to position 2 + 7 - 1
    only = {**cfg, "canon": {"taps": 1}, "layers": [cfg["layers"][1]]}
    s1 = LY.spec_from_config(only, {"l0.mix.rel": (8, 4)})
    w1 = LY.init_weights(s1, seed=4)
    w1["l0.canon1"][:] = 0
    with torch.no_grad():
        a = O.forward(only, w1, toks)
        b = O.forward(only, w1, toks[:2] + [(toks[2] + 1) % spec.vocab] + toks[3:])
        assert (a[8] - b[8]).abs().max() > 1e-6 and (a[9:] - b[9:]).abs().max() == 0
        c = O.forward(only, w1, [toks[0], (toks[1] + 1) % spec.vocab] + toks[2:])
        assert (a[29] - c[29]).abs().max() > 1e-6                     # a kept token is seen from the end
