"""Fivedra without a device: the configuration reader (every size and constant from config.json or the checkpoint's tensor shapes), the
registry, and checks of the oracle itself."""
import numpy as np
import pytest
import torch

import fivedra_oracle as O
from test_gpu_fivedra import CONFIGS, _rows, config, gru, lat, make_weights, par, rel_err, t64


def _native(cs, seed=1):
    from sglang.srt.models.fivedra import FivedraConfig
    w = make_weights(cs, seed)
    c = FivedraConfig.from_dict(cs[0], {k: v.shape for k, v in w.items()})
    return c, c.native_layers()


def test_registry_resolves_the_architecture():
    from wf_bitnet import registry
    assert registry.resolve({"architecture": "Fivedra"}).__name__ == "FivedraForCausalLM"
    assert registry.resolve({"architectures": ["FivedraForCausalLM"]}).reads_shapes


def test_config_reader_takes_every_size_from_config_and_shapes():
    from wf_bitnet import _lib
    for name, cs in CONFIGS.items():
        c, nat = _native(cs)
        layers = cs[0]["layers"]
        assert len(nat) == len(layers) + sum(L["type"] == "parallel" for L in layers)
        nxt = len(layers)
        for i, (L, s) in enumerate(zip(layers, nat)):
            m = L["mixer"]
            assert s.has_ff == (_lib.WF_SEQ_FF_DENSE if L["mlp"] else _lib.WF_SEQ_FF_NONE) and (not L["mlp"] or (s.ff == L["mlp"]["ff"] and s.ff_act == _lib.WF_SEQ_ACT_RELU2))
            if L["type"] == "mingru":
                assert (s.type, s.heads, s.dim, s.vdim, s.pair) == (_lib.WF_SEQ_MINGRU, 1, 1, m["width"], 0)
            elif L["type"] == "parallel":
                a, r, x = m["left"], m["right"], nat[nxt]
                assert s.pair == nxt
                nxt += 1
                assert (s.type, s.heads, s.kv_heads, s.dim, s.vdim, s.window) == (_lib.WF_SEQ_GQA_ATTENTION, a["heads"], a["kv_heads"], a["dim"], a["dim"], a["mask"]["size"])
                assert (s.v_is_k, s.sink, s.proj_bias, s.qk_norm, s.head_gate, s.rope_dims, s.chunk, s.rel_rows) == (1, 1, 2, 0, 0, 0, 0, cs[1][i]["rel_rows"])
                assert s.scale == pytest.approx(a["scale"]) and s.rel_far == pytest.approx(a["bias_max"]) and s.softcap == 0.0
                assert s.mix_scale == pytest.approx(m["left_scale"]) and s.pair_scale == pytest.approx(m["right_scale"])
                assert (x.type, x.heads, x.dim, x.vdim) == (_lib.WF_SEQ_MLSTM, r["heads"], r["dim"], r["vdim"]) and x.gate_cap == pytest.approx(r["gate_cap"])
            else:
                assert (s.type, s.heads, s.dim, s.rot_dim, s.vdim, s.kv_rank, s.q_rank) == (_lib.WF_SEQ_LATENT_ATTENTION, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"])
                assert (s.sink, s.head_gate, s.rope_interleaved, s.rope_dims) == (2, 0, 1, m["rot"]["dims"]) and s.window >= 1 << 30
                assert s.scale == pytest.approx(m["scale"]) and s.rope_base == pytest.approx(m["rot"]["base"])
                sc = m["rot"].get("scaling")
                if sc:
                    assert (s.rope_factor, s.rope_orig, s.rope_fast, s.rope_slow) == pytest.approx((sc["factor"], sc["original"], sc["fast"], sc["slow"]))
                else:
                    assert s.rope_factor == 0.0
        nc = _lib.SeqConfig()
        c.fill_native(nc)
        assert (nc.block_form, nc.tied_head, nc.norm_offset) == (_lib.WF_SEQ_BLOCK_PARALLEL, 0, 1.0) and nc.embed_scale == pytest.approx(cs[0]["embedding"]["scale"])


def test_config_reader_rejects_what_it_cannot_serve():
    from sglang.srt.models.fivedra import FivedraConfig
    cs = CONFIGS["mixed"]
    shapes = {k: v.shape for k, v in make_weights(cs, 1).items()}
    bad = dict(cs[0], layers=[dict(cs[0]["layers"][0], type="convolution")])
    with pytest.raises(ValueError):
        FivedraConfig.from_dict(bad, shapes).native_layers()
    bad = dict(cs[0], layers=[dict(cs[0]["layers"][1], mlp={"kind": "moe", "ff": 8})])
    with pytest.raises(ValueError):
        FivedraConfig.from_dict(bad, shapes).native_layers()
    with pytest.raises(ValueError):
        FivedraConfig.from_dict(cs[0], {}).native_layers()           # the bias table's size is in the shapes only
    with pytest.raises(ValueError):
        FivedraConfig.from_dict(dict(cs[0], layers=[]), shapes)
    p = par()
    p["mixer"]["left"]["vdim"] = 24                                   # values that are the keys cannot have a size of their own
    with pytest.raises(ValueError):
        FivedraConfig.from_dict(config([p]), {"l0.mix.left.rel": (8, 4)}).native_layers()


def test_oracle_pieces():
    """The bias table's rows by distance, the candidate's two branches, the interpolated frequencies, and what each constant moves."""
    assert [O.distance_bucket(n, 8, 20.0) for n in (0, 3, 4, 5, 9, 19, 20, 400)] == [0, 3, 4, 4, 6, 7, 7, 7]
    assert [O.distance_bucket(n, 7, 7.5) for n in (0, 2, 3, 4, 7, 8)] == [0, 2, 3, 4, 6, 6]
    u = torch.tensor([-2.0, -1e-9, 0.0, 1.5], dtype=torch.float64)
    assert torch.allclose(O.mingru_candidate(u), torch.tensor([1 / (1 + np.e ** 2), 0.5, 0.5, 2.0], dtype=torch.float64))
    f, mag = O.rotary_frequencies({"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}})
    plain, one = O.rotary_frequencies({"dims": 8, "base": 100.0})
    assert one == 1.0 and mag == pytest.approx(0.1 * np.log(4.0) + 1.0)
    assert f[0] == plain[0] and f[-1] == pytest.approx(plain[-1] / 4.0) and all(plain[i] / 4 <= f[i] <= plain[i] for i in range(4))




def test_oracle_is_sensitive_to_every_mechanism():
    """Each constant and each special rule moves the oracle's output: a product path that ignored one of them could not agree with it."""
    rows = torch.from_numpy(_rows(40, 48, 5)).double()

    def moved(layer, change, sizes=None, seed=7, edit=None):
        cfg = config([layer])
        w = t64(make_weights((cfg, sizes or {0: {"rel_rows": 10}}), seed))
        base = O.MIXERS[layer["type"]](rows, w, "l0.mix.", layer["mixer"], 2e-5).numpy()
        other = {k: (dict(v) if isinstance(v, dict) else v) for k, v in layer["mixer"].items()}
        w2 = dict(w)
        change(other, w2)
        return rel_err(O.MIXERS[layer["type"]](rows, w2, "l0.mix.", other, 2e-5).numpy(), base).max()

    L = par(ls=1.0, rs=0.0)
    assert moved(L, lambda m, w: m["left"].update(mask={"size": 8})) > 1e-2                 # the window, by one token
    assert moved(L, lambda m, w: m["left"].update(bias_max=40)) > 1e-3                      # the reach of the bias table
    assert moved(L, lambda m, w: m["left"].update(scale=0.3)) > 1e-2
    assert moved(L, lambda m, w: w.update({"l0.mix.left.rel": w["l0.mix.left.rel"] * 0})) > 1e-2
    assert moved(L, lambda m, w: w.update({"l0.mix.left.k.b": w["l0.mix.left.k.b"] * 0})) > 1e-3
    R = par(ls=0.0, rs=1.0)
    assert moved(R, lambda m, w: m["right"].update(gate_cap=1.0)) > 1e-2
    assert moved(R, lambda m, w: w.update({"l0.mix.right.f.b": w["l0.mix.right.f.b"] - 3})) > 1e-2
    assert moved(R, lambda m, w: w.update({"l0.mix.right.i.b": w["l0.mix.right.i.b"] + 1})) > 1e-4
    A = lat()
    assert moved(A, lambda m, w: m["rot"].pop("scaling")) > 1e-3
    assert moved(A, lambda m, w: m["rot"].update(base=500.0)) > 1e-3
    assert moved(A, lambda m, w: w.update({"l0.mix.sink": w["l0.mix.sink"] + 1})) > 1e-2
    assert moved(A, lambda m, w: w.update({"l0.mix.dq.norm": w["l0.mix.dq.norm"] * 0 + 1})) > 1e-3
    G = gru()
    assert moved(G, lambda m, w: w.update({"l0.mix.x.b": w["l0.mix.x.b"] + 1})) > 1e-2
    assert moved(G, lambda m, w: w.update({"l0.mix.z.b": w["l0.mix.z.b"] - 2})) > 1e-2


def test_matrix_memory_equals_its_unstabilised_form():
    """The running maximum only rescales state and normaliser together: with small gates the recurrence equals the direct sums
    S_t = sum_j (prod_{j < u <= t} f_u) i_j k_j v_j^T, as long as the maximum of the denominator is taken against exp(-m_t)."""
    cfg = config([par(ls=0.0, rs=1.0, mh=1, md=4, mv=3, cap=3.0)], width=16)
    w = t64(make_weights((cfg, {0: {"rel_rows": 8}}), 9))
    m, p = cfg["layers"][0]["mixer"]["right"], "l0.mix.right."
    h = torch.from_numpy(_rows(12, 16, 10)).double()
    got = O.matrix_memory(h, w, p, m, 2e-5)
    q = (h @ w[p + "q"].T) * 4 ** -0.5
    k, v = h @ w[p + "k"].T, h @ w[p + "v"].T
    li = O.capped(h @ w[p + "i"].T + w[p + "i.b"], 3.0)[:, 0]
    lf = O.log_sigmoid(O.capped(h @ w[p + "f"].T + w[p + "f.b"], 3.0))[:, 0]
    rows, mx = [], 0.0
    for t in range(12):
        mx = max(float(lf[t]) + mx, float(li[t]))
        wt = torch.stack([torch.exp(li[j] + lf[j + 1:t + 1].sum()) for j in range(t + 1)])
        S = (wt[:, None, None] * k[:t + 1, :, None] * v[:t + 1, None, :]).sum(0)
        n = (wt[:, None] * k[:t + 1]).sum(0)
        rows.append((S.T @ q[t]) / (torch.maximum((n @ q[t]).abs(), torch.tensor(1.0, dtype=torch.float64)) + 1e-6 * np.exp(mx)))
    o = O.rms_unit(torch.stack(rows), 2e-5) * w[p + "norm"]
    want = (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T
    assert rel_err(got.numpy(), want.numpy()).max() < 1e-9
