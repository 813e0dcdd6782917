"""Nukezen without a device: the configuration reader (every size and constant from config.json or the checkpoint's tensor shapes), the
registry, and checks of the oracle itself."""
import numpy as np
import pytest
import torch

import nukezen_oracle as O
from test_gpu_nukezen import CONFIGS, _rows, make_weights, rel_err, t64


def _native(cs, seed=1):
    from sglang.srt.models.nukezen import NukezenConfig
    w = make_weights(cs, seed)
    c = NukezenConfig.from_dict(cs[0], {k: v.shape for k, v in w.items()})
    return c, c.native_layers()


def test_registry_resolves_the_architecture():
    from wf_bitnet import registry
    assert registry.resolve({"architecture": "Nukezen"}).__name__ == "NukezenForCausalLM"
    assert registry.resolve({"architectures": ["NukezenForCausalLM"]}).reads_shapes


def test_config_reader_takes_every_size_from_config_and_shapes():
    from wf_bitnet import _lib
    for name, cs in CONFIGS.items():
        c, nat = _native(cs)
        layers = cs[0]["layers"]
        n_par = sum(L["type"] == "parallel" for L in layers)
        assert len(nat) == len(layers) + n_par
        nxt = len(layers)
        for i, (L, s) in enumerate(zip(layers, nat)):
            m = L["mixer"]
            assert s.tied == (1 if "weights_of" in L else 0) and (not s.tied or s.tied_to == L["weights_of"])
            assert s.has_ff == (_lib.WF_SEQ_FF_DENSE if L["mlp"] else _lib.WF_SEQ_FF_NONE) and (not L["mlp"] or (s.ff == L["mlp"]["ff"] and s.ff_act == _lib.WF_SEQ_ACT_GELU_TANH))
            if L["type"] == "parallel":
                a, r, x = m["left"], m["right"], nat[nxt]
                assert s.pair == nxt
                nxt += 1
                assert (s.type, s.heads, s.kv_heads, s.dim, s.vdim, s.window) == (_lib.WF_SEQ_GQA_ATTENTION, a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"])
                assert (s.rope_dims, s.rope_interleaved, s.qk_norm, s.head_gate, s.proj_bias, s.chunk, s.sink) == (a["rot"]["dims"], 1, _lib.WF_SEQ_QKNORM_HEAD, 2, 2, 0, 0)
                assert s.rope_base == pytest.approx(a["rot"]["base"]) and s.scale == pytest.approx(a["scale"])
                assert s.mix_scale == pytest.approx(m["left_scale"]) and s.pair_scale == pytest.approx(m["right_scale"])
                assert (x.type, x.heads, x.vdim, x.dim, x.kv_heads, x.conv, x.out_norm_groups) == (_lib.WF_SEQ_SSD, r["heads"], r["vdim"], r["state"], r["groups"], r["conv"], r["norm_groups"])
            elif L["type"] == "channel_delta":
                src = L.get("weights_of", i)
                assert (s.type, s.heads, s.kv_heads, s.dim, s.vdim, s.conv) == (_lib.WF_SEQ_DELTA, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"])
                assert (s.decay_channels, s.gate_act, s.decay_rank, s.gate_rank) == (1, 1, cs[1][src]["rank_a"], cs[1][src]["rank_g"])
            else:
                src = L.get("weights_of", i)
                assert (s.type, s.chunk, s.sink, s.qk_norm, s.rel_rows, s.rope_dims) == (_lib.WF_SEQ_GQA_ATTENTION, m["mask"]["size"], 1, _lib.WF_SEQ_QKNORM_FULL, cs[1][src]["rel_rows"], 0)
                assert s.softcap == pytest.approx(m["softcap"]) and s.rel_far == pytest.approx(m["bias_max"])
        nc = _lib.SeqConfig()
        c.fill_native(nc)
        assert (nc.block_form, nc.norm_weights, nc.tied_head) == (_lib.WF_SEQ_BLOCK_POST, 1, 1) and nc.embed_scale == pytest.approx(cs[0]["embedding"]["scale"])


def test_config_reader_rejects_what_it_cannot_serve():
    from sglang.srt.models.nukezen import NukezenConfig
    cs = CONFIGS["mixed"]
    shapes = {k: v.shape for k, v in make_weights(cs, 1).items()}
    bad = dict(cs[0], layers=[dict(cs[0]["layers"][0], type="mystery")])
    with pytest.raises(ValueError):
        NukezenConfig.from_dict(bad, shapes).native_layers()
    fwd = dict(cs[0], layers=[dict(cs[0]["layers"][2], weights_of=0)])
    with pytest.raises(ValueError):
        NukezenConfig.from_dict(fwd, shapes).native_layers()
    with pytest.raises(ValueError):
        NukezenConfig.from_dict(cs[0], {}).native_layers()          # ranks and table sizes come from the checkpoint


def test_distance_buckets():
    assert [O.distance_bucket(n, 10, 20.0) for n in range(5)] == [0, 1, 2, 3, 4]
    b = [O.distance_bucket(n, 10, 20.0) for n in range(5, 40)]
    # five logarithmic steps between distances 5 and 20: the last row starts at 5 * 4^(4/5) = 15.2
    assert b[0] == 5 and b == sorted(b) and b[-1] == 9 and O.distance_bucket(15, 10, 20.0) == 8 and O.distance_bucket(16, 10, 20.0) == 9


def test_recurrences_token_by_token_equal_a_closed_form():
    """The state-space oracle against the explicit sum y_t = sum_s (prod_{s<r<=t} a_r) dt_s (C_t . B_s) x_s + D x_t for one head."""
    torch.manual_seed(0)
    T, N, P = 9, 3, 4
    a, dt = torch.rand(T, dtype=torch.float64), torch.rand(T, dtype=torch.float64)
    B, C, x = (torch.randn(T, n, dtype=torch.float64) for n in (N, N, P))
    S = torch.zeros(N, P, dtype=torch.float64)
    for t in range(T):
        S = a[t] * S + dt[t] * torch.outer(B[t], x[t])
        want = sum(torch.prod(a[s + 1:t + 1]) * dt[s] * (C[t] @ B[s]) * x[s] for s in range(t + 1))
        assert torch.allclose(S.T @ C[t], want)


def test_oracle_is_sensitive_to_every_mechanism():
    """What the comparisons above can see: leaving out any one piece of a mixer moves the oracle's own output by far more than the
    tolerances (a check of the test's power; it needs no device)."""
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], t64(make_weights(cs, 111))
    eps = cfg["norm"]["eps"]
    h = torch.from_numpy(_rows(40, cfg["width"], 112)).double()

    def moved(fn, base, **change):
        return float(rel_err(fn(change).numpy(), base.numpy()).max())

    a = cfg["layers"][3]["mixer"]
    base = O.chunk_attention(h, w, "l3.mix.", a, eps)
    for k, v in (("softcap", 0.5), ("bias_max", 11), ("scale", 0.31)):
        assert moved(lambda c: O.chunk_attention(h, w, "l3.mix.", dict(a, **c), eps), base, **{k: v}) > 1e-2, k
    assert moved(lambda c: O.chunk_attention(h, w, "l3.mix.", dict(a, mask={"size": 11}), eps), base) > 1e-2
    w2 = dict(w); w2["l3.mix.rel"] = torch.zeros_like(w["l3.mix.rel"])
    assert float(rel_err(O.chunk_attention(h, w2, "l3.mix.", a, eps).numpy(), base.numpy()).max()) > 1e-2
    le = cfg["layers"][0]["mixer"]["left"]
    base = O.window_attention(h, w, "l2.mix.left.", le, eps)
    for change in ({"mask": {"size": 8}}, {"rot": {"dims": 6, "base": 1000.0}}, {"rot": {"dims": 8, "base": 900.0}}, {"kv_heads": 4}):
        if "kv_heads" in change:
            continue
        assert float(rel_err(O.window_attention(h, w, "l2.mix.left.", dict(le, **change), eps).numpy(), base.numpy()).max()) > 1e-3, change
    ri = cfg["layers"][0]["mixer"]["right"]
    base = O.state_space(h, w, "l2.mix.right.", ri, eps)
    for nm in ("D", "dt_bias", "A_log", "conv.b"):
        w2 = dict(w); w2["l2.mix.right." + nm] = w["l2.mix.right." + nm] + 0.5
        assert float(rel_err(O.state_space(h, w2, "l2.mix.right.", ri, eps).numpy(), base.numpy()).max()) > 1e-2, nm


