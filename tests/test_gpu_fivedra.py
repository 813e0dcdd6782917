"""Fivedra on the native sequence engine against the plain oracle (tests/fivedra_oracle.py): every mechanism alone, then whole models
through prompts, decoding, portions, mixed batches, reused slots and pages, the scheduler and the command line.  Configurations and
weights are made here; none of them has the sizes of a published model."""
import json

import numpy as np
import pytest
import torch

import fivedra_oracle as O

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------------------------------ configurations
def ffd(ff):
    return {"kind": "dense", "ff": ff} if ff else None


def gru(width=40, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": ffd(ff)}


def par(heads=4, kv=2, dim=16, scale=0.25, window=9, far=20, ls=0.8, rs=0.6, mh=2, md=6, mv=10, cap=5.0, ff=None):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window}, "bias_max": far}
    right = {"heads": mh, "dim": md, "vdim": mv, "gate_cap": cap}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": ls, "right": right, "right_scale": rs}, "mlp": ffd(ff)}


def lat(heads=3, dim=8, rot=6, vdim=10, rank=12, qrank=20, scale=0.3, base=1000.0, scaling=(3.0, 24, 16.0, 2.0), ff=None):
    r = {"dims": rot, "base": base}
    if scaling:
        r["scaling"] = {"factor": scaling[0], "original": scaling[1], "fast": scaling[2], "slow": scaling[3]}
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": qrank, "scale": scale, "rot": r},
            "mlp": ffd(ff)}


def config(layers, width=48, vocab=61, eps=2e-5, escale=1.7):
    return {"architecture": "Fivedra", "vocab": vocab, "width": width, "embedding": {"scale": escale}, "norm": {"eps": eps}, "layers": layers}


# (config, sizes the tensor shapes give).  Layer orders, head groupings, table sizes, ranks and constants all differ between them.
CFG_MIXED = (config([lat(ff=40), gru(ff=56), par(ff=40), par(heads=2, kv=1, window=5, ls=-0.5, rs=1.25, mh=3, md=10, mv=6, cap=2.0), lat(scaling=None, ff=24), gru(width=52)]),
             {2: {"rel_rows": 10}, 3: {"rel_rows": 6}})
# nothing a multiple of 8, one head, one key/value head for all, a window of one token, an odd bias table, layers without feed-forward first
CFG_ODD = (config([par(heads=3, kv=1, dim=6, scale=0.5, window=1, far=7.5, ls=1.0, rs=1.0, mh=1, md=5, mv=7, cap=30.0),
                   gru(width=19, ff=28), lat(heads=1, dim=5, rot=2, vdim=7, rank=9, qrank=5, scale=0.6, base=50.0, scaling=(1.5, 8, 4.0, 0.5), ff=21),
                   par(heads=3, kv=3, dim=10, window=4, far=33.0, ls=0.3, rs=1.5, mh=3, md=7, mv=5, cap=1.0, ff=17), gru(width=36)],
                  width=36, vocab=33, eps=1e-3, escale=0.6), {0: {"rel_rows": 7}, 3: {"rel_rows": 5}})
# sizes that the tensor-core kernels take
CFG_WIDE = (config([lat(heads=8, dim=32, rot=32, vdim=32, rank=64, qrank=96, scale=0.125, base=10000.0, scaling=(4.0, 64, 32.0, 1.0), ff=160),
                    par(heads=8, kv=2, dim=64, scale=0.125, window=37, far=90, mh=2, md=32, mv=64, cap=10.0, ff=96), gru(width=128, ff=64),
                    lat(heads=20, dim=16, rot=16, vdim=24, rank=128, qrank=64, scale=0.2, scaling=None)],
                   width=128, vocab=150, escale=2.5), {1: {"rel_rows": 12}})
CONFIGS = {"mixed": CFG_MIXED, "odd": CFG_ODD, "wide": CFG_WIDE}


def make_weights(cs, seed):
    """name -> float32 array whose values are exactly representable in bfloat16 (so both engine dtypes hold the same model)."""
    return {k: v.numpy() for k, v in O.random_weights(cs[0], seed, cs[1]).items()}


def build(cfg, weights, dtype="float32", max_tokens=256, slots=4, page_size=4, max_step_tokens=64):
    from wf_bitnet import registry
    cls = registry.resolve(cfg)
    model = cls(cfg, dtype=dtype, max_tokens=max_tokens, slots=slots, page_size=page_size, max_step_tokens=max_step_tokens,
                shapes={k: tuple(v.shape) for k, v in weights.items()})
    model.load_weights((k, v, "F32") for k, v in weights.items())
    return model


def t64(weights):
    return {k: torch.from_numpy(np.asarray(v)).double() for k, v in weights.items()}


def oracle_logits(cfg, weights, tokens, streams=None):
    return O.forward(cfg, t64(weights), list(tokens), streams).numpy()


def rel_err(got, want):
    """per row: RMS of the difference (mean taken off) over the RMS of the expected row"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-12)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def assert_close(got, want, dtype, what, factor=1.0):
    """float32: every row within tolerance.  bfloat16: a position where the random model happens to be ill-conditioned (two keys that
    nearly tie under a sharp softmax, a state that is still almost empty) multiplies the rounding of the layers below it; such positions
    are few, so four rows in five must be within tolerance, the typical row well within it, and none far off."""
    err = rel_err(np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64))
    if dtype == "float32" or err.size <= 4:
        assert err.max() < factor * TOL[dtype], (what, int(err.argmax()), float(err.max()))
    else:
        assert (err < factor * TOL[dtype]).mean() >= 0.8 and np.median(err) < 0.5 * TOL[dtype] and err.max() < 0.5, (what, int(err.argmax()), float(err.max()), float(np.median(err)))


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def bf16_exact(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _rows(n, W, seed, scale=1.0):
    return bf16_exact(np.random.default_rng(seed).standard_normal((n, W)) * scale)


def run_alone(m, tokens, cuts):
    """one request through the engine in portions `cuts`; logits of every position"""
    s = m.admit()
    out, a = [], 0
    for c in cuts:
        out.append(m.step([s], [c], tokens[a:a + c], list(range(c))))
        a += c
    m.release(s)
    return np.concatenate(out)


def part_alone(m, layer, part, rows, cuts):
    """one part of one layer on given rows, in portions, through the cache and state of one slot"""
    s = m.admit()
    out, a = [], 0
    for c in cuts:
        out.append(m.engine.run_part(layer, part, [s], [c], rows[a:a + c]))
        a += c
    m.release(s)
    return np.concatenate(out)


def oracle_mixer(cfg, w, li, rows):
    L = cfg["layers"][li]
    return O.MIXERS[L["type"]](torch.from_numpy(rows).double(), t64(w), f"l{li}.mix.", L["mixer"], cfg["norm"]["eps"]).numpy()


# ---------------------------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixers_alone_whole_and_in_portions(name, dtype):
    """Every layer's mixer on random rows: as one portion, in portions of 1 / 2 / 3 / ... tokens through cache and state, and token by
    token."""
    cfg = CONFIGS[name][0]
    w = make_weights(CONFIGS[name], 11)
    m = build(cfg, w, dtype, max_tokens=512)
    n = 45
    for li in range(len(cfg["layers"])):
        rows = _rows(n, cfg["width"], 20 + li)
        want = oracle_mixer(cfg, w, li, rows)
        for cuts in ([n], [1, 2, 3, 5, 7, 2, 11, 14], [1] * n):
            assert_close(part_alone(m, li, 2, rows, cuts), want, dtype, (name, li, cuts[:3]))
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_half_of_a_paired_mixer(dtype):
    """With one of the two constants zero the paired mixer is the other half alone."""
    for ls, rs in ((1.0, 0.0), (0.0, 1.0), (-0.5, 2.0)):
        cfg = config([par(ls=ls, rs=rs, kv=4, mh=3, md=12, mv=4)], width=40)
        w = make_weights((cfg, {0: {"rel_rows": 9}}), 31)
        rows = _rows(30, 40, 32)
        tw, mm, eps = t64(w), cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
        h = torch.from_numpy(rows).double()
        want = ls * O.keyvalue_attention(h, tw, "l0.mix.left.", mm["left"]) + rs * O.matrix_memory(h, tw, "l0.mix.right.", mm["right"], eps)
        m = build(cfg, w, dtype)
        assert_close(part_alone(m, 0, 2, rows, [7, 1, 22]), want.numpy(), dtype, (ls, rs))
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_and_both_norms_alone(dtype):
    cfg = config([gru(ff=52)], width=40)
    w = make_weights((cfg, {}), 41)
    m = build(cfg, w, dtype, max_step_tokens=256)
    tw = t64(w)
    for n in (1, 7, 150):
        rows = _rows(n, 40, 42 + n, 2.0)
        h = torch.from_numpy(rows).double()
        assert_close(part_alone(m, 0, 3, rows, [n]), O.dense_ff(h, tw, "l0.mlp.").numpy(), dtype, ("ff", n))
        assert_close(part_alone(m, 0, 0, rows, [n]), O.offset_norm(h, tw["l0.norm1"], cfg["norm"]["eps"]).numpy(), "float32", ("norm1", n))
        assert_close(part_alone(m, 0, 5, rows, [n]), O.offset_norm(h, tw["l0.norm2"], cfg["norm"]["eps"]).numpy(), "float32", ("norm2", n))
    # the stored weight is the gain's distance from one: a reader that took it for the gain itself would be far off
    assert rel_err((O.rms_unit(h, 2e-5) * tw["l0.norm1"]).numpy(), O.offset_norm(h, tw["l0.norm1"], 2e-5).numpy()).min() > 0.5
    m.close()


# ------------------------------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = CONFIGS[name][0]
    w = make_weights(CONFIGS[name], 51)
    m = build(cfg, w, dtype, max_tokens=512)
    n = 61
    toks = tokens_for(cfg, n, 52)
    want = oracle_logits(cfg, w, toks)
    for cuts in ([n], [1] * n, [40] + [1] * 21, [2, 2, 3, 2, 5, 7, 11, 2, 13, 14], [17, 1, 1, 19, 1, 22]):
        assert_close(run_alone(m, toks, cuts), want, dtype, (name, cuts[:4]), 1.5)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_streams_and_first_positions(dtype):
    """Prompts of one to five tokens (shorter than every window): the stream after every layer and the logits."""
    for name in ("odd", "mixed"):
        cs = CONFIGS[name]
        cfg, w = cs[0], make_weights(cs, 61)
        m = build(cfg, w, dtype)
        for n in (1, 2, 3, 4, 5):
            toks = tokens_for(cfg, n, 62 + n)
            streams = []
            want = oracle_logits(cfg, w, toks, streams)
            s = m.admit()
            out, tap = m.engine.step_with_layer_tap([s], [n], toks, list(range(n)))
            m.release(s)
            for li, st in enumerate(streams):
                assert_close(tap[li], st.numpy(), dtype, ("stream", n, li))
            assert_close(out, want, dtype, ("logits", n))
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    """Four unequal requests advance together — portions of some beside single tokens of others, one of them paused for a step — and
    every position equals the oracle of its request alone."""
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], make_weights(cs, 71)
    m = build(cfg, w, dtype, max_tokens=512)
    reqs = [tokens_for(cfg, n, 72 + n) for n in (37, 9, 23, 50)]
    want = [oracle_logits(cfg, w, r) for r in reqs]
    plan = [[5, 9, 1, 20], [1, 0, 2, 1], [13, 0, 1, 1], [1, 0, 0, 7], [17, 0, 19, 21]]
    slots = [m.admit() for _ in reqs]
    fed = [0] * 4
    for step in plan:
        sl, cn, tk, rows = [], [], [], []
        for i, c in enumerate(step):
            if c:
                sl.append(slots[i]); cn.append(c); tk += reqs[i][fed[i]:fed[i] + c]
                rows += [(i, fed[i] + k) for k in range(c)]
                fed[i] += c
        out = m.step(sl, cn, tk, list(range(len(tk))))
        assert_close(out, np.stack([want[i][p] for i, p in rows]), dtype, step, 1.5)
    assert fed == [len(r) for r in reqs]
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_are_used_again(dtype):
    """Six requests through a pool of 12 pages and 2 slots, a neighbour stepping in between: a slot's recurrent state and running maxima
    and a page's rows must not leak into the next request."""
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], make_weights(cs, 81)
    m = build(cfg, w, dtype, max_tokens=48, slots=2, page_size=4)
    other = m.admit()
    filler = tokens_for(cfg, 40, 82)
    used = 0
    for k, n in enumerate((19, 7, 24, 1, 13, 22)):
        toks = tokens_for(cfg, n, 83 + k)
        want = oracle_logits(cfg, w, toks)
        s = m.admit()
        assert s >= 0
        half = n // 2
        got = []
        if half:
            got.append(m.step([s], [half], toks[:half], list(range(half))))
        if used + 2 > 20:                          # the neighbour starts over before it outgrows its share of the pool
            m.release(other); other = m.admit(); used = 0
        m.step([other], [2], filler[used:used + 2], [])
        used += 2
        got.append(m.step([s], [n - half], toks[half:], list(range(n - half))))
        assert_close(np.concatenate(got), want, dtype, (k, n), 1.5)
        m.release(s)
    assert m.free_slots() == 1
    m.close()


# --------------------------------------------------------------------------------------------- one key that decides, at every edge
def _half_matrix(rows, W, seed):
    return _rows(rows, W // 2, seed, 1.0 / np.sqrt(W // 2))


def _window_model(dtype, span, page_size, n):
    """The windowed attention alone, its keys reading the first half of the input row and its queries the second half through the SAME
    matrix: a probe row that carries in its second half what a marked row carries in its first meets that key with the largest score
    there is (sharp softmax); its own key is an ordinary one.  The values being the keys, the output then IS the marked key."""
    W, d = 64, 64
    cfg = config([par(heads=2, kv=1, dim=d, scale=0.7, window=span, far=3 * span, ls=1.0, rs=0.0, mh=1, md=4, mv=4)], width=W)
    pre = "l0.mix.left."
    w = make_weights((cfg, {0: {"rel_rows": 6}}), 91)
    A = _half_matrix(d, W, 92)
    w[pre + "k"] = np.concatenate([A, np.zeros_like(A)], 1)
    w[pre + "q"] = np.concatenate([np.concatenate([np.zeros_like(A), A], 1)] * 2, 0)
    w[pre + "q.b"] = np.zeros_like(w[pre + "q.b"]); w[pre + "k.b"] = np.zeros_like(w[pre + "k.b"])
    w[pre + "rel"] = w[pre + "rel"] * 0.25
    return cfg, w, build(cfg, w, dtype, max_tokens=n + 64, page_size=page_size, max_step_tokens=n + 8)


def _latent_model(dtype, page_size, n):
    """Latent attention alone with the same device: the query latent reads the second half of the row and the key latent the first half
    through the same matrix and norm weight, and the unrotated query and key up-projections are equal, so a probe meets the marked
    position's key with the score |A c|^2 (the rotated query part is zero)."""
    W, R = 64, 32
    cfg = config([lat(heads=2, dim=24, rot=4, vdim=8, rank=R, qrank=R, scale=2.0, base=100.0, scaling=(2.0, 16, 8.0, 1.0))], width=W)
    pre = "l0.mix."
    w = make_weights((cfg, {}), 95)
    B = _half_matrix(R, W, 96)
    w[pre + "dkv"][:R] = np.concatenate([B, np.zeros_like(B)], 1)
    w[pre + "dq"] = np.concatenate([np.zeros_like(B), B], 1)
    w[pre + "dq.norm"] = w[pre + "dkv.norm"].copy()
    A = _rows(2 * 24, R, 97, 1.0 / np.sqrt(R))
    w[pre + "uk"] = A
    uq = np.zeros_like(w[pre + "uq"]).reshape(2, 28, R)
    uq[:, :24] = A.reshape(2, 24, R)
    w[pre + "uq"] = uq.reshape(2 * 28, R)
    return cfg, w, build(cfg, w, dtype, max_tokens=n + 64, page_size=page_size, max_step_tokens=n + 8)


def _edge_rows(n, probe, marked, seed):
    rows = _rows(n, 64, seed)
    rows[probe, 32:] = rows[marked, :32]
    return rows


def _cuts(points, n):
    edges = sorted({p for p in points if 0 < p < n} | {0, n})
    return [b - a for a, b in zip(edges, edges[1:])]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("span,page_size,n,probe_back", [(6, 4, 40, 0), (37, 4, 90, 1), (300, 16, 340, 2), (64, 16, 200, 3), (16, 16, 70, 0)])
def test_a_deciding_key_just_inside_and_just_outside_the_window(dtype, span, page_size, n, probe_back):
    """The marked key sits on the last position the probe still sees or one before it; the probe comes at the end of a prompt, in the
    middle of a portion, as a single decoded token, and after portions cut at the marked key.  The two placements differ by tens of
    percent in the oracle, so a window one token off cannot pass."""
    cfg, w, m = _window_model(dtype, span, page_size, n)
    probe = n - 1 - probe_back
    first_seen = probe - span + 1
    outs = {}
    for where, marked in (("inside", first_seen), ("outside", first_seen - 1), ("near", probe - 1)):
        rows = _edge_rows(n, probe, marked, 93)
        want = oracle_mixer(cfg, w, 0, rows)
        outs[where] = want[probe]
        for points in ((), (probe, probe + 1), (marked, marked + 2, probe), (marked + 1, probe)):
            cuts = _cuts(points, n)
            got = part_alone(m, 0, 2, rows, cuts)
            assert_close(got[probe:probe + 1], want[probe:probe + 1], dtype, (span, where, cuts), 2.0)
            if dtype == "float32":                 # in bfloat16 two ordinary keys that nearly tie under the sharp softmax may swap
                assert_close(got, want, dtype, (span, where, cuts, "all"), 2.0)
    gap = np.linalg.norm(outs["inside"] - outs["outside"]) / np.linalg.norm(outs["inside"])
    assert gap > 0.3, gap
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size,n,marked", [(64, 400, 0), (64, 400, 1), (64, 400, 63), (64, 400, 64), (64, 400, 65), (16, 330, 127), (16, 330, 128), (4, 90, 3)])
def test_a_far_key_decides_in_causal_latent_attention(dtype, page_size, n, marked):
    """One key hundreds of positions back, on both sides of page borders and on the very first positions, is the one the last query
    wants; the probe comes at the end of a prompt, after a cut at the marked key, and as a single decoded token.  A reader blind to
    that position differs by tens of percent."""
    cfg, w, m = _latent_model(dtype, page_size, n)
    probe = n - 1
    rows = _edge_rows(n, probe, marked, 98)
    want = oracle_mixer(cfg, w, 0, rows)
    blind = rows.copy()
    blind[marked] = _rows(1, 64, 99)[0]
    assert rel_err(oracle_mixer(cfg, w, 0, blind)[probe:], want[probe:]).max() > 0.3
    for points in ((), (probe,), (marked + 1, probe), (marked, marked + 2, n - 3, n - 2, probe)):
        got = part_alone(m, 0, 2, rows, _cuts(points, n))
        assert_close(got[probe:], want[probe:], dtype, (marked, points), 2.0)
        if dtype == "float32":
            assert_close(got, want, dtype, (marked, points, "all"), 2.0)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sinks_take_weight(dtype):
    """Large learned sinks in latent attention, and the extra unit of the windowed attention with few, weakly scored keys: both move the
    output by tens of percent, so leaving either out cannot pass."""
    cfg = config([lat(heads=4, dim=8, rot=4, vdim=6, rank=10, qrank=12, scale=0.1, scaling=None)], width=32)
    w = make_weights((cfg, {}), 171)
    w["l0.mix.sink"] = bf16_exact(np.array([3.0, -1.0, 1.5, 0.25]))
    rows = _rows(24, 32, 172)
    want = oracle_mixer(cfg, w, 0, rows)
    none = dict(w); none["l0.mix.sink"] = np.full(4, -60.0, dtype=np.float32)
    assert rel_err(oracle_mixer(cfg, none, 0, rows), want).min() > 0.1
    m = build(cfg, w, dtype)
    for cuts in ([24], [1] * 24, [5, 2, 17]):
        assert_close(part_alone(m, 0, 2, rows, cuts), want, dtype, ("learned", cuts[:2]))
    m.close()
    cfg = config([par(heads=2, kv=2, dim=8, scale=0.05, window=3, ls=1.0, rs=0.0)], width=32)
    w = make_weights((cfg, {0: {"rel_rows": 4}}), 173)
    w["l0.mix.left.rel"] = w["l0.mix.left.rel"] * 0.1
    want = oracle_mixer(cfg, w, 0, rows)
    assert np.abs(want[0]).max() > 0            # one visible key of score near zero shares its weight with the unit: about one half
    h = torch.from_numpy(rows[:1]).double()
    k0 = (h @ t64(w)["l0.mix.left.k"].T + t64(w)["l0.mix.left.k.b"]) @ t64(w)["l0.mix.left.o"].T
    assert 0.35 < np.linalg.norm(want[0]) / np.linalg.norm(k0.numpy()[0]) < 0.65
    m = build(cfg, w, dtype)
    for cuts in ([24], [1] * 24):
        assert_close(part_alone(m, 0, 2, rows, cuts), want, dtype, ("unit", cuts[:2]))
    m.close()


def test_state_is_carried_over_hundreds_of_tokens():
    """Recurrent mixers made to forget slowly (forget gate almost one; update gate almost zero): 300 tokens in seven portions with a
    neighbour stepping in another slot.  A state that lost its first half would move the last outputs by more than a tenth."""
    for layer, fix in ((par(ls=0.0, rs=1.0, mh=2, md=16, mv=8, cap=8.0), ("l0.mix.right.f.b", 6.0)), (gru(width=24), ("l0.mix.z.b", -5.0))):
        cfg = config([layer], width=32)
        w = make_weights((cfg, {0: {"rel_rows": 8}}), 101)
        w[fix[0]] = np.full_like(w[fix[0]], fix[1])
        n = 300
        rows = _rows(n, 32, 102)
        want = oracle_mixer(cfg, w, 0, rows)
        tail_only = oracle_mixer(cfg, w, 0, rows[150:])
        assert rel_err(tail_only[-20:], want[-20:]).max() > 0.1
        for dtype in ("float32", "bfloat16"):
            m = build(cfg, w, dtype, max_tokens=1024, max_step_tokens=128)
            s, nb = m.admit(), m.admit()
            out, a = [], 0
            for c in (3, 64, 1, 100, 2, 90, 40):
                out.append(m.engine.run_part(0, 2, [s], [c], rows[a:a + c]))
                m.engine.run_part(0, 2, [nb], [5], _rows(5, 32, 103 + a))
                a += c
            assert_close(np.concatenate(out), want, dtype, (fix[0], dtype), 2.0)
            m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_of_the_recurrences(dtype):
    """Portions of several hundred tokens run the recurrences in parallel pieces (matrix memory: chunks from a zero state, start states
    chained, every chunk again; element-wise recurrence: time slices of a block chained through shared memory): a long portion after a
    short one, then a ragged batch of a long, a short and a chunk-sized portion in three slots, against the token-by-token oracle."""
    for layer in (par(ls=0.0, rs=1.0, mh=3, md=12, mv=10, cap=6.0), gru(width=45)):
        cfg = config([layer], width=32)
        w = make_weights((cfg, {0: {"rel_rows": 8}}), 161)
        m = build(cfg, w, dtype, max_tokens=4096, page_size=16, max_step_tokens=1024)
        rows = [_rows(n, 32, 162 + n) for n in (37 + 600, 5 + 128, 300 + 1)]
        want = [oracle_mixer(cfg, w, 0, r) for r in rows]
        assert_close(part_alone(m, 0, 2, rows[0], [37, 600]), want[0], dtype, "one slot", 2.0)
        slots = [m.admit() for _ in rows]
        got = m.engine.run_part(0, 2, slots, [37, 5, 300], np.concatenate([rows[0][:37], rows[1][:5], rows[2][:300]]))
        got2 = m.engine.run_part(0, 2, slots, [600, 128, 1], np.concatenate([rows[0][37:], rows[1][5:], rows[2][300:]]))
        assert_close(np.concatenate([got, got2]), np.concatenate([want[0][:37], want[1][:5], want[2][:300], want[0][37:], want[1][5:], want[2][300:]]), dtype, "ragged", 2.0)
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_page_borders(dtype):
    """150 decoded tokens on 4-token pages: windows and bias buckets slide over decoded tokens only, rotation angles grow."""
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], make_weights(cs, 121)
    m = build(cfg, w, dtype, max_tokens=256, page_size=4)
    toks = tokens_for(cfg, 160, 122)
    assert_close(run_alone(m, toks, [10] + [1] * 150), oracle_logits(cfg, w, toks), dtype, "decode", 1.5)
    m.close()


def test_tensor_core_attention_with_key_splits_in_a_ragged_batch():
    """bfloat16, sizes the tensor-core kernels take, contexts long enough that decoding cuts the keys over several blocks: three sequences
    of unequal length, prompts in portions and then decoded together; float32 (the plain kernels) beside it."""
    le = par(heads=8, kv=2, dim=64, scale=0.125, window=700, far=400, mh=2, md=8, mv=8)
    la = lat(heads=8, dim=32, rot=16, vdim=32, rank=64, qrank=48, scale=0.15, base=10000.0, scaling=(4.0, 128, 32.0, 1.0))
    cfg = config([le, la], width=64, vocab=90)
    w = make_weights((cfg, {0: {"rel_rows": 14}}), 131)
    lens = (650, 300, 41)
    reqs = [tokens_for(cfg, n + 6, 132 + n) for n in lens]
    want = [oracle_logits(cfg, w, r) for r in reqs]
    for dtype in ("bfloat16", "float32"):
        m = build(cfg, w, dtype, max_tokens=1200, page_size=16, max_step_tokens=512)
        slots = [m.admit() for _ in reqs]
        for i, n in enumerate(lens):
            a = 0
            for c in (n // 3, n - n // 3):
                out = m.step([slots[i]], [c], reqs[i][a:a + c], list(range(c)))
                assert_close(out, want[i][a:a + c], dtype, ("prompt", i, a), 1.5)
                a += c
        for k in range(6):
            out = m.step(slots, [1, 1, 1], [reqs[i][lens[i] + k] for i in range(3)], [0, 1, 2])
            assert_close(out, np.stack([want[i][lens[i] + k] for i in range(3)]), dtype, ("decode", k), 1.5)
        m.close()


def _random_config(rng):
    """1-5 layers of random kinds with sizes drawn independently of each other"""
    W = rng.choice([24, 40, 72, 96, 136, 200])
    layers, sizes = [], {}
    for i in range(rng.randint(1, 5)):
        ff = rng.choice([None, W, rng.randint(8, 3 * W)])
        kind = rng.choice(["mingru", "parallel", "latent_attention"])
        if kind == "mingru":
            layers.append(gru(width=rng.choice([W, rng.randint(5, 2 * W)]), ff=ff))
        elif kind == "parallel":
            G, rep, B = rng.choice([1, 2, 3]), rng.choice([1, 2, 4, 8]), rng.choice([4, 10, 16, 24])
            d = rng.choice([6, 16, 24, 64, 128, 192])
            layers.append(par(heads=G * rep, kv=G, dim=d, scale=rng.choice([d ** -0.5, 0.2]), window=rng.choice([1, 2, 7, 16, 50, 120]), far=rng.choice([B // 2 + 1, 3 * B, 100.5]),
                              ls=rng.choice([0.6, 1.0, -0.4]), rs=rng.choice([0.5, 1.3]), mh=rng.choice([1, 2, 5]), md=rng.choice([4, 16, 33, 72, 160]), mv=rng.choice([4, 24, 40, 136]),
                              cap=rng.choice([1.5, 9.0, 25.0]), ff=ff))
            sizes[i] = {"rel_rows": B}
        else:
            r, d = rng.choice([2, 4, 12, 32, 48]), rng.choice([8, 24, 40, 64])
            sc = rng.choice([None, (rng.choice([2.0, 8.0]), rng.choice([16, 200]), rng.choice([32.0, 8.0]), rng.choice([1.0, 0.5]))])
            layers.append(lat(heads=rng.choice([1, 2, 5, 12, 33, 40]), dim=d, rot=r, vdim=rng.choice([8, 20, 48]), rank=rng.choice([16, 40, 96, 256]), qrank=rng.choice([8, 36, 100]),
                              scale=rng.choice([(d + r) ** -0.5, 0.1]), base=rng.choice([100.0, 10000.0, 5e5]), scaling=sc, ff=ff))
    return config(layers, width=W, vocab=rng.choice([50, 97, 300]), eps=rng.choice([1e-6, 1e-4]), escale=rng.choice([1.0, W ** 0.5, 0.3])), sizes


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations(seed):
    """Layer orders, head counts, sizes, windows and constants drawn at random: one prompt whole, prompt + decoded tail, and in random
    portions, in both dtypes."""
    import random
    rng = random.Random(1000 + seed)
    cfg, sizes = _random_config(rng)
    n = rng.choice([3, 17, 64, 130, 290])
    w = make_weights((cfg, sizes), 200 + seed)
    toks = tokens_for(cfg, n, 300 + seed)
    want = oracle_logits(cfg, w, toks)
    k = max(1, n - rng.randint(1, 8))
    cuts, left = [], n
    while left:
        cuts.append(min(left, rng.choice([1, 2, 3, 5, 16, 33, 64, 100])))
        left -= cuts[-1]
    for dtype in ("float32", "bfloat16"):
        m = build(cfg, w, dtype, max_tokens=512, page_size=rng.choice([4, 16, 64]), max_step_tokens=512)
        for c in ([n], [k] + [1] * (n - k), cuts):
            assert_close(run_alone(m, toks, c), want, dtype, (seed, dtype, c[:4]), 1.5)
        m.close()


# ------------------------------------------------------------------------------------------------- scheduler and command line
def _greedy_matches(cfg, w, prompt, output):
    seq = list(prompt)
    for t in output:
        lg = oracle_logits(cfg, w, seq)[-1]
        top2 = np.sort(lg)[-2:]
        if top2[1] - top2[0] > 1e-3 * np.abs(lg).max():
            assert int(np.argmax(lg)) == t
        seq.append(t)


def test_greedy_generation_through_the_scheduler():
    from wf_bitnet.scheduler import Request, Scheduler
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], make_weights(cs, 141)
    m = build(cfg, w, "float32", max_tokens=96, slots=2, page_size=4, max_step_tokens=16)
    sched = Scheduler(m, max_prefill_chunk=5)
    prompts = [tokens_for(cfg, n, 142 + n) for n in (11, 3, 17, 6, 1)]
    for i, p in enumerate(prompts):
        sched.add(Request(f"r{i}", p, max_new_tokens=6))
    done = {r.rid: r for r in sched.run()}
    assert len(done) == 5 and m.free_slots() == 2
    for i, p in enumerate(prompts):
        _greedy_matches(cfg, w, p, done[f"r{i}"].output)
    m.close()


def _write_model_dir(path, cfg, weights):
    import struct
    header, blob = {}, b""
    for name, a in weights.items():
        a = np.asarray(a, dtype=np.float32)
        raw = torch.from_numpy(a.copy()).to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    (path / "config.json").write_text(json.dumps(cfg))
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + blob)


def test_command_line_trace_replay_and_generate(tmp_path):
    """`trace` (bin/trace_run) replays a schedule with mixed batches, a pause, and a finished request whose slot and pages go to the next
    one; `generate` runs the scheduler.  The model class comes from config.json, the table sizes from the checkpoint's shapes."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cs = CONFIGS["mixed"]
    cfg, w = cs[0], make_weights(cs, 151)
    _write_model_dir(tmp_path, cfg, w)
    reqs = {"a": tokens_for(cfg, 21, 152), "b": tokens_for(cfg, 9, 153), "c": tokens_for(cfg, 14, 154)}
    want = {k: oracle_logits(cfg, w, v) for k, v in reqs.items()}
    plan = [[("a", 6)], [("a", 1), ("b", 8)], [("a", 10), ("b", 1)], [("a", 4)], [("c", 2)], [("c", 11)], [("c", 1)]]
    fed, lines, expect = {k: 0 for k in reqs}, [], []
    for n, step in enumerate(plan):
        ents, end, rows = [], [], []
        for rid, c in step:
            ents.append({"id": rid, "tokens": reqs[rid][fed[rid]:fed[rid] + c], "want": list(range(c))})
            rows += [(rid, fed[rid] + k) for k in range(c)]
            fed[rid] += c
            if fed[rid] == len(reqs[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": ents, "end": end}))
        expect.append(rows)
    out = tmp_path / "out"
    out.mkdir()
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", dtype, "--out", str(out), "--max-tokens", "64", "--slots", "2"],
                           input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
        got = [np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"]) for n, rows in enumerate(expect)]
        assert_close(np.concatenate(got), np.stack([want[rid][pos] for rows in expect for rid, pos in rows]), dtype, dtype, 1.5)
    r = subprocess.run([sys.executable, "-m", "wf_bitnet.cli", "generate", "--model", str(tmp_path), "--dtype", "float32", "--max-new-tokens", "5",
                        "--prompt-ids", ",".join(map(str, reqs["a"])), "--prompt-ids", ",".join(map(str, reqs["b"])), "--slots", "1", "--prefill-chunk", "4"],
                       capture_output=True, text=True, timeout=600, env=dict(__import__("os").environ, PYTHONPATH=str(root / "wrinklefree-inference-engine_b200")))
    assert r.returncode == 0, r.stderr[-2000:]
    outs = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [o["id"] for o in outs] == ["r0", "r1"]
    for o, rid in zip(outs, ("a", "b")):
        _greedy_matches(cfg, w, reqs[rid], o["output_ids"])
