"""Host-side pieces of the sequence-model serving path that need no GPU: checkpoint reader, configuration reader, registry, the
scheduler's batching policy and the batch splitter (against a fake model), and sanity checks of the plain oracle itself."""
import json
import struct

import numpy as np
import pytest
import torch

import karusun_oracle as O
from wf_bitnet import checkpoint, registry
from wf_bitnet.scheduler import Request, SamplingParams, Scheduler, execute


def write_safetensors(path, tensors):
    header, blob = {}, b""
    for name, (dtype, arr) in tensors.items():
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + blob)


def test_checkpoint_reader_roundtrip(tmp_path):
    x = torch.randn(5, 7)
    bits = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    table = np.arange(6, dtype=np.int32).reshape(2, 3)
    write_safetensors(tmp_path / "m.safetensors", {"a": ("BF16", bits), "t": ("I32", table), "f": ("F32", x.numpy())})
    f = checkpoint.SafetensorsFile(tmp_path / "m.safetensors")
    assert sorted(f.names()) == ["a", "f", "t"] and f.info("a") == ("BF16", (5, 7))
    a, dt = f.get("a")
    assert dt == "BF16" and np.array_equal(checkpoint.to_float32(a, dt), x.to(torch.bfloat16).float().numpy())
    assert np.array_equal(checkpoint.to_bfloat16_bits(f.get("f")[0], "F32"), bits)          # round to nearest even, as torch
    assert np.array_equal(f.get("t")[0], table)
    f.close()


def test_config_reader_fills_native_layers():
    from sglang.srt.models.karusun import NO_WINDOW, KarusunConfig
    cfg = {"architecture": "Karusun", "vocab": 50, "width": 32, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 2}, "layers": [
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "mask": {"size": 7}, "rot": {"base": 500.0, "dims": 4}, "scale": 0.25},
         "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "identity": 1, "top": 2, "groups": {"count": 3, "keep": 2}}}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "rot_dim": 0, "vdim": 6, "kv_rank": 10}},
    ]}
    c = KarusunConfig.from_dict(cfg)
    a, b, d = c.native_layers()
    assert (c.vocab, c.width, c.norm_groups, c.canon_taps) == (50, 32, 4, 2) and abs(c.eps - 1e-5) < 1e-12
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.window, a.rope_dims) == (3, 8, 4, 6, 10, 7, 4) and a.scale == 0.25 and a.rope_base == 500.0
    assert (a.has_ff, a.experts, a.identity, a.top, a.groups, a.keep, a.ff) == (1, 5, 1, 2, 3, 2, 12)
    assert (b.heads, b.kv_heads, b.conv, b.has_ff) == (4, 2, 3, 0)
    assert d.window == NO_WINDOW and d.has_ff == 0 and abs(d.scale - 8 ** -0.5) < 1e-7
    with pytest.raises(ValueError):
        KarusunConfig.from_dict(dict(cfg, layers=[{"type": "conv", "mixer": {"heads": 1, "dim": 1, "vdim": 1}}])).native_layers()


def test_registry_resolves_lazily():
    assert registry.resolve({"architecture": "Karusun"}).__name__ == "KarusunForCausalLM"
    assert "BitNetForCausalLM" in registry.known_architectures()
    with pytest.raises(KeyError):
        registry.resolve({"architectures": ["Unknown"]})


class FakeModel:
    """Step interface with a trivial 'model': the logit row of a token is one-hot at (position + token) % vocab."""

    def __init__(self, vocab=11, slots=2, pages=6, page_size=4, max_step_tokens=8):
        self.vocab, self.max_step_tokens, self.page_size = vocab, max_step_tokens, page_size
        self._free_slots, self._pages, self._len = list(range(slots)), pages, {}
        self.batches = []
        self._last = None

    def pages_for(self, n):
        return (n + self.page_size - 1) // self.page_size

    def free_slots(self):
        return len(self._free_slots)

    def free_pages(self):
        return self._pages - sum(self.pages_for(n) for n in self._len.values())

    def admit(self):
        if not self._free_slots:
            return -1
        s = self._free_slots.pop()
        self._len[s] = 0
        return s

    def release(self, s):
        del self._len[s]
        self._free_slots.append(s)

    def step(self, slots, counts, tokens, want=(), fetch=True):
        assert sum(counts) == len(tokens) <= self.max_step_tokens and len(set(slots)) == len(slots)
        rows, at = [], 0
        for s, c in zip(slots, counts):
            for k in range(c):
                row = np.zeros(self.vocab, dtype=np.float32)
                row[(self._len[s] + k + tokens[at + k]) % self.vocab] = 1.0
                rows.append(row)
            self._len[s] += c
            at += c
        assert self.free_pages() >= 0
        self.batches.append(list(zip(slots, counts)))
        self._last = np.stack([rows[w] for w in want]) if len(want) else None
        return self._last if fetch else None

    def sample(self, n, temperature=0.0, top_k=0, top_p=1.0, uniforms=None):
        return self._last[:n].argmax(-1).astype(np.int32)


def test_execute_splits_long_entries_and_keeps_the_order_of_wanted_rows():
    m = FakeModel(max_step_tokens=5, pages=20)
    a, b = m.admit(), m.admit()
    ta, tb = list(range(12)), [3, 1, 4]
    want = [(1, 2), (0, 11), (0, 0), (0, 5)]
    rows = execute(m, [(a, ta), (b, tb)], want)
    assert [len(x) for x in m.batches] == [1, 1, 2] and sum(c for bt in m.batches for _, c in bt) == 15
    expect = [(2 + 4) % 11, (11 + 11) % 11, 0, (5 + 5) % 11]
    assert rows.argmax(-1).tolist() == expect


def test_scheduler_batches_decodes_with_prompt_portions_and_reuses_slots():
    m = FakeModel(slots=2, pages=8, page_size=4, max_step_tokens=8)
    sched = Scheduler(m, max_prefill_chunk=5)
    prompts = [[1] * 9, [2] * 3, [3] * 6, [4] * 2]
    for i, p in enumerate(prompts):
        sched.add(Request(f"r{i}", p, max_new_tokens=4))
    done = sched.run()
    assert sorted(r.rid for r in done) == ["r0", "r1", "r2", "r3"] and all(len(r.output) == 4 for r in done)
    assert m.free_slots() == 2 and m.free_pages() == 8 and sched.reserved == 0
    assert any(len(b) == 2 and sorted(c for _, c in b)[0] == 1 and sorted(c for _, c in b)[1] > 1 for b in m.batches)   # a decode beside a portion
    # the fake model's next token is a function of position and token only: replay it
    for r in done:
        seq = list(r.prompt)
        for t in r.output:
            assert t == (len(seq) - 1 + seq[-1]) % m.vocab
            seq.append(t)
    # a lone request whose prompt takes several steps: steps in which no logits are wanted must still run
    m1 = FakeModel(slots=1, pages=8, page_size=4, max_step_tokens=8)
    s1 = Scheduler(m1, max_prefill_chunk=4)
    s1.add(Request("solo", [5] * 9, max_new_tokens=3))
    (solo,) = s1.run()
    assert [c for bt in m1.batches for _, c in bt] == [4, 4, 1, 1, 1]
    seq = list(solo.prompt)
    for t in solo.output:
        assert t == (len(seq) - 1 + seq[-1]) % m1.vocab
        seq.append(t)
    with pytest.raises(RuntimeError):
        s2 = Scheduler(FakeModel(pages=2))
        s2.add(Request("big", [0] * 20, max_new_tokens=4))
        s2.run()


def test_oracle_convolution_and_recurrence_identities():
    torch.manual_seed(0)
    h, w = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    y = O.causal_taps(h, w)
    assert torch.allclose(y[0], w[:, 2] * h[0]) and torch.allclose(y[4], w[:, 0] * h[2] + w[:, 1] * h[3] + w[:, 2] * h[4])
    # delta rule with decay 1 and write strength 1 stores v exactly along a unit key: reading with that key returns v
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3}
    S = torch.zeros(4, 3, dtype=torch.float64)
    k = torch.tensor([0.0, 1.0, 0.0, 0.0], dtype=torch.float64)
    v = torch.tensor([1.0, -2.0, 0.5], dtype=torch.float64)
    S = S + torch.outer(k, 1.0 * (v - S.T @ k))
    assert torch.allclose(S.T @ k, v)
    # groups: only experts of kept groups are ever chosen, weights are the uncorrected scores
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}
    P = {"router": torch.randn(6, 8, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 5.0, 0.0, 0.0, 0.0], dtype=torch.float64)}
    x = torch.randn(7, 8, dtype=torch.float64)
    idx, wt = O.route(x, P, r)
    assert set(idx.flatten().tolist()) <= {2, 3}
    s = torch.softmax(x @ P["router"].T, -1)
    assert torch.allclose(wt, s.gather(1, idx))


def test_sequence_engine_abi_matches_its_header():
    """libwf_seq.so exports every function include/wf_seq.h declares, each has a ctypes signature, struct sizes follow the header, and
    the engine refuses to exist without a device instead of falling back to anything."""
    import ctypes as C
    import re
    from pathlib import Path

    from wf_bitnet import _lib
    header = (Path(__file__).resolve().parent.parent / "include" / "wf_seq.h").read_text()
    decl = sorted(set(re.findall(r"\b(wf_seq_[a-z0-9_]+)\s*\(", header)))
    L = _lib.seq_lib()
    assert len(decl) >= 20
    for name in decl:
        assert hasattr(L, name), f"{name} declared in wf_seq.h but not exported"
        assert name in _lib.SEQ_SYMBOLS, f"{name} has no ctypes signature"
    for name in _lib.SEQ_SYMBOLS:
        assert name in decl or name == "wf_last_error"
    assert C.sizeof(_lib.SeqLayer) == 56 * 4 and C.sizeof(_lib.SeqConfig) == 20 * 4
    if not torch.cuda.is_available():
        assert L.wf_seq_available() == 0
        from sglang.srt.models.karusun import KarusunForCausalLM
        cfg = {"architecture": "Karusun", "vocab": 8, "width": 8, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 1},
               "layers": [{"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1}, "mlp": None}]}
        with pytest.raises(_lib.WfError):
            KarusunForCausalLM(cfg)
