"""Fivedra: a decoder-only stack whose layers add two branches that read the SAME residual stream, each behind its own RMS norm with a
weight stored as an offset from one: x <- x + mixer(n1(x)) + ff(n2(x)).  The embedding is scaled by a constant, the feed-forward is
down(relu(up h)^2), the head is a matrix of its own behind a norm of the same kind.  Three kinds of mixer:

  'mingru'            an element-wise gated recurrence: gate z = sigmoid(W_z h + b), candidate from W_x h + b (u + 1/2 right of zero, the
                      logistic function left of it), S <- (1 - z) S + z c, read out as W_o (S * silu(W_g h));
  'parallel'          two mixers side by side on the same input, summed with two constants: grouped-query sliding-window attention
                      whose VALUES ARE ITS KEYS (biased q / k projections, no value projection, no rotation, a learned bias by bucketed
                      distance, one extra unit in the softmax denominator), and a matrix memory with exponential input gate, sigmoid
                      forget gate (both capped by a tanh), a running maximum of the log gates, a normaliser vector, per-head unit RMS,
                      a weight vector and a sigmoid output gate;
  'latent_attention'  causal attention over a cached low-rank latent and one rotated key part shared by all heads; the queries pass a
                      normalised latent of their own; rotation in interleaved pairs with interpolated frequencies; a learned per-head
                      sink in the softmax denominator; no output gate.

This module is the model's configuration reader and its binding to the native engine (libwf_seq.so); it computes nothing itself.
config.json keys read here: architecture, vocab, width, embedding.scale, norm.eps, layers[].{type, mlp.{kind, ff}, mixer.{width, heads,
kv_heads, dim, vdim, rot_dim, kv_rank, q_rank, scale, mask.size, bias_max, gate_cap, left, right, left_scale, right_scale,
rot.{dims, base, scaling.{factor, original, fast, slow}}}}.  The row count of a layer's distance-bias table is read from the checkpoint's
tensor shapes (`mix.left.rel`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from wf_bitnet import _lib
from wf_bitnet._lib import SeqConfig, SeqLayer
from wf_bitnet.seq_model import SeqCausalLM

NO_WINDOW = 1 << 30


@dataclass
class FivedraConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: List[dict] = field(default_factory=list)
    shapes: Dict[str, tuple] = field(default_factory=dict)      # tensor name -> shape, from the checkpoint header

    @staticmethod
    def from_dict(cfg: Dict, shapes: Optional[Dict[str, tuple]] = None) -> "FivedraConfig":
        out = FivedraConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                            embed_scale=float(cfg["embedding"]["scale"]), layers=list(cfg["layers"]), shapes=dict(shapes or {}))
        if not out.layers:
            raise ValueError("config: 'layers' is empty")
        return out

    def fill_native(self, nc: SeqConfig) -> None:
        nc.block_form = _lib.WF_SEQ_BLOCK_PARALLEL
        nc.norm_weights, nc.tied_head = 1, 0
        nc.norm_offset = 1.0                      # the design stores its norm weights around zero
        nc.embed_scale = self.embed_scale

    def _rows(self, name: str, what: str) -> int:
        if name not in self.shapes:
            raise ValueError(f"config: {what} is the row count of tensor {name!r}; pass the checkpoint's tensor shapes")
        return int(self.shapes[name][0])

    @staticmethod
    def _mingru(m: Dict) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_MINGRU
        s.heads, s.dim, s.vdim = 1, 1, int(m["width"])
        return s

    def _keyvalue_attention(self, m: Dict, prefix: str) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_GQA_ATTENTION
        s.heads, s.dim = int(m["heads"]), int(m["dim"])
        s.vdim = int(m.get("vdim", s.dim))
        if s.vdim != s.dim:
            raise ValueError(f"config: {prefix}: the values are the keys, so vdim ({s.vdim}) must equal dim ({s.dim})")
        s.kv_heads = int(m.get("kv_heads", s.heads))
        s.scale = float(m["scale"])
        s.window = int(m["mask"]["size"]) if m.get("mask") else NO_WINDOW
        s.v_is_k, s.proj_bias, s.sink = 1, 2, 1
        s.qk_norm, s.head_gate, s.rope_dims = _lib.WF_SEQ_QKNORM_NONE, 0, 0
        s.rel_rows = self._rows(prefix + "rel", "the size of the distance-bias table")
        s.rel_far = float(m["bias_max"])
        return s

    @staticmethod
    def _matrix_memory(m: Dict) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_MLSTM
        s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s.gate_cap = float(m["gate_cap"])
        return s

    @staticmethod
    def _latent_attention(m: Dict) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_LATENT_ATTENTION
        s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s.rot_dim, s.kv_rank, s.q_rank = int(m["rot_dim"]), int(m["kv_rank"]), int(m["q_rank"])
        s.scale = float(m["scale"])
        s.window = NO_WINDOW                      # causal: every earlier position is visible
        s.sink, s.head_gate, s.rope_interleaved = 2, 0, 1
        rot = m.get("rot") or {}
        s.rope_dims = int(rot.get("dims", s.rot_dim))
        s.rope_base = float(rot.get("base", 10000.0))
        sc = rot.get("scaling")
        if sc:
            s.rope_factor, s.rope_orig = float(sc["factor"]), float(sc["original"])
            s.rope_fast, s.rope_slow = float(sc["fast"]), float(sc["slow"])
        return s

    def native_layers(self) -> List[SeqLayer]:
        main, extra = [], []
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            m, kind = L["mixer"], L["type"]
            if kind == "mingru":
                s = self._mingru(m)
            elif kind == "parallel":
                s = self._keyvalue_attention(m["left"], f"l{i}.mix.left.")
                s.pair = n + len(extra)
                s.mix_scale, s.pair_scale = float(m["left_scale"]), float(m["right_scale"])
                extra.append(self._matrix_memory(m["right"]))
            elif kind == "latent_attention":
                s = self._latent_attention(m)
            else:
                raise ValueError(f"config: layer {i} has unknown mixer type {kind!r}")
            f = L.get("mlp")
            if f is None:
                s.has_ff = _lib.WF_SEQ_FF_NONE
            elif f.get("kind") == "dense":
                s.has_ff, s.ff_act, s.ff = _lib.WF_SEQ_FF_DENSE, _lib.WF_SEQ_ACT_RELU2, int(f["ff"])
            else:
                raise ValueError(f"config: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
            main.append(s)
        return main + extra


class FivedraForCausalLM(SeqCausalLM):
    """Model class of the registry (weights, engine and step interface: wf_bitnet.seq_model.SeqCausalLM)."""

    architecture_names = ("Fivedra", "FivedraForCausalLM")
    reads_shapes = True

    @staticmethod
    def read_config(config: Dict, shapes: Optional[Dict[str, tuple]] = None) -> FivedraConfig:
        return FivedraConfig.from_dict(config, shapes)


EntryClass = FivedraForCausalLM
