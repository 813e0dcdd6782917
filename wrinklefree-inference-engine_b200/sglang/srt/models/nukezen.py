"""Nukezen: a decoder-only stack whose layers come in three kinds, each followed by an optional dense feed-forward (tanh-form gelu gate).
Every sublayer reads the residual stream itself; its OUTPUT is RMS-normalised with a weight vector and added.  The embedding is scaled by
a constant and the logits are products with the unscaled embedding table.

  'parallel'       two mixers side by side on the same input, summed with two constants: grouped-query attention (biased projections,
                   per-head RMS norm of queries and keys with one shared weight vector, rotation of the first `rot.dims` entries in
                   interleaved pairs, sliding window, element-wise sigmoid output gate) and a state-space recurrence with one decay per
                   head (short biased convolution + silu on x | B | C, softplus step size, skip term, silu gate, grouped output norm);
  'channel_delta'  a delta-rule recurrence with short convolutions on q / k / v, unit-length q and k, one decay per head AND key
                   channel from a two-matrix projection, per-head output norm and a two-matrix sigmoid gate;
  'attention'      grouped-query attention without rotation: RMS norm over the whole query / key projection, tanh-capped scores, a learned
                   bias by bucketed distance, visibility limited to the query's own chunk of positions, and one extra unit in the
                   softmax denominator.
A layer may name an earlier layer whose weights it uses (`weights_of`); its cache rows and its recurrent state are its own.

This module is the model's configuration reader and its binding to the native engine (libwf_seq.so); it computes nothing itself.
config.json keys read here: architecture, vocab, width, embedding.scale, norm.eps, layers[].{type, weights_of, mlp.{kind, ff},
mixer.{heads, kv_heads, dim, vdim, scale, mask.size, rot.{dims, base}, softcap, bias_max, conv, left, right, left_scale, right_scale,
groups, state, norm_groups}}.  The row count of a layer's bias table and the ranks of the two-matrix projections are read from the
checkpoint's tensor shapes (`mix.rel`, `mix.a1`, `mix.g1`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from wf_bitnet import _lib
from wf_bitnet._lib import SeqConfig, SeqLayer
from wf_bitnet.seq_model import SeqCausalLM

NO_WINDOW = 1 << 30


@dataclass
class NukezenConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: List[dict] = field(default_factory=list)
    shapes: Dict[str, tuple] = field(default_factory=dict)      # tensor name -> shape, from the checkpoint header

    @staticmethod
    def from_dict(cfg: Dict, shapes: Optional[Dict[str, tuple]] = None) -> "NukezenConfig":
        out = NukezenConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                            embed_scale=float(cfg["embedding"]["scale"]), layers=list(cfg["layers"]), shapes=dict(shapes or {}))
        if not out.layers:
            raise ValueError("config: 'layers' is empty")
        return out

    def fill_native(self, nc: SeqConfig) -> None:
        nc.block_form = _lib.WF_SEQ_BLOCK_POST
        nc.residual_mult = 1.0
        nc.norm_weights, nc.tied_head = 1, 1
        nc.embed_scale = self.embed_scale

    # ---- sizes that only the checkpoint states
    def _rows(self, name: str, what: str) -> int:
        if name not in self.shapes:
            raise ValueError(f"config: {what} is the row count of tensor {name!r}; pass the checkpoint's tensor shapes")
        return int(self.shapes[name][0])

    def _window_attention(self, m: Dict) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_GQA_ATTENTION
        s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s.kv_heads = int(m.get("kv_heads", s.heads))
        s.scale = float(m["scale"])
        s.window = int(m["mask"]["size"]) if m.get("mask") else NO_WINDOW
        s.qk_norm, s.proj_bias, s.head_gate = _lib.WF_SEQ_QKNORM_HEAD, 2, 2
        rot = m.get("rot") or {}
        s.rope_dims, s.rope_base, s.rope_interleaved = int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), 1
        return s

    def _state_space(self, m: Dict) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_SSD
        s.heads, s.vdim, s.dim = int(m["heads"]), int(m["vdim"]), int(m["state"])
        s.kv_heads, s.conv, s.out_norm_groups = int(m.get("groups", 1)), int(m["conv"]), int(m.get("norm_groups", 1))
        return s

    def _channel_delta(self, m: Dict, prefix: str) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_DELTA
        s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s.kv_heads, s.conv = int(m.get("kv_heads", s.heads)), int(m["conv"])
        s.decay_channels, s.gate_act = 1, 1
        s.decay_rank = self._rows(prefix + "mix.a1", "the rank of the decay projection")
        s.gate_rank = self._rows(prefix + "mix.g1", "the rank of the gate projection")
        return s

    def _chunk_attention(self, m: Dict, prefix: str) -> SeqLayer:
        s = SeqLayer()
        s.type = _lib.WF_SEQ_GQA_ATTENTION
        s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s.kv_heads = int(m.get("kv_heads", s.heads))
        s.scale = float(m["scale"])
        s.window = NO_WINDOW
        s.chunk = int(m["mask"]["size"]) if m.get("mask") else 0
        s.qk_norm, s.sink = _lib.WF_SEQ_QKNORM_FULL, 1
        s.softcap = float(m.get("softcap", 0.0))
        s.rel_rows = self._rows(prefix + "mix.rel", "the size of the distance-bias table")
        s.rel_far = float(m["bias_max"])
        return s

    def native_layers(self) -> List[SeqLayer]:
        main, extra = [], []
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            src = L.get("weights_of")
            if src is not None and not (0 <= int(src) < n and int(src) != i and self.layers[int(src)].get("weights_of") is None):
                raise ValueError(f"config: layer {i} takes its weights from layer {src}, which is not another layer with weights of its own")
            prefix = f"l{i if src is None else int(src)}."
            m, kind = L["mixer"], L["type"]
            if kind == "parallel":
                s = self._window_attention(m["left"])
                s.pair = n + len(extra)
                s.mix_scale, s.pair_scale = float(m["left_scale"]), float(m["right_scale"])
                extra.append(self._state_space(m["right"]))
            elif kind == "channel_delta":
                s = self._channel_delta(m, prefix)
            elif kind == "attention":
                s = self._chunk_attention(m, prefix)
            else:
                raise ValueError(f"config: layer {i} has unknown mixer type {kind!r}")
            if src is not None:
                s.tied, s.tied_to = 1, int(src)
            f = L.get("mlp")
            if f is None:
                s.has_ff = _lib.WF_SEQ_FF_NONE
            elif f.get("kind") == "dense":
                s.has_ff, s.ff_act, s.ff = _lib.WF_SEQ_FF_DENSE, _lib.WF_SEQ_ACT_GELU_TANH, int(f["ff"])
            else:
                raise ValueError(f"config: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
            main.append(s)
        return main + extra


class NukezenForCausalLM(SeqCausalLM):
    """Model class of the registry (weights, engine and step interface: wf_bitnet.seq_model.SeqCausalLM)."""

    architecture_names = ("Nukezen", "NukezenForCausalLM")
    reads_shapes = True

    @staticmethod
    def read_config(config: Dict, shapes: Optional[Dict[str, tuple]] = None) -> NukezenConfig:
        return NukezenConfig.from_dict(config, shapes)


EntryClass = NukezenForCausalLM
