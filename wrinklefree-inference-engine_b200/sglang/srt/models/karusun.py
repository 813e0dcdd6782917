"""Karusun: a decoder-only stack whose layers each hold one mixer — sliding-window latent attention (a cached low-rank latent plus one
rotated key part shared by all heads, gated output) or a gated delta rule with short convolutions — followed by an optional routed
feed-forward (softmax router with a choice correction, group-limited top-k, identity experts).  Every sublayer is wrapped in grouped RMS
norms before and after, and reads its input through a short causal convolution whose tail is part of the sequence state.

This module is the model's configuration reader and its binding to the native engine (libwf_seq.so); it computes nothing itself.
config.json keys read here: architecture, vocab, width, norm.{eps,groups}, canon.taps, layers[].{type,mixer,mlp}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

from wf_bitnet import _lib
from wf_bitnet._lib import SeqConfig, SeqLayer
from wf_bitnet.seq_model import SeqCausalLM

NO_WINDOW = 1 << 30


@dataclass
class KarusunConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    canon_taps: int
    layers: List[dict] = field(default_factory=list)
    has_canon: bool = True

    @staticmethod
    def from_dict(cfg: Dict) -> "KarusunConfig":
        norm = cfg.get("norm", {})
        out = KarusunConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(norm.get("eps", 1e-6)), norm_groups=int(norm.get("groups", 1)),
                            canon_taps=int((cfg.get("canon") or {}).get("taps", 1)), layers=list(cfg["layers"]), has_canon=bool(cfg.get("canon")))
        if not out.layers:
            raise ValueError("config: 'layers' is empty")
        return out

    def fill_native(self, nc: SeqConfig) -> None:
        nc.block_form = _lib.WF_SEQ_BLOCK_SANDWICH
        nc.norm_groups, nc.canon_taps = self.norm_groups, self.canon_taps

    def native_layers(self) -> List[SeqLayer]:
        res = []
        for i, L in enumerate(self.layers):
            m = L["mixer"]
            s = SeqLayer()
            s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "latent_attention":
                s.type = _lib.WF_SEQ_LATENT_ATTENTION
                s.rot_dim, s.kv_rank = int(m.get("rot_dim", 0)), int(m["kv_rank"])
                s.window = int(m["mask"]["size"]) if m.get("mask") else NO_WINDOW
                rot = m.get("rot") or {}
                s.rope_dims = int(rot.get("dims", s.rot_dim))
                s.rope_base = float(rot.get("base", 10000.0))
                s.scale = float(m["scale"]) if "scale" in m else float((s.dim + s.rot_dim) ** -0.5)
                s.head_gate = 2                                   # this design gates every output element
            elif L["type"] == "delta":
                s.type = _lib.WF_SEQ_DELTA
                s.kv_heads, s.conv = int(m.get("kv_heads", s.heads)), int(m.get("conv", 1))
            else:
                raise ValueError(f"config: layer {i} has unknown mixer type {L['type']!r}")
            f = L.get("mlp")
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"config: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
                r = f["router"]
                s.has_ff = _lib.WF_SEQ_FF_ROUTED
                s.experts, s.identity, s.top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
                g = r.get("groups") or {}
                s.groups, s.keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
                s.ff = int(f.get("expert", {}).get("ff", 0))
            res.append(s)
        return res


class KarusunForCausalLM(SeqCausalLM):
    """Model class of the registry (weights, engine and step interface: wf_bitnet.seq_model.SeqCausalLM)."""

    architecture_names = ("Karusun", "KarusunForCausalLM")

    @staticmethod
    def read_config(config: Dict) -> KarusunConfig:
        return KarusunConfig.from_dict(config)

    def neutral_tensor(self, name: str) -> bool:
        # parts the configuration does not mention are neutral: no input convolution (zero taps), no choice correction
        return (not self.config.has_canon and name.endswith((".canon1", ".canon2"))) or name.endswith(".mlp.correction")


EntryClass = KarusunForCausalLM
