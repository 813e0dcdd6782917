"""Model-class base of the layer-stack sequence models served by the native engine (libwf_seq.so): weight loading by checkpoint name
and the step interface (admit / release / step / sample) that the scheduler, `generate` and the trace replay drive.  A design's module
supplies the configuration reader that turns config.json into the engine's native structs; it computes nothing itself."""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import numpy as np

from . import _lib, checkpoint
from ._lib import SeqConfig, SeqLayer
from .seq_engine import SeqEngine


class SeqCausalLM:
    """Owns a native engine sized for `max_tokens` cached tokens and `slots` live sequences.  Subclasses implement
    `read_config(config_dict)` -> object with vocab, width, eps, layers, `native_layers()` (one descriptor per layer; the descriptors of
    second mixers that layers name through `pair` follow them) and `fill_native(SeqConfig)`."""

    architecture_names: Tuple[str, ...] = ()
    min_page_size = 1
    reads_shapes = False       # True: read_config(config, shapes) also gets the checkpoint's tensor shapes (sizes that config.json leaves to them)

    @staticmethod
    def read_config(config: Dict):
        raise NotImplementedError

    def neutral_tensor(self, name: str) -> bool:
        """True for an expected tensor that may be absent from a checkpoint and is then all zeros."""
        return False

    def __init__(self, config: Dict, *, dtype: str = "bfloat16", max_tokens: int = 4096, slots: int = 4, page_size: int = 16,
                 max_step_tokens: int = 1024, build: bool = False, shapes: Dict[str, tuple] = None):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
        self.config = self.read_config(config, shapes) if self.reads_shapes else self.read_config(config)
        c = self.config
        self.dtype = dtype
        self.page_size = page_size
        pages = max(1, (max_tokens + page_size - 1) // page_size)
        nc = SeqConfig()
        nc.dtype = _lib.WF_SEQ_F32 if dtype == "float32" else _lib.WF_SEQ_BF16
        nc.vocab, nc.width, nc.n_layers, nc.eps = c.vocab, c.width, len(c.layers), c.eps
        nc.norm_groups, nc.canon_taps = 1, 1
        nc.page_size, nc.max_pages, nc.slots, nc.max_step_tokens = page_size, pages, slots, max_step_tokens
        c.fill_native(nc)
        layers = c.native_layers()                   # one descriptor per layer, then the second mixers of paired layers
        nc.n_extra = len(layers) - nc.n_layers
        self.native_config = nc
        self.engine = SeqEngine(nc, layers, build=build)
        self.vocab = c.vocab
        self.max_step_tokens = max_step_tokens

    @classmethod
    def from_pretrained(cls, model_dir, config=None, **serving):
        """Model folder (config.json + model.safetensors) -> a loaded model; `serving`: dtype, max_tokens, slots, page_size,
        max_step_tokens, build."""
        from pathlib import Path
        cfg = config if config is not None else checkpoint.read_config(model_dir)
        if cls.reads_shapes and "shapes" not in serving:
            f = checkpoint.SafetensorsFile(Path(model_dir) / "model.safetensors")
            try:
                serving["shapes"] = {n: f.info(n)[1] for n in f.names()}
            finally:
                f.close()
        m = cls(cfg, **serving)
        m.load_safetensors(Path(model_dir) / "model.safetensors")
        return m

    # ---- weights
    def load_weights(self, weights: Iterable[Tuple[str, np.ndarray, str]]) -> None:
        """weights: (checkpoint name, array, safetensors dtype string) — bfloat16 as uint16 bit patterns (wf_bitnet.checkpoint)."""
        wanted = {n: count for n, count, _ in self.engine.expected_tensors()}
        for name, a, dt in weights:
            if name not in wanted:
                continue
            if int(np.asarray(a).size) != wanted[name]:
                raise ValueError(f"tensor {name!r} holds {int(np.asarray(a).size)} elements, the configuration needs {wanted[name]}")
            a = np.asarray(a).reshape(-1)
            self.engine.set_tensor(name, checkpoint.to_float32(a, dt) if self.dtype == "float32" else checkpoint.to_bfloat16_bits(a, dt))
        for n, count, loaded in self.engine.expected_tensors():
            if not loaded and self.neutral_tensor(n):
                self.engine.set_tensor(n, np.zeros(count, dtype=np.float32 if self.dtype == "float32" else np.uint16))
        missing = [n for n, _, loaded in self.engine.expected_tensors() if not loaded]
        if missing:
            raise KeyError(f"checkpoint lacks {len(missing)} tensors, first: {missing[:4]}")
        self.engine.finalize()

    def load_safetensors(self, path) -> None:
        f = checkpoint.SafetensorsFile(path)
        try:
            self.load_weights(f.items())
        finally:
            f.close()

    # ---- the step interface the scheduler and the trace replay drive
    def admit(self) -> int:
        return self.engine.admit()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def free_pages(self) -> int:
        return self.engine.free_pages()

    def free_slots(self) -> int:
        return self.engine.free_slots()

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def step(self, slots: Sequence[int], counts: Sequence[int], tokens: Sequence[int], want: Sequence[int] = (), fetch: bool = True):
        return self.engine.step(slots, counts, tokens, want, fetch)

    def sample(self, nrows: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, uniforms=None) -> np.ndarray:
        return self.engine.sample(nrows, temperature, top_k, top_p, uniforms)

    def close(self) -> None:
        self.engine.close()
