"""Model registry: config.json -> model class.

Model modules live in `sglang.srt.models` (the layout of the reference's fork) and export `EntryClass` (one class or a list), the way
that package's loader discovers models.  A class is found by its own name or by any string in its `architecture_names`; config.json names
its class under `architectures` (a list, the Hugging Face convention) or `architecture` (a single string).  Modules are imported lazily,
so resolving one model does not import another's dependencies (the BitNet module needs torch, the sequence models only numpy)."""
from __future__ import annotations

import importlib
from typing import Dict, List

# module of each known architecture name; importing the module is deferred until the name is asked for
_MODULES: Dict[str, str] = {
    "BitNetForCausalLM": "sglang.srt.models.bitnet",
    "BitnetForCausalLM": "sglang.srt.models.bitnet",
    "Karusun": "sglang.srt.models.karusun",
    "KarusunForCausalLM": "sglang.srt.models.karusun",
    "Tutizen": "sglang.srt.models.tutizen",
    "TutizenForCausalLM": "sglang.srt.models.tutizen",
    "Nukezen": "sglang.srt.models.nukezen",
    "NukezenForCausalLM": "sglang.srt.models.nukezen",
    "Fivedra": "sglang.srt.models.fivedra",
    "FivedraForCausalLM": "sglang.srt.models.fivedra",
}


def register(name: str, module: str) -> None:
    _MODULES[name] = module


def architectures_of(config: Dict) -> List[str]:
    names = config.get("architectures") or config.get("architecture") or []
    return [names] if isinstance(names, str) else list(names)


def known_architectures() -> List[str]:
    return sorted(_MODULES)


def resolve(config: Dict):
    """-> the model class for a parsed config.json."""
    names = architectures_of(config)
    for n in names:
        mod = _MODULES.get(n)
        if mod is None:
            continue
        entry = importlib.import_module(mod).EntryClass
        for cls in (entry if isinstance(entry, (list, tuple)) else [entry]):
            if n == cls.__name__ or n in getattr(cls, "architecture_names", ()):
                return cls
    raise KeyError(f"no model class for architecture {names!r}; known: {known_architectures()}")
