"""Swaps this package's classes into the reference's ``memory_transformer`` modules.

The reference builds its memory layer from three classes that it imports by name
(memory_transformer/model.py:15-31 ``ChapteredMemoryBank``, ``ChapterRouter``;
memory_transformer/memory_block.py:15 ``MemoryCrossAttention``).  Rebinding those names is the whole
integration: ``MemoryTransformer.__init__`` and ``forward`` (model.py:46-727) then run unchanged on the
CUDA operators.  Constructor arguments, attribute names and state-dict keys are the reference's, so
checkpoints load either way.

    import memory_transformer
    from memory_b200.dropin import use_b200_memory_layer
    with use_b200_memory_layer(memory_transformer):      # or call .install() / .restore() yourself
        model = memory_transformer.model.MemoryTransformer(config)
"""
from __future__ import annotations

import importlib
from typing import Dict, Tuple

from .memory_attention import MemoryCrossAttention
from .memory_bank import ChapteredMemoryBank
from .router import ChapterRouter

# (submodule, attribute) -> replacement
_BINDINGS = {
    ("model", "ChapterRouter"): ChapterRouter,
    ("model", "ChapteredMemoryBank"): ChapteredMemoryBank,
    ("memory_block", "MemoryCrossAttention"): MemoryCrossAttention,
}


class use_b200_memory_layer:
    """Context manager / handle that rebinds the three class names and puts them back."""

    def __init__(self, memory_transformer_pkg):
        self.pkg = memory_transformer_pkg
        self._saved: Dict[Tuple[str, str], object] = {}

    def install(self) -> "use_b200_memory_layer":
        for (sub, attr), cls in _BINDINGS.items():
            mod = importlib.import_module(f"{self.pkg.__name__}.{sub}")
            if (sub, attr) not in self._saved:
                self._saved[(sub, attr)] = getattr(mod, attr)
            setattr(mod, attr, cls)
        return self

    def restore(self) -> None:
        for (sub, attr), orig in self._saved.items():
            setattr(importlib.import_module(f"{self.pkg.__name__}.{sub}"), attr, orig)
        self._saved.clear()

    def __enter__(self):
        return self.install()

    def __exit__(self, *exc):
        self.restore()
        return False
