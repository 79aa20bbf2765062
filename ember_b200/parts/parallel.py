"""Two mixers side by side on the same input: result = left_scale * left + right_scale * right.

Each inner mixer keeps a cache of its own (pages, a state slot, ...): ``cache_needs`` names them "left" and "right"
and ``forward`` receives a mapping with those names.  The inner mixers store their fp32 results in buffers
(``can_store``) and one kernel forms the scaled sum.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .registry import build_part, register_part


class ParallelMixer(Mixer):
    can_store = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.left = build_part("mixer", spec.left, prefix + spec.left_prefix)
        self.right = build_part("mixer", spec.right, prefix + spec.right_prefix)
        for m in (self.left, self.right):
            if not getattr(m, "can_store", False):
                raise ConfigError(f"a parallel mixer needs inner mixers that can store their result; {type(m).__name__} cannot")
            if list(m.cache_needs()) != [""]:
                raise ConfigError("a parallel mixer's inner mixers are plain mixers")

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def weight_decls(self) -> List[WeightDecl]:
        return self.left.weight_decls() + self.right.weight_decls()

    def load(self, store, rt: Runtime) -> None:
        self.rt = rt
        self.left.load(store, rt)
        self.right.load(store, rt)

    def cache_needs(self) -> Dict[str, Optional[CacheNeed]]:
        return {"left": self.left.cache_need(), "right": self.right.cache_need()}

    def tile_requests(self):
        keys = []
        for m in (self.left, self.right):
            fn = getattr(m, "tile_requests", None)
            keys += [k for k in (fn() if fn else ()) if k not in keys]
        return keys

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, hidden = self.spec, self.spec.hidden_size
        a = ctx.buf("parallel.left", (ctx.max_tokens, hidden), torch.float32)
        b = ctx.buf("parallel.right", (ctx.max_tokens, hidden), torch.float32)
        self.left.forward(ctx, x, a, cache["left"], owns_cache, accumulate=False)
        self.right.forward(ctx, x, b, cache["right"], owns_cache, accumulate=False)
        ops.scaled_sum(a, s.left_scale, b, s.right_scale, out, ctx.T * hidden, accumulate=accumulate, stream=ctx.stream)


register_part("mixer", "parallel", ParallelMixer)
