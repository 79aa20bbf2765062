"""Gates on a sublayer's result.

"sigmoid_linear": the result is multiplied element by element by sigmoid(W h + b), h being the sublayer's input.
The part computes W h in fp32 and holds b; the arrangement's fused gate + norm + add kernel adds b and takes the
sigmoid.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from .base import Gate, Runtime, WeightDecl
from .linear import Linear
from .registry import register_part


class SigmoidLinearGate(Gate):
    graph_safe = True

    def _names(self):
        return self.prefix + self.spec.weight_suffix, self.prefix + self.spec.bias_suffix

    def weight_decls(self) -> List[WeightDecl]:
        w, b = self._names()
        n = self.spec.size
        return [WeightDecl(w, (n, n)), WeightDecl(b, (n,), init="zeros")]

    def load(self, store, rt: Runtime) -> None:
        n = self.spec.size
        wn, bn = self._names()
        w, b = store.take(wn, (n, n)), store.take(bn, (n,))
        if w is None or b is None:
            return
        self.proj = Linear.from_host(w, rt)
        self.bias = rt.to_device(b, torch.float32)

    def forward(self, ctx, x: torch.Tensor, logits: torch.Tensor) -> None:
        """logits[t] = W x[t]; ``self.bias`` (fp32 [size]) is added by whoever takes the sigmoid."""
        self.proj(ctx, x, logits, ctx.T, ops.EPI_STORE_F32)


register_part("gate", "sigmoid_linear", SigmoidLinearGate)
