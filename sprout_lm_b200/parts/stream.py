"""What travels from one layer call to the next when that is not simply the layer's result.

``depth_weighted_average``: every layer call's result X_(n+1) is kept (X_0 is the embedding's
output), and what the next call (or the final norm) reads is sum_{j <= n+1} w_n[j] X_j with a learned
weight vector per call.  The history lives for one step: float32 [calls + 1, tokens, hidden].
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part


@register_part("stream", "depth_weighted_average")
class DepthWeightedAverage(Part):
    def __init__(self, prefix: str, names: tuple):
        """``names[n]`` is the tensor of call n's weights; it has n + 2 entries."""
        self.names = tuple(prefix + name for name in names)
        self.weights: list = []

    def tensor_decls(self):
        # a fresh model passes the latest result on (the last entry is 1 + noise, the others noise)
        return [TensorDecl(name, (n + 2,), "pass_last") for n, name in enumerate(self.names)]

    def load(self, source: WeightSource):
        self.weights = [source.vector(name) for name in self.names]

    def begin(self, x: torch.Tensor, calls: int):
        if calls != len(self.names):
            raise ValueError(f"depth_weighted_average: {len(self.names)} weight vectors for {calls} layer calls")
        history = torch.empty((calls + 1, *x.shape), dtype=torch.float32, device=x.device)
        history[0].copy_(x)
        return history

    def after(self, history, n: int, x: torch.Tensor) -> None:
        kernels.depth_average(history, x, self.weights[n], n)

    def norm_after(self, history, n: int, y, gain, eps: float, x, y2=None, h=None, alpha: float = 1.0) -> None:
        """``after`` for a layer that ends in an RMS norm of ``y``: the norm, the average into ``x`` and, when given, the
        next layer's readers ``y2 = alpha x`` and ``h`` (x in h's dtype) in one launch."""
        kernels.sum_norm(y, gain, x, eps, y2=y2, h=h, alpha=alpha, history=history, weights=self.weights[n], n=n)
