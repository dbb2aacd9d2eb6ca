"""Linear attention with a per-head decay and a float32 state per request ("lightning attention").

q = act(W_q h), k = act(W_k h) (heads x dim), v = act(W_v h) (heads x value_dim), act = silu; per head
S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, nothing else scaled.  The heads side by side are divided by their
root mean square (``eps``), multiplied by a learned weight and by sigmoid(W_g h), and projected by W_o.  The state
[heads, dim, value_dim] starts at zero, is float32 and is carried from step to step in the request's state slot; the
mixer keeps nothing per token.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, StateSpec, StateView, TensorDecl, WeightSource, register_part
from .linear import Linear

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}


@register_part("mixer", "decay_linear_attention")
class DecayLinearAttention(Part):
    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, value_dim: int, decay, eps: float,
                 activation: str = "silu", names: dict | None = None):
        decay = tuple(float(d) for d in decay)
        if heads <= 0 or dim <= 0 or value_dim <= 0 or len(decay) != heads:
            raise ValueError("decay_linear_attention: sizes must be positive, one decay per head")
        if activation not in ("silu", "none"):
            raise ValueError("decay_linear_attention: activation must be 'silu' or 'none'")
        self.hidden_size, self.heads, self.dim, self.value_dim = hidden_size, heads, dim, value_dim
        self.decay_values, self.eps, self.silu = decay, float(eps), activation == "silu"
        # the chunked kernel takes powers of the decays (through their logarithms): decays in (0, 1] only
        self.chunkable = all(0.0 < d <= 1.0 for d in decay)
        self.names = {key: prefix + value for key, value in {**DEFAULT_NAMES, **(names or {})}.items()}
        self.runtime = None

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec(shape=(self.heads, self.dim, self.value_dim), dtype=torch.float32)

    def tensor_decls(self):
        n, qk, vw = self.names, self.heads * self.dim, self.heads * self.value_dim
        return [TensorDecl(n["q"], (qk, self.hidden_size)), TensorDecl(n["k"], (qk, self.hidden_size)),
                TensorDecl(n["v"], (vw, self.hidden_size)), TensorDecl(n["g"], (vw, self.hidden_size)),
                TensorDecl(n["o"], (self.hidden_size, vw)), TensorDecl(n["norm"], (vw,), "gain")]

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime
        fused = torch.cat([source.raw(n[key]) for key in ("q", "k", "v", "g")], dim=0)
        self.qkvg = Linear(source.to_device_matrix(fused), None, status, any_inner_size=True)
        self.out = Linear(source.matrix(n["o"]), None, status, any_inner_size=True)
        self.gain = source.vector(n["norm"])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=source.runtime.device)

    def forward(self, h, x, ctx, cache, state: StateView):
        """x (float32) += W_o (rmsnorm(o) * w * sigmoid(W_g h)); the requests' states advance by this step's tokens."""
        if state is None:
            raise RuntimeError("decay_linear_attention: the layer needs a state slot per request")
        rows = self.qkvg.forward(h)
        width = self.heads * self.value_dim
        o = torch.empty((rows.shape[0], width), dtype=torch.float32, device=rows.device)
        kernels.decay_attention(rows, ctx, state, self.decay, o, self.heads, self.dim, self.value_dim, self.silu,
                                self.runtime.status, chunked=self.chunkable)
        gated = torch.empty((rows.shape[0], width), dtype=rows.dtype, device=rows.device)
        kernels.gated_rmsnorm(o, self.gain, rows[:, rows.shape[1] - width:], gated, self.eps)
        self.out.forward(gated, residual=x)
