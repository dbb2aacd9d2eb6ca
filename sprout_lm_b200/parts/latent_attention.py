"""Attention over a cached low-rank latent: per token the cache holds one row [c | k_rot] shared by
all heads, c = RMSNorm(W_dkv h)[:rank] * w and k_rot = the last ``rot_dim`` outputs of W_dkv h rotated by
the token's position.  Head n's key is [W_uk,n c | k_rot], its value W_uv,n c, its query
[q_n (dim, unrotated) | q_rot,n (rot_dim, rotated)]; the score is scale * (q_n . W_uk,n c + q_rot,n . k_rot),
the mask causal, and the softmax's denominator may hold one more term exp(sink_n) per head.

The up-projections are folded to the query's side, so that nothing per head is ever made of the cache:
q_lat,n = W_uk,n^T q_n (rank wide), score = scale * ([q_lat,n | q_rot,n] . [c | k_rot]), the weighted sum of
the rows' c parts is taken once per head (rank wide) and W_uv,n is applied to that sum.  Prefill and
decode, whole prompts and portions all run this one form over the same rows.

Queries come from a latent of their own (``q_rank``: q = W_uq RMSNorm(W_dq h) * w) or straight from h.
A layer may read the rows another layer cached (its run-order entry has ``writes_cache=False``): it
then has no W_dkv and only brings queries, W_uk and W_uv of its own.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import PartSpec
from .base import CacheSpec, CacheView, Part, TensorDecl, WeightSource, build_part, register_part
from .linear import Linear

DEFAULT_NAMES = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                 "uk": "uk", "uv": "uv", "sink": "sink", "o": "o"}


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 scale: float, eps: float, position: PartSpec, q_rank: int | None = None, own_kv: bool = True,
                 sink: bool = True, names: dict | None = None):
        for label, value in (("hidden_size", hidden_size), ("heads", heads), ("value_dim", value_dim), ("kv_rank", kv_rank)):
            if value <= 0:
                raise ValueError(f"latent_attention: {label} must be positive (got {value})")
        if dim < 0 or rot_dim < 0 or dim + rot_dim == 0:
            raise ValueError("latent_attention: a head needs unrotated or rotated query/key dimensions")
        if q_rank is not None and q_rank <= 0:
            raise ValueError("latent_attention: q_rank must be positive when given")
        self.hidden_size, self.heads, self.dim, self.rot_dim = hidden_size, heads, dim, rot_dim
        self.value_dim, self.kv_rank, self.q_rank = value_dim, kv_rank, q_rank
        self.scale, self.eps, self.own_kv, self.has_sink = float(scale), float(eps), bool(own_kv), bool(sink)
        self.names = {key: prefix + value for key, value in {**DEFAULT_NAMES, **(names or {})}.items()}
        self.position = build_part("position", position)
        self.width = kv_rank + rot_dim                 # a cache row
        self.runtime = None

    # ---- what it keeps: one row per token, no values of their own
    def cache_spec(self):
        return CacheSpec(kv_heads=1, head_dim=self.width, kind="full", value_dim=0)

    def state_spec(self):
        return None

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        """How a step of one token per request divides its keys among CTAs: it follows the contexts' length."""
        return kernels.latent_split_plan(requests, self.heads, self.kv_rank, planned_context, self.width)

    # ---- weights
    def tensor_decls(self):
        n, q_width = self.names, self.heads * (self.dim + self.rot_dim)
        decls = []
        if self.q_rank is None:
            decls.append(TensorDecl(n["q"], (q_width, self.hidden_size)))
        else:
            decls += [TensorDecl(n["dq"], (self.q_rank, self.hidden_size)), TensorDecl(n["dq_norm"], (self.q_rank,), "gain"),
                      TensorDecl(n["uq"], (q_width, self.q_rank))]
        if self.own_kv:
            decls += [TensorDecl(n["dkv"], (self.width, self.hidden_size)), TensorDecl(n["dkv_norm"], (self.kv_rank,), "gain")]
        decls += [TensorDecl(n["uk"], (self.heads * self.dim, self.kv_rank)),
                  TensorDecl(n["uv"], (self.heads * self.value_dim, self.kv_rank))]
        if self.has_sink:
            decls.append(TensorDecl(n["sink"], (self.heads,), "bias"))
        decls.append(TensorDecl(n["o"], (self.hidden_size, self.heads * self.value_dim)))
        return decls

    def load(self, source: WeightSource):
        n, status = self.names, source.runtime.status
        self.runtime = source.runtime

        def linear(name):
            return Linear(source.matrix(name), None, status, any_inner_size=True)
        if self.q_rank is None:
            self.q = linear(n["q"])
        else:
            self.dq, self.uq = linear(n["dq"]), linear(n["uq"])
            self.dq_gain = source.vector(n["dq_norm"])
        if self.own_kv:
            self.dkv = linear(n["dkv"])
            self.dkv_gain = source.vector(n["dkv_norm"])
        # folded to the query's side: per head W_uk^T [rank, dim]; W_uv stays [value_dim, rank] per head
        uk = source.raw(n["uk"]).reshape(self.heads, self.dim, self.kv_rank).transpose(1, 2)
        self.uk_t = source.to_device_matrix(uk.contiguous()) if self.dim else None
        self.uv = source.matrix(n["uv"]).reshape(self.heads, self.value_dim, self.kv_rank)
        self.sink = source.vector(n["sink"]) if self.has_sink else None
        self.out = linear(n["o"])
        self.tables = self.position.rotary_tables(source.runtime) if self.rot_dim else None
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        if self.tables is not None and 2 * self.tables[0].shape[1] > self.rot_dim:
            raise ValueError("latent_attention: the rotation is wider than the rotated part")

    # ---- the step
    def forward(self, h, x, ctx, cache: CacheView, state=None):
        """x (float32) += W_o attention(h); appends this step's rows to the cache slot when it is this layer's."""
        status, tokens = self.runtime.status, h.shape[0]
        cos, sin = self.tables if self.tables is not None else (None, None)
        if cache.write != self.own_kv:
            raise RuntimeError("latent_attention: a layer with a down-projection of its own writes its cache slot, "
                               "a layer without one reads another layer's")
        if self.own_kv:
            rows = self.dkv.forward_float32(h)
            kernels.latent_kv_append(rows, self.dkv_gain, ctx.positions, ctx.seq_of_token, cache.block_table, cos, sin,
                                     self.interleaved, cache.k, self.kv_rank, self.eps, status)
        if self.q_rank is None:
            q = self.q.forward(h)
        else:
            cq = torch.empty((tokens, self.q_rank), dtype=h.dtype, device=h.device)
            kernels.rmsnorm(self.dq.forward_float32(h), self.dq_gain, cq, self.eps)
            q = self.uq.forward(cq)
        q_lat = (torch.empty if self.dim else torch.zeros)((tokens, self.heads * self.width), dtype=h.dtype, device=h.device)
        if self.dim:
            kernels.headwise_gemm(q, self.uk_t, q_lat, self.heads, self.dim + self.rot_dim, self.width)
        kernels.latent_query_tail(q, q_lat, ctx.positions, cos, sin, self.interleaved, self.heads, self.dim, self.rot_dim,
                                  self.kv_rank, status)
        mixed = torch.empty((tokens, self.heads * self.kv_rank), dtype=h.dtype, device=h.device)
        kernels.latent_attention(q_lat, cache, ctx, self.sink, mixed, self.heads, self.kv_rank, self.scale, status)
        attended = torch.empty((tokens, self.heads * self.value_dim), dtype=h.dtype, device=h.device)
        kernels.headwise_gemm(mixed, self.uv, attended, self.heads, self.kv_rank, self.value_dim)
        self.out.forward(attended, residual=x)
