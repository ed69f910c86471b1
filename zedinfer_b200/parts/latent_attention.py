"""Latent attention: keys and values of all heads are up-projections of one small vector per token, the latent,
and only the latent is cached.

Per token, with ``H`` heads of ``qk_dim`` query/key and ``v_dim`` value dimensions and a latent of ``rank``:

    q = Wq x                                   c = rmsnorm(Wdkv x) * g            (plain weight g, float32 norm)
    k_h = Wuk_h c,  v_h = Wuv_h c              s_j = scale * (q_h . k_h,j)  for the keys j the query may see
    p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j'))      (``sink``: a learned logit per head, no key, no value)
    y = Wo concat_h(sum_j p_j v_h,j)

The up-projections never touch the cache: ``q_h . (Wuk_h c) = (Wuk_h^T q_h) . c`` and ``sum_j p_j Wuv_h c_j =
Wuv_h (sum_j p_j c_j)``, so a step projects its queries into the latent space (one product per head), attends over
the cached latents as both keys and values (one cache plane, one "head" shared by all query heads), and projects the
result back (one product per head).  No position rule is applied.

A query at position P sees keys ``max(0, P - window + 1) .. P`` (all keys without a window).  A layer built with
``own_latent=False`` has no ``Wdkv``: it reads the latents another call of the schedule cached (``LayerCall.cache_of``)
with its own up-projections, queries, window and sinks.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView, PagedKVNeed
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, register_mixer
from .mlp import _stack

_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "o": "o"}


@register_mixer("latent_attention")
class LatentAttentionMixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, rank: int, eps: float,
                 scale: Optional[float] = None, window: Optional[int] = None, cache_window="own",
                 own_latent: bool = True, sinks: bool = True, names: Optional[Mapping[str, str]] = None):
        """``window``: this layer's mask; ``cache_window``: the window of the cache it reads or writes (the largest mask
        among the layers that share the latents; None keeps every latent; by default this layer's own window).  ``names``: local tensor names, by role."""
        if num_heads <= 0 or qk_dim <= 0 or v_dim <= 0:
            raise ValueError("latent_attention: heads and head sizes must be positive")
        if rank <= 0 or rank % 8 or rank > 512:
            raise ValueError(f"latent_attention: rank={rank} is not supported; the kernels take multiples of 8 up to 512")
        if window is not None and window <= 0:
            raise ValueError(f"latent_attention: window={window} must be positive (or None for all keys)")
        if cache_window == "own":
            cache_window = window
        if cache_window is not None and (window is None or cache_window < window):
            raise ValueError(f"latent_attention: a cache that keeps {cache_window} latents cannot serve a window of {window}")
        self.hidden_size, self.num_heads, self.qk_dim, self.v_dim = int(hidden_size), int(num_heads), int(qk_dim), int(v_dim)
        self.rank, self.eps = int(rank), float(eps)
        self.scale = float(scale) if scale is not None else float(qk_dim) ** -0.5
        self.window = int(window) if window is not None else None
        self.cache_window = int(cache_window) if cache_window is not None else None
        self.own_latent, self.has_sinks = bool(own_latent), bool(sinks)
        self.names = dict(_NAMES)
        self.names.update(names or {})
        self.q_dim, self.o_dim = self.num_heads * self.qk_dim, self.num_heads * self.v_dim
        self.w_in = self.g = self.w_uk_t = self.w_uv = self.sinks = self.w_o = None

    def cache_need(self):
        return PagedKVNeed(1, self.rank, self.cache_window, planes=1)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        specs = {nm["q"]: TensorSpec((self.q_dim, h)), nm["uk"]: TensorSpec((self.q_dim, self.rank)),
                 nm["uv"]: TensorSpec((self.o_dim, self.rank)), nm["o"]: TensorSpec((h, self.o_dim))}
        if self.own_latent:
            specs[nm["dkv"]] = TensorSpec((self.rank, h))
            specs[nm["dkv_norm"]] = TensorSpec((self.rank,), init=("one_plus_normal", 0.01))
        if self.has_sinks:
            specs[nm["sink"]] = TensorSpec((self.num_heads,), init=("normal", 0.05))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        # the query and the latent's down-projection read the same input: one stacked product
        self.w_in = _stack([tensors[nm["q"]], tensors[nm["dkv"]]]) if self.own_latent else tensors[nm["q"]].contiguous()
        if self.own_latent:
            self.g = tensors[nm["dkv_norm"]].contiguous()
        # [heads, rank, qk_dim]: the rows of Wuk_h^T, so that q_h -> latent space is an ordinary "x @ w.T" per head
        self.w_uk_t = tensors[nm["uk"]].view(self.num_heads, self.qk_dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[nm["uv"]].view(self.num_heads, self.v_dim, self.rank).contiguous()
        self.sinks = tensors[nm["sink"]].float().contiguous() if self.has_sinks else None
        self.w_o = tensors[nm["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._attend(x, ctx, cache, owns_cache), self.w_o, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView,
                             owns_cache: bool) -> torch.Tensor:
        return ops.linear_for_residual(self._attend(x, ctx, cache, owns_cache), self.w_o, None)

    def _attend(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        """Everything up to the output projection: ``[tokens, heads * v_dim]``."""
        if cache.kind != "paged" or cache.kv_stride != 0:
            raise RuntimeError("latent attention needs a paged cache with one plane")
        if owns_cache != self.own_latent:
            raise RuntimeError("latent attention: a layer with a down-projection owns its cache, one without borrows one")
        n, heads = x.shape[0], self.num_heads
        proj = ctx.empty(n, self.w_in.shape[0])
        ops.linear(x, self.w_in, None, proj)
        if self.own_latent:
            ops.rmsnorm_append(proj[:, self.q_dim:], self.g, self.eps, cache.tensor, ctx.tables[cache.group],
                               ctx.tok_seg, ctx.positions, cache.page_size, cache.page_stride)
        q_lat = ctx.empty(n, heads, self.rank)
        ops.linear_per_head(proj[:, :self.q_dim], self.w_uk_t, q_lat)
        o_lat = ctx.empty(n, heads, self.rank)
        ops.attention(q_lat, cache, o_lat, ctx, heads, 1, self.rank, self.window, self.scale, sinks=self.sinks)
        o = ctx.empty(n, heads, self.v_dim)
        ops.linear_per_head(o_lat, self.w_uv, o)
        return o.view(n, self.o_dim)
