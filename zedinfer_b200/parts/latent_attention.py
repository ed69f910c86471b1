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

Options:

* ``rot_dim`` r > 0, a rotated key part shared by all heads: ``Wdkv`` has ``rank + r`` rows, the last r of which (not
  normed) are turned by the token's position (``rot_base``, ``rot_dims`` of them, pairing ``rot_interleaved``) and cached
  behind the latent; a query head is ``[qk_dim plain | r turned]`` and ``s_j = scale * (q_plain . k_h,j + q_rot . kr_j)``.
  In the latent space the query is ``[Wuk_h^T q_plain | q_rot]`` against the cache row ``[c | kr]``, and the values are the
  first ``rank`` entries of that row: the per-head weights are padded with an identity block and with zeros accordingly.
* ``q_rank``: the queries go through a latent of their own, ``q = Wuq (rmsnorm(Wdq x) * gq)``.
* ``out_gate``: the concatenated heads are multiplied by ``sigmoid(Wg x)`` before ``Wo``.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView, PagedKVNeed
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, register_mixer
from .mlp import _stack

_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "o": "o",
          "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "g": "g"}


@register_mixer("latent_attention")
class LatentAttentionMixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, rank: int, eps: float,
                 scale: Optional[float] = None, window: Optional[int] = None, cache_window="own",
                 own_latent: bool = True, sinks: bool = True, names: Optional[Mapping[str, str]] = None,
                 rot_dim: int = 0, rot_dims: Optional[int] = None, rot_base: float = 10000.0, rot_interleaved: bool = True,
                 q_rank: Optional[int] = None, out_gate: bool = False):
        """``window``: this layer's mask; ``cache_window``: the window of the cache it reads or writes (the largest mask
        among the layers that share the latents; None keeps every latent; by default this layer's own window).  ``names``: local tensor names, by role."""
        if num_heads <= 0 or qk_dim <= 0 or v_dim <= 0:
            raise ValueError("latent_attention: heads and head sizes must be positive")
        rot_dim = int(rot_dim or 0)
        rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if rot_dim < 0 or rot_dims < 0 or rot_dims % 2 or rot_dims > rot_dim:
            raise ValueError(f"latent_attention: {rot_dims} of {rot_dim} rotated key entries cannot turn (an even number, at most all)")
        if rot_dim == 0 and (rank <= 0 or rank % 8 or rank > 512):
            raise ValueError(f"latent_attention: rank={rank} is not supported; the kernels take multiples of 8 up to 512")
        if rank <= 0 or rank + rot_dim > 1024:
            raise ValueError(f"latent_attention: rank={rank} with {rot_dim} rotated entries is not supported; the kernels take "
                             f"cache rows of at most 1024 entries")
        if q_rank is not None and q_rank <= 0:
            raise ValueError(f"latent_attention: q_rank={q_rank} must be positive (or None for a direct query projection)")
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
        self.rot_dim, self.rot_dims, self.rot_base, self.rot_interleaved = rot_dim, rot_dims, float(rot_base), bool(rot_interleaved)
        self.q_rank, self.out_gate = (int(q_rank) if q_rank is not None else None), bool(out_gate)
        self.q_head = self.qk_dim + self.rot_dim                     # a query head: plain entries, then the turned ones
        self.key_dim = self.rank + self.rot_dim                      # what a token caches: the latent, then the turned key part
        self.row_width = (self.key_dim + 7) // 8 * 8                 # ... in a cache row padded to what the kernels take
        self.q_dim, self.o_dim = self.num_heads * self.q_head, self.num_heads * self.v_dim
        self.w_in = self.g = self.gq = self.w_uq = self.w_uk_t = self.w_uv = self.sinks = self.w_o = None
        self._inv_freq: Optional[torch.Tensor] = None
        # where the parts of the stacked input product lie: [query (latent) | latent + key part | gate]
        self.q_cols = self.q_rank if self.q_rank is not None else self.q_dim
        self.c_off = self.q_cols
        self.g_off = self.c_off + (self.key_dim if self.own_latent else 0)

    def cache_need(self):
        return PagedKVNeed(1, self.row_width, self.cache_window, planes=1)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        specs = {nm["uk"]: TensorSpec((self.num_heads * self.qk_dim, self.rank)),
                 nm["uv"]: TensorSpec((self.o_dim, self.rank)), nm["o"]: TensorSpec((h, self.o_dim))}
        if self.q_rank is not None:
            specs[nm["dq"]] = TensorSpec((self.q_rank, h))
            specs[nm["dq_norm"]] = TensorSpec((self.q_rank,), init=("one_plus_normal", 0.01))
            specs[nm["uq"]] = TensorSpec((self.q_dim, self.q_rank))
        else:
            specs[nm["q"]] = TensorSpec((self.q_dim, h))
        if self.own_latent:
            specs[nm["dkv"]] = TensorSpec((self.key_dim, h))
            specs[nm["dkv_norm"]] = TensorSpec((self.rank,), init=("one_plus_normal", 0.01))
        if self.has_sinks:
            specs[nm["sink"]] = TensorSpec((self.num_heads,), init=("normal", 0.05))
        if self.out_gate:
            specs[nm["g"]] = TensorSpec((self.o_dim, h))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm, heads = self.names, self.num_heads
        # the query (or its latent), the latent's down-projection and the gate read the same input: one stacked product
        parts = [tensors[nm["dq"] if self.q_rank is not None else nm["q"]]]
        if self.own_latent:
            parts.append(tensors[nm["dkv"]])
            self.g = tensors[nm["dkv_norm"]].contiguous()
        if self.out_gate:
            parts.append(tensors[nm["g"]])
        self.w_in = _stack(parts) if len(parts) > 1 else parts[0].contiguous()
        if self.q_rank is not None:
            self.gq, self.w_uq = tensors[nm["dq_norm"]].contiguous(), tensors[nm["uq"]].contiguous()
        # [heads, row_width, q_head]: the rows of Wuk_h^T, so that q_h -> latent space is an ordinary "x @ w.T" per head;
        # with a turned part an identity block carries it across unchanged (1 * x + 0 + ... is exact), zeros pad the row
        uk = tensors[nm["uk"]].view(heads, self.qk_dim, self.rank)
        w = torch.zeros((heads, self.row_width, self.q_head), dtype=uk.dtype, device=uk.device)
        w[:, :self.rank, :self.qk_dim] = uk.transpose(1, 2)
        if self.rot_dim:
            w[:, self.rank:self.key_dim, self.qk_dim:] = torch.eye(self.rot_dim, dtype=uk.dtype, device=uk.device)
        self.w_uk_t = w.contiguous()
        uv = tensors[nm["uv"]].view(heads, self.v_dim, self.rank)
        w = torch.zeros((heads, self.v_dim, self.row_width), dtype=uv.dtype, device=uv.device)
        w[:, :, :self.rank] = uv                                      # the values are the latent: what lies behind it meets zeros
        self.w_uv = w.contiguous()
        self.sinks = tensors[nm["sink"]].float().contiguous() if self.has_sinks else None
        self.w_o = tensors[nm["o"]].contiguous()

    def _frequencies(self, device: torch.device) -> torch.Tensor:
        """float32: 1 / powf(rot_base, float(2i) / float(rot_dims))."""
        if self._inv_freq is None or self._inv_freq.device != device:
            expo = torch.arange(0, self.rot_dims, 2, dtype=torch.float32) / torch.tensor(float(self.rot_dims), dtype=torch.float32)
            self._inv_freq = (1.0 / torch.pow(torch.tensor(self.rot_base, dtype=torch.float32), expo)).to(device)
        return self._inv_freq

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
        plain = self.rot_dim == 0 and self.q_rank is None and self.row_width == self.rank
        if plain:
            if self.own_latent:
                ops.rmsnorm_append(proj[:, self.q_dim:], self.g, self.eps, cache.tensor, ctx.tables[cache.group],
                                   ctx.tok_seg, ctx.positions, cache.page_size, cache.page_stride)
            q = proj[:, :self.q_dim]
        else:
            freq = self._frequencies(x.device) if self.rot_dims else None
            cq = ctx.empty(n, self.q_rank) if self.q_rank is not None else None
            if self.own_latent or cq is not None:
                # the query latent's norm, and the latent's norm with the key part's turn, straight into the pages
                ops.latent_prepare(proj, 0, self.q_rank or 0, self.gq, cq, self.c_off, self.rank, self.g if self.own_latent else self.gq,
                                   self.rot_dim, self.rot_dims, self.rot_interleaved, freq, self.eps,
                                   cache if self.own_latent else None, ctx.tables[cache.group], ctx.tok_seg, ctx.positions)
            if cq is not None:
                q = ctx.empty(n, self.q_dim)
                ops.linear(cq, self.w_uq, None, q)
            else:
                q = proj[:, :self.q_dim]
            if self.rot_dims:
                ops.rotary(q, q, ctx.positions, freq, heads, 0, self.q_head, self.qk_dim, self.rot_dims, self.rot_interleaved)
        q_lat = ctx.empty(n, heads, self.row_width)
        ops.linear_per_head(q, self.w_uk_t, q_lat)
        o_lat = ctx.empty(n, heads, self.row_width)
        ops.attention(q_lat, cache, o_lat, ctx, heads, 1, self.row_width, self.window, self.scale, sinks=self.sinks)
        o = ctx.empty(n, heads, self.v_dim)
        ops.linear_per_head(o_lat, self.w_uv, o)
        o = o.view(n, self.o_dim)
        if self.out_gate:
            ops.sigmoid_mul(o, proj[:, self.g_off: self.g_off + self.o_dim])
        return o
