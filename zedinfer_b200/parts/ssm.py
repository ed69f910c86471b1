"""Selective state-space mixer in the Mamba-2 form: a recurrent state per request instead of cached keys and values.

Per token, with ``H`` heads of ``vdim`` columns, a state of ``N`` rows, ``G`` groups that share B and C, and
``inner = H * vdim``:

    [z | x | B | C | dt] = Win h                      (inner, inner, G N, G N, H columns)
    [x | B | C] <- silu(conv([x | B | C]) + bias)     causal, per channel, ``taps`` wide, zeros before the start
    dt <- softplus(dt + dt_bias)                      float32, no clamp
    per head a (group a // (H / G)):   S_t = exp(-exp(A_log_a) dt_t) S_(t-1) + dt_t B_t x_t^T     (S is N x vdim, float32)
                                       y_t = S_t^T C_t + D_a x_t
    out = Wo (unit_rms_per_part(y * silu(z)) * g)     the gate first, then the norm in ``norm_groups`` equal parts

What a request carries from step to step is one slot of fixed-size float32 state: S of every head and the convolution's
last ``taps - 1`` inputs (the pre-activation columns of x, B and C).  A step runs the tokens it brings from that state and
leaves the state behind its last token, so a prompt may be cut anywhere and a decoded token is a portion of one.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView, StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, register_mixer

STRETCHWISE_MIN_TOKENS = 256      # steps of at least this many tokens (bfloat16) run their segments in stretches side by side

_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D", "norm": "norm",
          "o": "o"}


def step_segment_bounds(ctx: StepContext) -> Optional[torch.Tensor]:
    """int32 ``[segments, 2]`` on the device: first and one-past-last token of every segment of the step, made once per
    step and shared by the layers that walk segments; None for a step of single tokens (segment s is token s)."""
    if ctx.decode_only:
        return None
    key = ("segment_bounds",)
    b = ctx.step_cache.get(key)
    if b is None:
        b = torch.empty((ctx.n_segments, 2), dtype=torch.int32, device=ctx.device)
        ops.segment_bounds(ctx.tok_seg, ctx.n_segments, b)
        ctx.step_cache[key] = b
    return b


@register_mixer("mamba2")
class Mamba2Mixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, heads: int, vdim: int, state: int, groups: int, conv: int, norm_groups: int,
                 eps: float, names: Optional[Mapping[str, str]] = None):
        if min(hidden_size, heads, vdim, state, groups, conv, norm_groups) <= 0:
            raise ValueError("mamba2: every size must be positive")
        if heads % groups:
            raise ValueError(f"mamba2: {heads} heads cannot share {groups} groups of B and C")
        if (heads * vdim) % norm_groups:
            raise ValueError(f"mamba2: {norm_groups} norm groups do not divide the inner width {heads * vdim}")
        if state > 512:
            raise ValueError(f"mamba2: state={state} is not supported; the scan kernel takes at most 512")
        self.hidden_size, self.heads, self.vdim, self.n_state = int(hidden_size), int(heads), int(vdim), int(state)
        self.groups, self.taps, self.norm_groups, self.eps = int(groups), int(conv), int(norm_groups), float(eps)
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state          # what the convolution sees: x | B | C
        self.proj_width = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.state_elems = self.inner * self.n_state
        self.names = dict(_NAMES)
        self.names.update(names or {})
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.d = self.g = self.w_o = None

    def cache_need(self):
        # the recurrent state [heads, vdim, state], then the convolution's ring [taps - 1, channels]
        return StateNeed((self.state_elems + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        return {nm["in"]: TensorSpec((self.proj_width, h)), nm["conv"]: TensorSpec((self.channels, self.taps), init=("normal", 0.2)),
                nm["conv_bias"]: TensorSpec((self.channels,)), nm["dt_bias"]: TensorSpec((self.heads,)),
                nm["a_log"]: TensorSpec((self.heads,)), nm["d"]: TensorSpec((self.heads,), init=("one_plus_normal", 0.01)),
                nm["norm"]: TensorSpec((self.inner,), init=("one_plus_normal", 0.01)), nm["o"]: TensorSpec((h, self.inner))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = tensors[nm["in"]].contiguous()
        self.w_conv, self.b_conv = tensors[nm["conv"]].contiguous(), tensors[nm["conv_bias"]].contiguous()
        # what enters the recurrence is float32
        self.dt_bias, self.a_log, self.d = (tensors[nm[k]].float().contiguous() for k in ("dt_bias", "a_log", "d"))
        self.g, self.w_o = tensors[nm["norm"]].contiguous(), tensors[nm["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._mix(x, ctx, cache, owns_cache), self.w_o, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        return ops.linear_for_residual(self._mix(x, ctx, cache, owns_cache), self.w_o, None)

    def _mix(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        """Everything up to the output projection: ``[tokens, inner]``."""
        if cache.kind != "state" or not owns_cache:
            raise RuntimeError("a state-space mixer needs a state slot of its own")
        if ctx.slots is None:
            raise RuntimeError("a state-space mixer needs the step's state slots")
        n, inner = x.shape[0], self.inner
        state = cache.tensor
        proj = ctx.empty(n, self.proj_width)
        ops.linear(x, self.w_in, None, proj)
        raw = proj[:, inner: inner + self.channels]
        bounds = step_segment_bounds(ctx)
        tok_seg = None if ctx.decode_only else ctx.tok_seg
        xbc = ctx.empty(n, self.channels)
        # a step of single tokens: a thread reads its channel's ring alone, so it writes the token's input there itself;
        # otherwise the ring is written by a second launch, once every token of the portion has read it
        single = tok_seg is None
        ops.causal_conv_silu(raw, self.w_conv, self.b_conv, state, self.state_elems, ctx.slots, tok_seg, ctx.positions, xbc,
                             update_state=single)
        if not single:
            ops.conv_state_update(raw, self.taps, state, self.state_elems, ctx.slots, bounds, ctx.positions, ctx.n_segments)
        y = ctx.empty(n, inner, dtype=torch.float32)
        # float32 steps walk every segment in one order whatever the cut; long bfloat16 portions run in stretches side by side
        stretchwise = bounds is not None and x.dtype == torch.bfloat16 and n >= STRETCHWISE_MIN_TOKENS
        ops.ssm_scan(xbc, proj[:, inner + self.channels:], self.dt_bias, self.a_log, self.d, state, ctx.slots, bounds, y,
                     ctx.n_segments, self.heads, self.vdim, self.n_state, self.groups, stretchwise=stretchwise)
        out = ctx.empty(n, inner)
        ops.gated_group_rmsnorm(y, proj[:, :inner], self.g, self.norm_groups, self.eps, out)
        return out
