"""Gated feed-forward: ``down(up(x) * act(gate(x)))`` with SiLU, no biases unless asked
(src/frontend/models/transformer_forward.cpp:128-137, src/backend/ops/swiglu/cpu/swiglu_cpu.cpp:13-20).
Gate and up weights are stacked at load so one product makes both."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, StepContext, register_feed_forward


def _stack(tensors):
    """Concatenate along dim 0; if storage dtypes differ, float32 wins."""
    dtype = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype
    return torch.cat([t.to(dtype) for t in tensors], dim=0).contiguous()


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (only 'silu')")
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("gated_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size, self.bias = int(hidden_size), int(intermediate_size), bool(bias)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.b_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.b_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                 "down_proj.weight": TensorSpec((h, i))}
        if self.bias:
            specs.update({"gate_proj.bias": TensorSpec((i,)), "up_proj.bias": TensorSpec((i,)),
                          "down_proj.bias": TensorSpec((h,))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = _stack([tensors["gate_proj.weight"], tensors["up_proj.weight"]])
        self.w_down = tensors["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gate_up = _stack([tensors["gate_proj.bias"], tensors["up_proj.bias"]])
            self.b_down = tensors["down_proj.bias"].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_silu_mul(x, self.w_gate_up, self.b_gate_up, act)     # activation in the product's epilogue where it can be
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, self.b_down, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, self.b_down)   # the product, or partial sums over K


@register_feed_forward("squared_relu_mlp")
class SquaredReluMLP(FeedForward):
    """``down(relu(up(x))^2)``, no gate, no biases."""
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, up_name: str = "up", down_name: str = "down"):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("squared_relu_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.up_name, self.down_name = up_name, down_name
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.up_name: TensorSpec((self.intermediate_size, self.hidden_size)),
                self.down_name: TensorSpec((self.hidden_size, self.intermediate_size))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_relu2(x, self.w_up, act)               # the activation in the product's epilogue where it can be
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, None)


@register_feed_forward("clamped_gated_mlp")
class ClampedGatedMLP(FeedForward):
    """``down(g * sigmoid(slope * g) * (u + up_offset))`` with ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit,
    limit)``; no biases.  ``limit=None``: no clamping."""
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: Optional[float], slope: float = 1.0,
                 up_offset: float = 0.0, gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("clamped_gated_mlp: sizes must be positive")
        if limit is not None and not limit > 0.0:
            raise ValueError(f"clamped_gated_mlp: limit={limit} must be positive (or None)")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.slope, self.up_offset = (float(limit) if limit is not None else 0.0), float(slope), float(up_offset)
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {self.gate_name: TensorSpec((i, h)), self.up_name: TensorSpec((i, h)), self.down_name: TensorSpec((h, i))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = _stack([tensors[self.gate_name], tensors[self.up_name]])
        self.w_down = tensors[self.down_name].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_gated_clamp_mul(x, self.w_gate_up, act, self.limit, self.slope, self.up_offset)
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, None)
