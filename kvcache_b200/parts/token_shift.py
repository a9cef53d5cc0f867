"""Token shift: a mixer reads a blend of each row with the row of the token before it.

s_t = x_t + (x_{t-1} - x_t) * w, element by element, with x_{-1} = 0 for a request's first token.  The row of the last
token a request has run is part of its state (one row per request, float32 holding the rows' own values), so that a
portion's first token finds its predecessor whatever way the request was cut.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, Mixer, StateSpec

PREVIOUS = "shift.previous"
INNER = "inner"


class TokenShiftMixer(Mixer):
    """Wraps a mixer: shifts the rows, then runs it.  The wrapped mixer's states are kept under `inner` / `inner.<name>`."""

    def __init__(self, width: int, inner: Mixer, weight_name: str, dtype: str):
        self.width, self.inner, self.weight_name = width, inner, weight_name
        self.dtype = TORCH_DTYPES[dtype]
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {**self.inner.tensor_specs(), self.weight_name: TensorSpec((self.width,))}

    def init_kinds(self) -> Dict[str, str]:
        return self.inner.init_kinds()

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.inner.bind(tensors, device)
        self.weight = tensors[self.weight_name].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.inner.weight_bytes() + self.width * 4

    def cache_spec(self):
        return self.inner.cache_spec()

    def state_spec(self):
        spec = self.inner.state_spec()
        named = {} if spec is None else ({f"{INNER}.{name}": s for name, s in spec.items()} if isinstance(spec, dict) else {INNER: spec})
        return {PREVIOUS: StateSpec((self.width,)), **named}

    def step_planners(self, kernels):
        return self.inner.step_planners(kernels)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        shifted = ctx.workspace.buffer("shift.rows", (x.shape[0], self.width), self.dtype)
        ctx.kernels.token_shift(x, self.weight, ctx.state[PREVIOUS], ctx.batch, shifted)
        spec = self.inner.state_spec()
        state = None
        if isinstance(spec, dict):
            state = {name: ctx.state[f"{INNER}.{name}"] for name in spec}
        elif spec is not None:
            state = ctx.state[INNER]
        inner = LayerContext(batch=ctx.batch, kernels=ctx.kernels, workspace=ctx.workspace, kv=ctx.kv, state=state,
                             call_index=ctx.call_index, embedded=ctx.embedded)
        return self.inner.forward(shifted, inner)
