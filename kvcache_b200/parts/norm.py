"""RMSNorm with the residual add folded in (reference: src/qwen_kernels.cu:26-43 after :55-61)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import LayerContext, Norm, NormedDelta, ScaledDelta


class RMSNorm(Norm):
    """y = v * rsqrt(mean(v^2) + eps) * weight * gain, v = h + delta, in float32; the weight stays float32.  `gain`: a
    constant of the architecture that multiplies the normalised rows (a residual multiplier); it is folded into the
    device copy of the weight.  `offset`: the checkpoint stores weight - offset (a weight kept around zero: offset 1);
    the sum is made in float32 when the weight is bound."""

    def __init__(self, width: int, eps: float, weight_name: str, gain: float = 1.0, offset: float = 0.0):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.gain = float(gain)
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,))}

    def init_kinds(self) -> Dict[str, str]:
        return {self.weight_name: "ones_plus_normal" if self.offset == 0.0 else "normal"}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        weight = tensors[self.weight_name].to(torch.float32) + self.offset
        self.weight = (weight if self.gain == 1.0 else weight * self.gain).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.width * 4

    def add_norm(self, h, delta, out, ctx: LayerContext, rows=None, tail=None) -> None:
        if isinstance(delta, ScaledDelta):
            if out is None or tail is not None:
                raise ValueError("a delta with a scale per channel is added by the launch that also normalises the rows")
            ctx.kernels.add_rmsnorm(h, delta.delta, self.weight, self.eps, out, rows, delta_scale=delta.scale)
            return
        if isinstance(delta, NormedDelta) or out is None or tail is not None:
            # h += post.norm(delta), then this norm: one launch for both sums of squares.
            post = delta.post.fold_params() if isinstance(delta, NormedDelta) else None
            if isinstance(delta, NormedDelta) and post is None:
                raise ValueError("a delta can be normalised before the add only by a norm of the form v * rsqrt(mean(v^2) + eps) * w")
            d = delta.delta if isinstance(delta, NormedDelta) else delta
            gate = delta.gate if isinstance(delta, NormedDelta) else None
            extra = {} if gate is None else {"delta_gate": gate}
            ctx.kernels.norm_add_rmsnorm(h, d, post[0] if post else None, post[1] if post else 0.0, self.weight, self.eps, out,
                                         rows, tail, **extra)
            return
        ctx.kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)

    def fold_params(self):
        return self.weight, self.eps


class PassNorm(Norm):
    """No normalisation: adds the pending delta (normalised by its own norm if it is a `NormedDelta`) and hands the
    rows on as they are, rounded to the compute type - the place of a norm in a block whose sublayers read the
    residual stream itself."""

    def add_norm(self, h, delta, out, ctx: LayerContext, rows=None, tail=None) -> None:
        post = delta.post.fold_params() if isinstance(delta, NormedDelta) else None
        if isinstance(delta, NormedDelta) and post is None:
            raise ValueError("a delta can be normalised before the add only by a norm of the form v * rsqrt(mean(v^2) + eps) * w")
        d = delta.delta if isinstance(delta, NormedDelta) else delta
        gate = delta.gate if isinstance(delta, NormedDelta) else None
        extra = {} if gate is None else {"delta_gate": gate}
        ctx.kernels.norm_add_rmsnorm(h, d, post[0] if post else None, post[1] if post else 0.0, None, 0.0, out, rows, tail, **extra)
