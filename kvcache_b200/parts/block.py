"""The arrangement of parts in one layer: pre-norm residual block
(reference order: apps/qwen_serve.cu:101-116)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, Block, FeedForward, LayerContext, Mixer, Norm, Part, ScaledDelta


class LayerScale(Part):
    """A learned number per residual channel that multiplies a sublayer's result before it is added (float32 on the
    device); the multiplication runs inside the launch that adds the result (`ScaledDelta`)."""

    def __init__(self, width: int, name: str):
        self.width, self.name = width, name
        self.scale: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.width,))}

    def init_kinds(self) -> Dict[str, str]:
        return {self.name: "ones_plus_normal"}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.scale = tensors[self.name].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.width * 4


class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += ffn(norm2(h)).

    Each add is folded into the norm that follows it, so the block takes the
    previous layer's delta as `pending` and hands its own feed-forward delta on.
    `ffn` (with `norm2`) may be None: the layer then ends after its mixer.  `scale1` / `scale2` (`LayerScale`): the
    sublayer's result is multiplied channel by channel before the add, h += scale * sublayer(norm(h)).
    """

    def __init__(self, width: int, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: str,
                 scale1: Optional[LayerScale] = None, scale2: Optional[LayerScale] = None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        if ffn is None and scale2 is not None:
            raise ValueError("a scale of the feed-forward's result without a feed-forward")
        self.width = width
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.scale1, self.scale2 = scale1, scale2
        self.dtype = TORCH_DTYPES[dtype]

    def _parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.scale1, self.scale2) if p is not None)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def init_kinds(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for part in self._parts():
            out.update(part.init_kinds())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        for part in self._parts():
            part.bind(tensors, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self._parts())

    def supports_fold(self, kernels, num_rows: int) -> bool:
        return (self.ffn is not None and self.scale1 is None and self.scale2 is None
                and self.mixer.supports_fold(self.norm1, kernels, num_rows)
                and self.ffn.supports_fold(self.norm2, kernels, num_rows))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, ctx: LayerContext) -> None:
        self.mixer.forward_folded(h, h16, self.norm1, ctx)
        self.ffn.forward_folded(h, h16, self.norm2, ctx)

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: LayerContext) -> Optional[torch.Tensor]:
        T = h.shape[0]
        x = ctx.workspace.buffer("block.normed", (T, self.width), self.dtype)
        self.norm1.add_norm(h, pending, x, ctx)
        delta = self.mixer.forward(x, ctx)
        if self.scale1 is not None:
            delta = ScaledDelta(delta, self.scale1.scale)
        if self.ffn is None:
            return delta
        self.norm2.add_norm(h, delta, x, ctx)
        delta = self.ffn.forward(x, ctx)
        return ScaledDelta(delta, self.scale2.scale) if self.scale2 is not None else delta


class SandwichBlock(Block):
    """h += post1(mixer(pre1(h))); h += post2(ffn(pre2(h))): a norm before and after each sublayer.

    The normalisation of a sublayer's result and its add are folded into the norm that follows (one launch computes
    both sums of squares), so the block takes the layer before's `NormedDelta` as `pending` and hands its own on.
    `ffn` may be None: the layer then ends after its mixer.  `gate1` / `gate2` (`ResidualGate`): the sublayer's result is
    multiplied by sigmoid(W x + b), x being the rows the norm before the sublayer made, before its own norm; the
    multiplication runs inside the launch that normalises and adds the result.
    """

    def __init__(self, width: int, pre1: Norm, mixer: Mixer, post1: Norm, pre2: Optional[Norm], ffn: Optional[FeedForward],
                 post2: Optional[Norm], dtype: str, gate1: Optional["ResidualGate"] = None, gate2: Optional["ResidualGate"] = None):
        if (ffn is None) != (pre2 is None) or (ffn is None) != (post2 is None):
            raise ValueError("a feed-forward comes with its two norms, or none of the three is given")
        if ffn is None and gate2 is not None:
            raise ValueError("a gate of the feed-forward's result without a feed-forward")
        self.width = width
        self.pre1, self.mixer, self.post1, self.pre2, self.ffn, self.post2 = pre1, mixer, post1, pre2, ffn, post2
        self.gate1, self.gate2 = gate1, gate2
        self.dtype = TORCH_DTYPES[dtype]

    def _parts(self):
        return tuple(p for p in (self.pre1, self.mixer, self.post1, self.pre2, self.ffn, self.post2, self.gate1, self.gate2)
                     if p is not None)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def init_kinds(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for part in self._parts():
            out.update(part.init_kinds())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        for part in self._parts():
            part.bind(tensors, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self._parts())

    def forward(self, h: torch.Tensor, pending, ctx: LayerContext):
        from .base import NormedDelta
        T = h.shape[0]
        x = ctx.workspace.buffer("block.normed", (T, self.width), self.dtype)
        self.pre1.add_norm(h, pending, x, ctx)
        gate = self.gate1.forward(x, ctx, "block.gate1") if self.gate1 is not None else None
        delta = NormedDelta(self.mixer.forward(x, ctx), self.post1, gate)
        if self.ffn is None:
            return delta
        self.pre2.add_norm(h, delta, x, ctx)
        gate = self.gate2.forward(x, ctx, "block.gate2") if self.gate2 is not None else None
        return NormedDelta(self.ffn.forward(x, ctx), self.post2, gate)


class ResidualGate(Part):
    """Logits of a gate on a sublayer's result: W x + b, one number per residual channel, in the compute type.  The
    sigmoid and the multiplication happen where the result is normalised and added (`NormedDelta.gate`)."""

    def __init__(self, width: int, weight_name: str, bias_name: str, dtype: str):
        self.width = width
        self.weight_name, self.bias_name = weight_name, bias_name
        self.dtype = TORCH_DTYPES[dtype]
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width, self.width)), self.bias_name: TensorSpec((self.width,))}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.weight = tensors[self.weight_name].to(self.dtype).to(device).contiguous()
        self.bias = tensors[self.bias_name].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size() + self.width * 4

    def forward(self, x: torch.Tensor, ctx: LayerContext, buffer_name: str) -> torch.Tensor:
        logits = ctx.workspace.buffer(buffer_name, (x.shape[0], self.width), self.dtype)
        ctx.kernels.linear(x, self.weight, logits, self.bias)
        return logits
