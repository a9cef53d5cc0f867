"""Dense gated feed-forward (reference: apps/qwen_serve.cu:112-116, src/qwen_kernels.cu:102-105)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, FeedForward, LayerContext


GATED_ACTIVATIONS = ("silu", "clamped_swiglu")


class GatedMLP(FeedForward):
    """delta = act(x Wg^T, x Wu^T) Wd^T; no biases.  act is "silu": silu(g) * u, or "clamped_swiglu":
    g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit) and u' = clamp(u, -limit, limit)."""

    def __init__(self, hidden: int, intermediate: int, *, activation: str, prefix: str, dtype: str,
                 names: Sequence[str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight"), limit: float = 0.0):
        """`names`: what the gate, up and down matrices are called after `prefix` in the checkpoint."""
        self.names = tuple(names)
        if activation not in GATED_ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not supported by the gated feed-forward kernel")
        if activation == "clamped_swiglu" and not limit > 0.0:
            raise ValueError("the clamped activation needs a positive limit")
        self.activation, self.limit = activation, float(limit)
        self.hidden, self.intermediate = hidden, intermediate
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.interleaved = False
        self.delta_name = "ffn.delta"          # the workspace buffer of the result (another name where two run in one layer)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        gate, up, down = self.names
        return {
            f"{p}{gate}": TensorSpec((self.intermediate, self.hidden)),
            f"{p}{up}": TensorSpec((self.intermediate, self.hidden)),
            f"{p}{down}": TensorSpec((self.hidden, self.intermediate)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        gate, up = tensors[f"{p}{self.names[0]}"], tensors[f"{p}{self.names[1]}"]
        # One projection for gate and up.  When the width allows, rows are interleaved in eights (gate rows
        # 8 b .. 8 b + 7, then the up rows of the same indices) so that a kernel's thread holds both values
        # of an index and can write the activation without a second pass.
        self.interleaved = self.intermediate % 8 == 0
        if self.interleaved:
            both = torch.stack([gate.view(-1, 8, self.hidden), up.view(-1, 8, self.hidden)], dim=1).reshape(-1, self.hidden)
        else:
            both = torch.cat([gate, up], dim=0)
        self.w_gate_up = both.to(self.dtype).to(device).contiguous()
        self.w_down = tensors[f"{p}{self.names[2]}"].to(self.dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def supports_fold(self, norm, kernels, num_rows: int) -> bool:
        can = getattr(kernels, "can_fold", None)
        return (can is not None and self.interleaved and self.activation == "silu" and norm.fold_params() is not None
                and can(self.dtype, num_rows, self.hidden, 2 * self.intermediate)
                and can(self.dtype, num_rows, self.intermediate, self.hidden))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm, ctx: LayerContext) -> None:
        T = h.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        weight, eps = norm.fold_params()
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.norm_gate_up_act(h16, self.w_gate_up, weight, eps, act)
        k.linear_into_residual(act, self.w_down, h, h16)


    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        if self.activation == "silu":
            k.gate_up_act(x, self.w_gate_up, act, ws, self.interleaved)
        else:
            k.gate_up_act(x, self.w_gate_up, act, ws, self.interleaved, activation=self.activation, limit=self.limit)
        delta = ws.buffer(self.delta_name, (T, self.hidden), self.dtype)
        k.linear(act, self.w_down, delta)
        return delta


class ReluSquaredMLP(FeedForward):
    """delta = Wdown relu(Wup x)^2; no biases, no gate."""

    def __init__(self, hidden: int, intermediate: int, *, prefix: str, dtype: str, names: Sequence[str] = ("up", "down")):
        self.hidden, self.intermediate = hidden, intermediate
        self.prefix, self.names = prefix, tuple(names)
        self.dtype = TORCH_DTYPES[dtype]
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        up, down = self.names
        return {self.prefix + up: TensorSpec((self.intermediate, self.hidden)),
                self.prefix + down: TensorSpec((self.hidden, self.intermediate))}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.w_up = tensors[self.prefix + self.names[0]].to(self.dtype).to(device).contiguous()
        self.w_down = tensors[self.prefix + self.names[1]].to(self.dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.linear(x, self.w_up, act)
        k.activation_(act, "relu2")
        delta = ws.buffer("ffn.delta", (T, self.hidden), self.dtype)
        k.linear(act, self.w_down, delta)
        return delta


ROUTED_ACTIVATIONS = ("relu2", "clamped_swiglu", "swiglu")


class RoutedMLP(FeedForward):
    """A mixture of small feed-forwards: delta = sum over the `top` chosen experts e of w_e * expert_e(x) (+ shared(x));
    no biases.  The router's logits are float32 (from the rows in the compute type).

    `scores`: "chosen" - the experts with the largest logits, weights = softmax over the chosen logits only;
    "all" - weights = the softmax over all experts' logits at the chosen ones, as they are (they do not sum to 1).
    `activation`: "relu2" - expert(x) = Wdown relu(Wup x)^2 (`expert_names` = up, down); "clamped_swiglu" - expert(x) =
    Wdown (g sigmoid(1.702 g) (u + 1)) with g = min(Wgate x, limit), u = clamp(Wup x, -limit, limit) (`expert_names` =
    gate, up, down); "swiglu" - expert(x) = Wdown (silu(Wgate x) * (Wup x)), the same three names.  `shared`: a
    feed-forward that every row takes, added to the routed sum.  `router_bias`: the name of a bias of the router's logits
    (one float32 number per expert), or None.

    The experts' matrices are stacked ([experts, ff, hidden] - gate and up rows in turn, [experts, 2 ff, hidden], for the
    gated form - and [experts, hidden, ff]) so that one grouped product serves all of them; which rows go to which expert
    is decided on the device, and the launches do not depend on it.
    """

    def __init__(self, hidden: int, expert_ff: int, experts: int, top: int, *, activation: str, prefix: str, dtype: str,
                 router_name: str = "router", expert_names: Optional[Sequence[str]] = None, scores: str = "chosen",
                 limit: float = 0.0, shared: Optional[FeedForward] = None, router_bias: Optional[str] = None):
        if activation not in ROUTED_ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not supported by the routed feed-forward kernels")
        if not 1 <= top <= experts:
            raise ValueError(f"top {top} of {experts} experts")
        if scores not in ("chosen", "all"):
            raise ValueError(f"scores '{scores}' (chosen, all)")
        if activation == "clamped_swiglu" and not limit > 0.0:
            raise ValueError("the clamped activation needs a positive limit")
        self.hidden, self.expert_ff, self.experts, self.top = hidden, expert_ff, experts, top
        self.activation, self.scores, self.limit = activation, scores, float(limit)
        self.gated = activation in ("clamped_swiglu", "swiglu")
        self.router_bias = router_bias
        self.b_router: Optional[torch.Tensor] = None
        if expert_names is None:
            expert_names = ("e{e}.gate", "e{e}.up", "e{e}.down") if self.gated else ("e{e}.up", "e{e}.down")
        if len(expert_names) != (3 if self.gated else 2):
            raise ValueError(f"{len(expert_names)} expert matrix names for activation '{activation}'")
        self.prefix, self.router_name, self.expert_names = prefix, router_name, tuple(expert_names)
        self.shared = shared
        if shared is not None and hasattr(shared, "delta_name"):
            shared.delta_name = "ffn.shared_delta"
        self.dtype = TORCH_DTYPES[dtype]
        self.w_router: Optional[torch.Tensor] = None
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _expert(self, which: int, e: int) -> str:
        return self.prefix + self.expert_names[which].format(e=e)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.router_name: TensorSpec((self.experts, self.hidden))}
        if self.router_bias is not None:
            specs[self.prefix + self.router_bias] = TensorSpec((self.experts,))
        for e in range(self.experts):
            for which in range(len(self.expert_names) - 1):
                specs[self._expert(which, e)] = TensorSpec((self.expert_ff, self.hidden))
            specs[self._expert(len(self.expert_names) - 1, e)] = TensorSpec((self.hidden, self.expert_ff))
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        return specs

    def init_kinds(self) -> Dict[str, str]:
        return self.shared.init_kinds() if self.shared is not None else {}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        place = lambda t: t.to(self.dtype).to(device).contiguous()
        E = range(self.experts)
        self.w_router = place(tensors[self.prefix + self.router_name])
        if self.router_bias is not None:
            self.b_router = tensors[self.prefix + self.router_bias].to(torch.float32).to(device).contiguous()
        if self.gated:
            # Row 2 i is gate row i, row 2 i + 1 up row i: a product's thread holds both numbers of an index.
            self.w_up = place(torch.stack([torch.stack([tensors[self._expert(0, e)], tensors[self._expert(1, e)]], dim=1)
                                           .reshape(2 * self.expert_ff, self.hidden) for e in E]))
        else:
            self.w_up = place(torch.stack([tensors[self._expert(0, e)] for e in E]))
        self.w_down = place(torch.stack([tensors[self._expert(len(self.expert_names) - 1, e)] for e in E]))
        if self.shared is not None:
            self.shared.bind(tensors, device)

    def weight_bytes(self) -> int:
        """Bytes one row reads: the router and its `top` experts (a step of many rows reads up to all experts)."""
        size = self.w_up.element_size()
        per_expert = (3 if self.gated else 2) * self.expert_ff * self.hidden
        shared = self.shared.weight_bytes() if self.shared is not None else 0
        return (self.w_router.numel() + self.top * per_expert) * size + shared

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        base = self.shared.forward(x, ctx) if self.shared is not None else None
        logits = ws.buffer("moe.logits", (T, self.experts), torch.float32)
        k.linear(x, self.w_router, logits, self.b_router)
        chosen = ws.buffer("moe.chosen", (T, self.top), torch.int32)
        share = ws.buffer("moe.share", (T, self.top), torch.float32)
        delta = ws.buffer("ffn.delta", (T, self.hidden), self.dtype)
        if self.scores == "chosen" and not self.gated and base is None:
            k.route_top(logits, chosen, share)
            k.routed_experts(x, self.w_up, self.w_down, chosen, share, delta, self.activation, ws)
        else:
            k.route_top(logits, chosen, share, scores=self.scores)
            k.routed_experts(x, self.w_up, self.w_down, chosen, share, delta, self.activation, ws, limit=self.limit, base=base)
        return delta
