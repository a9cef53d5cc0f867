"""Mixers that carry a matrix of fixed size per request and head from token to token instead of keys and values.

Both keep a state S [key channels, value channels] per head with S_t = decay_t S_{t-1} + gain_t k_t v_t^T and read it
with the query, o_t = S_t^T q_t.  They differ in the decay (one number per key channel, or one per head with an input
gate and a running maximum that keeps the exponentials in range) and in what follows the read-out.  The state lives in
float32 in the request's slot (`StateSpec`), is zero at admission, and everything that enters the recurrence besides
the projections themselves is float32: the projections are written as float32 rows, and the decays, gates and norms
are computed from them inside the kernels.  The same kernel serves prompts, portions and single tokens (a token's
result is bit for bit the same however the request was cut).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec, WeightError
from .base import TORCH_DTYPES, LayerContext, Mixer, StateSpec


class _MatrixStateMixer(Mixer):
    """What the two mixers share: sizes, the fused input projection with float32 rows, the output matrix."""

    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, *, eps: float, prefix: str, dtype: str):
        self.hidden, self.num_heads, self.dim, self.vdim = hidden, num_heads, dim, vdim
        self.eps = float(eps)
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.qk_size, self.heads_width = num_heads * dim, num_heads * vdim
        self.q_scale = 1.0 / math.sqrt(dim)
        self.w_in: Optional[torch.Tensor] = None
        self.b_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        # Columns of the fused projection: [q | k | v | gate of the result | ...].
        self.q_col, self.k_col, self.v_col, self.g_col = 0, self.qk_size, 2 * self.qk_size, 2 * self.qk_size + self.heads_width

    def _base_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        return {p + "q": TensorSpec((self.qk_size, self.hidden)), p + "k": TensorSpec((self.qk_size, self.hidden)),
                p + "v": TensorSpec((self.heads_width, self.hidden)), p + "g": TensorSpec((self.heads_width, self.hidden)),
                p + "o": TensorSpec((self.hidden, self.heads_width))}

    def init_kinds(self) -> Dict[str, str]:
        return {self.prefix + "norm": "ones_plus_normal"}

    def _place(self, t: torch.Tensor, device: torch.device) -> torch.Tensor:
        return t.to(self.dtype).to(device).contiguous()

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def weight_bytes(self) -> int:
        mats = [m for m in (self.w_in, self.w_o) if m is not None]
        return sum(m.numel() * m.element_size() for m in mats)

    def _project(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        proj = ctx.workspace.buffer("recurrent.proj", (x.shape[0], self.w_in.shape[0]), torch.float32)
        ctx.kernels.linear(x, self.w_in, proj, self.b_in)
        return proj

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        gated = ctx.workspace.buffer("recurrent.gated", (T, self.heads_width), self.dtype)
        self.forward_heads(x, ctx, gated)
        delta = ctx.workspace.buffer("attn.delta", (T, self.hidden), self.dtype)
        ctx.kernels.linear(gated, self.w_o, delta)
        return delta


class GatedLinearAttention(_MatrixStateMixer):
    """q = Wq h / sqrt(dim), k = Wk h, v = Wv h; a decay per key channel a = sigmoid(Wa2 (Wa1 h) + b)^(1 / tau);
    S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; each head's o divided by its root mean square, times a weight
    of vdim numbers that the heads share, times silu(Wg h); then the output matrix."""

    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, decay_rank: Optional[int], tau: float, *, eps: float,
                 prefix: str, dtype: str):
        super().__init__(hidden, num_heads, dim, vdim, eps=eps, prefix=prefix, dtype=dtype)
        self.decay_rank = decay_rank          # None: whatever the checkpoint's Wa1 and Wa2 agree on
        self.tau = float(tau)
        self.w_a1 = self.w_a2 = self.b_a2 = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        specs = self._base_specs()
        specs.update({p + "norm": TensorSpec((self.vdim,)), p + "a1": TensorSpec((self.decay_rank, self.hidden)),
                      p + "a2": TensorSpec((self.qk_size, self.decay_rank)), p + "a2.b": TensorSpec((self.qk_size,))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        self.w_in = self._place(torch.cat([tensors[p + n] for n in "qkvg"], dim=0), device)
        if tensors[p + "a1"].shape[0] != tensors[p + "a2"].shape[1]:
            raise WeightError(f"{p}a1 has {tensors[p + 'a1'].shape[0]} rows but {p}a2 has {tensors[p + 'a2'].shape[1]} columns")
        self.w_a1, self.w_a2 = self._place(tensors[p + "a1"], device), self._place(tensors[p + "a2"], device)
        self.b_a2 = tensors[p + "a2.b"].to(torch.float32).to(device).contiguous()
        self.w_o = self._place(tensors[p + "o"], device)
        self.norm = tensors[p + "norm"].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return super().weight_bytes() + sum(m.numel() * m.element_size() for m in (self.w_a1, self.w_a2))

    def state_spec(self):
        # [head, key channel, value channel]: the scan's lanes own value channels, so a key channel's row is read at once.
        return {"memory": StateSpec((self.num_heads, self.dim, self.vdim))}

    def forward_heads(self, x: torch.Tensor, ctx: LayerContext, out: torch.Tensor, out_col: int = 0, scale: float = 1.0) -> None:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        proj = self._project(x, ctx)
        low = ws.buffer("recurrent.low", (T, self.w_a1.shape[0]), self.dtype)
        k.linear(x, self.w_a1, low)
        z = ws.buffer("recurrent.z", (T, self.qk_size), torch.float32)
        k.linear(low, self.w_a2, z, self.b_a2)
        o = ws.buffer("recurrent.o", (T, self.heads_width), torch.float32)
        k.gated_linear_scan(proj, (self.q_col, self.k_col, self.v_col), z, self.tau, self.q_scale, ctx.batch,
                            ctx.state["memory"], o, self.num_heads, self.dim, self.vdim, ws)
        k.head_norm_gate(o, self.norm, self.eps, (proj, self.g_col), "silu", scale, out, out_col, self.num_heads, self.vdim)


class LightningAttention(_MatrixStateMixer):
    """Linear attention with one constant decay per head: q = silu(Wq h), k = silu(Wk h), v = silu(Wv h);
    S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t (no other scale); the heads' results, all of a token's at once, are
    divided by their root mean square, multiplied by a weight over all heads' channels and by sigmoid(Wg h); then the
    output matrix.  `decay`: one number per head, a constant of the model."""

    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, decay, *, eps: float, prefix: str, dtype: str):
        super().__init__(hidden, num_heads, dim, vdim, eps=eps, prefix=prefix, dtype=dtype)
        decay = tuple(float(d) for d in decay)
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.decay_values = decay
        self.decay: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = self._base_specs()
        specs[self.prefix + "norm"] = TensorSpec((self.heads_width,))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        self.w_in = self._place(torch.cat([tensors[p + n] for n in "qkvg"], dim=0), device)
        self.w_o = self._place(tensors[p + "o"], device)
        self.norm = tensors[p + "norm"].to(torch.float32).to(device).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)

    def state_spec(self):
        return {"memory": StateSpec((self.num_heads, self.dim, self.vdim))}

    def forward_heads(self, x: torch.Tensor, ctx: LayerContext, out: torch.Tensor, out_col: int = 0, scale: float = 1.0) -> None:
        k, ws = ctx.kernels, ctx.workspace
        proj = self._project(x, ctx)
        o = ws.buffer("recurrent.o", (x.shape[0], self.heads_width), torch.float32)
        k.lightning_scan(proj, (self.q_col, self.k_col, self.v_col), self.decay, ctx.batch, ctx.state["memory"], o,
                         self.num_heads, self.dim, self.vdim, ws)
        k.head_norm_gate(o, self.norm, self.eps, (proj, self.g_col), "sigmoid", scale, out, out_col, self.num_heads, self.vdim,
                         scope="all")


class MatrixMemory(_MatrixStateMixer):
    """q = Wq h / sqrt(dim), k, v; per head i = cap tanh((Wi h + bi) / cap), f = logsigmoid(cap tanh((Wf h + bf) / cap));
    m_t = max(f + m_{t-1}, i) with m = 0 before the first token; S_t = e^{f + m_{t-1} - m_t} S_{t-1} + e^{i - m_t} k v^T and
    n_t likewise with k alone; o = S_t^T q / (max(|n_t . q|, e^{-m_t}) + 1e-6); each head's o divided by its root mean
    square, times a weight over all heads' value channels, times sigmoid(Wg h); then the output matrix."""

    DENOMINATOR_FLOOR = 1e-6

    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, gate_cap: float, *, eps: float, prefix: str, dtype: str):
        super().__init__(hidden, num_heads, dim, vdim, eps=eps, prefix=prefix, dtype=dtype)
        self.gate_cap = float(gate_cap)
        self.i_col = self.g_col + self.heads_width
        self.f_col = self.i_col + num_heads

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, H = self.prefix, self.num_heads
        specs = self._base_specs()
        specs.update({p + "norm": TensorSpec((self.heads_width,)), p + "i": TensorSpec((H, self.hidden)), p + "i.b": TensorSpec((H,)),
                      p + "f": TensorSpec((H, self.hidden)), p + "f.b": TensorSpec((H,))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        self.w_in = self._place(torch.cat([tensors[p + n] for n in "qkvgif"], dim=0), device)
        bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32)
        bias[self.i_col:self.i_col + self.num_heads] = tensors[p + "i.b"].to(torch.float32)
        bias[self.f_col:self.f_col + self.num_heads] = tensors[p + "f.b"].to(torch.float32)
        self.b_in = bias.to(device).contiguous()
        self.w_o = self._place(tensors[p + "o"], device)
        self.norm = tensors[p + "norm"].to(torch.float32).to(device).contiguous()

    def state_spec(self):
        H = self.num_heads
        return {"memory": StateSpec((H, self.dim, self.vdim)), "normalizer": StateSpec((H, self.dim)), "maximum": StateSpec((H,))}

    def forward_heads(self, x: torch.Tensor, ctx: LayerContext, out: torch.Tensor, out_col: int = 0, scale: float = 1.0) -> None:
        k, ws = ctx.kernels, ctx.workspace
        proj = self._project(x, ctx)
        o = ws.buffer("recurrent.o", (x.shape[0], self.heads_width), torch.float32)
        k.matrix_memory_scan(proj, (self.q_col, self.k_col, self.v_col, self.i_col, self.f_col), self.gate_cap, self.q_scale,
                             self.DENOMINATOR_FLOOR, ctx.batch, ctx.state["memory"], ctx.state["normalizer"], ctx.state["maximum"],
                             o, self.num_heads, self.dim, self.vdim, ws)
        k.head_norm_gate(o, self.norm, self.eps, (proj, self.g_col), "sigmoid", scale, out, out_col, self.num_heads, self.vdim)


class DeltaRuleMixer(_MatrixStateMixer):
    """The generalized delta rule.  r = Wr h, k = Wk h, v = Wv h per head (dim numbers each); a decay per key channel
    w = exp(-DECAY_RATE sigmoid(Ww2 tanh(Ww1 h) + w0)) and a removal rate per key channel a = sigmoid(Wa h + ba); with the
    unit key u = k / sqrt(sum k^2 + UNIT_KEY_EPS) of a head, S_t = diag(w) S_{t-1} - (a u) (u^T S_{t-1}) + k v^T (both terms
    read the old state) and o_t = S_t^T r; each head's o divided by its root mean square, times a weight over all heads'
    channels, times sigmoid(Wg h); then the output matrix.  The state is [head, key channel, value channel] in float32."""

    DECAY_RATE = math.exp(-0.5)
    UNIT_KEY_EPS = 1e-6

    def __init__(self, hidden: int, num_heads: int, dim: int, decay_rank: Optional[int], *, eps: float, prefix: str, dtype: str):
        super().__init__(hidden, num_heads, dim, dim, eps=eps, prefix=prefix, dtype=dtype)
        self.decay_rank = decay_rank          # None: whatever the checkpoint's Ww1 and Ww2 agree on
        self.a_col = self.g_col + self.heads_width
        self.w_w1 = self.w_w2 = self.b_w2 = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, n = self.prefix, self.qk_size
        specs = {p + name: TensorSpec((n, self.hidden)) for name in ("r", "k", "v", "g", "a")}
        specs.update({p + "a.b": TensorSpec((n,)), p + "w1": TensorSpec((self.decay_rank, self.hidden)),
                      p + "w2": TensorSpec((n, self.decay_rank)), p + "w0": TensorSpec((n,)), p + "norm": TensorSpec((n,)),
                      p + "o": TensorSpec((self.hidden, n))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        # One projection for everything that reads the rows directly: [r | k | v | gate of the result | removal logits].
        self.w_in = self._place(torch.cat([tensors[p + n] for n in ("r", "k", "v", "g", "a")], dim=0), device)
        bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32)
        bias[self.a_col:self.a_col + self.qk_size] = tensors[p + "a.b"].to(torch.float32)
        self.b_in = bias.to(device).contiguous()
        if tensors[p + "w1"].shape[0] != tensors[p + "w2"].shape[1]:
            raise WeightError(f"{p}w1 has {tensors[p + 'w1'].shape[0]} rows but {p}w2 has {tensors[p + 'w2'].shape[1]} columns")
        self.w_w1, self.w_w2 = self._place(tensors[p + "w1"], device), self._place(tensors[p + "w2"], device)
        self.b_w2 = tensors[p + "w0"].to(torch.float32).to(device).contiguous()
        self.w_o = self._place(tensors[p + "o"], device)
        self.norm = tensors[p + "norm"].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return super().weight_bytes() + sum(m.numel() * m.element_size() for m in (self.w_w1, self.w_w2))

    def state_spec(self):
        return {"memory": StateSpec((self.num_heads, self.dim, self.dim))}

    def forward_heads(self, x: torch.Tensor, ctx: LayerContext, out: torch.Tensor, out_col: int = 0, scale: float = 1.0) -> None:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        proj = self._project(x, ctx)
        low = ws.buffer("recurrent.low", (T, self.w_w1.shape[0]), self.dtype)
        k.linear(x, self.w_w1, low)
        k.activation_(low, "tanh")
        z = ws.buffer("recurrent.z", (T, self.qk_size), torch.float32)
        k.linear(low, self.w_w2, z, self.b_w2)
        o = ws.buffer("recurrent.o", (T, self.heads_width), torch.float32)
        k.delta_rule_scan(proj, (self.q_col, self.k_col, self.v_col, self.a_col), z, self.DECAY_RATE, self.UNIT_KEY_EPS, ctx.batch,
                          ctx.state["memory"], o, self.num_heads, self.dim, ws)
        k.head_norm_gate(o, self.norm, self.eps, (proj, self.g_col), "sigmoid", scale, out, out_col, self.num_heads, self.dim)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same rows: delta = left_scale * left(x) + right_scale * right(x).

    Both sides hand over what their output matrices multiply (`forward_heads`, already times the side's scale) into
    one buffer [left heads | right heads], and one product with [Wo_left | Wo_right] makes the sum.  At most one side
    may want cache pages; per-request states of both are kept under `left.` / `right.` names."""

    def __init__(self, hidden: int, left: Mixer, right: Mixer, left_scale: float, right_scale: float, dtype: str):
        for side in (left, right):
            if not hasattr(side, "forward_heads") or not hasattr(side, "out_weight"):
                raise ValueError(f"{type(side).__name__} cannot run beside another mixer (no forward_heads / out_weight)")
        if left.cache_spec() is not None and right.cache_spec() is not None:
            raise ValueError("only one side of a parallel mixer may keep keys and values in pages")
        self.hidden = hidden
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.dtype = TORCH_DTYPES[dtype]
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {**self.left.tensor_specs(), **self.right.tensor_specs()}

    def init_kinds(self) -> Dict[str, str]:
        return {**self.left.init_kinds(), **self.right.init_kinds()}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.left.bind(tensors, device)
        self.right.bind(tensors, device)
        self.w_o = torch.cat([self.left.out_weight(), self.right.out_weight()], dim=1).contiguous()

    def weight_bytes(self) -> int:
        return self.left.weight_bytes() + self.right.weight_bytes()

    def cache_spec(self):
        return self.left.cache_spec() or self.right.cache_spec()

    @staticmethod
    def _named(spec, side: str) -> Dict[str, StateSpec]:
        if spec is None:
            return {}
        return {f"{side}.{name}": s for name, s in spec.items()} if isinstance(spec, dict) else {side: spec}

    def state_spec(self):
        both = {**self._named(self.left.state_spec(), "left"), **self._named(self.right.state_spec(), "right")}
        return both or None

    def step_planners(self, kernels):
        return tuple(self.left.step_planners(kernels)) + tuple(self.right.step_planners(kernels))

    @staticmethod
    def _side_context(ctx: LayerContext, spec, side: str) -> LayerContext:
        state = None
        if isinstance(spec, dict):
            state = {name: ctx.state[f"{side}.{name}"] for name in spec}
        elif spec is not None:
            state = ctx.state[side]
        return LayerContext(batch=ctx.batch, kernels=ctx.kernels, workspace=ctx.workspace, kv=ctx.kv, state=state,
                            call_index=ctx.call_index, embedded=ctx.embedded)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        wl = self.left.heads_width
        both = ctx.workspace.buffer("parallel.heads", (T, wl + self.right.heads_width), self.dtype)
        self.left.forward_heads(x, self._side_context(ctx, self.left.state_spec(), "left"), both, 0, self.left_scale)
        self.right.forward_heads(x, self._side_context(ctx, self.right.state_spec(), "right"), both, wl, self.right_scale)
        delta = ctx.workspace.buffer("attn.delta", (T, self.hidden), self.dtype)
        ctx.kernels.linear(both, self.w_o, delta)
        return delta
