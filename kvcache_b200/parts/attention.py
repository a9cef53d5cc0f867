"""Grouped-query attention over the paged cache: the mixer of this architecture.

Reference: the attention part of the layer loop, apps/qwen_serve.cu:102-110
(q/k/v projections with bias, rotation of q and k, write into the pool, causal
paged attention with scale 1/sqrt(D), output projection without bias).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional, Sequence

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, Mixer, PagedKVSpec, PositionEncoding


class GQAAttention(Mixer):
    """Options beyond the reference's layer: `value_dim` (values of another size than keys), `qk_norm_eps` (queries and
    keys divided by their root mean square per head and multiplied by a weight of head_dim numbers that all heads share,
    `<q name>.norm` / `<k name>.norm`, before the rotation), `head_gate` (a head's result times sigmoid of one number per
    head, a projection of the mixer's input), `names` (what the q, k, v and output matrices are called after `prefix`).

    `qk_norm_scope` "all": the root mean square is taken over a token's whole query (key) projection, all heads at once,
    and the weights have that size.  `qk_norm_weight` False: no weights.  `qk_norm_after_rotation`: the norm follows the
    rotation instead of preceding it.  `sink`: the softmax's denominator also holds exp(sink) of a key that has no value -
    "learned": one number per head, `<prefix>sink`; a number: that logit for every head.  `keep_first`: with a window, the
    request's first tokens stay visible to every later query.  `value_mix`: "source" - this layer's values are also kept
    for the step; "mix" - v = (1 - lam) v + lam v_source with lam the scalar `<prefix><value_mix_name>`, before the values
    are cached; the source is the layer of the model that ran with "source" in the same step.

    `q_temperature` = (coef, every): the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).
    `score_cap`: score <- cap tanh(score / cap), after the scale.  `distance_bias` "geometric": head h of H then loses
    2^(-8 (h + 1) / H) (i - j) for a key i - j tokens back (after the cap, before the softmax).  `pad_values`: values
    narrower than keys are cached as wide as the keys, with zeros after their numbers, where that brings the layer to the
    tensor-core kernels, which take one size for both (bfloat16, keys of up to 128 numbers in steps of 16); the heads'
    results then carry those zero columns, which the step after attention leaves out."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, *, qkv_bias: bool,
                 out_bias: bool, position: Optional[PositionEncoding], window: Optional[int], prefix: str,
                 dtype: str, scale: Optional[float] = None, value_dim: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, head_gate: Optional[str] = None,
                 names: Sequence[str] = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight"),
                 qk_norm_scope: str = "head", qk_norm_weight: bool = True, qk_norm_after_rotation: bool = False,
                 sink=None, keep_first: int = 0, value_mix: Optional[str] = None, value_mix_name: str = "vmix",
                 q_temperature=None, score_cap: Optional[float] = None, distance_bias: Optional[str] = None,
                 pad_values: bool = False):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if out_bias:
            raise ValueError("an output-projection bias is not supported")
        self.hidden, self.num_heads, self.num_kv_heads, self.head_dim = hidden, num_heads, num_kv_heads, head_dim
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.qkv_bias = qkv_bias
        self.position = position
        self.window = window
        self.prefix = prefix
        self.names = tuple(names)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.head_gate = head_gate
        if qk_norm_scope not in ("head", "all"):
            raise ValueError(f"qk_norm_scope '{qk_norm_scope}' (head, all)")
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix '{value_mix}' (source, mix)")
        if sink is not None and sink != "learned" and not isinstance(sink, (int, float)):
            raise ValueError(f"sink {sink!r} (None, 'learned' or a number)")
        if keep_first and window is None:
            keep_first = 0                       # without a window every key is visible anyway
        self.qk_norm_scope, self.qk_norm_weight, self.qk_norm_after_rotation = qk_norm_scope, bool(qk_norm_weight), bool(qk_norm_after_rotation)
        self.sink, self.keep_first = sink, int(keep_first)
        self.value_mix, self.value_mix_name = value_mix, value_mix_name
        if distance_bias not in (None, "geometric"):
            raise ValueError(f"distance_bias '{distance_bias}' (None, geometric)")
        self.q_temperature = None if q_temperature is None else (float(q_temperature[0]), int(q_temperature[1]))
        self.score_cap = None if score_cap is None else float(score_cap)
        self.distance_bias = distance_bias
        self.slopes: Optional[torch.Tensor] = None
        self.sink_logits: Optional[torch.Tensor] = None
        self.mix_weight: Optional[torch.Tensor] = None
        self.dtype = TORCH_DTYPES[dtype]
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.v_size = num_kv_heads * self.value_dim
        self.heads_width = num_heads * self.value_dim        # what the output matrix multiplies
        # The plain layer (equal key and value sizes, no norm of q and k, no gate) has fused and folded forms.
        self.plain = (self.value_dim == head_dim and self.qk_norm_eps is None and head_gate is None and sink is None
                      and not self.keep_first and value_mix is None and q_temperature is None and score_cap is None
                      and distance_bias is None)
        # Keys narrower than values are cached as wide as the values, with zeros after their numbers (which add nothing
        # to a score), where that brings the layer to the tensor-core attention kernels, which take one size for both:
        # bfloat16, values of up to 128 numbers in steps of 16.  The cache then holds 2 value_dim numbers a token and
        # key/value head instead of head_dim + value_dim.
        self.key_store = head_dim
        if dtype == "bfloat16" and head_dim < self.value_dim <= 128 and self.value_dim % 16 == 0 and num_heads // num_kv_heads <= 16:
            self.key_store = self.value_dim
        # What a cached value is as wide as: its own numbers, or the keys' (zeros after them, see `pad_values`).
        self.value_store = self.value_dim
        if (pad_values and dtype == "bfloat16" and self.value_dim < head_dim <= 128 and head_dim % 16 == 0
                and num_heads // num_kv_heads <= 16):
            self.value_store = head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm = self.k_norm = None

    def _bias_name(self, i: int) -> str:
        name = self.names[i]
        return self.prefix + (name[:-len("weight")] + "bias" if name.endswith("weight") else name + ".b")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        q, k, v, o = self.names
        specs = {
            p + q: TensorSpec((self.q_size, self.hidden)),
            p + k: TensorSpec((self.kv_size, self.hidden)),
            p + v: TensorSpec((self.v_size, self.hidden)),
            p + o: TensorSpec((self.hidden, self.heads_width)),
        }
        if self.qkv_bias:
            specs[self._bias_name(0)] = TensorSpec((self.q_size,))
            specs[self._bias_name(1)] = TensorSpec((self.kv_size,))
            specs[self._bias_name(2)] = TensorSpec((self.v_size,))
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            whole = self.qk_norm_scope == "all"
            specs[p + q + ".norm"] = TensorSpec((self.q_size if whole else self.head_dim,))
            specs[p + k + ".norm"] = TensorSpec((self.kv_size if whole else self.head_dim,))
        if self.head_gate is not None:
            specs[p + self.head_gate] = TensorSpec((self.num_heads, self.hidden))
        if self.sink == "learned":
            specs[p + "sink"] = TensorSpec((self.num_heads,))
        if self.value_mix is not None:
            # The source has nothing to blend with; a checkpoint may carry its scalar all the same.
            specs[p + self.value_mix_name] = TensorSpec((), optional=self.value_mix == "source")
        return specs

    def init_kinds(self) -> Dict[str, str]:
        if self.qk_norm_eps is None or not self.qk_norm_weight:
            return {}
        return {self.prefix + self.names[0] + ".norm": "ones_plus_normal", self.prefix + self.names[1] + ".norm": "ones_plus_normal"}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        # One projection for q, k and v (and the heads' gates): rows [q heads | k heads | v heads | gates].
        rows = [tensors[p + n] for n in self.names[:3]]
        if self.head_gate is not None:
            rows.append(tensors[p + self.head_gate])
        self.w_qkv = torch.cat(rows, dim=0).to(self.dtype).to(device).contiguous()
        if self.qkv_bias:
            bias = [tensors[self._bias_name(i)] for i in range(3)]
            if self.head_gate is not None:
                bias.append(torch.zeros(self.num_heads))
            self.b_qkv = torch.cat(bias, dim=0).to(torch.float32).to(device).contiguous()
        self.w_o = tensors[p + self.names[3]].to(self.dtype).to(device).contiguous()
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = tensors[p + self.names[0] + ".norm"].to(torch.float32).to(device).contiguous()
            self.k_norm = tensors[p + self.names[1] + ".norm"].to(torch.float32).to(device).contiguous()
        if self.sink == "learned":
            self.sink_logits = tensors[p + "sink"].to(torch.float32).to(device).contiguous()
        elif self.sink is not None:
            self.sink_logits = torch.full((self.num_heads,), float(self.sink), dtype=torch.float32, device=device)
        if self.distance_bias == "geometric":
            H = self.num_heads
            self.slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64).to(torch.float32).to(device)
        if self.value_mix == "mix":
            self.mix_weight = tensors[p + self.value_mix_name].to(torch.float32).reshape(1).to(device).contiguous()
        if self.position is not None:
            self.position.bind(tensors, device)
        # The folded projection of decode steps rotates inside the product and wants a second copy of the q/k/v weight
        # with each head's rows reordered (made when first asked for): possible in bfloat16, with whole-head rotation (or
        # none) and heads in steps of 16.
        self.w_qkv_paired = self.b_qkv_paired = None
        self._can_pair = self.plain and self.dtype == torch.bfloat16 and self.head_dim % 16 == 0 and device.type == "cuda"

    def _pair_rows(self, kernels) -> bool:
        """Makes the row-paired copy of the q/k/v weight and bias if the kernel set can use one."""
        rotation = self.position.rotation() if self.position is not None else None
        whole = rotation is None or rotation.cos.shape[1] * 2 == self.head_dim
        if self.w_qkv_paired is None and self._can_pair and whole and hasattr(kernels, "pair_rotation_rows"):
            order = kernels.pair_rotation_rows(self.num_heads + 2 * self.num_kv_heads, self.head_dim).to(self.w_qkv.device)
            self.w_qkv_paired = self.w_qkv.index_select(0, order).contiguous()
            if self.b_qkv is not None:
                self.b_qkv_paired = self.b_qkv.index_select(0, order).contiguous()
        return self.w_qkv_paired is not None

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        return n + (self.b_qkv.numel() * 4 if self.b_qkv is not None else 0)

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.key_store, self.window,
                           None if self.value_store == self.key_store else self.value_store, self.keep_first)

    def step_planners(self, kernels):
        planner = getattr(kernels, "paged_attention_planner", None)
        return () if planner is None else (planner(),)

    def supports_fold(self, norm, kernels, num_rows: int) -> bool:
        can = getattr(kernels, "can_fold", None)
        return (self.plain and can is not None and norm.fold_params() is not None
                and can(self.dtype, num_rows, self.hidden, self.q_size + 2 * self.kv_size)
                and can(self.dtype, num_rows, self.q_size, self.hidden) and self._pair_rows(kernels))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm, ctx: LayerContext) -> None:
        T = h.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        weight, eps = norm.fold_params()
        rotation = self.position.rotation() if self.position is not None else None
        cos, sin = (rotation.cos, rotation.sin) if rotation else (None, None)
        q = ws.buffer("attn.q", (T, self.q_size), self.dtype)
        k.norm_qkv_rope_append(h16, self.w_qkv_paired, self.b_qkv_paired, weight, eps, cos, sin, ctx.batch, ctx.kv, q,
                               self.num_heads)
        attn = ws.buffer("attn.out", (T, self.q_size), self.dtype)
        k.paged_attention(q, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws)
        k.linear_into_residual(attn, self.w_o, h, h16)


    def forward_heads(self, x: torch.Tensor, ctx: LayerContext, out: torch.Tensor, out_col: int = 0, scale: float = 1.0) -> None:
        """The heads' results, gated and times `scale`, into columns out_col .. out_col + heads_width of `out` (what the
        output matrix multiplies): the form a mixer that runs beside another one is asked for."""
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        qkv = ws.buffer("attn.qkv", (T, self.w_qkv.shape[0]), self.dtype)
        k.linear(x, self.w_qkv, qkv)
        rotation = self.position.rotation() if self.position is not None else None
        cos, sin = (rotation.cos, rotation.sin) if rotation else (None, None)
        q = ws.buffer("attn.q", (T, self.num_heads * self.key_store), self.dtype)
        extra = {}
        if self.qk_norm_eps is not None and (self.qk_norm_scope != "head" or self.qk_norm_after_rotation or not self.qk_norm_weight):
            extra.update(norm_scope=self.qk_norm_scope, norm_after_rotation=self.qk_norm_after_rotation)
        if self.value_mix is not None:
            # The source's values of this step's tokens, in the compute type: written by the source, read by the mixing layers.
            kept = ws.buffer("attn.value_source", (T, self.v_size), self.dtype)
            extra["value_mix"] = (kept, self.mix_weight)
        if self.q_temperature is not None:
            extra["q_temperature"] = self.q_temperature
        if self.value_store != self.value_dim:
            extra["value_dim"] = self.value_dim
        k.qkv_rope_append(qkv, self.b_qkv, cos, sin, ctx.batch, ctx.kv, q, self.num_heads, q_norm=self.q_norm, k_norm=self.k_norm,
                          norm_eps=self.qk_norm_eps or 0.0, key_dim=self.head_dim, **extra)
        padded = self.value_store != self.value_dim
        direct = self.head_gate is None and scale == 1.0 and out_col == 0 and out.shape[1] == self.heads_width and not padded
        attn = out if direct else ws.buffer("attn.out", (T, self.num_heads * self.value_store), self.dtype)
        more = {}
        if self.sink_logits is not None:
            more["sink"] = self.sink_logits
        if self.score_cap is not None:
            more["score_cap"] = self.score_cap
        if self.slopes is not None:
            more["slopes"] = self.slopes
        k.paged_attention(q, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws, **more)
        if not direct:
            gate = (qkv, self.q_size + self.kv_size + self.v_size) if self.head_gate is not None else None
            if padded:
                k.head_gate(attn, gate, self.num_heads, self.value_dim, scale, out, out_col, x_head_stride=self.value_store)
            else:
                k.head_gate(attn, gate, self.num_heads, self.value_dim, scale, out, out_col)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        delta = ws.buffer("attn.delta", (T, self.hidden), self.dtype)
        if not self.plain:
            gated = ws.buffer("attn.gated", (T, self.heads_width), self.dtype)
            self.forward_heads(x, ctx, gated)
            k.linear(gated, self.w_o, delta)
            return delta
        qkv = ws.buffer("attn.qkv", (T, self.q_size + 2 * self.kv_size), self.dtype)
        k.linear(x, self.w_qkv, qkv)
        rotation = self.position.rotation() if self.position is not None else None
        cos, sin = (rotation.cos, rotation.sin) if rotation else (None, None)
        attn = ws.buffer("attn.out", (T, self.q_size), self.dtype)
        # A kernel set may do bias, rotation, append and attention in one launch where it has a kernel for that.
        fused = getattr(k, "rope_append_attention", None)
        if fused is None or not fused(qkv, self.b_qkv, cos, sin, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws):
            q = ws.buffer("attn.q", (T, self.q_size), self.dtype)
            k.qkv_rope_append(qkv, self.b_qkv, cos, sin, ctx.batch, ctx.kv, q, self.num_heads)
            k.paged_attention(q, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws)
        k.linear(attn, self.w_o, delta)
        return delta
