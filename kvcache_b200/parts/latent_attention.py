"""Latent attention: keys and values of all heads are expanded from one small latent per token, and only the
latent (with one rotated key part that all heads share) is cached.

With h the mixer's input, per token:
    cq = norm(Wdq h),  q = Wuq cq                      per head [dim unrotated | rot_dim rotated]
    [c_raw | kr] = Wdkv h,  c = norm(c_raw)            c: kv_rank, kr: rot_dim, rotated by the position, not normed
    per head: k = Wuk c, v = Wuv c
    score(i, j) = scale * (q_i[:dim] . k_j + R_i(q_i[dim:]) . R_j(kr_j)),  j <= i;  softmax over j
    out = Wo (concat_heads(sum_j p_ij v_j) * sigmoid(Wg h))

This part never expands a cached token.  Since k_j = Wuk c_j, the unrotated score is (Wuk^T q_i[:dim]) . c_j: the
query is taken into the latent's space once (a product per head with Wuk^T), attention then runs with one shared
"key" row [c_j | R_j(kr_j)] of kv_rank + rot_dim numbers per token, whose first kv_rank numbers are also the "value",
and the head's result sum_j p_ij c_j goes through Wuv afterwards.  The cache entry is one key head of that width and
no value pool (`PagedKVSpec.value_dim == 0`); a step reads kv_rank + rot_dim numbers per cached token, whatever the
number of heads.

Options.  `q_rank` None: the query comes straight from the input, q = Wq h (tensor `q`; no `dq`, `dq.norm`, `uq`).
`window`: a query sees its own key and the window - 1 before it.  `sink` "learned": the softmax's denominator also holds
exp(sink_h), one learned logit per head (`sink`), a key without a value.  `gate` "head": one gate number per head
(`g` has H rows) instead of one per value channel.  `rotary_layout` "interleaved": the rotation pairs neighbours
(2 t, 2 t + 1); a score is a sum over the rotated numbers, so it does not change when the rotated parts of queries and keys
are reordered alike, and the rows of the projections that make them are reordered once, when the weights are bound, into
the order in which partners lie half the rotated numbers apart - the kernels and the cache then see the other layout.
`own_latent` False: the layer projects no latent; its layer call reads the cache entry that another layer writes
(sizes and rotation equal), and expands it with its own Wuk and Wuv.  `cache_window`: what the cache entry has to keep
when layers with other windows read it too.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, Mixer, PagedKVSpec, PositionEncoding


class LatentAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: Optional[int], *,
                 scale: float, eps: float, position: PositionEncoding, prefix: str, dtype: str, window: Optional[int] = None,
                 sink: Optional[str] = None, gate: str = "channel", rotary_layout: str = "half", own_latent: bool = True,
                 cache_window: Optional[int] = None):
        if sink not in (None, "learned"):
            raise ValueError(f"sink {sink!r} (None, 'learned')")
        if gate not in ("channel", "head"):
            raise ValueError(f"gate '{gate}' (channel, head)")
        if rotary_layout not in ("half", "interleaved"):
            raise ValueError(f"rotary_layout '{rotary_layout}' (half, interleaved)")
        self.hidden, self.num_heads = hidden, num_heads
        self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank = dim, rot_dim, vdim, kv_rank, q_rank
        self.scale, self.eps = float(scale), float(eps)
        self.position = position
        self.window = window
        self.cache_window = cache_window if cache_window is not None or window is None else window
        self.sink, self.gate, self.rotary_layout, self.own_latent = sink, gate, rotary_layout, bool(own_latent)
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.q_head = dim + rot_dim                 # a head's query as the checkpoint lays it out
        self.key_dim = kv_rank + rot_dim            # a cached row, and a head's query after it was taken to the latent's space
        self.gate_width = num_heads * (vdim if gate == "channel" else 1)
        # Columns of the fused projection's rows: [query latent, or the heads' queries | key/value latent | shared key part | gate].
        self.q_width = q_rank if q_rank is not None else num_heads * self.q_head
        self.kv_col = self.q_width
        self.gate_col = self.q_width + (self.key_dim if self.own_latent else 0)
        self.w_in: Optional[torch.Tensor] = None
        self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.q_norm = self.kv_norm = self.sink_logits = None

    def keep_for_window(self, window: Optional[int]) -> None:
        """Another layer reads this layer's cache entry with `window`: the entry keeps what the widest reader sees."""
        if self.cache_window is not None:
            self.cache_window = None if window is None else max(self.cache_window, window)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, H = self.prefix, self.num_heads
        specs = {
            f"{p}uk": TensorSpec((H * self.dim, self.kv_rank)),
            f"{p}uv": TensorSpec((H * self.vdim, self.kv_rank)),
            f"{p}g": TensorSpec((self.gate_width, self.hidden)),
            f"{p}o": TensorSpec((self.hidden, H * self.vdim)),
        }
        if self.q_rank is not None:
            specs.update({f"{p}dq": TensorSpec((self.q_rank, self.hidden)), f"{p}dq.norm": TensorSpec((self.q_rank,)),
                          f"{p}uq": TensorSpec((H * self.q_head, self.q_rank))})
        else:
            specs[f"{p}q"] = TensorSpec((H * self.q_head, self.hidden))
        if self.own_latent:
            specs.update({f"{p}dkv": TensorSpec((self.kv_rank + self.rot_dim, self.hidden)), f"{p}dkv.norm": TensorSpec((self.kv_rank,))})
        if self.sink == "learned":
            specs[f"{p}sink"] = TensorSpec((H,))
        return specs

    def init_kinds(self) -> Dict[str, str]:
        return {f"{self.prefix}dq.norm": "ones_plus_normal", f"{self.prefix}dkv.norm": "ones_plus_normal"}

    def _rotated_order(self) -> torch.Tensor:
        """Where each of the rot_dim rotated numbers comes from: the identity, or, for the interleaved layout, the even
        members of the rotated pairs, then the odd ones, then what is not rotated."""
        if self.rotary_layout == "half":
            return torch.arange(self.rot_dim)
        rotation = self.position.rotation()
        dims = 2 * rotation.cos.shape[1] if rotation is not None else self.position.rotary_dim
        return torch.cat([torch.arange(0, dims, 2), torch.arange(1, dims, 2), torch.arange(dims, self.rot_dim)])

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p, H = self.prefix, self.num_heads
        place = lambda t: t.to(self.dtype).to(device).contiguous()
        self.position.bind(tensors, device)
        order = self._rotated_order()
        head_rows = torch.cat([torch.arange(self.dim), self.dim + order])          # a head's query rows, rotated part reordered
        query_rows = (torch.arange(H)[:, None] * self.q_head + head_rows[None, :]).reshape(-1)
        # One product for everything that reads the mixer's input: rows [query latent or queries | key/value latent |
        # shared key part | gate], zero rows after them up to a multiple of 8 (so that rows of the result start on 16 bytes).
        rows = [tensors[f"{p}dq"] if self.q_rank is not None else tensors[f"{p}q"][query_rows]]
        if self.own_latent:
            latent_rows = torch.cat([torch.arange(self.kv_rank), self.kv_rank + order])
            rows.append(tensors[f"{p}dkv"][latent_rows])
        rows.append(tensors[f"{p}g"])
        total = sum(r.shape[0] for r in rows)
        if self.q_rank is None and total % 8:
            rows.append(torch.zeros(8 - total % 8, self.hidden, dtype=rows[0].dtype))
        self.w_in = place(torch.cat(rows, dim=0))
        if self.q_rank is not None:
            self.w_uq = place(tensors[f"{p}uq"][query_rows])
            self.q_norm = tensors[f"{p}dq.norm"].to(torch.float32).to(device).contiguous()
        if self.own_latent:
            self.kv_norm = tensors[f"{p}dkv.norm"].to(torch.float32).to(device).contiguous()
        if self.sink == "learned":
            self.sink_logits = tensors[f"{p}sink"].to(torch.float32).to(device).contiguous()
        # [H, kv_rank, dim]: the transposed key expansion, which takes a head's unrotated query to the latent's space.
        self.w_uk_t = place(tensors[f"{p}uk"].view(H, self.dim, self.kv_rank).transpose(1, 2))
        self.w_uv = place(tensors[f"{p}uv"].view(H, self.vdim, self.kv_rank))
        self.w_o = place(tensors[f"{p}o"])

    def weight_bytes(self) -> int:
        mats = [m for m in (self.w_in, self.w_uq, self.w_uk_t, self.w_uv, self.w_o) if m is not None]
        return sum(m.numel() * m.element_size() for m in mats) + 4 * ((self.q_rank or 0) + self.kv_rank)

    def cache_spec(self) -> Optional[PagedKVSpec]:
        return PagedKVSpec(1, self.key_dim, self.cache_window, value_dim=0) if self.own_latent else None

    def step_planners(self, kernels):
        planner = getattr(kernels, "latent_attention_planner", None)
        if planner is None:
            return ()
        return (planner(self.num_heads, self.key_dim, self.kv_rank, self.window) if self.window else
                planner(self.num_heads, self.key_dim, self.kv_rank),)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T, H = x.shape[0], self.num_heads
        k, ws = ctx.kernels, ctx.workspace
        rotation = self.position.rotation()
        if ctx.kv.writes != self.own_latent:
            raise ValueError("a latent-attention layer writes the cache entry of its layer call exactly if it projects a latent of its own")
        proj = ws.buffer("latent.proj", (T, self.w_in.shape[0]), self.dtype)
        k.linear(x, self.w_in, proj)
        rotate = (rotation.cos, rotation.sin, ctx.batch.positions)
        q_lat = ws.buffer("latent.q_lat", (T, H * self.key_dim), self.dtype)
        if self.q_rank is not None:
            cq = ws.buffer("latent.cq", (T, self.q_rank), self.dtype)
            k.latent_norm_rope_append(proj, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps,
                                      rotation.cos, rotation.sin, ctx.batch, ctx.kv, cq)
            q = ws.buffer("latent.q", (T, H * self.q_head), self.dtype)
            k.linear(cq, self.w_uq, q)
            k.head_linear(q, self.w_uk_t, q_lat, rotate=rotate)
        else:
            if self.own_latent:
                k.latent_norm_rope_append(proj, 0, self.kv_rank, self.rot_dim, None, self.kv_norm, self.eps, rotation.cos,
                                          rotation.sin, ctx.batch, ctx.kv, None, kv_col=self.kv_col)
            k.head_linear(proj, self.w_uk_t, q_lat, rotate=rotate, x_col=0)
        o_lat = ws.buffer("latent.o_lat", (T, H * self.kv_rank), self.dtype)
        if self.sink_logits is None and self.window == ctx.kv.spec.window:
            k.latent_attention(q_lat, ctx.batch, ctx.kv, o_lat, H, self.kv_rank, self.scale, ws)
        else:
            k.latent_attention(q_lat, ctx.batch, ctx.kv, o_lat, H, self.kv_rank, self.scale, ws, window=self.window,
                               sink=self.sink_logits)
        o = ws.buffer("latent.o", (T, H * self.vdim), self.dtype)
        if self.gate == "channel":
            k.head_linear(o_lat, self.w_uv, o, gate=(proj, self.gate_col))
        else:
            k.head_linear(o_lat, self.w_uv, o, gate=(proj, self.gate_col), gate_per_head=True)
        delta = ws.buffer("attn.delta", (T, self.hidden), self.dtype)
        k.linear(o, self.w_o, delta)
        return delta
