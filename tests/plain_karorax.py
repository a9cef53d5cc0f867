"""Plain, slow implementation of the Karorax decoder: whole sequences, no cache, token-by-token recurrence, one function
for each mechanism, float64 by default.  It shares no code with `kvcache_b200` (it reads the model folder with the
`safetensors` package and `json`) and states every formula directly.

The design, in this file's notation.  W = width, residual stream x[T, W]; unit(v) = v / sqrt(mean(v^2) + eps).

* embedding: x_t = embed[tok_t] + bigram[b_t], b_0 = buckets (the table's last row), b_t = (tok_{t-1} mul_prev +
  tok_t mul_cur) mod buckets.
* layer: x += ls1 * mixer(unit(x) (1 + norm1)); x += ls2 * ff(unit(x) (1 + norm2)) (the second line only if the layer
  has a feed-forward); ls1, ls2 multiply channel by channel.
* latent attention: q = Wq h, per head [dim numbers that are not rotated | rot_dim that are]; [c_raw | kr] = Wdkv h,
  c = unit(c_raw) * dkv.norm (kv_rank numbers), kr (rot_dim numbers) is one key part for all heads; per head
  k = Wuk c, v = Wuv c; score(i, j) = scale (q_i[:dim] . k_j + R_i(q_i[dim:]) . R_j(kr_j)) for 0 <= i - j < window;
  p_ij = e^{s_ij} / (e^{sink_h} + sum_j e^{s_ij}); head h's sum of values times sigmoid(Wg h)_h; out = Wo concat.
  R_p turns the pair (2 t, 2 t + 1) of the first `dims` numbers by the angle p base^(-2 t / dims).  A layer with
  `kv_from` = j projects no c and kr of its own: it takes layer j's (of the same tokens) and expands them with its own
  Wuk and Wuv.
* attention with grouped keys (left side of a parallel layer): q = Wq h, k = Wk h, v = Wv h, no rotation; the query at
  position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1); s = scale q_i . k_j, s <- cap tanh(s / cap),
  s <- s - 2^(-8 (h + 1) / H) (i - j) for head h of H; all j <= i; softmax; out = Wo concat.
* lightning attention (right side): q = silu(Wq h), k = silu(Wk h), v = silu(Wv h); per head S_t = decay_h S_{t-1} +
  k_t v_t^T, o_t = S_t^T q_t; out = Wo (unit(concat_heads(o)) * norm * sigmoid(Wg h)), the unit taken over all heads'
  channels at once.
* the parallel mixer: left_scale * left + right_scale * right, both reading the same h.
* feed-forwards: dense - Wdown relu(Wup h)^2.  Routed - z = Wrouter h + b; the `top` largest z, weights softmax over
  those alone; expert(h) = Wdown (silu(Wgate h) * (Wup h)); a shared expert of the same form is added for every token.
* logits = cap tanh(head (unit(x) (1 + final.norm)) / cap).
"""
from __future__ import annotations

import contextlib
import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        config = json.load(fh)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """A norm whose stored weight lies around zero."""
    return unit(x, eps) * (1.0 + weight)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


_ROUND_TO: Optional[torch.dtype] = None


@contextlib.contextmanager
def rounding(dtype: torch.dtype = torch.bfloat16):
    """Within the block every matrix product rounds its input rows and its result to `dtype` (the arithmetic stays as
    wide as the weights): what rounding alone does to a position's logits."""
    global _ROUND_TO
    saved, _ROUND_TO = _ROUND_TO, dtype
    try:
        yield
    finally:
        _ROUND_TO = saved


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if _ROUND_TO is None:
        return x @ weight.t()
    return (x.to(_ROUND_TO).to(weight.dtype) @ weight.t()).to(_ROUND_TO).to(weight.dtype)


# ---- embedding --------------------------------------------------------------------------------------------------------
def bigram_rows(tokens: Sequence[int], bigram: dict) -> List[int]:
    buckets, mul_prev, mul_cur = int(bigram["buckets"]), int(bigram["mul_prev"]), int(bigram["mul_cur"])
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embed(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    x = w["embed"][list(tokens)].clone()
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        x = x + w["bigram"][bigram_rows(tokens, bigram)]
    return x


# ---- rotation ---------------------------------------------------------------------------------------------------------
def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, D]: of each head's first rot.dims numbers, neighbours (2 t, 2 t + 1) are turned by p base^(-2 t / dims)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = x.clone()
    for t in range(dims // 2):
        angle = positions.to(torch.float64) * base ** (-2.0 * t / dims)
        c, s = torch.cos(angle)[:, None].to(x.dtype), torch.sin(angle)[:, None].to(x.dtype)
        u, v = x[..., 2 * t], x[..., 2 * t + 1]
        out[..., 2 * t], out[..., 2 * t + 1] = u * c - v * s, v * c + u * s
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------------
def latent_kv(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor, eps: float):
    """What a latent-attention layer keeps per token: the normalised latent c [T, kv_rank] and the turned key part [T, rot_dim]."""
    rank, rot_dim = int(m["kv_rank"]), int(m["rot_dim"])
    down = linear(h, w[p + "dkv"])
    c = unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    kr = rotate_pairs(down[:, None, rank:rank + rot_dim], positions, m["rot"])[:, 0]
    return c, kr


def latent_attention(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor, eps: float, kept=None):
    """`kept`: (c, kr) of the layer named by `kv_from`, or None for a layer that projects its own.  Returns (out, (c, kr))."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    window = int(m["mask"]["size"]) if m.get("mask") else None
    c, kr = kept if kept is not None else latent_kv(m, w, p, h, positions, eps)
    q = linear(h, w[p + "q"]).view(T, H, dim + rot_dim)
    q_plain, q_turned = q[..., :dim], rotate_pairs(q[..., dim:], positions, m["rot"])
    k = linear(c, w[p + "uk"]).view(T, H, dim)
    v = linear(c, w[p + "uv"]).view(T, H, vdim)
    gate = torch.sigmoid(linear(h, w[p + "g"]))                                   # [T, H]
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for head in range(H):
            s = (k[lo:i + 1, head] @ q_plain[i, head] + kr[lo:i + 1] @ q_turned[i, head]) * float(m["scale"])
            sink = w[p + "sink"][head]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[i, head] = (e / (e.sum() + torch.exp(sink - top))) @ v[lo:i + 1, head]
    out = out * gate[:, :, None]
    return linear(out.reshape(T, H * vdim), w[p + "o"]), (c, kr)


def query_temperature(positions: torch.Tensor, q_temp: Optional[dict]) -> torch.Tensor:
    if not q_temp:
        return torch.ones(len(positions), dtype=torch.float64)
    steps = torch.div(positions + 1, int(q_temp["every"]), rounding_mode="floor").to(torch.float64)
    return 1.0 + float(q_temp["coef"]) * torch.log(steps + 1.0)


def distance_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def biased_attention(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """The left side: grouped keys, no rotation, query temperature, capped scores, a bias that grows with the distance."""
    T = h.shape[0]
    H, G, dim, vdim = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    q = linear(h, w[p + "q"]).view(T, H, dim) * query_temperature(positions, m.get("q_temp")).to(h.dtype)[:, None, None]
    k = linear(h, w[p + "k"]).view(T, G, dim)
    v = linear(h, w[p + "v"]).view(T, G, vdim)
    slopes = distance_slopes(H).to(h.dtype)
    cap = float(m["softcap"]) if m.get("softcap") else None
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for i in range(T):
        distance = (i - torch.arange(i + 1)).to(h.dtype)
        for head in range(H):
            g = head // (H // G)
            s = (k[:i + 1, g] @ q[i, head]) * float(m["scale"])
            if cap is not None:
                s = cap * torch.tanh(s / cap)
            s = s - slopes[head] * distance
            out[i, head] = torch.softmax(s, dim=0) @ v[:i + 1, g]
    return linear(out.reshape(T, H * vdim), w[p + "o"])


def lightning_attention(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, eps: float, state: Optional[torch.Tensor] = None):
    """The right side, token by token.  Returns (out, the state after the last token [heads, dim, vdim])."""
    T = h.shape[0]
    H, dim, vdim = (int(m[k]) for k in ("heads", "dim", "vdim"))
    decay = [float(d) for d in m["decay"]]
    q = silu(linear(h, w[p + "q"])).view(T, H, dim)
    k = silu(linear(h, w[p + "k"])).view(T, H, dim)
    v = silu(linear(h, w[p + "v"])).view(T, H, vdim)
    S = torch.zeros(H, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, vdim, dtype=h.dtype)
    for t in range(T):
        for head in range(H):
            S[head] = decay[head] * S[head] + torch.outer(k[t, head], v[t, head])
            o[t, head] = S[head].t() @ q[t, head]
    y = unit(o.reshape(T, H * vdim), eps) * w[p + "norm"] * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(y, w[p + "o"]), S


def parallel_mixer(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, positions: torch.Tensor, eps: float) -> torch.Tensor:
    left = biased_attention(m["left"], w, p + "left.", h, positions)
    right, _ = lightning_attention(m["right"], w, p + "right.", h, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- feed-forwards ----------------------------------------------------------------------------------------------------
def dense_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return linear(torch.relu(linear(h, w[p + "up"])) ** 2, w[p + "down"])


def gated_expert(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return linear(silu(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def route(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ w[p + "router"].t() + w[p + "router.b"]
    best, which = torch.topk(z, int(mlp["router"]["top"]), dim=-1)
    return which, torch.softmax(best, dim=-1)


def routed_ff(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    which, share = route(mlp, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s in range(which.shape[1]):
            out[t] += share[t, s] * gated_expert(w, f"{p}e{int(which[t, s])}.", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + gated_expert(w, p + "shared.", h)
    return out


def feed_forward(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return dense_ff(w, p, h) if mlp["kind"] == "dense" else routed_ff(mlp, w, p, h)


# ---- the model --------------------------------------------------------------------------------------------------------
def layer_forward(config: dict, w: Dict[str, torch.Tensor], i: int, x: torch.Tensor, positions: torch.Tensor, kept: dict) -> torch.Tensor:
    """One layer on the whole sequence.  `kept`: {layer: (c, kr)} of the latent-attention layers that ran before."""
    layer, eps, p = config["layers"][i], float(config["norm"]["eps"]), f"l{i}."
    h = offset_norm(x, w[p + "norm1"], eps)
    if layer["type"] == "latent_attention":
        source = layer["mixer"].get("kv_from")
        delta, kept[i] = latent_attention(layer["mixer"], w, p + "mix.", h, positions, eps, None if source is None else kept[int(source)])
    else:
        delta = parallel_mixer(layer["mixer"], w, p + "mix.", h, positions, eps)
    x = x + w[p + "ls1"] * delta
    if layer.get("mlp"):
        x = x + w[p + "ls2"] * feed_forward(layer["mlp"], w, p + "mlp.", offset_norm(x, w[p + "norm2"], eps))
    return x


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of every place of one sequence; `trace` receives the residual stream after every layer."""
    positions = torch.arange(len(tokens))
    x = embed(config, w, tokens)
    kept: dict = {}
    for i in range(len(config["layers"])):
        x = layer_forward(config, w, i, x, positions, kept)
        if trace is not None:
            trace.append(x.clone())
    logits = linear(offset_norm(x, w["final.norm"], float(config["norm"]["eps"])), w["head"])
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(torch.argmax(forward(config, w, tokens)[-1])))
    return tokens[len(prompt):]
