"""Plain, slow implementation of the Lipelix decoder: whole sequences, no cache, token-by-token recurrences, one
function for each mechanism, float64 by default.  It shares no code with `kvcache_b200` (it takes the configuration
as the dict config.json holds and the weights as a dict of tensors) and states every formula directly.

The design, in this file's notation.  W = width, residual stream x[T, W]; unit(v) = v / sqrt(mean(v^2) + eps);
sig = the logistic function; m = residual_mult.

* embedding: x_t = embed[tok_t] * scale.
* layer: a = unit(x) * norm1; g = sig(rg1 a + rg1.b); s_t = a_t + (a_{t-1} - a_t) * shift (a_{-1} = 0);
  x += m * unit(mixer(s) * g) * norm1b; then, if the layer has a feed-forward, b = unit(x) * norm2;
  x += m * unit(ff(b) * sig(rg2 b + rg2.b)) * norm2b.
* attention with a learned sink: q, k, v = Wq s, Wk s, Wv s; q and k are each normalised over ALL their numbers at once
  (unit over the whole row, times a weight of that size), then the first `dims` numbers of every head are rotated
  (t pairs with t + dims/2, angle p base^(-2t/dims)); e_ij = exp(scale q_i . k_j) for j <= i;
  out_i = sum_j e_ij v_j / (exp(sink_head) + sum_j e_ij).
* attention over a window with kept first tokens: q and k rotated first, then every head divided by its own root mean
  square (no weight); j is seen from i if j <= i and (i - j < size or j < keep_first); the denominator is 1 + sum_j e_ij.
* value mixing: among the layers with v_mix, the first keeps its values as they are; every later one uses
  (1 - lam) v + lam v_first with its own scalar lam = vmix and v_first the first such layer's values of that token.
* generalized delta rule: r, k, v = Wr s, Wk s, Wv s per head; decay w = exp(-e^{-1/2} sig(Ww2 tanh(Ww1 s) + w0));
  removal a = sig(Wa s + a.b); u = k / sqrt(sum k^2 + 1e-6) per head;
  S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T; o_t = S_t^T r_t;
  out = Wo (concat_heads(unit(o)) * norm * sig(Wg s)).
* feed-forward: Wdown relu(Wup b)^2.
* logits = head (unit(x) * final.norm).
"""
from __future__ import annotations

import contextlib
import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

UNIT_KEY_EPS = 1e-6
DECAY_RATE = math.exp(-0.5)


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


_ROUND_TO: Optional[torch.dtype] = None


@contextlib.contextmanager
def rounding(dtype: torch.dtype = torch.bfloat16):
    """Within the block every matrix product rounds its input rows and its result to `dtype` (the arithmetic stays as
    wide as the weights): what rounding alone does to a position's logits, which is what a reduced-precision run of the
    engine may be held to where a position is badly conditioned."""
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


def embed(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    return w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))


def token_shift(a: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    before = torch.cat([torch.zeros_like(a[:1]), a[:-1]], dim=0)
    return a + (before - a) * shift


def residual_gate(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    return torch.sigmoid(linear(a, weight) + bias)


def rotate(x: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, dim]; row t is at position t.  No `rot`: no rotation."""
    if rot is None:
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    angle = torch.arange(x.shape[0], dtype=torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor,
                           window: Optional[int], keep_first: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv], sink [H] (logits of a key without value); returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)      # head h reads key/value head h // (H / G)
    e = torch.exp(torch.einsum("ihd,jhd->hij", q, k) * scale) * seen[None, :, :]
    weights = e / (torch.exp(sink)[:, None, None] + e.sum(dim=-1, keepdim=True))
    return torch.einsum("hij,jhd->ihd", weights, v)


def mixed_values(v: torch.Tensor, lam: Optional[torch.Tensor], v_first: Optional[torch.Tensor]) -> torch.Tensor:
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def attention(s: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, v_first: Optional[torch.Tensor]):
    """The mixer with norms over whole projections and a learned sink.  Returns (result [T, W], this layer's values)."""
    T, H, G, D, Dv = s.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = unit(linear(s, w[p + "q"]), eps) * w[p + "q.norm"]
    k = unit(linear(s, w[p + "k"]), eps) * w[p + "k.norm"]
    v = linear(s, w[p + "v"])
    if m.get("v_mix"):
        v = mixed_values(v, w.get(p + "vmix"), v_first)
    q, k = rotate(q.view(T, H, D), m.get("rot")), rotate(k.view(T, G, D), m.get("rot"))
    o = sink_softmax_attention(q, k, v.view(T, G, Dv), float(m["scale"]), w[p + "sink"].to(s.dtype), None, 0)
    return linear(o.reshape(T, H * Dv), w[p + "o"]), v


def attention_2(s: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, v_first: Optional[torch.Tensor]):
    """The mixer with per-head unit norms after the rotation, a window that keeps the first tokens, and a sink at 0."""
    T, H, G, D, Dv = s.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = linear(s, w[p + "q"]).view(T, H, D), linear(s, w[p + "k"]).view(T, G, D), linear(s, w[p + "v"])
    if m.get("v_mix"):
        v = mixed_values(v, w.get(p + "vmix"), v_first)
    q, k = unit(rotate(q, m.get("rot")), eps), unit(rotate(k, m.get("rot")), eps)
    mask = m.get("mask") or {}
    window = int(mask["size"]) if "size" in mask else None
    o = sink_softmax_attention(q, k, v.view(T, G, Dv), float(m["scale"]), torch.zeros(H, dtype=s.dtype), window,
                               int(mask.get("keep_first", 0)))
    return linear(o.reshape(T, H * Dv), w[p + "o"]), v


def delta_rule_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, removal: torch.Tensor,
                    state: Optional[torch.Tensor] = None):
    """r, k, v, decay, removal [T, H, D]; state [H, D, D] ([head, key channel, value channel]).  Returns (o [T, H, D], state)."""
    T, H, D = r.shape
    S = torch.zeros(H, D, D, dtype=r.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, D, dtype=r.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(dim=-1, keepdim=True) + UNIT_KEY_EPS)
        read = torch.einsum("hk,hkv->hv", u, S)                       # u^T S, from the old state
        S = decay[t][:, :, None] * S - (removal[t] * u)[:, :, None] * read[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, r[t])
    return out, S


def general_delta(s: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T, H, D = s.shape[0], int(m["heads"]), int(m["dim"])
    r, k, v = (linear(s, w[p + n]).view(T, H, D) for n in "rkv")
    decay = torch.exp(-DECAY_RATE * torch.sigmoid(linear(torch.tanh(linear(s, w[p + "w1"])), w[p + "w2"]) + w[p + "w0"]))
    removal = torch.sigmoid(linear(s, w[p + "a"]) + w[p + "a.b"])
    o, _ = delta_rule_scan(r, k, v, decay.view(T, H, D), removal.view(T, H, D))
    gated = unit(o, eps).reshape(T, H * D) * w[p + "norm"] * torch.sigmoid(linear(s, w[p + "g"]))
    return linear(gated, w[p + "o"])


def feed_forward(b: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] != "dense":
        raise ValueError(f"feed-forward kind {mlp['kind']}")
    return linear(torch.relu(linear(b, w[p + "up"])) ** 2, w[p + "down"])


def residual_streams(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> List[torch.Tensor]:
    """The residual stream after the embedding and after every layer."""
    eps, mult = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    x = embed(config, w, tokens)
    streams = [x]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        a = unit(x, eps) * w[p + "norm1"]
        s = token_shift(a, w[p + "shift"])
        kind, m = layer["type"], layer["mixer"]
        if kind == "general_delta":
            y = general_delta(s, w, p + "mix.", m, eps)
        else:
            y, values = (attention if kind == "attention" else attention_2)(s, w, p + "mix.", m, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = values
        x = x + mult * unit(y * residual_gate(a, w[p + "rg1"], w[p + "rg1.b"]), eps) * w[p + "norm1b"]
        if layer.get("mlp") is not None:
            b = unit(x, eps) * w[p + "norm2"]
            y = feed_forward(b, w, p + "mlp.", layer["mlp"])
            x = x + mult * unit(y * residual_gate(b, w[p + "rg2"], w[p + "rg2.b"]), eps) * w[p + "norm2b"]
        streams.append(x)
    return streams


def logits_of(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    x = residual_streams(config, w, tokens)[-1]
    return linear(unit(x, float(config["norm"]["eps"])) * w["final.norm"], w["head"])


def greedy_generate(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(torch.argmax(logits_of(config, w, tokens)[-1])))
    return tokens[len(prompt):]
