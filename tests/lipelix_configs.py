"""Tiny Lipelix configurations for the tests: they differ from one another in every size, in the order and kinds of
layers, in windows, kept first tokens, rotation and score constants.  Sizes that tend to coincide or to be 1 each occur
somewhere: one key/value head, as many as query heads, values as wide as keys, narrower and wider; rotation of a whole
head, of part of it, none; a window of one token, of one page, across pages; no kept tokens, one, a page and a half of
them, more than the window; a layer without feed-forward; value mixing whose source is not the model's first layer, a
layer that opts out of it; a model of one kind of layer only; residual multiplier and embedding scale of 1."""
from __future__ import annotations

import copy
import os

import torch


def _attention(heads, kv_heads, dim, vdim, scale, rot, v_mix=True):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot is not None:
        out["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": out}


def _window(heads, kv_heads, dim, vdim, scale, rot, size, keep_first, v_mix=True):
    out = _attention(heads, kv_heads, dim, vdim, scale, rot, v_mix)
    out["type"] = "attention_2"
    out["mixer"]["mask"] = {"size": size, "keep_first": keep_first}
    return out


def _delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def _layer(mixer, ff):
    return dict(mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# A: every kind of layer; the source of the mixed values is a window layer; keys narrower than values; a layer without
# feed-forward; a window across pages with kept tokens inside one page.
LIP_A = {
    "architecture": "Lipelix", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "embedding": {"scale": 0.7},
    "layers": [
        _layer(_delta(3, 8, 4), 40),
        _layer(_window(4, 2, 12, 16, 0.21, (10000.0, 8), 11, 3), 48),
        _layer(_attention(4, 2, 16, 16, 0.3, (500.0, 16)), None),
        _layer(_window(2, 1, 8, 32, 0.35, (2000.0, 8), 5, 9), 24),
        _layer(_delta(2, 20, 1), None),
    ],
}
# B: one key/value head; a window of one token that keeps one; whole-head rotation and none; a mixing layer whose values
# are not mixed beside ones that are; residual multiplier and embedding scale of 1.
LIP_B = {
    "architecture": "Lipelix", "vocab": 331, "width": 96, "norm": {"eps": 3e-5}, "residual_mult": 1.0, "embedding": {"scale": 1.0},
    "layers": [
        _layer(_attention(3, 1, 32, 24, 0.05, (777.0, 32), v_mix=False), 72),
        _layer(_attention(6, 3, 8, 16, 0.2, None), 40),
        _layer(_window(3, 3, 16, 16, 0.25, (300000.0, 4), 1, 1), None),
        _layer(_window(12, 6, 4, 8, 0.5, None, 16, 0), 56),
    ],
}
# C: only delta-rule layers (no cache pages at all), sizes that are no power of two, one head.
LIP_C = {
    "architecture": "Lipelix", "vocab": 150, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.25, "embedding": {"scale": 3.0},
    "layers": [_layer(_delta(1, 33, 7), 56), _layer(_delta(5, 6, 2), None), _layer(_delta(2, 40, 16), 24)],
}
# D: only window layers with different windows and kept tokens (a cache group each): kept tokens over a page and a half,
# more kept tokens than the window is wide, five query heads on one key/value head.
LIP_D = {
    "architecture": "Lipelix", "vocab": 500, "width": 120, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "embedding": {"scale": 0.45},
    "layers": [
        _layer(_window(5, 1, 24, 40, 0.125, (300000.0, 12), 37, 6), 88),
        _layer(_window(10, 2, 8, 20, 0.3, (100.0, 8), 3, 7), 40),
        _layer(_window(4, 4, 20, 10, 0.2, (5000.0, 20), 9, 0), None),
    ],
}
# E: sizes in steps of 16 as real models have them (in bfloat16 these reach the tensor-core kernels): keys of 64 beside
# values of 64 and keys of 32 beside values of 64, delta-rule heads of 64 and 128 key channels.
LIP_E = {
    "architecture": "Lipelix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.35, "embedding": {"scale": 0.8},
    "layers": [
        _layer(_attention(4, 2, 64, 64, 0.11, (8000.0, 64)), 192),
        _layer(_window(4, 2, 32, 64, 0.16, (30000.0, 32), 40, 3), 192),
        _layer(_delta(2, 64, 8), None),
        _layer(_delta(1, 128, 16), 64),
        _layer(_attention(2, 2, 64, 64, 0.14, (8000.0, 32)), 64),
    ],
}
CONFIGS = {"A": LIP_A, "B": LIP_B, "C": LIP_C, "D": LIP_D, "E": LIP_E}
PAGE_SIZE = {"A": 8, "B": 16, "C": 16, "D": 4, "E": 16}


def config_dict(name: str, **changes) -> dict:
    out = copy.deepcopy(CONFIGS[name])
    out.update(changes)
    return out


def make_lipelix_folder(tmp_path, name: str, seed: int = 0, dtype=torch.float32, sharpen: float = 1.0, std: float = 0.08,
                        data: dict = None) -> str:
    """A random-weights folder for configuration `name` (or for `data`).  `sharpen` multiplies every attention's score
    scale, so that the softmax picks out single keys and a wrong or missing key shows in the logits.  Sinks, mixing
    scalars and token-shift weights are drawn wide enough to matter."""
    import kvcache_b200  # registers the architectures  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    data = copy.deepcopy(data) if data is not None else config_dict(name)
    data["initializer_range"] = std
    for layer in data["layers"]:
        if layer["type"] != "general_delta":
            layer["mixer"]["scale"] *= sharpen
    folder = os.path.join(str(tmp_path), f"lip_{name}_{seed}_{sharpen}")
    write_random_model(folder, config_from_dict(data), seed, dtype)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    g = torch.Generator().manual_seed(1000 + seed)
    for key in list(tensors):
        t = tensors[key]
        if key.endswith(".shift"):
            tensors[key] = torch.rand(t.shape, generator=g).to(t.dtype)
        elif key.endswith(".vmix"):
            tensors[key] = (0.2 + 0.6 * torch.rand(t.shape, generator=g)).to(t.dtype)
        elif key.endswith(".sink"):
            tensors[key] = (torch.randn(t.shape, generator=g) * 1.5).to(t.dtype)
        elif key.endswith((".w0", ".a.b", ".rg1.b", ".rg2.b")):
            tensors[key] = torch.randn(t.shape, generator=g).to(t.dtype)
    save_file(tensors, path)
    return folder
