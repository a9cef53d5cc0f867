"""Tiny Karorax configurations for the tests: they differ from one another in every size, in the order and kinds of
layers, in windows, rotation, caps and decays; values that tend to coincide or to be 1 (one key/value head, as many as
query heads, values as wide as keys, one expert chosen, all chosen, no shared expert, a layer without feed-forward, a
window of one page, of one token, none at all, only part of the rotated numbers turned, a decay of 1 and of 0, no query
temperature, no cap, no pair table, a layer that reads the latent of a layer that is not the first) each occur somewhere."""
from __future__ import annotations

import copy
import os

import torch


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, window, rot, kv_from=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
           "rot": {"base": rot[0], "dims": rot[1]}}
    if window is not None:
        out["mask"] = {"size": window}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": out}


def _left(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        out["softcap"] = softcap
    if q_temp is not None:
        out["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return out


def _parallel(left, right, left_scale, right_scale):
    heads, dim, vdim, decay = right
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                          "right": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}}


def _moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# A: every kind of layer; the second latent layer reads the first one's cache with a wider window than its owner's.
KAR_A = {
    "architecture": "Karorax", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "logit_softcap": 9.0,
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        _layer(_latent(3, 8, 4, 12, 20, 0.3, 11, (10000.0, 4)), _dense(48)),
        _layer(_parallel(_left(4, 2, 16, 8, 0.25, 20.0, (0.4, 7)), (3, 8, 12, (0.5, 0.97, 0.8)), 1.3, 0.7), _moe(5, 2, 24, 40)),
        _layer(_latent(2, 12, 4, 8, 20, 0.2, 19, (10000.0, 4), kv_from=0), _moe(5, 2, 24, 40)),
        _layer(_parallel(_left(4, 2, 16, 8, 0.25, 20.0, (0.4, 7)), (3, 8, 12, (0.5, 0.97, 0.8)), 0.6, 1.1), None),
    ],
}
# B: no window in the latent layer, only part of the rotated numbers turned, one key/value head, values as wide as keys,
# one lightning head, all experts chosen and no shared expert, no temperature, no cap, no pair table, no cap of the logits.
KAR_B = {
    "architecture": "Karorax", "vocab": 331, "width": 96, "norm": {"eps": 3e-5},
    "layers": [
        _layer(_parallel(_left(3, 1, 24, 24, 0.2), (1, 40, 24, (1.0,)), 1.0, 1.0), _moe(3, 3, 40)),
        _layer(_latent(2, 16, 8, 16, 24, 0.25, None, (500.0, 6)), _moe(4, 1, 16, 16)),
        _layer(_parallel(_left(2, 2, 8, 40, 0.35, 3.0), (2, 16, 40, (0.0, 0.9)), 2.0, 0.25), _dense(24)),
    ],
}
# C: only latent layers; the source of the shared latent is not the first layer; windows of one token and across pages.
KAR_C = {
    "architecture": "Karorax", "vocab": 150, "width": 40, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
    "embedding": {"bigram": {"buckets": 50, "mul_prev": 1, "mul_cur": 1000003}},
    "layers": [
        _layer(_latent(1, 12, 6, 20, 10, 0.4, 1, (100.0, 6)), _moe(2, 1, 56, 24)),
        _layer(_latent(5, 4, 2, 8, 14, 0.5, 21, (3000.0, 2)), None),
        _layer(_latent(3, 6, 2, 4, 14, 0.3, 9, (3000.0, 2), kv_from=1), _dense(32)),
        _layer(_latent(2, 10, 2, 6, 14, 0.3, 21, (3000.0, 2), kv_from=1), _dense(32)),
    ],
}
# D: only parallel layers (no latent cache at all), five query heads on one key/value head, keys narrower than values.
KAR_D = {
    "architecture": "Karorax", "vocab": 500, "width": 120, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "embedding": {"bigram": {"buckets": 1, "mul_prev": 7, "mul_cur": 3}},
    "layers": [
        _layer(_parallel(_left(5, 1, 24, 40, 0.125, 8.0, (0.25, 3)), (2, 48, 24, (0.99, 0.6)), 1.0, 0.5), _moe(9, 3, 40, 72)),
        _layer(_parallel(_left(10, 5, 8, 16, 0.35, 45.0, (1.0, 16)), (4, 16, 8, (0.2, 0.4, 0.9, 0.998)), 0.9, 1.2), _moe(9, 3, 40, 72)),
    ],
}
# E: sizes in steps of 16 as real models have them (in bfloat16 the tensor-core kernels): values narrower than keys on the
# left side (cached as wide as the keys), windows across pages, a shared latent.
KAR_E = {
    "architecture": "Karorax", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "logit_softcap": 20.0,
    "embedding": {"bigram": {"buckets": 211, "mul_prev": 17, "mul_cur": 3}},
    "layers": [
        _layer(_latent(4, 32, 16, 48, 48, 0.14, 40, (50000.0, 16)), _dense(192)),
        _layer(_parallel(_left(4, 2, 32, 16, 0.17, 30.0, (0.3, 16)), (2, 32, 32, (0.7, 0.995)), 1.1, 0.8), _moe(4, 2, 32, 64)),
        _layer(_latent(4, 32, 16, 48, 48, 0.14, 40, (50000.0, 16), kv_from=0), _moe(4, 2, 32, 64)),
        _layer(_parallel(_left(2, 2, 64, 64, 0.125, 30.0, (0.3, 16)), (2, 64, 32, (0.7, 0.995)), 1.1, 0.8), _moe(4, 2, 32, 64)),
    ],
}
CONFIGS = {"A": KAR_A, "B": KAR_B, "C": KAR_C, "D": KAR_D, "E": KAR_E}
PAGE_SIZE = {"A": 8, "B": 16, "C": 4, "D": 16, "E": 16}


def config_dict(name: str, **changes) -> dict:
    out = copy.deepcopy(CONFIGS[name])
    out.update(changes)
    return out


def make_karorax_folder(tmp_path, name: str, seed: int = 0, dtype=torch.float32, sharpen: float = 1.0, std: float = 0.08,
                        all_experts: bool = False, data: dict = None) -> str:
    """A random-weights folder for configuration `name` (or for `data`).  `sharpen` multiplies every attention's score scale,
    so that the softmax picks out single keys and a wrong or missing key shows in the logits.  `all_experts`: every routed
    layer chooses all its experts - for comparisons in bfloat16, where rounding may turn a close call between two experts
    the other way than the plain implementation's float64 does."""
    import kvcache_b200  # registers the architectures  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    data = config_dict(name, initializer_range=std) if data is None else dict(copy.deepcopy(data), initializer_range=std)
    for layer in data["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= sharpen
        else:
            layer["mixer"]["scale"] *= sharpen
        if all_experts and layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    folder = os.path.join(str(tmp_path), f"kar_{name}_{seed}_{sharpen}_{int(all_experts)}")
    write_random_model(folder, config_from_dict(data), seed, dtype)
    return folder
