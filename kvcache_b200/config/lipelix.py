"""Configuration of the Lipelix decoder, read from its own config.json keys.

config.json of this design is nested: `layers` is a list with one object per layer (`type` names the mixer, its sizes
lie under `mixer`, the feed-forward under `mlp` or null), beside `embedding.scale`, `residual_mult`, `norm.eps`,
`vocab` and `width`.  Mixer types: `attention` (grouped heads, queries and keys normalised over their whole
projection, a learned sink per head), `attention_2` (queries and keys divided by their root mean square per head after
the rotation, a window of keys that also keeps the sequence's first tokens, a sink at 0) and `general_delta` (a matrix
state per head under the generalized delta rule).  Every size and every constant that can differ between models is
read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .base import KeyReader, ModelConfig

LIPELIX_ARCHITECTURE = "Lipelix"
MIXER_TYPES = ("attention", "attention_2", "general_delta")


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int


@dataclass(frozen=True)
class AttentionSpec:
    """Both attention mixers; `kind` tells which norm, mask and sink go with it (see models/lipelix.py)."""
    kind: str
    heads: int
    kv_heads: int
    dim: int                         # numbers of a head's query and key
    vdim: int                        # numbers of a head's value
    scale: float
    rot: Optional[RotarySpec]
    v_mix: bool
    window: Optional[int] = None     # `mask.size`: keys a query sees, its own included; None: all
    keep_first: int = 0              # `mask.keep_first`: the sequence's first tokens stay visible beyond the window


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    dim: int
    decay_rank: Optional[int] = None   # inner size of the decay's two matrices; None: the checkpoint's shapes decide


@dataclass(frozen=True)
class DenseSpec:
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: Union[AttentionSpec, DeltaSpec, None]
    mlp: Optional[DenseSpec]


def _read_rot(m: KeyReader) -> Optional[RotarySpec]:
    rot = m.sub("rot", required=False)
    if rot is None:
        return None
    spec = RotarySpec(rot.number("base", positive=True), rot.integer("dims", minimum=2))
    if spec.dims is not None and spec.dims % 2:
        rot.fail(f"'dims' must be even, got {spec.dims}")
    m.absorb(rot)
    return spec


def _read_mixer(lr: KeyReader, kind: Optional[str]):
    m = lr.sub("mixer")
    if m is None or kind is None:
        return None
    if kind == "general_delta":
        spec = DeltaSpec(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("decay_rank", default=None, minimum=1))
        lr.absorb(m)
        return spec
    window, keep_first = None, 0
    mask = m.sub("mask", required=False)
    if mask is not None:
        if kind == "attention":
            m.fail("'mask' belongs to attention_2")
        window = mask.integer("size", minimum=1)
        keep_first = mask.integer("keep_first", default=0, minimum=0)
        m.absorb(mask)
    spec = AttentionSpec(kind=kind, heads=m.integer("heads", minimum=1), kv_heads=m.integer("kv_heads", minimum=1),
                         dim=m.integer("dim", minimum=1), vdim=m.integer("vdim", minimum=1),
                         scale=m.number("scale", positive=True), rot=_read_rot(m), v_mix=m.boolean("v_mix", default=False),
                         window=window, keep_first=keep_first or 0)
    if None not in (spec.heads, spec.kv_heads) and spec.heads % spec.kv_heads:
        m.fail(f"heads {spec.heads} is not a multiple of kv_heads {spec.kv_heads}")
    if spec.rot is not None and None not in (spec.rot.dims, spec.dim) and spec.rot.dims > spec.dim:
        m.fail(f"rot.dims {spec.rot.dims} exceeds dim {spec.dim}")
    lr.absorb(m)
    return spec


def _read_mlp(lr: KeyReader) -> Optional[DenseSpec]:
    m = lr.sub("mlp", required=False)
    if m is None:
        return None
    kind = m.string("kind")
    spec = None
    if kind == "dense":
        spec = DenseSpec(m.integer("ff", minimum=1))
    elif kind is not None:
        m.fail(f"unknown feed-forward kind '{kind}' (dense)")
    lr.absorb(m)
    return spec


@dataclass(frozen=True)
class LipelixConfig(ModelConfig):
    vocab_size: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    layers: Tuple[LayerSpec, ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "LipelixConfig":
        r = KeyReader(data, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = r.sub("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        r.absorb(norm)
        emb = r.sub("embedding", required=False)
        scale = emb.number("scale", default=1.0) if emb is not None else 1.0
        r.absorb(emb)
        mult = r.number("residual_mult", default=1.0)
        raw_layers = data.get("layers")
        layers = []
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            r.fail("'layers' must be a non-empty list")
        else:
            for i, item in enumerate(raw_layers):
                if not isinstance(item, Mapping):
                    r.fail(f"layers[{i}] must be an object")
                    continue
                lr = KeyReader(item, f"{where}: layers[{i}]")
                kind = lr.string("type")
                if kind is not None and kind not in MIXER_TYPES:
                    lr.fail(f"unknown mixer type '{kind}' ({', '.join(MIXER_TYPES)})")
                    kind = None
                layers.append(LayerSpec(kind, _read_mixer(lr, kind), _read_mlp(lr)))
                r.absorb(lr)
        # Layers that mix values take them from the first such layer, number by number: they must have as many.
        mixing = [(i, l.mixer) for i, l in enumerate(layers) if isinstance(l.mixer, AttentionSpec) and l.mixer.v_mix]
        for i, m in mixing[1:]:
            first = mixing[0][1]
            if None not in (m.kv_heads, m.vdim, first.kv_heads, first.vdim) and m.kv_heads * m.vdim != first.kv_heads * first.vdim:
                r.fail(f"layers[{i}]: v_mix needs kv_heads * vdim = {first.kv_heads * first.vdim} as in layers[{mixing[0][0]}], "
                       f"got {m.kv_heads * m.vdim}")
        eos = r.int_list("eos_token_id", default=())
        init_range = r.number("initializer_range", default=0.05, positive=True)
        r.finish()
        return cls(architecture=LIPELIX_ARCHITECTURE, vocab_size=vocab, width=width, norm_eps=eps, residual_mult=mult,
                   embedding_scale=scale, layers=tuple(layers), eos_token_ids=eos, initializer_range=init_range)

    def to_dict(self) -> Dict[str, Any]:
        def mixer(s):
            if isinstance(s, DeltaSpec):
                return {"heads": s.heads, "dim": s.dim, **({} if s.decay_rank is None else {"decay_rank": s.decay_rank})}
            out: Dict[str, Any] = {"heads": s.heads, "kv_heads": s.kv_heads, "dim": s.dim, "vdim": s.vdim, "scale": s.scale,
                                   "v_mix": s.v_mix}
            if s.rot is not None:
                out["rot"] = {"base": s.rot.base, "dims": s.rot.dims}
            if s.window is not None:
                out["mask"] = {"size": s.window, "keep_first": s.keep_first}
            return out

        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff}}
                       for l in self.layers],
            "initializer_range": self.initializer_range,
        }
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif len(self.eos_token_ids) > 1:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
