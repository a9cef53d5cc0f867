"""Configuration of the Karorax decoder, read from its own config.json keys.

config.json of this design is nested: `layers` is a list with one object per layer (`type` names the mixer, its sizes
lie under `mixer`, the feed-forward under `mlp` or null), `embedding.bigram` gives the hashed pair table, `norm.eps`,
`logit_softcap`, `vocab`, `width`.  Mixer types: `latent_attention` (keys and values expanded from one cached latent per
token, a window, a sink in the softmax, optionally the latent of an earlier layer: `kv_from`) and `parallel` (attention
with grouped keys, a capped score and a bias that grows with the distance, beside lightning attention with one decay per
head).  Feed-forwards: `dense` or `moe`.  Every size and every constant that can differ between models is read here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .base import KeyReader, ModelConfig

KARORAX_ARCHITECTURE = "Karorax"


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int                         # numbers of a head's query and key that are not rotated
    rot_dim: int                     # numbers of the rotated part (of a head's query, and of the key part all heads share)
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]            # keys a query sees, its own included; None: all
    rot: RotarySpec
    kv_from: Optional[int] = None    # the layer whose cached latent and key part this layer reads instead of its own


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int


@dataclass(frozen=True)
class BiasedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    q_temp: Optional[QueryTemperature]


@dataclass(frozen=True)
class LightningSpec:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]         # one per head


@dataclass(frozen=True)
class ParallelSpec:
    left: BiasedAttentionSpec
    right: LightningSpec
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseSpec:
    ff: int


@dataclass(frozen=True)
class RoutedSpec:
    expert_ff: int
    experts: int
    top: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: Union[LatentSpec, ParallelSpec, None]
    mlp: Union[DenseSpec, RoutedSpec, None]


@dataclass(frozen=True)
class BigramSpec:
    buckets: int
    mul_prev: int
    mul_cur: int


def _read_latent(m: KeyReader) -> LatentSpec:
    mask = m.sub("mask", required=False)
    window = mask.integer("size", minimum=1) if mask is not None else None
    m.absorb(mask)
    rot = m.sub("rot")
    rotary = None
    if rot is not None:
        rotary = RotarySpec(rot.number("base", positive=True), rot.integer("dims", minimum=2))
        if rotary.dims is not None and rotary.dims % 2:
            rot.fail(f"'dims' must be even, got {rotary.dims}")
        m.absorb(rot)
    spec = LatentSpec(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1), rot_dim=m.integer("rot_dim", minimum=2),
                      vdim=m.integer("vdim", minimum=1), kv_rank=m.integer("kv_rank", minimum=1),
                      scale=m.number("scale", positive=True), window=window, rot=rotary,
                      kv_from=m.integer("kv_from", default=None, minimum=0))
    if rotary is not None and None not in (rotary.dims, spec.rot_dim) and rotary.dims > spec.rot_dim:
        m.fail(f"rot.dims {rotary.dims} exceeds rot_dim {spec.rot_dim}")
    return spec


def _read_left(parent: KeyReader) -> Optional[BiasedAttentionSpec]:
    m = parent.sub("left")
    if m is None:
        return None
    temp = m.sub("q_temp", required=False)
    q_temp = None
    if temp is not None:
        q_temp = QueryTemperature(temp.number("coef"), temp.integer("every", minimum=1))
        m.absorb(temp)
    spec = BiasedAttentionSpec(heads=m.integer("heads", minimum=1), kv_heads=m.integer("kv_heads", minimum=1),
                               dim=m.integer("dim", minimum=1), vdim=m.integer("vdim", minimum=1),
                               scale=m.number("scale", positive=True), softcap=m.number("softcap", default=None, positive=True),
                               q_temp=q_temp)
    if None not in (spec.heads, spec.kv_heads) and spec.heads % spec.kv_heads:
        m.fail(f"heads {spec.heads} is not a multiple of kv_heads {spec.kv_heads}")
    parent.absorb(m)
    return spec


def _read_right(parent: KeyReader) -> Optional[LightningSpec]:
    m = parent.sub("right")
    if m is None:
        return None
    heads = m.integer("heads", minimum=1)
    raw = m.data.get("decay")
    decay: Tuple[float, ...] = ()
    if isinstance(raw, (int, float)) and not isinstance(raw, bool) and heads is not None:
        raw = [raw] * heads
    if not isinstance(raw, (list, tuple)) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in raw):
        m.fail("'decay' must be a list of numbers, one per head")
    else:
        decay = tuple(float(d) for d in raw)
        if heads is not None and len(decay) != heads:
            m.fail(f"'decay' has {len(decay)} numbers for {heads} heads")
        if any(not 0.0 <= d <= 1.0 for d in decay):
            m.fail("every 'decay' must lie in [0, 1]")
    spec = LightningSpec(heads, m.integer("dim", minimum=1), m.integer("vdim", minimum=1), decay)
    parent.absorb(m)
    return spec


def _read_mixer(lr: KeyReader, kind: Optional[str]):
    m = lr.sub("mixer")
    if m is None or kind is None:
        return None
    spec = None
    if kind == "latent_attention":
        spec = _read_latent(m)
    elif kind == "parallel":
        spec = ParallelSpec(_read_left(m), _read_right(m), m.number("left_scale"), m.number("right_scale"))
    lr.absorb(m)
    return spec


def _read_mlp(lr: KeyReader):
    m = lr.sub("mlp", required=False)
    if m is None:
        return None
    kind = m.string("kind")
    spec = None
    if kind == "dense":
        spec = DenseSpec(m.integer("ff", minimum=1))
    elif kind == "moe":
        router, expert, shared = m.sub("router"), m.sub("expert"), m.sub("shared", required=False)
        experts = router.integer("experts", minimum=1) if router is not None else None
        top = router.integer("top", minimum=1) if router is not None else None
        if None not in (experts, top) and top > experts:
            m.fail(f"router.top {top} exceeds router.experts {experts}")
        spec = RoutedSpec(expert.integer("ff", minimum=1) if expert is not None else None, experts or 0, top or 0,
                          shared.integer("ff", minimum=1) if shared is not None else None)
        for child in (router, expert, shared):
            m.absorb(child)
    elif kind is not None:
        m.fail(f"unknown feed-forward kind '{kind}' (dense, moe)")
    lr.absorb(m)
    return spec


@dataclass(frozen=True)
class KaroraxConfig(ModelConfig):
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    bigram: Optional[BigramSpec]
    logit_softcap: Optional[float]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "KaroraxConfig":
        r = KeyReader(data, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = r.sub("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        r.absorb(norm)
        bigram = None
        emb = r.sub("embedding", required=False)
        if emb is not None:
            b = emb.sub("bigram", required=False)
            if b is not None:
                bigram = BigramSpec(b.integer("buckets", minimum=1), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0))
                emb.absorb(b)
            r.absorb(emb)
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
                if kind is not None and kind not in ("latent_attention", "parallel"):
                    lr.fail(f"unknown mixer type '{kind}' (latent_attention, parallel)")
                    kind = None
                layers.append(LayerSpec(kind, _read_mixer(lr, kind), _read_mlp(lr)))
                r.absorb(lr)
            # A layer that reads another's latent: the other lies before it, projects its own, and agrees in what is cached.
            for i, layer in enumerate(layers):
                m = layer.mixer
                if not isinstance(m, LatentSpec) or m.kv_from is None:
                    continue
                j = m.kv_from
                src = layers[j].mixer if j < i else None
                if not isinstance(src, LatentSpec) or src.kv_from is not None:
                    r.fail(f"layers[{i}]: kv_from {j} must name an earlier latent_attention layer that keeps its own latent")
                elif (src.kv_rank, src.rot_dim, src.rot) != (m.kv_rank, m.rot_dim, m.rot):
                    r.fail(f"layers[{i}]: kv_rank, rot_dim and rot must equal those of layer {j}, whose latent it reads")
        softcap = r.number("logit_softcap", default=None, positive=True)
        eos = r.int_list("eos_token_id", default=())
        init_range = r.number("initializer_range", default=0.05, positive=True)
        r.finish()
        return cls(architecture=KARORAX_ARCHITECTURE, vocab_size=vocab, width=width, norm_eps=eps, layers=tuple(layers),
                   bigram=bigram, logit_softcap=softcap, eos_token_ids=eos, initializer_range=init_range)

    def to_dict(self) -> Dict[str, Any]:
        def mixer(s):
            if isinstance(s, LatentSpec):
                out: Dict[str, Any] = {"heads": s.heads, "dim": s.dim, "rot_dim": s.rot_dim, "vdim": s.vdim, "kv_rank": s.kv_rank,
                                       "scale": s.scale, "rot": {"base": s.rot.base, "dims": s.rot.dims}}
                if s.window is not None:
                    out["mask"] = {"size": s.window}
                if s.kv_from is not None:
                    out["kv_from"] = s.kv_from
                return out
            left: Dict[str, Any] = {"heads": s.left.heads, "kv_heads": s.left.kv_heads, "dim": s.left.dim, "vdim": s.left.vdim,
                                    "scale": s.left.scale}
            if s.left.softcap is not None:
                left["softcap"] = s.left.softcap
            if s.left.q_temp is not None:
                left["q_temp"] = {"coef": s.left.q_temp.coef, "every": s.left.q_temp.every}
            return {"left": left, "left_scale": s.left_scale, "right_scale": s.right_scale,
                    "right": {"heads": s.right.heads, "dim": s.right.dim, "vdim": s.right.vdim, "decay": list(s.right.decay)}}

        def mlp(s):
            if s is None:
                return None
            if isinstance(s, DenseSpec):
                return {"kind": "dense", "ff": s.ff}
            out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": s.expert_ff}, "router": {"experts": s.experts, "top": s.top}}
            if s.shared_ff is not None:
                out["shared"] = {"ff": s.shared_ff}
            return out

        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
            "initializer_range": self.initializer_range,
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif len(self.eos_token_ids) > 1:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
