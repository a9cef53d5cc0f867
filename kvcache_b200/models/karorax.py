"""The Karorax decoder put together from parts, layer by layer, from its configuration.

Tensor names: `embed`, `bigram`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`,
`l<i>.mix.*` (the mixer; the two sides of a parallel mixer under `left.` and `right.`), `l<i>.mlp.*` (dense: `up`, `down`;
routed: `router`, `router.b`, experts `e<j>.`, `shared.`).  A layer is x += ls1 * mixer(norm1(x)); x += ls2 * ff(norm2(x));
the norms' weights are stored around zero (the factor is 1 + w).  The embedding adds a row of a hashed table of token
pairs; the logits pass through cap * tanh(. / cap).  Layer kinds: `latent_attention` - keys and values expanded from one
cached latent per token, queries straight from the input, neighbouring numbers rotated as pairs, a window, a learned
sink per head in the softmax, a gate per head; with `kv_from` the layer reads the cache entry of an earlier layer instead
of projecting a latent.  `parallel` - attention with grouped keys (no rotation; a query temperature that grows with the
position, capped scores, a bias that grows with the distance) beside lightning attention (a constant decay per head),
summed with two scales.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.karorax import KARORAX_ARCHITECTURE, DenseSpec, KaroraxConfig, LatentSpec, ParallelSpec, RotarySpec
from ..config.registry import register_architecture
from ..parts.attention import GQAAttention
from ..parts.block import LayerScale, PreNormBlock
from ..parts.embedding import HashedBigramEmbedding
from ..parts.feedforward import GatedMLP, ReluSquaredMLP, RoutedMLP
from ..parts.latent_attention import LatentAttention
from ..parts.model import DecoderModel, LayerCall
from ..parts.norm import RMSNorm
from ..parts.position import RotaryHalf
from ..parts.recurrent import LightningAttention, ParallelMixer

# Until the engine tells how long a request may get (it always does), rotation tables are made for this many positions.
DEFAULT_POSITIONS = 4096
# The norms' weights are stored as their distance from this.
NORM_WEIGHT_OFFSET = 1.0


def build_karorax(config: KaroraxConfig, dtype: str = "bfloat16", device: str = "cuda:0",
                  max_positions: Optional[int] = None) -> DecoderModel:
    c = config
    positions = max_positions or DEFAULT_POSITIONS
    rotations: Dict[tuple, RotaryHalf] = {}          # layers with equal rotation constants share one table

    def rotation(spec: RotarySpec) -> RotaryHalf:
        key = (spec.dims, spec.base)
        if key not in rotations:
            rotations[key] = RotaryHalf(spec.dims, spec.base, positions)
        return rotations[key]

    def norm(name: str) -> RMSNorm:
        return RMSNorm(c.width, c.norm_eps, name, offset=NORM_WEIGHT_OFFSET)

    def mixer(spec, p: str):
        if isinstance(spec, LatentSpec):
            return LatentAttention(c.width, spec.heads, spec.dim, spec.rot_dim, spec.vdim, spec.kv_rank, None, scale=spec.scale,
                                   eps=c.norm_eps, position=rotation(spec.rot), prefix=p, dtype=dtype, window=spec.window,
                                   sink="learned", gate="head", rotary_layout="interleaved", own_latent=spec.kv_from is None)
        assert isinstance(spec, ParallelSpec)
        a, g = spec.left, spec.right
        left = GQAAttention(c.width, a.heads, a.kv_heads, a.dim, qkv_bias=False, out_bias=False, position=None, window=None,
                            prefix=p + "left.", dtype=dtype, scale=a.scale, value_dim=a.vdim, names=("q", "k", "v", "o"),
                            q_temperature=None if a.q_temp is None else (a.q_temp.coef, a.q_temp.every), score_cap=a.softcap,
                            distance_bias="geometric", pad_values=True)
        right = LightningAttention(c.width, g.heads, g.dim, g.vdim, g.decay, eps=c.norm_eps, prefix=p + "right.", dtype=dtype)
        return ParallelMixer(c.width, left, right, spec.left_scale, spec.right_scale, dtype)

    blocks, schedule, cache_of = [], [], {}
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = norm2 = scale2 = None
        if isinstance(layer.mlp, DenseSpec):
            ffn = ReluSquaredMLP(c.width, layer.mlp.ff, prefix=p + "mlp.", dtype=dtype)
        elif layer.mlp is not None:
            m = layer.mlp
            shared = None
            if m.shared_ff is not None:
                shared = GatedMLP(c.width, m.shared_ff, activation="silu", prefix=p + "mlp.shared.", dtype=dtype,
                                  names=("gate", "up", "down"))
            ffn = RoutedMLP(c.width, m.expert_ff, m.experts, m.top, activation="swiglu", scores="chosen", prefix=p + "mlp.",
                            dtype=dtype, shared=shared, router_bias="router.b")
        if ffn is not None:
            norm2, scale2 = norm(p + "norm2"), LayerScale(c.width, p + "ls2")
        part = mixer(layer.mixer, p + "mix.")
        blocks.append(PreNormBlock(c.width, norm(p + "norm1"), part, norm2, ffn, dtype, scale1=LayerScale(c.width, p + "ls1"),
                                   scale2=scale2))
        # A layer that reads another's latent has no cache entry of its own: its call reads the other's, which then keeps
        # what the wider of their windows sees.
        source = layer.mixer.kv_from if isinstance(layer.mixer, LatentSpec) else None
        if source is None:
            cache_of[i] = len(cache_of)
            schedule.append(LayerCall(i, cache_of[i]))
        else:
            blocks[source].mixer.keep_for_window(layer.mixer.window)
            schedule.append(LayerCall(i, cache_of[source], writes_cache=False))
    # A checkpoint may carry the second norm and scale of a layer that has no feed-forward: they are left alone.
    unused = [f"l{i}.{name}" for i, layer in enumerate(c.layers) if layer.mlp is None for name in ("norm2", "ls2")]
    embedding_parts = []
    if c.bigram is not None:
        embedding_parts.append(HashedBigramEmbedding(c.width, c.bigram.buckets, c.bigram.mul_prev, c.bigram.mul_cur, c.vocab_size,
                                                     "bigram", dtype))
    return DecoderModel(config=c, dtype=dtype, vocab_size=c.vocab_size, width=c.width, embed_name="embed", head_name="head",
                        blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), position=None,
                        embedding_parts=embedding_parts, ignorable_tensors=unused, logit_softcap=c.logit_softcap)


register_architecture(KARORAX_ARCHITECTURE, KaroraxConfig, build_karorax, replace=True)
