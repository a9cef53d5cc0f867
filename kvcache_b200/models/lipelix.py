"""The Lipelix decoder put together from parts, layer by layer, from its configuration.

Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`
(the norms before and after the two sublayers), `l<i>.shift` (token shift of the mixer's input), `l<i>.rg1` / `.rg1.b`
and `l<i>.rg2` / `.rg2.b` (gates on the sublayers' results), `l<i>.mix.*` (the mixer), `l<i>.mlp.up` / `.down`.
A layer is x += m * norm1b(gate1 * mixer(shift(norm1(x)))); x += m * norm2b(gate2 * ff(norm2(x))), with m the
configuration's residual multiplier (folded into the weights of the norms after the sublayers); the embedded rows are
multiplied by the configuration's embedding scale.  Mixers: `attention` (queries and keys normalised over their whole
projections before the rotation, a learned sink per head), `attention_2` (rotation first, then each head divided by its
root mean square; a window that keeps the first tokens; a sink at 0), `general_delta` (the generalized delta rule).
Attention layers with `v_mix` blend their values with those of the first such layer.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.lipelix import LIPELIX_ARCHITECTURE, AttentionSpec, DeltaSpec, LipelixConfig, RotarySpec
from ..config.registry import register_architecture
from ..parts.attention import GQAAttention
from ..parts.block import ResidualGate, SandwichBlock
from ..parts.feedforward import ReluSquaredMLP
from ..parts.model import DecoderModel, LayerCall
from ..parts.norm import RMSNorm
from ..parts.position import RotaryHalf
from ..parts.recurrent import DeltaRuleMixer
from ..parts.token_shift import TokenShiftMixer

# Until the engine tells how long a request may get (it always does), rotation tables are made for this many positions.
DEFAULT_POSITIONS = 4096
# The sink of `attention_2`: a key without value whose score is 0, so the softmax's denominator is one larger.
WINDOW_ATTENTION_SINK = 0.0


def build_lipelix(config: LipelixConfig, dtype: str = "bfloat16", device: str = "cuda:0",
                  max_positions: Optional[int] = None) -> DecoderModel:
    c = config
    positions = max_positions or DEFAULT_POSITIONS
    rotations: Dict[tuple, RotaryHalf] = {}          # layers with equal rotation constants share one table

    def rotation(spec: Optional[RotarySpec]) -> Optional[RotaryHalf]:
        if spec is None:
            return None
        key = (spec.dims, spec.base)
        if key not in rotations:
            rotations[key] = RotaryHalf(spec.dims, spec.base, positions)
        return rotations[key]

    first_mixing = next((i for i, l in enumerate(c.layers) if isinstance(l.mixer, AttentionSpec) and l.mixer.v_mix), None)

    def mixer(i: int, spec, p: str):
        if isinstance(spec, DeltaSpec):
            return DeltaRuleMixer(c.width, spec.heads, spec.dim, spec.decay_rank, eps=c.norm_eps, prefix=p, dtype=dtype)
        assert isinstance(spec, AttentionSpec)
        value_mix = None if not spec.v_mix else "source" if i == first_mixing else "mix"
        common = dict(qkv_bias=False, out_bias=False, position=rotation(spec.rot), prefix=p, dtype=dtype, scale=spec.scale,
                      value_dim=spec.vdim, qk_norm_eps=c.norm_eps, names=("q", "k", "v", "o"), value_mix=value_mix)
        if spec.kind == "attention":
            return GQAAttention(c.width, spec.heads, spec.kv_heads, spec.dim, window=None, qk_norm_scope="all", sink="learned",
                                **common)
        return GQAAttention(c.width, spec.heads, spec.kv_heads, spec.dim, window=spec.window, keep_first=spec.keep_first,
                            qk_norm_weight=False, qk_norm_after_rotation=True, sink=WINDOW_ATTENTION_SINK, **common)

    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = pre2 = post2 = gate2 = None
        if layer.mlp is not None:
            ffn = ReluSquaredMLP(c.width, layer.mlp.ff, prefix=p + "mlp.", dtype=dtype)
            pre2, post2 = RMSNorm(c.width, c.norm_eps, p + "norm2"), RMSNorm(c.width, c.norm_eps, p + "norm2b", gain=c.residual_mult)
            gate2 = ResidualGate(c.width, p + "rg2", p + "rg2.b", dtype)
        shifted = TokenShiftMixer(c.width, mixer(i, layer.mixer, p + "mix."), p + "shift", dtype)
        blocks.append(SandwichBlock(c.width, RMSNorm(c.width, c.norm_eps, p + "norm1"), shifted,
                                    RMSNorm(c.width, c.norm_eps, p + "norm1b", gain=c.residual_mult), pre2, ffn, post2, dtype,
                                    gate1=ResidualGate(c.width, p + "rg1", p + "rg1.b", dtype), gate2=gate2))
    # A checkpoint may carry the feed-forward's norms and gate of a layer that has none: they are left alone.
    unused = [f"l{i}.{name}" for i, layer in enumerate(c.layers) if layer.mlp is None
              for name in ("norm2", "norm2b", "rg2", "rg2.b")]
    return DecoderModel(config=c, dtype=dtype, vocab_size=c.vocab_size, width=c.width, embed_name="embed", head_name="head",
                        blocks=blocks, schedule=[LayerCall(i, i) for i in range(len(c.layers))],
                        final_norm=RMSNorm(c.width, c.norm_eps, "final.norm"), position=None, ignorable_tensors=unused,
                        embed_scale=c.embedding_scale)


register_architecture(LIPELIX_ARCHITECTURE, LipelixConfig, build_lipelix, replace=True)
