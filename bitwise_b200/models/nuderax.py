"""Nuderax assembled from parts, and its entry in the architecture registry.

A decoder of parallel blocks: every layer adds ``mixer(norm1(x)) + feed_forward(norm2(x))`` to
the stream, both norms layer norms with a weight and no bias.  The mixers are latent attention
(queries straight from the input, or through a latent of their own), some of them reading the
cache of an earlier layer; the feed-forward is routed (sigmoid scores with a correction for the
choice, groups of experts, a shared expert).  The embedded rows pass a layer norm before the
first layer, the head is the embedding table after a last layer norm.

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q | dq, dq.norm, uq}``, ``l<i>.mix.{dkv, dkv.norm}`` (absent where the
layer reads another's cache), ``l<i>.mix.{uk, uv, o}``, ``l<i>.mlp.e<k>.{gate, up, down}``,
``l<i>.mlp.{router, correction}``, ``l<i>.mlp.shared.{gate, up, down}``.  Matrices are stored
[out, in].
"""
from __future__ import annotations

from ..config.nuderax import NuderaxConfig
from ..config.registry import register_architecture
from ..parts.block import ParallelBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.latent_attention import LatentAttention
from ..parts.norm import LayerNorm
from ..parts.rope import RotaryEncoding
from ..parts.routed_ffn import ClampedGLU, RoutedFFN
from .decoder import DecoderModel, LayerRun

BLOCK_NAMES = {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "feed_forward": "mlp"}
GLU_ALPHA = 1.702  # the constant inside the experts' sigmoid


def build_nuderax(config: NuderaxConfig) -> DecoderModel:
    c = config
    rotaries = {}   # one table per (turned entries, base)
    blocks, schedule, entry_of = [], [], {}
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        rotary = rotaries.setdefault((m.rot_dims, m.rot_base), RotaryEncoding(m.rot_dims, m.rot_base))
        mixer = LatentAttention(c.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale, c.eps, position=rotary,
                                q_rank=m.q_rank if m.kind == "latent_attention_2" else None,
                                shares_cache=m.kv_from is not None)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            f = layer.mlp
            shared = ClampedGLU(c.width, f.shared_ff, f.shared_limit, GLU_ALPHA) if f.shared_ff is not None else None
            ffn = RoutedFFN(c.width, f.experts, f.top, f.ff, f.limit, GLU_ALPHA, f.weight_scale, f.groups, f.keep_groups,
                            correction=True, shared=shared)
            ffn_norm = LayerNorm(c.width, c.eps, suffix="")
        blocks.append(ParallelBlock(c.width, mixer, ffn, LayerNorm(c.width, c.eps, suffix=""), ffn_norm, BLOCK_NAMES))
        if m.kv_from is None:
            entry_of[i] = len(entry_of)
            schedule.append(LayerRun(i, entry_of[i], True))
        else:
            schedule.append(LayerRun(i, entry_of[m.kv_from], False))
    embedding = TokenEmbedding(c.vocab, c.width, tensor="embed", norm=LayerNorm(c.width, c.eps, suffix=""),
                               norm_tensor="embed.norm")
    head = OutputHead(c.vocab, c.width, LayerNorm(c.width, c.eps, suffix=""), tied_to=embedding, norm_name="final.norm")
    return DecoderModel(c, embedding, blocks, head, schedule=schedule, position_encodings=list(rotaries.values()),
                        block_prefix="l{}", embed_prefix="")


register_architecture("Nuderax", NuderaxConfig.from_json, build_nuderax)
