"""Favudra assembled from parts, and its entry in the architecture registry.

A decoder whose layers carry a norm before and after each sublayer (``SandwichBlock``), every
norm a root-mean-square norm with its weight held around zero.  Three kinds of mixer, in any
order: softmax attention with a short convolution on q, k and v, normed and partly rotated q and
k, capped scores and a sink (``attention``; such a layer may read the keys and values of an
earlier one), attention whose values are its keys, with a penalty on distance inside a window
(``attention_2``), and gated linear attention (``gla``).  The feed-forward is the dense gated one
and may be absent.  The embedded rows are scaled, the logits too.

Tensor names: ``embed``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*`` (see the mixers), ``l<i>.mlp.{gate, up, down}``.
Matrices are stored [out, in].
"""
from __future__ import annotations

from ..config.favudra import FavudraConfig
from ..config.registry import register_architecture
from ..parts.block import SandwichBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.linear_recurrence import GatedLinearAttention
from ..parts.mlp import SwiGLU
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEncoding
from ..parts.scored_attention import ScoredAttention, distance_slopes
from .decoder import DecoderModel, LayerRun

BLOCK_NAMES = {"mixer_norm": "norm1", "mixer_post": "norm1b", "mixer": "mix", "ffn_norm": "norm2", "ffn_post": "norm2b",
               "feed_forward": "mlp"}
SLOPE_EXPONENT = 8.0  # attention_2: slope_h = 2 ** (-8 (h + 1) / heads)


def build_favudra(config: FavudraConfig) -> DecoderModel:
    c = config

    def norm():
        return RMSNorm(c.width, c.eps, suffix="", offset=1.0)

    rotaries = {}   # one table per (turned entries, base)
    blocks, schedule, entry_of = [], [], {}
    entries = 0
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        state_entry = None
        if m.kind == "gla":
            mixer = GatedLinearAttention(c.width, m.heads, m.dim, m.vdim, m.tau, m.decay_rank or max(1, m.dim // 2), c.eps)
        elif m.kind == "attention_2":
            mixer = ScoredAttention(c.width, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, c.eps,
                                    slopes=distance_slopes(m.heads, SLOPE_EXPONENT), window=m.window, values_are_keys=True)
        else:
            rotary = None
            if m.rot_dims:
                rotary = rotaries.setdefault((m.rot_dims, m.rot_base), RotaryEncoding(m.rot_dims, m.rot_base))
            mixer = ScoredAttention(c.width, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, c.eps, conv_taps=m.conv or 0,
                                    qk_norm=True, position=rotary, rot_dims=m.rot_dims or 0, softcap=m.softcap, sink=True,
                                    shares_cache=m.kv_from is not None)
        ffn = SwiGLU(c.width, layer.ff, names=("gate", "up", "down"), suffix="") if layer.ff else None
        blocks.append(SandwichBlock(c.width, mixer, ffn, norm(), norm(), norm() if ffn else None, norm() if ffn else None,
                                    BLOCK_NAMES))
        if m.kv_from is None:
            entry_of[i] = entries
            entries += 1
        if mixer.state_need() is not None:
            state_entry = entries
            entries += 1
        schedule.append(LayerRun(i, entry_of[i if m.kv_from is None else m.kv_from], m.kv_from is None, state_entry))
    embedding = TokenEmbedding(c.vocab, c.width, tensor="embed", scale=c.embedding_scale)
    final = RMSNorm(c.width, c.eps, suffix="", offset=1.0, gain=c.logit_scale)
    head = OutputHead(c.vocab, c.width, final, norm_name="final.norm", head_name="head", suffix="")
    return DecoderModel(c, embedding, blocks, head, schedule=schedule, position_encodings=list(rotaries.values()),
                        block_prefix="l{}", embed_prefix="")


register_architecture("Favudra", FavudraConfig.from_json, build_favudra)
