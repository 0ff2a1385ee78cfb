"""Small Nuderax configurations for the tests, and weights for them.

The configurations differ from one another in every size: widths that are no multiple of 8,
head counts 1 to 40, latent sizes beside and beyond a multiple of 32, rotated parts of which
only some entries turn, one group of experts and several, one choice and several, layers with
and without a feed-forward or a shared expert, a layer that reads an earlier layer's cache.
Weights are drawn so that scores, router logits and activations are of order one (the clamps
bite, the groups and the correction decide choices, the softmax is far from flat).
"""
import numpy as np
import torch

from bitwise_b200.config import LatentMixerConfig, NuderaxConfig, NuderaxLayerConfig, RoutedMlpConfig


def mixer(kind="latent_attention", heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=0.2, base=10000.0,
          dims=None, q_rank=None, kv_from=None):
    return LatentMixerConfig(kind, heads, dim, rot_dim, vdim, kv_rank, scale, base, dims if dims is not None else rot_dim,
                             q_rank, kv_from)


def mlp(experts=6, top=2, scale=1.0, groups=1, keep=1, ff=24, limit=1.0, shared_ff=None, shared_limit=None):
    return RoutedMlpConfig(experts, top, scale, groups, keep, ff, limit, shared_ff, shared_limit)


CONFIGS = {
    # two kinds of mixer, groups of experts, a shared expert, a layer reading layer 1's cache
    "a": NuderaxConfig(vocab=131, width=72, eps=1e-5, layers=(
        NuderaxLayerConfig(mixer("latent_attention_2", heads=2, dim=16, rot_dim=16, vdim=24, kv_rank=48, scale=0.17,
                                 base=5000.0, q_rank=40), mlp(8, 3, 1.3, 4, 2, 20, 1.2, 28, 1.7)),
        NuderaxLayerConfig(mixer(heads=5, dim=16, rot_dim=8, vdim=16, kv_rank=40, scale=0.21, base=200000.0),
                           mlp(8, 3, 1.3, 4, 2, 20, 1.2, 28, 1.7)),
        NuderaxLayerConfig(mixer(heads=5, dim=16, rot_dim=8, vdim=16, kv_rank=40, scale=0.21, base=200000.0, kv_from=1),
                           mlp(8, 3, 1.3, 4, 2, 20, 1.2, 28, 1.7)))),
    # odd sizes everywhere, one head, one choice, one group, no shared expert, a layer without feed-forward,
    # only part of the rotated entries turn
    "b": NuderaxConfig(vocab=97, width=50, eps=1e-6, layers=(
        NuderaxLayerConfig(mixer(heads=1, dim=10, rot_dim=6, vdim=7, kv_rank=33, scale=0.3, base=100.0, dims=4),
                           mlp(5, 1, 2.0, 1, 1, 9, 0.8)),
        NuderaxLayerConfig(mixer("latent_attention_2", heads=3, dim=6, rot_dim=10, vdim=12, kv_rank=70, scale=0.25,
                                 base=777.0, q_rank=19), None),
        NuderaxLayerConfig(mixer(heads=1, dim=10, rot_dim=6, vdim=7, kv_rank=33, scale=0.3, base=100.0, dims=4, kv_from=0),
                           mlp(6, 2, 0.7, 6, 3, 11, 3.0, 5, 0.5)))),
    # many heads (more than a block of the attention kernel takes), a latent beyond 128, groups of one expert
    "c": NuderaxConfig(vocab=64, width=64, eps=1e-5, layers=(
        NuderaxLayerConfig(mixer(heads=40, dim=8, rot_dim=4, vdim=8, kv_rank=136, scale=0.3, base=10000.0),
                           mlp(4, 2, 1.0, 4, 3, 16, 1.0, 16, 1.0)),)),
}


def random_weights(config, seed, std=None):
    """name -> bfloat16 CPU tensor (float32 for the router's correction and the norm weights)."""
    from bitwise_b200.config.registry import lookup_architecture
    g = torch.Generator().manual_seed(seed)
    specs = lookup_architecture("Nuderax").build(config).param_specs()
    out = {}
    for s in specs:
        if s.name.endswith("correction"):
            t = torch.randn(s.shape, generator=g) * 0.3
        elif len(s.shape) == 1:
            t = 1.0 + 0.2 * torch.randn(s.shape, generator=g)
        elif s.name == "embed":
            t = torch.randn(s.shape, generator=g)
        else:
            t = torch.randn(s.shape, generator=g) * (std or 1.6 / np.sqrt(s.shape[1]))
        out[s.name] = t.to(torch.bfloat16)
    return out


def tokens(config, n, seed):
    return np.random.default_rng(seed).integers(0, config.vocab, n).tolist()
