"""Small Favudra configurations for the tests, and weights for them.

The configurations differ from one another in every size and use every branch: attention with
one and with several key/value heads, value sizes unlike the key size, convolutions of 2, 3 and 5
taps and none, all and only some entries turned, with and without a cap, a layer that reads an
earlier layer's keys and values; window attention with and without a window, grouped and not;
recurrences with square and oblong states; layers with and without a feed-forward; more query
heads on a key/value head than a thread block takes at once.  Weights are drawn so that scores
are of order one to ten (caps bite, the softmax is far from flat, the sink matters), decays lie
between 0.5 and 1, and norm weights scatter around zero.
"""
import numpy as np
import torch

from bitwise_b200.config import FavudraConfig, FavudraLayerConfig, FavudraMixerConfig


def attention(heads, kv_heads, dim, vdim, scale, conv=None, rot=None, softcap=None, kv_from=None):
    return FavudraMixerConfig("attention", heads, dim, vdim, kv_heads=kv_heads, scale=scale, conv=conv,
                              rot_base=rot[1] if rot else None, rot_dims=rot[0] if rot else None, softcap=softcap,
                              kv_from=kv_from)


def window_attention(heads, kv_heads, dim, scale, window=None):
    return FavudraMixerConfig("attention_2", heads, dim, dim, kv_heads=kv_heads, scale=scale, window=window)


def gla(heads, dim, vdim, tau, rank):
    return FavudraMixerConfig("gla", heads, dim, vdim, tau=tau, decay_rank=rank)


def layer(mixer, ff=None):
    return FavudraLayerConfig(mixer, ff)


CONFIGS = {
    # every kind of layer, a layer reading layer 0's keys and values, two key/value heads, values
    # wider than keys, three taps, a quarter of the entries turned
    "a": FavudraConfig(vocab=101, width=64, eps=1e-5, embedding_scale=3.0, logit_scale=0.5, layers=(
        layer(attention(4, 2, 16, 24, 0.3, conv=3, rot=(8, 10000.0), softcap=5.0), 96),
        layer(gla(2, 8, 16, 4.0, 4)),
        layer(window_attention(4, 2, 16, 0.25, window=20), 48),
        layer(attention(4, 2, 16, 24, 0.3, conv=3, rot=(8, 10000.0), softcap=5.0, kv_from=0), 96),
        layer(gla(3, 12, 8, 9.0, 5), 32))),
    # odd sizes: a width that is no multiple of 8, one key/value head and as many as heads, every
    # entry turned, no cap, five and two taps, a window of seven and none at all, one head of state
    "b": FavudraConfig(vocab=67, width=50, eps=1e-6, embedding_scale=1.0, logit_scale=2.0, layers=(
        layer(window_attention(3, 1, 10, 0.4, window=7)),
        layer(attention(2, 2, 36, 12, 0.2, conv=5, rot=(36, 500.0)), 40),
        layer(gla(1, 40, 40, 2.0, 3), 40),
        layer(attention(6, 1, 20, 20, 0.35, conv=2, rot=(4, 77.0), softcap=30.0), 24),
        layer(window_attention(2, 2, 24, 0.3)))),
    # forty query heads on one key/value head, no convolution and no rotation, an oblong state
    # whose rows are no multiple of a thread's share, a window that ends inside a key tile
    "c": FavudraConfig(vocab=64, width=64, eps=1e-5, embedding_scale=8.0, logit_scale=0.25, layers=(
        layer(attention(40, 1, 8, 40, 0.5, softcap=8.0), 64),
        layer(gla(2, 72, 24, 16.0, 9)),
        layer(window_attention(8, 4, 32, 0.2, window=33), 64))),
}

# Layer combinations at the edges of what the cache manager sees: no pages at all, no state at all, two
# windows (two page groups beside the group of full contexts), a one-tap convolution (a factor per
# channel, no state) whose keys a layer with more query heads and a three-tap convolution reads.
EDGE_CONFIGS = {
    "only_gla": FavudraConfig(vocab=50, width=32, eps=1e-5, embedding_scale=2.0, logit_scale=1.0, layers=(
        layer(gla(2, 8, 8, 3.0, 4), 24), layer(gla(1, 16, 8, 5.0, 2)))),
    "only_attention": FavudraConfig(vocab=50, width=32, eps=1e-5, embedding_scale=2.0, logit_scale=1.0, layers=(
        layer(attention(2, 1, 16, 16, 0.3), 24), layer(attention(2, 1, 16, 16, 0.3, kv_from=0)))),
    "two_windows": FavudraConfig(vocab=50, width=32, eps=1e-5, embedding_scale=2.0, logit_scale=1.0, layers=(
        layer(window_attention(2, 1, 16, 0.3, window=5), 24), layer(window_attention(4, 4, 8, 0.3, window=40)),
        layer(attention(2, 2, 16, 8, 0.3, conv=1, rot=(2, 10.0), softcap=2.0), 16),
        layer(attention(4, 2, 16, 8, 0.3, conv=3, rot=(2, 10.0), kv_from=2)))),
}


def random_weights(config, seed):
    """name -> bfloat16 CPU tensor."""
    from bitwise_b200.config.registry import lookup_architecture
    g = torch.Generator().manual_seed(seed)
    specs = lookup_architecture("Favudra").build(config).param_specs()
    out = {}
    for s in specs:
        last = s.name.rsplit(".", 1)[-1]
        if s.name.endswith(".conv"):
            t = torch.randn(s.shape, generator=g) * 0.6
        elif s.name.endswith(".a2.b"):
            t = 1.0 + torch.randn(s.shape, generator=g)
        elif s.name.endswith(".norm") and ".mix." in s.name:
            t = 1.0 + 0.2 * torch.randn(s.shape, generator=g)           # plain weights: around one
        elif len(s.shape) == 1:
            t = 0.2 * torch.randn(s.shape, generator=g)                  # offset weights: around zero
        elif s.name == "embed":
            t = torch.randn(s.shape, generator=g)
        elif last in ("a1", "a2"):
            t = torch.randn(s.shape, generator=g) * (2.0 / np.sqrt(s.shape[1]))
        else:
            t = torch.randn(s.shape, generator=g) * (1.6 / np.sqrt(s.shape[1]))
        out[s.name] = t.to(torch.bfloat16)
    return out


def tokens(config, n, seed):
    return np.random.default_rng(seed).integers(0, config.vocab, n).tolist()
