"""The Nuderax design stated plainly: whole sequences, no cache, no batching, float64 on the CPU.

One function per mechanism, written from the design's equations and sharing nothing with the
package: the tests compare the package's kernels, cache and scheduler with these.

Notation: x is [tokens, width]; a weight W is stored [out, in] and applied as ``x @ W.T``.

* layer norm without bias: ``(x - mean) / sqrt(var + eps) * w`` (var = mean of squared deviations)
* root-mean-square norm: ``x / sqrt(mean(x^2) + eps) * w``
* rotation: the pair (2i, 2i+1) of a vector at position p turns by the angle ``p * base**(-2i/dims)``
* latent attention: keys and values of all heads are made from one latent vector per token plus
  one rotated key part that every head shares
* routed feed-forward: sigmoid scores, a correction that enters the choice only, groups of
  neighbouring experts of which the best stay eligible, a shared expert for every token
* a layer adds mixer(norm1(x)) + ff(norm2(x)) to x: both read the same x
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    d = x - mean
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_pairs(v, positions, base, dims):
    """v: [tokens, ..., n]; the first ``dims`` entries are turned pair by pair (2i with 2i+1),
    the rest pass unchanged."""
    out = v.clone()
    p = torch.as_tensor(positions, dtype=F64).reshape((-1,) + (1,) * (v.dim() - 1))
    for i in range(dims // 2):
        a = p * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[..., 0], torch.sin(a)[..., 0]
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_and_shared_key(h, w_dkv, w_norm, kv_rank, eps, positions, rot):
    """What a layer keeps per token: the normed latent and the rotated shared key part."""
    d = h @ w_dkv.T
    c = rms_norm(d[:, :kv_rank], w_norm, eps)
    kr = rotate_pairs(d[:, kv_rank:], positions, rot["base"], rot["dims"])
    return c, kr


def latent_attention(q, c, kr, w_uk, w_uv, heads, dim, rot_dim, vdim, scale, positions, rot):
    """q: [tokens, heads * (dim + rot_dim)] not yet rotated; c: [tokens, kv_rank]; kr: [tokens,
    rot_dim] already rotated.  Causal softmax attention; returns [tokens, heads * vdim]."""
    n = q.shape[0]
    q = q.reshape(n, heads, dim + rot_dim)
    q_plain = q[:, :, :dim]
    q_rot = rotate_pairs(q[:, :, dim:], positions, rot["base"], rot["dims"])
    k_plain = (c @ w_uk.T).reshape(n, heads, dim)
    v = (c @ w_uv.T).reshape(n, heads, vdim)
    out = torch.zeros(n, heads, vdim, dtype=q.dtype)
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for hd in range(heads):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ kr.T) * scale
        s = s.masked_fill(~mask, -math.inf)
        p = torch.softmax(s, dim=-1)
        out[:, hd] = p @ v[:, hd]
    return out.reshape(n, heads * vdim)


def mixer(kind, h, W, pre, m, eps, positions, shared_kv=None):
    """One latent-attention mixer.  ``W`` maps tensor names to tensors, ``pre`` is the mixer's
    prefix, ``m`` its sizes.  Returns (output, (c, kr)) so that a later layer can read the cache."""
    if kind == "latent_attention_2":
        cq = rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
        q = cq @ W[pre + "uq"].T
    else:
        q = h @ W[pre + "q"].T
    if shared_kv is None:
        c, kr = latent_and_shared_key(h, W[pre + "dkv"], W[pre + "dkv.norm"], m["kv_rank"], eps, positions, m["rot"])
    else:
        c, kr = shared_kv
    a = latent_attention(q, c, kr, W[pre + "uk"], W[pre + "uv"], m["heads"], m["dim"], m["rot_dim"], m["vdim"],
                         m["scale"], positions, m["rot"])
    return a @ W[pre + "o"].T, (c, kr)


def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, w_router, correction, r):
    """Chosen experts [tokens, top] and their weights."""
    s = torch.sigmoid(h @ w_router.T)
    choice = s + correction
    n, e = s.shape
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = e // groups["count"]
    by_group = choice.reshape(n, groups["count"], per)
    group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros(n, groups["count"], dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed.repeat_interleave(per, dim=1)
    masked = choice.masked_fill(~allowed, -math.inf)
    chosen = masked.topk(r["top"], dim=-1).indices
    weights = s.gather(1, chosen) * r["scale"]
    return chosen, weights


def feed_forward(h, W, pre, mlp):
    r = mlp["router"]
    chosen, weights = route(h, W[pre + "router"], W[pre + "correction"], r)
    out = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(chosen[t, j])
            out[t] += weights[t, j] * expert(h[t:t + 1], W[f"{pre}e{e}.gate"], W[f"{pre}e{e}.up"], W[f"{pre}e{e}.down"],
                                             mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + expert(h, W[pre + "shared.gate"], W[pre + "shared.up"], W[pre + "shared.down"], mlp["shared"]["limit"])
    return out


def forward(config, W, tokens, layers_out=None):
    """Logits [tokens, vocab] of one whole sequence.  ``W``: name -> tensor (any float dtype).
    ``layers_out``: a list that receives the stream after every layer."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    eps = config["norm"]["eps"]
    positions = list(range(len(tokens)))
    x = layer_norm(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        pre = f"l{i}."
        src = m.get("kv_from")
        y, kept[i] = mixer(layer["type"], layer_norm(x, W[pre + "norm1"], eps), W, pre + "mix.", m, eps, positions,
                           kept[src] if src is not None else None)
        if layer.get("mlp"):
            y = y + feed_forward(layer_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.", layer["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, W["final.norm"], eps) @ W["embed"].T
