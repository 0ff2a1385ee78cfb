"""The Favudra design stated plainly: whole sequences, no cache, no batching, float64 on the CPU.

One function per mechanism, written from the design's equations and sharing nothing with the
package: the tests compare the package's kernels, cache, state slots and scheduler with these.

Notation: x is [T, width] (T tokens at positions 0 .. T-1); a weight W is stored [out, in] and
applied as ``x @ W.T``; ``cfg`` is the dictionary of config.json, ``w`` maps tensor names to
float64 tensors.

* norm with an offset weight:  x / sqrt(mean(x^2) + eps) * (1 + g)
* norm with a plain weight:    x / sqrt(mean(x^2) + eps) * g
* a layer:  x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))  (the second only with a feed-forward)
* mixers: softmax attention with a short convolution on q, k, v, normed and partly rotated q and
  k, capped scores and one extra unit in the softmax denominator; attention whose values are its
  keys, with a linear penalty on distance inside a window; a linear recurrence with a decay per
  key channel.
"""
import math

import torch

F64 = torch.float64


# -- norms -------------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_offset(x, g, eps):
    return unit_rms(x, eps) * (1.0 + g)


def norm_plain(x, g, eps):
    return unit_rms(x, eps) * g


# -- activations -------------------------------------------------------------------------------
def silu(z):
    return z * torch.sigmoid(z)


# -- short causal convolution ------------------------------------------------------------------
def causal_conv(u, taps_w):
    """u: [T, C]; taps_w: [C, K].  y[t] = sum_j taps_w[:, j] * u[t - (K - 1) + j], u = 0 before 0."""
    T, C = u.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(u)
    for j in range(K):
        shift = K - 1 - j
        if shift < T:
            y[shift:] += taps_w[:, j] * u[:T - shift]
    return y


# -- rotation ----------------------------------------------------------------------------------
def rotate_pairs(v, dims, base):
    """v: [T, heads, n]; entries 2i and 2i + 1 (i < dims / 2) of every head turn by t * base^(-2i/dims)."""
    out = v.clone()
    t = torch.arange(v.shape[0], dtype=F64)[:, None]
    for i in range(dims // 2):
        a = t * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a), torch.sin(a)
        a0, a1 = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a0 * c - a1 * s
        out[..., 2 * i + 1] = a1 * c + a0 * s
    return out


# -- attention cores ---------------------------------------------------------------------------
def capped_sink_attention(q, k, v, scale, cap):
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv].  Causal.  Scores s = q.k * scale, then
    cap * tanh(s / cap) when a cap is given; weights exp(s_j) / (1 + sum_j exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        out[:, h] = (e / (torch.exp(-m) + e.sum(-1, keepdim=True))) @ v[:, g]
    return out


def distance_window_attention(q, k, scale, window):
    """q: [T, H, d], k: [T, G, d]; the values are the keys.  Token i sees j with 0 <= i - j < window
    (every j <= i without a window); score q.k * scale - slope_h * (i - j), slope_h = 2^(-8 (h + 1) / H);
    ordinary softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).to(F64)
    hidden = (j > i) | ((i - j >= window) if window else torch.zeros(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, k.shape[2], dtype=F64)
    for h in range(H):
        g = h // rep
        slope = 2.0 ** (-8.0 * (h + 1) / H)
        s = (q[:, h] @ k[:, g].T) * scale - slope * dist
        s = s.masked_fill(hidden, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ k[:, g]
    return out


# -- the three mixers --------------------------------------------------------------------------
def mixer_attention(h, w, pre, m, eps, shared=None):
    """Returns (output, (k, v)): the keys and values as a later layer may read them."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")

    def project(name, heads, size, normed, turned):
        u = h @ w[f"{pre}.{name}"].T
        if f"{pre}.{name}.conv" in w:
            u = causal_conv(u, w[f"{pre}.{name}.conv"])
        u = u.reshape(T, heads, size)
        if normed:
            u = norm_plain(u, w[f"{pre}.{name}.norm"], eps)
        if turned and rot:
            u = rotate_pairs(u, rot["dims"], rot["base"])
        return u

    q = project("q", H, d, True, True)
    if shared is None:
        k = project("k", G, d, True, True)
        v = project("v", G, dv, False, False)
    else:
        k, v = shared
    o = capped_sink_attention(q, k, v, m["scale"], m.get("softcap"))
    return o.reshape(T, H * dv) @ w[f"{pre}.o"].T, (k, v)


def mixer_attention_2(h, w, pre, m):
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[f"{pre}.q"].T).reshape(T, H, d)
    k = (h @ w[f"{pre}.k"].T).reshape(T, G, d)
    window = (m.get("mask") or {}).get("size")
    o = distance_window_attention(q, k, m["scale"], window)
    return o.reshape(T, H * d) @ w[f"{pre}.o"].T


def decayed_recurrence(q, k, v, decay):
    """q, k, decay: [T, H, d]; v: [T, H, dv].  S_t = diag(decay_t) S_(t-1) + k_t v_t^T (S is d x dv,
    zero before the first token); o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hd,hde->he", q[t], S)
    return out


def mixer_gla(h, w, pre, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{pre}.q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[f"{pre}.k"].T).reshape(T, H, d)
    v = (h @ w[f"{pre}.v"].T).reshape(T, H, dv)
    z = (h @ w[f"{pre}.a1"].T) @ w[f"{pre}.a2"].T + w[f"{pre}.a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / m["tau"]).reshape(T, H, d)
    o = norm_plain(decayed_recurrence(q, k, v, decay), w[f"{pre}.norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[f"{pre}.g"].T)) @ w[f"{pre}.o"].T


# -- feed-forward ------------------------------------------------------------------------------
def dense_ff(h, w, pre):
    return (silu(h @ w[f"{pre}.gate"].T) * (h @ w[f"{pre}.up"].T)) @ w[f"{pre}.down"].T


# -- the model ---------------------------------------------------------------------------------
def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence.  ``streams``: a list that receives x after every layer."""
    w = {n: t.to(F64) for n, t in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = norm_offset(x, w[f"{p}.norm1"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, kept[i] = mixer_attention(h, w, f"{p}.mix", m, eps, shared=None if src is None else kept[src])
        elif layer["type"] == "attention_2":
            y = mixer_attention_2(h, w, f"{p}.mix", m)
        elif layer["type"] == "gla":
            y = mixer_gla(h, w, f"{p}.mix", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_offset(y, w[f"{p}.norm1b"], eps)
        if layer.get("mlp"):
            y = dense_ff(norm_offset(x, w[f"{p}.norm2"], eps), w, f"{p}.mlp")
            x = x + norm_offset(y, w[f"{p}.norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return (norm_offset(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
