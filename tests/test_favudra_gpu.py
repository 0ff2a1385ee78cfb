"""Favudra on the device against the plain implementation (tests/plain_favudra.py).

Each mechanism alone (the norm after a sublayer, the scaled embedding, the convolution with its
state across steps, the norm and rotation of q and k and their way into the pages, scored
attention with cap, sink, distance slopes and windows, the gated recurrence with its state), with
inputs made so that a key far away, a key at a window's edge or the sink decides the result; then
whole models of several shapes in both precisions, the same requests cut in every way (whole,
token by token, portions down to two tokens, mixed batches over a pool whose pages and slots are
used again), long decoding, and greedy generation through the engine and its scheduler.
"""
import math

import numpy as np
import pytest
import torch

import plain_favudra as P
import replay_patterns as R
from favudra_configs import CONFIGS, EDGE_CONFIGS, random_weights, tokens

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}   # relative to the largest reference value
SEQ = 1 << 20                                  # the tile height that lists whole sequences


def ops_of(dtype):
    from bitwise_b200.kernels.ops import get_ops
    return get_ops(dtype)


def act(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def close(got, want, dtype, what="", factor=1.0):
    got, want = got.detach().to(F64).cpu(), want.to(F64)
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= TOL[dtype] * factor, f"{what}: relative error {err:.3g}"


class Batch:
    """What the kernels read of a step: rows of sequences, their positions, slots and tiles."""

    def __init__(self, seqs, slots=None):
        # seqs: list of (first position, rows); one block-table row each
        pos, row_seq, seq_pos0, seq_row0 = [], [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(seqs):
            seq_pos0.append(p0), seq_row0.append(r)
            pos += list(range(p0, p0 + cnt))
            row_seq += [s] * cnt
            r += cnt
        self.i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.n, self.seqs = r, seqs
        self.pos, self.row_seq = self.i32(pos), self.i32(row_seq)
        self.seq_pos0, self.seq_row0 = self.i32(seq_pos0), self.i32(seq_row0 + [r])
        self.seq_slot = self.i32(list(slots) if slots is not None else list(range(len(seqs))))
        self.max_keys = max(pos) + 1

    def query_tiles(self, tile_rows):
        t_seq, t_row0, t_rows = [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(self.seqs):
            for a in range(0, cnt, tile_rows):
                t_seq.append(s), t_row0.append(r + a), t_rows.append(min(tile_rows, cnt - a))
            r += cnt
        return self.i32(t_seq), self.i32(t_row0), self.i32(t_rows), len(t_seq)


def pages_in_no_order(seqs, total, page, g):
    """A block table [seqs, blocks] over a pool of ``total`` pages handed out in no order."""
    blocks = (max(p0 + cnt for p0, cnt in seqs) + page - 1) // page
    perm = torch.randperm(total, generator=g)[:len(seqs) * blocks]
    return perm.to(torch.int32).reshape(len(seqs), blocks).to(DEV)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [50, 256, 1500])
def test_norm_after_a_sublayer_and_scaled_embedding(dtype, width):
    ops = ops_of(dtype)
    g = torch.Generator().manual_seed(width)
    d = (torch.randn(6, width, generator=g) * 4).to(DEV)
    x = torch.randn(6, width, generator=g).to(DEV)
    w = (0.3 * torch.randn(width, generator=g)).to(DEV)
    want = x.cpu().to(F64) + P.norm_offset(d.cpu().to(F64), w.cpu().to(F64), 1e-5)
    got = x.clone()
    ops.rmsnorm_residual(d, w + 1.0, 1e-5, got)      # the part folds the offset into the weight when it loads it
    close(got, want, "float32", "x + norm(d)")
    # ... and the norm before the next sublayer from the same kernel
    w2 = (0.3 * torch.randn(width, generator=g)).to(DEV)
    got2, nxt = x.clone(), torch.empty(6, width, dtype=act(dtype), device=DEV)
    ops.rmsnorm_residual(d, w + 1.0, 1e-5, got2, next_weight=w2 + 1.0, next_eps=1e-5, next_out=nxt)
    assert torch.equal(got2, got)
    close(nxt, P.norm_offset(want, w2.cpu().to(F64), 1e-5), dtype, "norm(x + norm(d))")
    table = torch.randn(11, width, generator=g).to(act(dtype)).to(DEV)
    toks = torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, width, device=DEV)
    ops.embed_rows(table, toks, out, scale=7.5)
    assert torch.equal(out, table[toks.long()].float() * 7.5)


def conv_reference(u, w, heads, kv_heads, dim, vdim, qn, kn, eps, rot):
    """q, k, v of one whole sequence after convolution, norm and rotation (plain functions)."""
    T = u.shape[0]
    y = P.causal_conv(u, w) if w is not None else u
    q = y[:, :heads * dim].reshape(T, heads, dim)
    k = y[:, heads * dim:(heads + kv_heads) * dim].reshape(T, kv_heads, dim)
    v = y[:, (heads + kv_heads) * dim:].reshape(T, kv_heads, vdim)
    if qn is not None:
        q, k = P.norm_plain(q, qn, eps), P.norm_plain(k, kn, eps)
    if rot:
        q, k = P.rotate_pairs(q, rot[0], rot[1]), P.rotate_pairs(k, rot[0], rot[1])
    return q, k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps,rot", [(4, 2, 16, 24, 3, (8, 10000.0)), (2, 2, 36, 12, 5, (36, 500.0)),
                                                            (6, 1, 20, 20, 2, (4, 77.0)), (3, 1, 72, 40, 4, None),
                                                            (5, 5, 8, 8, 0, (8, 1e6)), (1, 1, 256, 256, 1, (64, 1e4))])
@pytest.mark.parametrize("by_four", [False, True])
def test_convolution_norm_rotation_and_state_across_steps(dtype, heads, kv_heads, dim, vdim, taps, rot, by_four):
    """One sequence fed in portions (single rows, pairs, portions shorter and longer than the taps)
    beside another sequence that starts late in a slot someone else left dirty."""
    from bitwise_b200.parts.rope import RotaryEncoding
    ops = ops_of(dtype)
    page, T = 16, 41
    g = torch.Generator().manual_seed(dim + taps)
    cols = heads * dim + kv_heads * (dim + vdim)
    seqs_u = [torch.randn(T, cols, generator=g) * 2, torch.randn(T, cols, generator=g) * 2]
    w = torch.randn(cols, taps, generator=g) * 0.6 if taps else None
    qn, kn = 1 + 0.3 * torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    cos = sin = None
    if rot:
        cos, sin = RotaryEncoding(rot[0], rot[1], positions=64).rotary_tables(DEV)
    want = [conv_reference(u.to(F64), w.to(F64) if taps else None, heads, kv_heads, dim, vdim, qn.to(F64), kn.to(F64), 1e-5, rot)
            for u in seqs_u]
    table = pages_in_no_order([(0, T), (0, T)], 9, page, g)
    kc = torch.zeros(10, kv_heads, page, dim, dtype=act(dtype), device=DEV)
    vc = torch.zeros(10, kv_heads, page, vdim, dtype=act(dtype), device=DEV)
    state = torch.full((3, max(taps - 1, 1), cols), 1e3, device=DEV) if taps > 1 else None   # dirty slots
    got_q = [torch.zeros(T, heads * dim, dtype=act(dtype)) for _ in range(2)]
    # (rows of sequence 0, rows of sequence 1) per step; sequence 1 begins at the third step
    cuts = [(1, 0), (1, 0), (2, 3), (1, 1), (taps + 2, 2), (2, 1), (1, 9), (7, 1), (3, 2)]
    at = [0, 0]
    while at[0] < T or at[1] < T:
        c = cuts.pop(0) if cuts else (5, 6)
        seqs, rows, who = [], [], []
        for s in range(2):
            n = min(c[s], T - at[s])
            if n:
                seqs.append((at[s], n)), rows.append(seqs_u[s][at[s]:at[s] + n]), who.append(s)
        b = Batch(seqs, slots=[2 - s for s in who])
        u = torch.cat(rows).to(DEV)
        q = torch.empty(b.n, heads * dim, dtype=act(dtype), device=DEV)
        # (with the taps transposed as well, shapes in steps of 4 take the kernel that reads four channels at a time)
        ops.qkv_prepare(u, w.to(DEV) if taps else None, state, qn.to(DEV), kn.to(DEV), 1e-5, cos, sin, b,
                        table[who].contiguous(), kc, vc, q, heads, kv_heads, dim, vdim,
                        conv_wt=w.t().contiguous().to(DEV) if taps and by_four else None)
        if taps > 1:
            ops.conv_state_update(u, state, b, taps, b.query_tiles(SEQ))
        r = 0
        for s, (p0, n) in zip(who, seqs):
            got_q[s][p0:p0 + n] = q[r:r + n].cpu()
            at[s] += n
            r += n
    for s in range(2):
        wq, wk, wv = want[s]
        close(got_q[s], wq.reshape(T, -1), dtype, f"queries of sequence {s}")
        idx = torch.arange(T)
        blocks, slots = table[s].cpu().long()[idx // page], idx % page
        close(kc.cpu()[blocks, :, slots, :], wk, dtype, f"keys of sequence {s}")
        close(vc.cpu()[blocks, :, slots, :], wv, dtype, f"values of sequence {s}")


def fill_pages(seq_tensors, table, page, kv_heads, size, dtype):
    cache = torch.zeros(int(table.max()) + 2, kv_heads, page, size, dtype=act(dtype), device=DEV)
    for s, t in enumerate(seq_tensors):
        idx = torch.arange(t.shape[0])
        cache[table[s].long()[idx // page], :, idx % page, :] = t.to(act(dtype)).to(DEV)
    return cache


# (the serving precision runs shapes with sizes in steps of 16 on the tensor cores, the others on the CUDA cores)
ATTENTION_SHAPES = [(4, 2, 16, 24), (8, 2, 128, 128), (3, 3, 40, 8), (40, 1, 8, 40), (2, 1, 96, 200), (6, 2, 64, 32),
                    (80, 1, 16, 16), (2, 2, 32, 256)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", ATTENTION_SHAPES)
@pytest.mark.parametrize("cap", [None, 6.0])
def test_capped_sink_attention(dtype, heads, kv_heads, dim, vdim, cap):
    """Prompt portions and single rows against the plain function.  One query is scaled so that a key
    hundreds of positions back takes nearly all its weight; another sees only very negative
    scores, so that the sink takes nearly all of it."""
    ops = ops_of(dtype)
    page, T = 16, 700
    g = torch.Generator().manual_seed(heads * dim)
    rt = lambda *s: torch.randn(*s, generator=g).to(act(dtype)).to(F64)   # values that the cache holds exactly
    q, k, v = rt(T, heads, dim), rt(T, kv_heads, dim), rt(T, kv_heads, vdim)
    scale = 1.0 / math.sqrt(dim)
    k[5] = (q[690, 0] * 3).to(act(dtype)).to(F64)        # a far key that query 690 of head 0 agrees with
    q[650] = (-q[650].abs() * (40 / math.sqrt(dim))).to(act(dtype)).to(F64)
    k[:651] = k[:651].abs()                              # every score of row 650 is very negative
    k[5] = k[5].abs()
    want = P.capped_sink_attention(q, k, v, scale, cap)
    table = pages_in_no_order([(0, T)], 60, page, g)
    kc, vc = fill_pages([k], table, page, kv_heads, dim, dtype), fill_pages([v], table, page, kv_heads, vdim, dtype)
    for seqs in ([(0, T)], [(600, 100)], [(649, 2)], [(690, 1)], [(650, 1)]):
        p0, n = seqs[0]
        b = Batch(seqs)
        out = torch.empty(n, heads * vdim, dtype=act(dtype), device=DEV)
        ops.scored_attention(q[p0:p0 + n].reshape(n, -1).to(act(dtype)).to(DEV).contiguous(), kc, vc, table, out, heads,
                             kv_heads, dim, vdim, scale, cap or 0.0, True, None, 0, b)
        close(out, want[p0:p0 + n].reshape(n, -1), dtype, f"rows {p0}..{p0 + n - 1}", 2.0)
    assert want[650].abs().max() < 0.05 * v.abs().max() or cap, "the sink did not take the weight"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim", [(4, 2, 96), (3, 1, 10), (8, 4, 32), (2, 2, 24)])
@pytest.mark.parametrize("window", [7, 33, 80, 0])
def test_distance_window_attention(dtype, heads, kv_heads, dim, window):
    """The values are the keys.  The key just outside a query's window is made to agree with it
    strongly (it would take all the weight if it were seen), the key just inside another query's
    window likewise (it must take it)."""
    from bitwise_b200.parts.scored_attention import distance_slopes
    ops = ops_of(dtype)
    page, T = 16, 300
    g = torch.Generator().manual_seed(dim + window)
    rt = lambda *s: torch.randn(*s, generator=g).to(act(dtype)).to(F64)
    q, k = rt(T, heads, dim), rt(T, kv_heads, dim)
    scale = 1.0 / math.sqrt(dim)
    W = window or T
    for i, inside in ((200, True), (250, False), (W + 1, False), (280, True)):
        j = i - W + 1 if inside else i - W
        if j >= 0 and i < T:
            q[i] = (k[j, 0] * 4).to(act(dtype)).to(F64)
    want = P.distance_window_attention(q, k, scale, window or None)
    # pages that the window has passed are given back in a live engine: their table entries are -1
    table = pages_in_no_order([(0, T)], 30, page, g)
    kc = fill_pages([k], table, page, kv_heads, dim, dtype)
    slopes = torch.tensor(distance_slopes(heads), dtype=torch.float32, device=DEV)
    for seqs in ([(0, T)], [(190, 70)], [(199, 2)], [(250, 1)], [(280, 1)], [(W + 1, 1)] if W + 1 < T else [(5, 1)]):  # noqa: E501
        p0, n = seqs[0]
        b = Batch(seqs)
        tb = table.clone()
        if window and p0 - window + 1 >= page:
            tb[0, :(p0 - window + 1) // page] = -1
        out = torch.empty(n, heads * dim, dtype=act(dtype), device=DEV)
        ops.scored_attention(q[p0:p0 + n].reshape(n, -1).to(act(dtype)).to(DEV).contiguous(), kc, None, tb, out, heads,
                             kv_heads, dim, dim, scale, 0.0, False, slopes, window, b)
        close(out, want[p0:p0 + n].reshape(n, -1), dtype, f"rows {p0}..{p0 + n - 1}", 2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_of_unequal_sequences_in_one_step(dtype):
    """Three sequences in one step (a long portion, a pair, a single row deep in its context)
    give what each gives alone."""
    ops = ops_of(dtype)
    heads, kv_heads, dim, vdim, page = 6, 2, 32, 16, 16
    g = torch.Generator().manual_seed(11)
    rt = lambda *s: torch.randn(*s, generator=g).to(act(dtype)).to(F64)
    lens = [90, 200, 333]
    ks, vs, qs = [rt(n, kv_heads, dim) for n in lens], [rt(n, kv_heads, vdim) for n in lens], [rt(n, heads, dim) for n in lens]
    seqs = [(20, 70), (198, 2), (332, 1)]
    table = pages_in_no_order([(0, n) for n in lens], 70, page, g)
    kc, vc = fill_pages(ks, table, page, kv_heads, dim, dtype), fill_pages(vs, table, page, kv_heads, vdim, dtype)
    b = Batch(seqs)
    qrows = torch.cat([qs[s][p0:p0 + n].reshape(n, -1) for s, (p0, n) in enumerate(seqs)])
    out = torch.empty(b.n, heads * vdim, dtype=act(dtype), device=DEV)
    ops.scored_attention(qrows.to(act(dtype)).to(DEV).contiguous(), kc, vc, table, out, heads, kv_heads, dim, vdim, 0.2, 9.0,
                         True, None, 0, b)
    want = torch.cat([P.capped_sink_attention(qs[s], ks[s], vs[s], 0.2, 9.0)[p0:p0 + n].reshape(n, -1)
                      for s, (p0, n) in enumerate(seqs)])
    close(out, want, dtype, "three sequences", 2.0)
    # single rows at unequal depths: one below the span of keys from which rows are spread over blocks
    seqs = [(89, 1), (199, 1), (332, 1)]
    b = Batch(seqs)
    qrows = torch.cat([qs[s][p0:p0 + n].reshape(n, -1) for s, (p0, n) in enumerate(seqs)])
    out = torch.empty(b.n, heads * vdim, dtype=act(dtype), device=DEV)
    ops.scored_attention(qrows.to(act(dtype)).to(DEV).contiguous(), kc, vc, table, out, heads, kv_heads, dim, vdim, 0.2, 9.0,
                         True, None, 0, b)
    want = torch.cat([P.capped_sink_attention(qs[s], ks[s], vs[s], 0.2, 9.0)[p0:p0 + n].reshape(n, -1)
                      for s, (p0, n) in enumerate(seqs)])
    close(out, want, dtype, "three single rows", 2.0)


def test_tensor_core_attention_agrees_with_the_plain_kernel():
    """bfloat16: the same step on both kernels (prompt portion, then single rows spread over spans)."""
    from bitwise_b200.parts.scored_attention import distance_slopes
    ops = ops_of("bfloat16")
    heads, kv_heads, dim, vdim, page, T = 8, 2, 64, 64, 16, 600
    g = torch.Generator().manual_seed(5)
    k = torch.randn(T, kv_heads, dim, generator=g).to(torch.bfloat16)
    v = torch.randn(T, kv_heads, vdim, generator=g).to(torch.bfloat16)
    table = pages_in_no_order([(0, T)], 40, page, g)
    kc, vc = fill_pages([k], table, page, kv_heads, dim, "bfloat16"), fill_pages([v], table, page, kv_heads, vdim, "bfloat16")
    slopes = torch.tensor(distance_slopes(heads), dtype=torch.float32, device=DEV)
    for seqs in ([(100, 500)], [(599, 1)]):
        b = Batch(seqs)
        q = torch.randn(b.n, heads * dim, generator=g).to(torch.bfloat16).to(DEV)
        outs = []
        for plain in (False, True):
            ops.plain_mixers(plain)
            try:
                o1 = torch.empty(b.n, heads * vdim, dtype=torch.bfloat16, device=DEV)
                ops.scored_attention(q, kc, vc, table, o1, heads, kv_heads, dim, vdim, 0.125, 12.0, True, None, 0, b)
                o2 = torch.empty(b.n, heads * dim, dtype=torch.bfloat16, device=DEV)
                ops.scored_attention(q, kc, None, table, o2, heads, kv_heads, dim, dim, 0.125, 0.0, False, slopes, 100, b)
            finally:
                ops.plain_mixers(False)
            outs.append((o1.float(), o2.float()))
        for a, c in zip(*outs):
            assert float((a - c).abs().max()) <= 0.02 * float(c.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,tau", [(2, 8, 16, 4.0), (4, 32, 48, 12.0), (1, 40, 40, 2.0), (2, 72, 24, 16.0),
                                                (3, 12, 8, 9.0), (2, 128, 128, 8.0), (1, 256, 64, 3.0)])
def test_gated_recurrence_with_state_across_steps(dtype, heads, dim, vdim, tau):
    """Two sequences fed in portions of changing size through dirty slots; the state lives between
    the steps.  The plain functions: decay from z, the recurrence, the norm, the gate."""
    ops = ops_of(dtype)
    T = 45
    g = torch.Generator().manual_seed(dim * vdim)
    hd, hv = heads * dim, heads * vdim
    us = [torch.randn(T, 2 * hd + 2 * hv, generator=g) for _ in range(2)]
    zs = [torch.randn(T, hd, generator=g) * 2 for _ in range(2)]
    bias, nw = 1 + torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(vdim, generator=g)
    want = []
    for u, z in zip(us, zs):
        u64, z64 = u.to(F64), z.to(F64)
        decay = torch.sigmoid(z64 + bias.to(F64)).pow(1.0 / tau).reshape(T, heads, dim)
        o = P.decayed_recurrence(u64[:, :hd].reshape(T, heads, dim) * dim ** -0.5, u64[:, hd:2 * hd].reshape(T, heads, dim),
                                 u64[:, 2 * hd:2 * hd + hv].reshape(T, heads, vdim), decay)
        want.append(P.norm_plain(o, nw.to(F64), 1e-5).reshape(T, hv) * P.silu(u64[:, 2 * hd + hv:]))
    state = torch.full((4, heads, dim, vdim), 1e3, device=DEV)   # dirty slots
    got = [torch.zeros(T, hv, dtype=act(dtype)) for _ in range(2)]
    cuts = [(1, 0), (2, 0), (9, 1), (1, 1), (1, 17), (3, 2), (8, 8)]
    at = [0, 0]
    while at[0] < T or at[1] < T:
        c = cuts.pop(0) if cuts else (11, 4)
        seqs, rows, zrows, who = [], [], [], []
        for s in range(2):
            n = min(c[s], T - at[s])
            if n:
                seqs.append((at[s], n)), rows.append(us[s][at[s]:at[s] + n]), zrows.append(zs[s][at[s]:at[s] + n]), who.append(s)
        b = Batch(seqs, slots=[3 - 2 * s for s in who])
        out = torch.empty(b.n, hv, dtype=act(dtype), device=DEV)
        ops.gla_scan(torch.cat(rows).to(DEV), torch.cat(zrows).to(DEV), bias.to(DEV), tau, state, nw.to(DEV), 1e-5, out, heads,
                     dim, vdim, dim ** -0.5, b, b.query_tiles(SEQ))
        r = 0
        for s, (p0, n) in zip(who, seqs):
            got[s][p0:p0 + n] = out[r:r + n].cpu()
            at[s] += n
            r += n
    for s in range(2):
        close(got[s], want[s], dtype, f"sequence {s}", 2.0)


# ---------------------------------------------------------------------------------------------
# whole models

_models, _plain = {}, {}


def model_of(name, dtype):
    from bitwise_b200 import Model
    if (name, dtype) not in _models:
        _models[(name, dtype)] = Model.from_tensors(CONFIGS[name], random_weights(CONFIGS[name], 7), dtype=dtype, device=DEV)
    return _models[(name, dtype)]


def plain_logits(name, toks):
    key = (name, tuple(toks))
    if key not in _plain:
        _plain[key] = P.forward(CONFIGS[name].to_json(), random_weights(CONFIGS[name], 7), toks).numpy()
    return _plain[key]


LENGTHS = {"a": [70, 45, 5, 300, 64, 17, 1, 131], "b": [100, 9, 330, 1, 65, 33], "c": [40, 290, 3, 17]}


def requests_of(name):
    return {f"{name}-{i}": tokens(CONFIGS[name], n, i) for i, n in enumerate(LENGTHS[name])}


def row_errors(got, want):
    """Per position: root mean square of the difference over that of the reference row."""
    return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))


def assess(errors, dtype, what):
    errors = np.concatenate([np.atleast_1d(e) for e in errors])
    if dtype == "float32":
        assert errors.max() <= 4 * TOL[dtype], f"{what}: worst relative error {errors.max():.3g}"
    else:
        assert errors.mean() <= 0.03 and errors.max() <= 0.12, \
            f"{what}: mean relative error {errors.mean():.3g}, worst {errors.max():.3g}"


def compare(name, dtype, got_by_request):
    errors = []
    for rid, toks in requests_of(name).items():
        want = plain_logits(name, toks)
        got = got_by_request[rid]
        assert got.shape == want.shape
        errors.append(row_errors(got, want))
    assess(errors, dtype, f"{name} {dtype} against the plain implementation")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts_and_layers(name, dtype):
    model = model_of(name, dtype)
    reqs = requests_of(name)
    steps = R.whole(reqs)
    compare(name, dtype, R.collect(steps, R.run_in_process(model, steps, 384), CONFIGS[name].vocab))
    # the stream after every layer, for one request
    toks = next(iter(reqs.values()))
    want = []
    P.forward(CONFIGS[name].to_json(), random_weights(CONFIGS[name], 7), toks, want)
    seen = []
    for b in model.decoder.blocks:
        def fwd(ctx, x, cache, orig=b.forward):
            orig(ctx, x, cache)
            seen.append(x.clone())
        b.forward = fwd
    try:
        model.logits(toks)
    finally:
        for b in model.decoder.blocks:
            del b.forward
    for i, (got, w) in enumerate(zip(seen, want)):
        assess([row_errors(got.float().cpu().numpy(), w.numpy())], dtype, f"stream after layer {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_gives_the_same_logits(name, dtype):
    model = model_of(name, dtype)
    reqs = requests_of(name)
    vocab = CONFIGS[name].vocab
    base = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), 384), vocab)
    patterns = {"tail": (R.tail_one_by_one(reqs, tail=40), 384), "portions": (R.portions(reqs), 384),
                "pairs": (R.portions(reqs, sizes=(2,)), 384), "mixed": (R.mixed(reqs, 704, seed=3), 704),
                "mixed-tight": (R.mixed(reqs, 448, seed=4), 448)}
    for pname, (steps, pool) in patterns.items():
        for graphs in ((None, False) if dtype == "bfloat16" and pname in ("tail", "mixed") else (None,)):
            got = R.collect(steps, R.run_in_process(model, steps, pool, use_graphs=graphs), vocab)
            compare(name, dtype, got)
            # between two cuts only rounding differs: far less than between precision and plain
            errs = np.concatenate([row_errors(got[rid], base[rid]) for rid in reqs])
            assert errs.max() <= (1e-5 if dtype == "float32" else 0.02), f"{name} {dtype} {pname}: cuts differ by {errs.max():.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(EDGE_CONFIGS))
def test_layer_combinations_at_the_edges(name, dtype):
    """Models without any pages, without any state, with two windows and a shared one-tap layer."""
    from bitwise_b200 import Model
    cfg = EDGE_CONFIGS[name]
    W = random_weights(cfg, 3)
    model = Model.from_tensors(cfg, W, dtype=dtype, device=DEV)
    reqs = {f"{name}{i}": tokens(cfg, n, i) for i, n in enumerate([37, 70, 5, 1, 18])}
    want = {rid: P.forward(cfg.to_json(), W, t).numpy() for rid, t in reqs.items()}
    for steps, pool in ((R.whole(reqs), 128), (R.portions(reqs, sizes=(3, 2, 11, 1)), 128), (R.mixed(reqs, 192, seed=5), 192)):
        got = R.collect(steps, R.run_in_process(model, steps, pool), cfg.vocab)
        assess([row_errors(got[rid], want[rid]) for rid in reqs], dtype, f"{name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_reused_pages(dtype):
    # one request decoded token by token from position 3 to past 600 (pages, key tiles and windows
    # are crossed one position at a time) while others come and go in the pool and in the slots
    name = "a"
    model = model_of(name, dtype)
    toks = tokens(CONFIGS[name], 620, 99)
    others = {f"o{i}": tokens(CONFIGS[name], n, 50 + i) for i, n in enumerate([30, 64, 100, 7, 65, 120])}
    from bitwise_b200.engine.replay import make_replay_stepper
    from bitwise_b200.engine.step import StepEntry
    stepper = make_replay_stepper(model, 640 + 128 + 64, max_live=3)
    want = plain_logits(name, toks)
    queue = list(others.items())
    live = None
    errors = []
    out = stepper.run([StepEntry("long", toks[:3], [2])])
    for p in range(3, len(toks)):
        entries = [StepEntry("long", toks[p:p + 1], [0])]
        if live is None and queue and p % 7 == 0:
            live = [queue.pop(0), 0]
        if live is not None:
            (rid, ot), at = live
            c = min(len(ot) - at, 1 + p % 9)
            entries.append(StepEntry(rid, ot[at:at + c], [c - 1]))
            live[1] += c
        out = stepper.run(entries).float().cpu().numpy()
        errors.append(row_errors(out[0], want[p]))
        if live is not None:
            w = plain_logits(name, live[0][1])
            errors.append(row_errors(out[1], w[live[1] - 1]))
            if live[1] == len(live[0][1]):
                stepper.finish(live[0][0])
                live = None
    assert not queue
    stepper.finish("long")
    assert stepper.manager.all_free()
    assess(errors, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    name = "a"
    model = model_of(name, dtype)
    cfg = CONFIGS[name]
    prompts = [tokens(cfg, n, 200 + i) for i, n in enumerate([5, 40, 17, 1, 33])]
    new = 12
    # a pool that does not hold all requests at once and a token budget below the longest prompt
    eng = Engine(model, EngineConfig(num_blocks=12, block_size=16, max_batched_tokens=24, max_num_seqs=3))
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True))
    W = random_weights(cfg, 7)
    for prompt, out in zip(prompts, got):
        assert len(out) == new
        seq = list(prompt)
        for t in out:
            row = P.forward(cfg.to_json(), W, seq)[-1].numpy()
            if dtype == "float32":
                assert t == int(row.argmax()) or row.max() - row[t] < 1e-4 * np.abs(row).max()
            else:
                assert row.max() - row[t] <= 0.05 * np.abs(row).max(), "the chosen token is no near-maximum"
            seq.append(t)
    assert eng.manager.all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_simulated_traces_reproduce_requests_run_alone(dtype):
    # the engine's simulator: random requests, budgets and pools, preemption with recomputation; a
    # request's tokens and the fingerprint of its logits must be those it yields alone on an idle
    # engine: every kernel of the design walks keys and tokens in an order of its own sizes
    from bitwise_b200.engine.simulate import run_traces
    out = run_traces(model_of("a", dtype), traces=8, seed=5)
    assert out.traces == 8 and out.requests_checked > 10
    assert out.violations == 0, (out.token_mismatch, out.fingerprint_mismatch, out.hangs, out.leaks)


def test_command_line_random_folder_replay_and_generation(tmp_path):
    """``bitwise_b200 random`` writes a Favudra folder from a config.json; ``bin/trace_run`` replays a mixed
    schedule on it and ``bitwise_b200 generate`` decodes greedily: both as a user calls them, both
    against the plain implementation on the folder's own tensors (the decay's inner size is read from
    the stored shapes)."""
    import json
    import os
    import subprocess
    import sys
    from bitwise_b200.weights.safetensors_io import SafetensorsFile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CONFIGS["b"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_json()))
    folder = tmp_path / "model"
    run = lambda *a, **k: subprocess.run([sys.executable, *a], capture_output=True, text=True, timeout=900, **k)
    p = run(os.path.join(root, "bin", "bitwise_b200"), "random", "--config", str(tmp_path / "config.json"), "--seed", "11",
            "--out", str(folder), "--dtype", "bfloat16", "--norm-jitter", "0.2")
    assert p.returncode == 0, p.stderr[-2000:]
    f = SafetensorsFile(str(folder / "model.safetensors"))
    W = {n: f.tensor(n).clone() for n in f.names()}
    raw = json.load(open(folder / "config.json"))
    reqs = {f"q{i}": tokens(cfg, n, 300 + i) for i, n in enumerate([33, 70, 2, 19])}
    steps = R.mixed(reqs, 192, seed=8)
    out = tmp_path / "out"
    p = run(os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
            "--max-tokens", "192", input="".join(json.dumps(s) + "\n" for s in steps))
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg.vocab) for s in steps}
    got = R.collect(steps, outs, cfg.vocab)
    for rid, toks in reqs.items():
        want = P.forward(raw, W, toks).numpy()
        assert np.abs(got[rid] - want).max() <= 1e-4 * np.abs(want).max(), rid
    prompt = reqs["q3"]
    p = run(os.path.join(root, "bin", "bitwise_b200"), "generate", "--model", str(folder), "--dtype", "float32",
            "--max-new-tokens", "6", "--ignore-eos", "--temperature", "0", "--prompt-ids", ",".join(map(str, prompt)))
    assert p.returncode == 0, p.stderr[-2000:]
    seq = list(prompt)
    for t in json.loads(p.stdout.strip().split("\n")[0])["tokens"]:
        row = P.forward(raw, W, seq)[-1].numpy()
        assert t == int(row.argmax()) or row.max() - row[t] < 1e-4 * np.abs(row).max()
        seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_cuts_agree_bit_for_bit(name, dtype):
    """Every kernel of the design walks keys, tokens and products in an order given by its own sizes
    (key tiles and spans at fixed absolute positions, the recurrence token by token), so the logits of
    a position are the same bits whole, token by token, in portions and in a crowd: also beyond the
    256 keys from which a context is walked in spans."""
    model = model_of(name, dtype)
    reqs = requests_of(name)
    vocab = CONFIGS[name].vocab
    base = R.collect(R.whole(reqs), R.run_in_process(model, R.whole(reqs), 384), vocab)
    for pname, (steps, pool) in {"tail": (R.tail_one_by_one(reqs, tail=40), 384), "portions": (R.portions(reqs), 384),
                                 "mixed": (R.mixed(reqs, 704, seed=3), 704)}.items():
        got = R.collect(steps, R.run_in_process(model, steps, pool), vocab)
        for rid in reqs:
            same = (got[rid].view(np.uint32) == base[rid].view(np.uint32)).all(axis=1)
            assert same.all(), f"{name} {dtype} {pname} {rid}: first position that differs {int(np.argmin(same))}"
