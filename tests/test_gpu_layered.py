"""GPU tests of the layered (Dolurax) family against the NumPy oracle tests/dolurax_ref.py: each kernel alone,
then whole models under every schedule the step function admits -- whole prompts, token-by-token decoding,
portions down to two tokens, batches of unequal requests, pages and slots that are freed and used again --
and greedy generation through the scheduler.  Small configurations with random weights, made so that a key
one position off a chunk edge, a far key or a page border decides the answer where random weights would hide
it.  float32 mode is held to 2e-4, bfloat16 mode to the rounding of bfloat16 products."""
import json
import os

import numpy as np
import pytest

import pygpukit_b200 as gk
from pygpukit_b200 import llm
from pygpukit_b200._lib import api
from pygpukit_b200.llm.config import layered_config_from_json
from pygpukit_b200.llm.paged_cache import PagedKVCache
from tests import dolurax_ref as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def dev_w(a, wdt):
    a = np.ascontiguousarray(a, np.float32)
    return keep(gk.from_numpy((a.view(np.uint32) >> 16).astype(np.uint16).reshape(a.shape)) if wdt == 2 else gk.from_numpy(a))


_KEEP = []


def keep(g):
    """A device array made inside a call expression dies (and is freed) before the asynchronous kernel runs unless
    something holds it: park it until the test ends."""
    _KEEP.append(g)
    return g


@pytest.fixture(autouse=True)
def _release_parked_arrays():
    yield
    gk.synchronize()
    _KEEP.clear()


def i32(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.int32)))


def f32(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.float32)))


# ================================================================ kernels alone
@pytest.mark.parametrize("M,N,K", [(70, 50, 36), (9, 130, 200), (200, 64, 96), (3, 64, 40), (1, 10, 7), (8, 33, 64), (65, 7, 13)])
@pytest.mark.parametrize("wdt", [0, 2])
def test_gemm_rows(M, N, K, wdt):
    rng = np.random.default_rng(M * 1000 + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Wt = bf16_round(rng.standard_normal((N, K)).astype(np.float32))
    ref = (bf16_round(A) if wdt == 2 else A).astype(np.float64) @ Wt.astype(np.float64).T
    a, w, c = gk.from_numpy(A), dev_w(Wt, wdt), gk.zeros((M, N), gk.float32)
    lin = llm.LinearRows(w)
    lin.forward(a.device_ptr, K, M, c.device_ptr, N)
    assert np.abs(c.to_numpy() - ref).max() < 1e-4 * np.sqrt(K)
    # the tiled kernel on the same rows (the few-row kernel serves M <= 8 above)
    api.gemm_rows_f32(a.device_ptr, K, None, w.device_ptr, wdt, 0, c.device_ptr, N, M, N, K, None, 1, M, 0, 1.0, 0.0, None)
    assert np.abs(c.to_numpy() - ref).max() < 1e-4 * np.sqrt(K)


@pytest.mark.parametrize("M", [5, 40])
@pytest.mark.parametrize("wdt", [0, 2])
def test_gemm_epilogues_and_row_gather(M, wdt):
    rng = np.random.default_rng(M)
    K, F = 24, 10
    A = bf16_round(rng.standard_normal((M + 3, K)).astype(np.float32))
    g, u = (bf16_round(rng.standard_normal((F, K)).astype(np.float32)) for _ in range(2))
    rows = rng.permutation(M + 3)[:M]
    x = A[rows].astype(np.float64)
    ref = R.silu(x @ g.T.astype(np.float64)) * (x @ u.T.astype(np.float64))
    lin = llm.LinearRows(dev_w(llm.interleave_gate_up(g, u), wdt), epilogue=1)
    a, c, r = gk.from_numpy(A), gk.zeros((M, F), gk.float32), i32(rows)
    lin.forward(a.device_ptr, K, M, c.device_ptr, F, r.device_ptr)
    assert np.abs(c.to_numpy() - ref).max() < 1e-4
    head = llm.LinearRows(dev_w(g, wdt), epilogue=2, scale=1.7, cap=2.5)
    c2 = gk.zeros((M, F), gk.float32)
    head.forward(a.device_ptr, K, M, c2.device_ptr, F, r.device_ptr)
    assert np.abs(c2.to_numpy() - 2.5 * np.tanh(x @ g.T.astype(np.float64) * 1.7 / 2.5)).max() < 1e-4
    head = llm.LinearRows(dev_w(g, wdt), epilogue=2, scale=0.5, cap=0.0)       # no cap
    head.forward(a.device_ptr, K, M, c2.device_ptr, F, r.device_ptr)
    assert np.abs(c2.to_numpy() - x @ g.T.astype(np.float64) * 0.5).max() < 1e-4


@pytest.mark.parametrize("wdt", [0, 2])
def test_gemm_grouped_and_per_row(wdt):
    rng = np.random.default_rng(3)
    E, N, K, T = 5, 12, 20, 90
    Wt = bf16_round(rng.standard_normal((E, N, K)).astype(np.float32))
    A = bf16_round(rng.standard_normal((T, K)).astype(np.float32))
    counts = np.array([30, 0, 70, 1, 9])                       # an empty expert, one with a single row
    off = np.concatenate([[0], np.cumsum(counts)])
    src = rng.integers(0, T, off[-1])
    grp = np.repeat(np.arange(E), counts)
    ref = np.einsum("rk,rnk->rn", A[src].astype(np.float64), Wt[grp].astype(np.float64))
    lin = llm.LinearRows(dev_w(Wt, wdt))
    a, c = gk.from_numpy(A), gk.zeros((off[-1], N), gk.float32)
    lin.forward_grouped(a.device_ptr, K, c.device_ptr, N, i32(src).device_ptr, i32(off).device_ptr, T)
    assert np.abs(c.to_numpy() - ref).max() < 1e-4
    n = 11
    c2 = gk.zeros((n, N), gk.float32)
    lin.forward_per_row(a.device_ptr, K, n, c2.device_ptr, N, i32(src[:n]).device_ptr, i32(grp[::10][:n]).device_ptr)
    ref2 = np.einsum("rk,rnk->rn", A[src[:n]].astype(np.float64), Wt[grp[::10][:n]].astype(np.float64))
    assert np.abs(c2.to_numpy() - ref2).max() < 1e-4


@pytest.mark.parametrize("E,top,gc,keep", [(16, 4, 2, 1), (16, 3, 4, 2), (8, 2, 1, 1), (12, 1, 3, 3), (6, 6, 2, 2), (40, 5, 5, 2), (64, 40, 1, 1)])
@pytest.mark.parametrize("wdt", [0, 2])
def test_router_and_row_lists(E, top, gc, keep, wdt):
    rng = np.random.default_rng(E + top)
    T, W = 37, 24
    x = bf16_round(rng.standard_normal((T, W)).astype(np.float32))
    Wr = bf16_round(rng.standard_normal((E, W)).astype(np.float32) * 0.8)
    ridx, rw = R.route(x.astype(np.float64) @ Wr.astype(np.float64).T, top, gc, keep)
    idx, wt, rank = gk.zeros((T * top,), gk.int32), gk.zeros((T * top,), gk.float32), gk.zeros((T * top,), gk.int32)
    counts = gk.zeros((E,), gk.int32)
    z = gk.zeros((T, E), gk.float32)
    llm.LinearRows(dev_w(Wr, wdt)).forward(f32(x).device_ptr, W, T, z.device_ptr, E)
    api.moe_route_grouped(z.device_ptr, E, T, E, top, gc, keep, idx.device_ptr, wt.device_ptr, rank.device_ptr,
                          counts.device_ptr, None)
    got_idx = idx.to_numpy().reshape(T, top)
    assert np.array_equal(got_idx, ridx)
    assert np.abs(wt.to_numpy().reshape(T, top) - rw).max() < 1e-5
    assert np.array_equal(counts.to_numpy(), np.bincount(ridx.reshape(-1), minlength=E))
    off, perm, inv = gk.zeros((E + 1,), gk.int32), gk.zeros((T * top,), gk.int32), gk.zeros((T * top,), gk.int32)
    api.moe_row_lists(counts.device_ptr, off.device_ptr, idx.device_ptr, rank.device_ptr, perm.device_ptr, inv.device_ptr,
                      E, T, top, None)
    o, p, v = off.to_numpy(), perm.to_numpy(), inv.to_numpy()
    assert np.array_equal(o, np.concatenate([[0], np.cumsum(np.bincount(ridx.reshape(-1), minlength=E))]))
    assert not counts.to_numpy().any()                                  # cleared for the next layer
    assert sorted(v) == list(range(T * top))                            # a permutation of the rows
    flat = ridx.reshape(-1)
    for i in range(T * top):
        assert o[flat[i]] <= v[i] < o[flat[i] + 1] and p[v[i]] == i // top


def test_combine_layernorm_with_and_without_parts():
    rng = np.random.default_rng(5)
    T, W, top = 6, 50, 3
    x0 = rng.standard_normal((T, W)).astype(np.float32)
    base = rng.standard_normal((T + 2, W)).astype(np.float32)
    parts = rng.standard_normal((T * top, W)).astype(np.float32)
    inv = rng.permutation(T * top)
    wts = rng.uniform(0, 1, (T, top)).astype(np.float32)
    g, b = rng.standard_normal(W).astype(np.float32), rng.standard_normal(W).astype(np.float32)
    src = rng.permutation(T + 2)[:T]
    y = base[src].astype(np.float64) + np.einsum("tk,tkw->tw", wts.astype(np.float64), parts[inv].reshape(T, top, W).astype(np.float64))
    ref = x0 + R.layer_norm(y, g, b, 1e-5)
    x = gk.from_numpy(x0)
    api.combine_layernorm_f32(f32(base).device_ptr, i32(src).device_ptr, f32(parts).device_ptr,
                              i32(inv).device_ptr, f32(wts).device_ptr, top, f32(g).device_ptr,
                              f32(b).device_ptr, 1e-5, x.device_ptr, T, W, 1, None)
    assert np.abs(x.to_numpy() - ref).max() < 1e-5
    out = gk.zeros((T, W), gk.float32)                                   # no parts, no add: plain LayerNorm of gathered rows
    api.combine_layernorm_f32(f32(base).device_ptr, i32(src).device_ptr, None, None, None, 0,
                              f32(g).device_ptr, f32(b).device_ptr, 1e-5, out.device_ptr, T, W, 0, None)
    assert np.abs(out.to_numpy() - R.layer_norm(base[src].astype(np.float64), g, b, 1e-5)).max() < 1e-5


# ---------------------------------------------------------------- attention kernels on a hand-made cache
class AttnHarness:
    """mixer_prep + attention on raw q / k / v rows (norm weights one, eps zero would change q: the oracle side applies
    the same RMS norm)."""

    def __init__(self, H, G, D, Dv, chunk, scale=0.3, softcap=0.0, page=4, dtype="float32", gate=False, splits=1):
        self.splits = splits
        self.decode_kernel = True          # one-token calls go through the decoding kernel
        self.H, self.G, self.D, self.Dv, self.chunk, self.scale, self.softcap, self.gate = H, G, D, Dv, chunk, scale, softcap, gate
        self.cache = PagedKVCache([(G, D, Dv)], dtype, page, 64, 2)
        self.qt = api.seq_queries_per_tile(H, G)
        self.slopes = gk.from_numpy(R.head_slopes(H).astype(np.float32))
        self.ones = gk.from_numpy(np.ones(D, np.float32))
        self.tickets = gk.zeros((4096,), gk.int32)
        self.cols = H * D + G * D + G * Dv + (H * Dv if gate else 0)

    def run(self, seq, q, k, v, gate=None):
        """Feed n tokens of sequence `seq` (q [n, H, D], k [n, G, D], v [n, G, Dv]); returns out [n, H, Dv]."""
        n = q.shape[0]
        slot, pos0 = self.cache.extend(seq, n)
        self.cache.sync_table()
        row = [q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)] + ([gate.reshape(n, -1)] if self.gate else [])
        proj = gk.from_numpy(np.concatenate(row, axis=1).astype(np.float32))
        c = self.cache
        api.seq_mixer_prep(proj.device_ptr, self.cols, n, self.H, self.G, self.D, self.Dv, self.ones.device_ptr,
                           self.ones.device_ptr, 1e-6, 0, 0.0, None, c.k[0].device_ptr, c.v[0].device_ptr, c.dtype_code,
                           c.table_dev.device_ptr, c.pool.max_pages, c.page_size, i32([slot] * n).device_ptr,
                           i32(np.arange(pos0, pos0 + n)).device_ptr, None)
        tiles = [(i, min(self.qt, n - i), slot, pos0 + i) for i in range(0, n, self.qt)]
        out = gk.zeros((n, self.H * self.Dv), gk.float32)
        api.seq_attention(proj.device_ptr, self.cols, 0, self.H * self.D + self.G * self.D + self.G * self.Dv, out.device_ptr,
                          self.H * self.Dv, c.k[0].device_ptr, c.v[0].device_ptr, c.dtype_code, c.table_dev.device_ptr,
                          c.pool.max_pages, c.page_size, i32(tiles).device_ptr, len(tiles), self.slopes.device_ptr, self.H,
                          self.G, self.D, self.Dv, self.chunk, self.scale, self.softcap, 1 if self.gate else 0, self.splits,
                          keep(gk.zeros((n * self.H * self.splits * (self.Dv + 2),), gk.float32)).device_ptr,
                          self.tickets.device_ptr, 1 if (n == 1 and self.decode_kernel) else 0, None)
        assert not self.tickets.to_numpy().any()                         # the tickets clear themselves
        return out.to_numpy().reshape(n, self.H, self.Dv)

    def oracle(self, q, k, v, gate=None):
        one = np.ones(self.D)
        o = R.attention_core(R.rms_norm(q.astype(np.float64), one, 1e-6), R.rms_norm(k.astype(np.float64), one, 1e-6),
                             v.astype(np.float64), self.scale, self.softcap, self.chunk)
        return o * R.sigmoid(gate.astype(np.float64)) if self.gate else o


@pytest.mark.parametrize("H,G,D,Dv,chunk,page,softcap", [(4, 1, 16, 8, 6, 4, 5.0), (4, 2, 8, 40, 5, 3, 0.0), (3, 3, 12, 8, 0, 4, 7.0),
                                                         (8, 2, 32, 32, 16, 8, 3.0), (2, 1, 20, 70, 7, 5, 0.0), (40, 1, 8, 8, 4, 4, 2.0)])
def test_attention_whole_portions_and_single_tokens_agree_with_the_oracle(H, G, D, Dv, chunk, page, softcap):
    rng = np.random.default_rng(H * 7 + D)
    T = 45
    q, k = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D))
    v, gate = rng.standard_normal((T, G, Dv)), rng.standard_normal((T, H, Dv))
    h = AttnHarness(H, G, D, Dv, chunk, softcap=softcap, page=page, gate=True)
    ref = h.oracle(q, k, v, gate)
    whole = h.run("w", q, k, v, gate)
    assert np.abs(whole - ref).max() < 1e-5
    cuts = [0, 2, 5, 6, 19, 20, 31, 45]                                  # portions of 2, 3, 1, 13, 1, 11, 14 tokens
    parts = np.concatenate([h.run("p", q[a:b], k[a:b], v[a:b], gate[a:b]) for a, b in zip(cuts, cuts[1:])])
    assert np.abs(parts - ref).max() < 1e-5
    h.cache.release("w")                                                 # its pages serve the next sequence
    single = np.concatenate([h.run("s", q[i:i + 1], k[i:i + 1], v[i:i + 1], gate[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < 1e-5
    h.cache.release("p")
    h.decode_kernel = False                                              # the same through the tile kernel
    single = np.concatenate([h.run("t", q[i:i + 1], k[i:i + 1], v[i:i + 1], gate[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < 1e-5


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("chunk,page", [(6, 4), (8, 8), (5, 16)])
def test_attention_standout_key_just_inside_and_just_outside_the_chunk(chunk, page, decoded):
    """One key carries a score far above the rest and a value nobody else has.  A query sees it exactly when it lies in
    the query's chunk: at the chunk's first position yes, one position earlier no."""
    H, G, D, Dv, T = 2, 1, 8, 4, 4 * chunk + 3
    rng = np.random.default_rng(chunk)
    for star in (2 * chunk, 2 * chunk - 1, 3 * chunk - 1):               # first of a chunk, last of the one before, last of a chunk
        q, k = 0.01 * rng.standard_normal((T, H, D)), 0.01 * rng.standard_normal((T, G, D))
        v = np.zeros((T, G, Dv))
        q[:, :, 0] = 3.0
        k[:, :, 0] = 0.0                                                  # only the standout key points along q
        k[star, 0, 0] = 3.0
        k[star, 0, 1:] = 0.0
        v[star, 0, 0] = 1.0
        h = AttnHarness(H, G, D, Dv, chunk, scale=20.0, page=page)
        ref = h.oracle(q, k, v)
        n0 = T if not decoded else star + 1
        got = h.run("a", q[:n0], k[:n0], v[:n0])
        if decoded:
            got = np.concatenate([got] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(n0, T)])
        assert np.abs(got - ref).max() < 1e-5
        lo, hi = (star // chunk) * chunk, (star // chunk + 1) * chunk
        for i in range(T):
            sees = star <= i < hi and i >= lo
            assert (got[i, :, 0] > 0.5).all() == sees and (sees or (got[i, :, 0] == 0).all()), (star, i)


def test_attention_far_key_among_hundreds_and_across_page_borders():
    H, G, D, Dv, T = 2, 2, 16, 8, 300
    rng = np.random.default_rng(9)
    q, k = 0.02 * rng.standard_normal((T, H, D)), 0.02 * rng.standard_normal((T, G, D))
    v = 0.01 * rng.standard_normal((T, G, Dv))
    q[:, :, 3] = 4.0
    k[:, :, 3] = 0.0
    for star in (3, 64, 127):                                            # early, first of a page, last of a page
        k[star, :, 3] = 4.0
        v[star, :, star % Dv] = 5.0
    h = AttnHarness(H, G, D, Dv, chunk=0, scale=30.0, softcap=25.0, page=64)
    h.slopes = gk.from_numpy(np.zeros(H, np.float32))                    # no distance penalty: the far keys keep their weight
    got = np.concatenate([h.run("a", q[:250], k[:250], v[:250])] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(250, T)])
    one = np.ones(D)
    qn, kn = R.rms_norm(q, one, 1e-6), R.rms_norm(k, one, 1e-6)
    ref = np.zeros((T, H, Dv))
    for hh in range(H):
        s = 25.0 * np.tanh((qn[:, hh] @ kn[:, hh].T) * 30.0 / 25.0)
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        ref[:, hh] = (p / p.sum(-1, keepdims=True)) @ v[:, hh]
    assert np.abs(got - ref).max() < 1e-5
    assert got[299, 0, 3] > 1.0 and got[299, 0, 0] > 1.0 and got[299, 0, 7] > 1.0   # all three far keys count at the end
    assert got[100, 0, 7] < 0.1                                          # key 127 is in the future of query 100


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_attention_key_slices_fold_to_the_same_answer(splits):
    H, G, D, Dv, T = 4, 2, 16, 40, 200
    rng = np.random.default_rng(splits)
    q, k = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D))
    v, gate = rng.standard_normal((T, G, Dv)), rng.standard_normal((T, H, Dv))
    h = AttnHarness(H, G, D, Dv, chunk=90, softcap=4.0, page=16, gate=True, splits=splits)
    ref = h.oracle(q, k, v, gate)
    got = np.concatenate([h.run("a", q[:150], k[:150], v[:150], gate[:150])] +
                         [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1], gate[i:i + 1]) for i in range(150, T)])
    assert np.abs(got - ref).max() < 1e-5


def test_value_mixing_records_and_mixes():
    H, G, D, Dv, n = 2, 2, 8, 4, 5
    rng = np.random.default_rng(2)
    cache = PagedKVCache([(G, D, Dv)], "float32", 4, 32, 1)
    slot, _ = cache.extend("a", n)
    cache.sync_table()
    cols = H * D + G * D + G * Dv
    rows1, rows2 = (rng.standard_normal((n, cols)).astype(np.float32) for _ in range(2))
    vf = gk.zeros((n, G * Dv), gk.float32)
    one = gk.from_numpy(np.ones(D, np.float32))
    for rows, mode in ((rows1, 1), (rows2, 2)):
        api.seq_mixer_prep(f32(rows).device_ptr, cols, n, H, G, D, Dv, one.device_ptr, one.device_ptr, 1e-5, mode,
                           0.25, vf.device_ptr, cache.k[0].device_ptr, cache.v[0].device_ptr, 0, cache.table_dev.device_ptr,
                           cache.pool.max_pages, 4, i32([slot] * n).device_ptr, i32(np.arange(n)).device_ptr, None)
    v1, v2 = rows1[:, -G * Dv:], rows2[:, -G * Dv:]
    assert np.array_equal(vf.to_numpy(), v1)
    vc = cache.v[0].to_numpy()                                           # [pages, G, 4, Dv]
    pages = cache.pool.page_list("a")
    got = np.stack([vc[pages[i // 4], :, i % 4, :].reshape(-1) for i in range(n)])
    assert np.abs(got - R.value_mix(v2.astype(np.float64), v1.astype(np.float64), 0.25)).max() < 1e-6


# ================================================================ whole models
def variants():
    """Configurations that leave the beaten track: one head group, as many KV heads as heads, value size = key size,
    top = 1, one group, every group kept, no shared expert, layers without feed-forward or value mixing, a late first
    mixing layer, no chunks, no caps, widths that are no multiple of 8."""
    base = R.make_config()
    yield "base", base
    yield "mha_vdim_eq_dim", R.make_config(heads=4, kv_heads=4, dim=8, vdim=8, chunk=5)
    yield "one_kv_head", R.make_config(heads=8, kv_heads=1, dim=16, vdim=24, chunk=7, groups=(4, 2), experts=12, top=3)
    yield "top1_one_group_no_shared", R.make_config(top=1, groups=(1, 1), shared_ff=0, softcap=0.0, logit_softcap=0.0)
    yield "all_groups_kept_odd_width", R.make_config(width=52, vocab=61, ff=10, shared_ff=14, groups=(2, 2), chunk=0)
    c = R.make_config(layers=4, chunk=6)
    c["layers"][0]["mixer"]["v_mix"] = False          # the first mixing layer is layer 1
    c["layers"][2]["mixer"]["v_mix"] = False          # a layer in between that does not mix
    c["layers"][1]["mlp"] = None
    c["layers"][3]["mixer"]["mask"] = {"size": 9}     # another chunk size
    c["layers"][3]["mixer"]["scale"] = 0.4
    c["layers"][3]["mlp"]["router"]["top"] = 3
    yield "mixed_stack", c
    c = R.make_config(v_mix=False, mlp=False, layers=2)
    yield "attention_only", c


VARIANTS = dict(variants())


def make(name, dtype="float32", page=4, seed=1, tokens_hint=64):
    cfg = VARIANTS[name]
    P = R.random_params(cfg, seed=seed)
    m = llm.build_layered_model(layered_config_from_json(cfg), P, dtype)
    m.init_cache(tokens_hint, page_size=page, slots=2)
    return cfg, P, m


def tokens(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_matches_the_oracle_float32(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 29)
    ref, layers = R.forward(cfg, P, toks, True)
    got = m.step([("a", toks, list(range(len(toks))))])
    assert np.abs(m.residual_rows(len(toks)) - layers[-1]).max() < F32_TOL
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "mixed_stack", "one_kv_head"])
def test_prefill_then_token_by_token_decoding(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 40, seed=3)
    ref = R.forward(cfg, P, toks)
    got = [m.step([("a", toks[:9], list(range(9)))])]
    got += [m.step([("a", [t], [0])]) for t in toks[9:]]                 # 31 decoded tokens pass several chunk edges
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "mixed_stack"])
def test_first_tokens_and_decoding_from_position_zero(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 12, seed=4)
    ref = R.forward(cfg, P, toks)
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks])      # a one-token prompt, then decoding
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("sizes", [[2] * 15, [3, 2, 7, 1, 11, 6], [16, 14], [1, 29]])
def test_prompt_portions(sizes):
    cfg, P, m = make("mixed_stack")
    toks = tokens(cfg, sum(sizes), seed=5)
    ref = R.forward(cfg, P, toks)
    got, at = [], 0
    for n in sizes:
        got.append(m.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "mixed_stack", "top1_one_group_no_shared"])
def test_batch_of_unequal_requests_equals_each_alone(name):
    cfg, P, m = make(name, tokens_hint=16)                               # small pool: it has to grow
    lens, new = [1, 23, 7, 40], 6
    seqs = [tokens(cfg, n + new, seed=10 + i) for i, n in enumerate(lens)]
    refs = [R.forward(cfg, P, s) for s in seqs]
    got = m.step([(i, s[:n], list(range(n))) for i, (s, n) in enumerate(zip(seqs, lens))])
    assert np.abs(got - np.concatenate([r[:n] for r, n in zip(refs, lens)])).max() < F32_TOL
    for j in range(new):                                                 # request 0 ends after two more tokens
        live = [i for i in range(4) if i != 0 or j < 2]
        got = m.step([(i, [seqs[i][lens[i] + j]], [0]) for i in live], end=[0] if j == 1 else [])
        assert np.abs(got - np.stack([refs[i][lens[i] + j] for i in live])).max() < F32_TOL
    assert m.cache.pool.live_sequences == 3


def test_more_than_eight_decoding_requests_use_the_sorted_expert_path():
    cfg, P, m = make("base", tokens_hint=256)
    seqs = [tokens(cfg, 5 + i, seed=30 + i) for i in range(11)]
    refs = [R.forward(cfg, P, s) for s in seqs]
    m.step([(i, s[:-2], []) for i, s in enumerate(seqs)])
    for back in (2, 1):
        got = m.step([(i, [s[-back]], [0]) for i, s in enumerate(seqs)])
        assert np.abs(got - np.stack([r[-back] for r in refs])).max() < F32_TOL


def test_pages_and_slots_are_used_again():
    cfg, P, m = make("base", page=4)
    a, b, c = tokens(cfg, 19, seed=20), tokens(cfg, 14, seed=21), tokens(cfg, 22, seed=22)
    m.step([("a", a, []), ("b", b[:6], [])])
    pages_a, slot_a = m.cache.pool.page_list("a"), m.cache.pool.slot("a")
    m.step([("b", b[6:], [])], end=["a"])
    got = m.step([("c", c[:13], list(range(13)))])                       # c inherits a's slot and (dirty) pages
    assert m.cache.pool.slot("c") == slot_a and set(m.cache.pool.page_list("c")) <= set(pages_a)
    got = np.concatenate([got] + [m.step([("c", [t], [0]), ("b", [1], [])])[:1] for t in c[13:]])
    assert np.abs(got - R.forward(cfg, P, c)).max() < F32_TOL


def test_long_decoding_and_wanted_places_subset():
    cfg, P, m = make("one_kv_head", page=8)
    toks = tokens(cfg, 150, seed=6)
    ref = R.forward(cfg, P, toks)
    want = [0, 6, 7, 8, 30, 69]
    got = m.step([("a", toks[:70], want)])
    assert np.abs(got - ref[want]).max() < F32_TOL
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[70:]])
    assert np.abs(got - ref[70:]).max() < F32_TOL


def test_decoding_over_a_long_unchunked_context_reads_the_cache_in_slices():
    cfg, P, m = make("all_groups_kept_odd_width", page=16, tokens_hint=512)      # chunk 0: every key stays visible
    toks = tokens(cfg, 300, seed=8)
    ref = R.forward(cfg, P, toks)
    m.step([("a", toks[:288], [])])
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[288:]])
    assert m._ws is not None                                             # the sliced path ran
    assert np.abs(got - ref[288:]).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "mixed_stack", "all_groups_kept_odd_width"])
def test_bfloat16_mode_stays_within_bfloat16_rounding(name):
    cfg, P, m = make(name, dtype="bfloat16")
    toks = tokens(cfg, 33, seed=7)
    ref = R.forward(cfg, P, toks)
    whole = m.step([("a", toks, list(range(33)))])
    scale = np.abs(ref).max()
    assert np.abs(whole - ref).max() < 0.03 * scale
    got = np.concatenate([m.step([("b", toks[:20], list(range(20)))])] + [m.step([("b", [t], [0])]) for t in toks[20:]])
    assert np.abs(got - whole).max() < 0.03 * scale                      # the same sequence cut differently: rounding only


def test_greedy_generation_through_the_scheduler():
    cfg, P, m = make("base", tokens_hint=256)
    prompts = [tokens(cfg, n, seed=40 + n) for n in (3, 17, 9)]
    outs = m.generate(prompts, max_new_tokens=12, temperature=0.0, prefill_chunk=5)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        seq = list(p)
        for t in o[len(p):]:
            z = R.forward(cfg, P, seq)[-1]
            top2 = np.sort(z)[-2:]
            if top2[1] - top2[0] < 1e-3:                                 # a near tie: either token is right, stop comparing
                break
            assert t == int(np.argmax(z))
            seq.append(t)
    assert m.cache.pool.live_sequences == 0 and m.generate(prompts[0], 2) == outs[0][:len(prompts[0]) + 2]


def test_sampling_and_eos_through_the_scheduler():
    cfg, P, m = make("base")
    p = tokens(cfg, 6, seed=50)
    first = m.generate(p, 1)[-1]
    assert m.generate(p, 8, eos_token_id=first) == p + [first]           # stops at the end token
    np.random.seed(0)
    out = m.generate(p, 5, temperature=0.8, top_k=10, top_p=0.9)
    assert len(out) == 11 and all(0 <= t < cfg["vocab"] for t in out)


def test_loader_picks_the_family_from_config_json(tmp_path):
    cfg = VARIANTS["mixed_stack"]
    P = R.random_params(cfg, seed=8)
    tensors = {k: ((np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(v.shape), "BF16")
               for k, v in P.items()}
    llm.save_safetensors(os.path.join(tmp_path, "model.safetensors"), tensors)
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(cfg, f)
    m = llm.load_model_from_safetensors(str(tmp_path), dtype="float32")
    assert isinstance(m, llm.LayeredCausalModel)
    toks = tokens(cfg, 10)
    assert np.abs(m.step([("a", toks, list(range(10)))]) - R.forward(cfg, P, toks)).max() < F32_TOL
    with pytest.raises(ValueError, match="shape"):
        bad = dict(P)
        bad["l0.mix.q"] = P["l0.mix.q"][:-1]
        llm.build_layered_model(layered_config_from_json(cfg), bad, "float32")
