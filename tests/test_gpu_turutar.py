"""GPU tests of the Turutar design in the layered family against the NumPy oracle tests/turutar_ref.py: the new kernels
alone (RMS norm of rows, the GEMM epilogues and per-head batches, whole-projection preparation, windowed attention with
a sink and a per-head gate, latent attention on one cached row), then whole models under every schedule the step
function admits, and greedy generation through the scheduler and the command line.  Configurations are small and
random; where random weights would hide a fault (a key at the window's edge, a far key among hundreds, the sink) the
inputs are made so that it decides the answer.  float32 mode is held to 2e-4."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import pygpukit_b200 as gk
from pygpukit_b200 import llm
from pygpukit_b200._lib import api
from pygpukit_b200.llm.config import layered_config_from_json
from pygpukit_b200.llm.paged_cache import PagedKVCache
from tests import turutar_ref as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_KEEP = []


def keep(g):
    """Park a device array until the test ends (kernels run asynchronously)."""
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


def f64(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.float64)))


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def dev_w(a, wdt):
    a = np.ascontiguousarray(a, np.float32)
    return keep(gk.from_numpy((a.view(np.uint32) >> 16).astype(np.uint16).reshape(a.shape)) if wdt == 2 else gk.from_numpy(a))


# ================================================================ kernels alone
@pytest.mark.parametrize("W", [48, 1030])
def test_rms_norm_rows_offset_gather_sum_and_accumulate(W):
    rng = np.random.default_rng(W)
    n = 7
    x, add, w = rng.standard_normal((n, W)), rng.standard_normal((n, W)), 0.3 * rng.standard_normal(W)
    out = gk.zeros((n, W), gk.float32)
    for off in (0.0, 1.0):
        api.rms_norm_rows_f32(f32(x).device_ptr, None, None, None, f32(w).device_ptr, off, 1e-5, out.device_ptr, n, W, 0, None)
        assert np.abs(out.to_numpy() - R.rms_norm(x, w, 1e-5, off)).max() < 1e-5
    src = [5, 0, 5, 2]
    api.rms_norm_rows_f32(f32(x).device_ptr, i32(src).device_ptr, None, None, f32(w).device_ptr, 1.0, 1e-5, out.device_ptr, 4, W, 0, None)
    assert np.abs(out.to_numpy()[:4] - R.rms_norm(x[src], w, 1e-5, 1.0)).max() < 1e-5
    xs, base = f32(x), f32(add)                          # x <- x + add (written back), out += norm(x + add)
    before = out.to_numpy().copy()
    api.rms_norm_rows_f32(xs.device_ptr, None, base.device_ptr, xs.device_ptr, f32(w).device_ptr, 0.0, 1e-5, out.device_ptr, n, W, 1, None)
    assert np.abs(xs.to_numpy() - (x + add)).max() < 1e-6
    assert np.abs(out.to_numpy() - (before + R.rms_norm(x + add, w, 1e-5))).max() < 1e-5
    api.rms_norm_rows_f32(xs.device_ptr, None, None, None, f32(w).device_ptr, 1.0, 1e-5, xs.device_ptr, n, W, 0, None)   # in place
    assert np.abs(xs.to_numpy() - R.rms_norm(x + add, w, 1e-5, 1.0)).max() < 1e-5


@pytest.mark.parametrize("W", [40, 1030])
def test_seam_of_two_norms_and_embedding_with_its_norm(W):
    rng = np.random.default_rng(W + 1)
    n = 6
    y, x, add = (rng.standard_normal((n, W)) for _ in range(3))
    w1, w2 = 0.5 + 0.2 * rng.standard_normal(W), 0.3 * rng.standard_normal(W)
    for extra in (None, add):
        xs, h = f32(x), gk.zeros((n, W), gk.float32)
        api.rms_norm_seam_f32(f32(y).device_ptr, f32(w1).device_ptr, 0.0, xs.device_ptr, f32(extra).device_ptr if extra is not None else None,
                              f32(w2).device_ptr, 1.0, 1e-5, h.device_ptr, n, W, None)
        want = x + R.rms_norm(y, w1, 1e-5) + (extra if extra is not None else 0.0)
        assert np.abs(xs.to_numpy() - want).max() < 1e-5
        assert np.abs(h.to_numpy() - R.rms_norm(want, w2, 1e-5, 1.0)).max() < 1e-5
    table = bf16_round(rng.standard_normal((11, W)))
    toks = [3, 10, 0, 3]
    for wdt in (0, 2):
        xs, keep_ = gk.zeros((4, W), gk.float32), gk.zeros((4, W), gk.float32)
        api.embed_norm_rows_f32(dev_w(table, wdt).device_ptr, wdt, i32(toks).device_ptr, f32(w2).device_ptr, 1.0, 1e-5, xs.device_ptr,
                                keep_.device_ptr, 4, W, 11, None)
        assert np.abs(xs.to_numpy() - R.rms_norm(table[toks], w2, 1e-5, 1.0)).max() < 1e-5
        assert np.array_equal(xs.to_numpy(), keep_.to_numpy())


@pytest.mark.parametrize("wdt", [0, 2])
@pytest.mark.parametrize("M", [3, 70])
def test_gemm_epilogues_clamped_gate_scaled_accumulate_and_gathered_gelu(M, wdt):
    rng = np.random.default_rng(M + wdt)
    K, F = 44, 13
    few = 8 if M <= 8 else 0
    x = rng.standard_normal((M, K)).astype(np.float32)
    xr = bf16_round(x) if wdt == 2 else x
    tol = 2e-5
    # clamped gate/up pairs: limit 0.8 cuts a good part of both
    wg, wu = (bf16_round(rng.standard_normal((F, K)) / 3) for _ in range(2))
    inter = np.empty((2 * F, K), np.float32)
    inter[0::2], inter[1::2] = wg, wu
    out = gk.zeros((M, F), gk.float32)
    api.gemm_seq_f32(f32(x).device_ptr, K, 0, dev_w(inter, wdt).device_ptr, wdt, 0, out.device_ptr, F, 0, M, 2 * F, K, 1, 3,
                     1.702, 0.8, None, None, 0, None, 0, 0, min(few, M), None)
    g, u = np.minimum(xr @ wg.T.astype(np.float64), 0.8), np.clip(xr @ wu.T.astype(np.float64), -0.8, 0.8)
    assert (g == 0.8).any() and (u == -0.8).any()
    assert np.abs(out.to_numpy() - g * R.sigmoid(1.702 * g) * (u + 1)).max() < tol
    # C += s * product
    N = 21
    w = bf16_round(rng.standard_normal((N, K)) / 3)
    c0, s = rng.standard_normal((M, N)).astype(np.float32), rng.standard_normal(N).astype(np.float32)
    c = f32(c0)
    api.gemm_seq_f32(f32(x).device_ptr, K, 0, dev_w(w, wdt).device_ptr, wdt, 0, c.device_ptr, N, 0, M, N, K, 1, 4, 0.0, 0.0,
                     f32(s).device_ptr, None, 0, None, 0, 0, min(few, M), None)
    assert np.abs(c.to_numpy() - (c0 + s * (xr @ w.T.astype(np.float64)))).max() < tol
    # gelu(product) * table[row index, offset + column]
    table = bf16_round(rng.standard_normal((9, 3 * N)))
    rows = rng.integers(0, 9, M)
    out = gk.zeros((M, N), gk.float32)
    api.gemm_seq_f32(f32(x).device_ptr, K, 0, dev_w(w, wdt).device_ptr, wdt, 0, out.device_ptr, N, 0, M, N, K, 1, 5, 0.0, 0.0,
                     None, dev_w(table, wdt).device_ptr, wdt, i32(rows).device_ptr, 3 * N, N, min(few, M), None)
    assert np.abs(out.to_numpy() - R.gelu_tanh(xr @ w.T.astype(np.float64)) * table[rows, N:2 * N]).max() < tol


@pytest.mark.parametrize("wdt", [0, 2])
@pytest.mark.parametrize("M", [2, 40])
def test_gemm_batches_one_product_per_head(M, wdt):
    rng = np.random.default_rng(M)
    H, K, N, pad_a, pad_c = 5, 12, 18, 7, 3              # head h reads x[:, h * (K + pad_a) ...], writes c[:, h * (N + pad_c) ...]
    x = rng.standard_normal((M, H * (K + pad_a))).astype(np.float32)
    w = bf16_round(rng.standard_normal((H, N, K)) / 2)
    c = gk.zeros((M, H * (N + pad_c)), gk.float32)
    api.gemm_seq_f32(f32(x).device_ptr, H * (K + pad_a), K + pad_a, dev_w(w, wdt).device_ptr, wdt, N * K, c.device_ptr,
                     H * (N + pad_c), N + pad_c, M, N, K, H, 0, 0.0, 0.0, None, None, 0, None, 0, 0, M if M <= 8 else 0, None)
    xr = (bf16_round(x) if wdt == 2 else x).reshape(M, H, K + pad_a)[:, :, :K]
    got = c.to_numpy().reshape(M, H, N + pad_c)
    assert np.abs(got[:, :, :N] - np.einsum("mhk,hnk->mhn", xr.astype(np.float64), w)).max() < 2e-5
    assert not got[:, :, N:].any()


# ---------------------------------------------------------------- windowed attention on a hand-made cache
class WindowHarness:
    """pgk_seq_mixer_prep_all + pgk_seq_attention_ex on raw q / k rows [q | k | gate per head]."""

    def __init__(self, H, G, D, window, scale=0.3, page=4, dtype="float32", sink=0.0, splits=1, gate=True):
        self.H, self.G, self.D, self.window, self.scale, self.splits, self.gate = H, G, D, window, scale, splits, gate
        self.cache = PagedKVCache([(G, D, D)], dtype, page, 64, 2)
        self.qt = api.seq_queries_per_tile(H, G)
        self.sinks = None if sink is None else gk.from_numpy(np.full(H, sink, np.float32))
        self.sink = sink
        self.tickets = gk.zeros((4096,), gk.int32)
        self.cols = H * D + G * D + H
        rng = np.random.default_rng(H * 31 + D)
        self.qb, self.kb = 0.2 * rng.standard_normal(H * D), 0.2 * rng.standard_normal(G * D)
        self.qw, self.kw = 1 + 0.2 * rng.standard_normal(H * D), 1 + 0.2 * rng.standard_normal(G * D)
        self.decode_kernel = True

    def run(self, seq, q, k, gate):
        n = q.shape[0]
        slot, pos0 = self.cache.extend(seq, n)
        self.cache.sync_table()
        proj = gk.from_numpy(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), gate.reshape(n, -1)], axis=1).astype(np.float32))
        c, H, G, D = self.cache, self.H, self.G, self.D
        api.seq_mixer_prep_all(proj.device_ptr, self.cols, n, H, G, D, H * D, f32(self.qb).device_ptr, f32(self.kb).device_ptr,
                               f32(self.qw).device_ptr, f32(self.kw).device_ptr, 0.0, 1e-6, c.k[0].device_ptr, c.v[0].device_ptr,
                               c.dtype_code, c.table_dev.device_ptr, c.pool.max_pages, c.page_size, i32([slot] * n).device_ptr,
                               i32(np.arange(pos0, pos0 + n)).device_ptr, None)
        tiles = [(i, min(self.qt, n - i), slot, pos0 + i) for i in range(0, n, self.qt)]
        out = gk.zeros((n, H * D), gk.float32)
        api.seq_attention_ex(proj.device_ptr, self.cols, 0, proj.device_ptr, self.cols, H * D + G * D, 2 if self.gate else 0,
                             out.device_ptr, H * D, c.k[0].device_ptr, c.v[0].device_ptr, D, D, c.dtype_code,
                             c.table_dev.device_ptr, c.pool.max_pages, c.page_size, i32(tiles).device_ptr, len(tiles), None,
                             self.sinks.device_ptr if self.sinks is not None else None, H, G, D, D, 0, self.window, self.scale,
                             0.0, self.splits, keep(gk.zeros((n * H * self.splits * (D + 2),), gk.float32)).device_ptr,
                             self.tickets.device_ptr, 1 if (n == 1 and self.decode_kernel) else 0, None)
        assert not self.tickets.to_numpy().any()
        return out.to_numpy().reshape(n, H, D)

    def oracle(self, q, k, gate):
        T = q.shape[0]
        qf, kf = q.reshape(T, -1) + self.qb, k.reshape(T, -1) + self.kb
        qn = R.rms_norm(qf, self.qw, 1e-6).reshape(T, self.H, self.D)
        kn = R.rms_norm(kf, self.kw, 1e-6).reshape(T, self.G, self.D)
        o = R.windowed_core(qn, kn, kf.reshape(T, self.G, self.D), self.scale, self.window, self.sink)
        return o * R.sigmoid(gate)[:, :, None] if self.gate else o


@pytest.mark.parametrize("H,G,D,window,page", [(4, 1, 16, 6, 4), (4, 2, 8, 1, 3), (3, 3, 12, 100, 4), (8, 2, 32, 17, 8),
                                               (2, 1, 20, 9, 5), (40, 1, 8, 5, 4), (1, 1, 6, 0, 4), (2, 1, 112, 11, 8)])
def test_windowed_attention_whole_portions_and_single_tokens_agree_with_the_oracle(H, G, D, window, page):
    rng = np.random.default_rng(H * 7 + D)
    T = 45
    q, k, gate = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, H))
    h = WindowHarness(H, G, D, window, page=page)
    ref = h.oracle(q, k, gate)
    assert np.abs(h.run("w", q, k, gate) - ref).max() < 1e-5
    cuts = [0, 2, 5, 6, 19, 20, 31, 45]
    parts = np.concatenate([h.run("p", q[a:b], k[a:b], gate[a:b]) for a, b in zip(cuts, cuts[1:])])
    assert np.abs(parts - ref).max() < 1e-5
    h.cache.release("w")                                                 # its pages serve the next sequence
    single = np.concatenate([h.run("s", q[i:i + 1], k[i:i + 1], gate[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < 1e-5
    h.cache.release("p")
    h.decode_kernel = False                                              # the same through the tile kernel
    single = np.concatenate([h.run("t", q[i:i + 1], k[i:i + 1], gate[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < 1e-5
    # (the layout with heads of 112, like the latent one with rows of 160, needs 40-48 KB of dynamic shared memory: together
    # with the kernels' static arrays that is past the limit a launch may use without opting in)


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,page", [(6, 4), (8, 8), (33, 16), (1, 4)])
def test_standout_key_just_inside_and_just_outside_the_window(window, page, decoded):
    """One key has a score far above the rest, and its value (the key as projected) is the only one with a large
    component.  Query i must see it exactly while 0 <= i - star < window."""
    H, G, D = 2, 1, 8
    T = 2 * window + 40
    rng = np.random.default_rng(window)
    for star in (0, 5, window + 3, 63):                                  # also the sequence's first token and a page's last row
        if star >= T:
            continue
        q, k = 0.01 * rng.standard_normal((T, H, D)), 0.01 * rng.standard_normal((T, G, D))
        q[:, :, 0] = 3.0
        k[:, :, 0] = -3.0                                                # every other key points away from the queries
        k[star, 0, 0] = 3.0
        h = WindowHarness(H, G, D, window, scale=6.0, page=page, gate=False)
        h.qb[:], h.kb[:], h.qw[:], h.kw[:] = 0.0, 0.0, 1.0, 1.0
        ref = h.oracle(q, k, np.zeros((T, H)))
        n0 = T if not decoded else min(star + 1, T - 1)
        got = h.run("a", q[:n0], k[:n0], np.zeros((n0, H)))
        if decoded:
            got = np.concatenate([got] + [h.run("a", q[i:i + 1], k[i:i + 1], np.zeros((1, H))) for i in range(n0, T)])
        assert np.abs(got - ref).max() < 1e-5
        for i in range(T):
            sees = 0 <= i - star < window
            assert (got[i, :, 0] > 2.5).all() == sees and (sees or (got[i, :, 0] < 0).all()), (star, i)


def test_the_sink_takes_the_weight_when_no_key_matches():
    """All scores are far below zero, so the fixed sink (score 0, no value) holds nearly all of the softmax mass and the
    output all but vanishes; a learned sink of -40 gives the mass back to the keys."""
    H, G, D, T = 2, 2, 8, 20
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D))
    q[:, :, 0], k[:, :, 0] = 6.0, -6.0
    for sink, small in ((0.0, True), (-40.0, False), (None, False)):
        h = WindowHarness(H, G, D, 7, scale=3.0, sink=sink, gate=False)
        h.qb[:], h.kb[:], h.qw[:], h.kw[:] = 0.0, 0.0, 1.0, 1.0
        ref = h.oracle(q, k, np.zeros((T, H)))
        got = np.concatenate([h.run("a", q[:11], k[:11], np.zeros((11, H)))] +
                             [h.run("a", q[i:i + 1], k[i:i + 1], np.zeros((1, H))) for i in range(11, T)])
        assert np.abs(got - ref).max() < 1e-5
        assert (np.abs(got[:, :, 0]).max() < 1e-3) == small


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_key_slices_with_window_and_sink_fold_to_the_same_answer(splits):
    H, G, D, T = 4, 2, 16, 260
    rng = np.random.default_rng(splits)
    q, k, gate = rng.standard_normal((T, H, D)), rng.standard_normal((T, G, D)), rng.standard_normal((T, H))
    h = WindowHarness(H, G, D, 170, page=16, splits=splits, sink=0.7)
    ref = h.oracle(q, k, gate)
    got = np.concatenate([h.run("a", q[:200], k[:200], gate[:200])] +
                         [h.run("a", q[i:i + 1], k[i:i + 1], gate[i:i + 1]) for i in range(200, T)])
    assert np.abs(got - ref).max() < 1e-5


# ---------------------------------------------------------------- latent attention on a hand-made cache
class LatentHarness:
    """pgk_seq_latent_prep + pgk_seq_rope_heads + pgk_seq_attention_ex on raw rows: absorbed queries qa [n, H, nc], query
    tails qr [n, H, Dr], latent c [n, nc], shared key part r [n, Dr], gate [n, H].  Output in latent space [n, H, nc]."""

    def __init__(self, H, nc, Dr, dims, base=100.0, scale=0.2, page=4, dtype="float32", splits=1):
        self.H, self.nc, self.Dr, self.dims, self.base, self.scale, self.splits = H, nc, Dr, dims, base, scale, splits
        self.cache = PagedKVCache([(1, nc + Dr, 0)], dtype, page, 64, 2)
        self.qt = api.seq_queries_per_tile(H, 1)
        rng = np.random.default_rng(H + nc)
        self.sink = rng.standard_normal(H)
        self.cw = 1 + 0.2 * rng.standard_normal(nc)
        self.inv = f64([base ** (-2.0 * i / dims) for i in range(dims // 2)] or [0.0])
        self.tickets = gk.zeros((4096,), gk.int32)

    def run(self, seq, qa, qr, c, r, gate):
        n, H, nc, Dr = qa.shape[0], self.H, self.nc, self.Dr
        row = nc + Dr
        slot, pos0 = self.cache.extend(seq, n)
        self.cache.sync_table()
        ch = self.cache
        proj = gk.from_numpy(np.concatenate([c, r, gate], axis=1).astype(np.float32))
        pos, slots = i32(np.arange(pos0, pos0 + n)), i32([slot] * n)
        api.seq_latent_prep(proj.device_ptr, row + H, n, 0, 0, nc, Dr, self.dims, None, f32(self.cw).device_ptr, 0.0, 1e-6,
                            self.inv.device_ptr, ch.k[0].device_ptr, ch.dtype_code, ch.table_dev.device_ptr, ch.pool.max_pages,
                            ch.page_size, slots.device_ptr, pos.device_ptr, None)
        full = np.zeros((n, H, row), np.float32)
        full[:, :, :nc] = qa
        qfull = gk.from_numpy(full.reshape(n, -1))
        api.seq_rope_heads(f32(qr.reshape(n, -1)).device_ptr, H * Dr, Dr, 0, qfull.device_ptr, H * row, row, nc, n, H, Dr,
                           self.dims, self.inv.device_ptr, pos.device_ptr, None)
        tiles = [(i, min(self.qt, n - i), slot, pos0 + i) for i in range(0, n, self.qt)]
        out = gk.zeros((n, H * nc), gk.float32)
        api.seq_attention_ex(qfull.device_ptr, H * row, 0, proj.device_ptr, row + H, row, 2, out.device_ptr, H * nc,
                             ch.k[0].device_ptr, ch.k[0].device_ptr, row, row, ch.dtype_code, ch.table_dev.device_ptr,
                             ch.pool.max_pages, ch.page_size, i32(tiles).device_ptr, len(tiles), None,
                             f32(self.sink).device_ptr, H, 1, row, nc, 0, 0, self.scale, 0.0, self.splits,
                             keep(gk.zeros((n * H * self.splits * (nc + 2),), gk.float32)).device_ptr,
                             self.tickets.device_ptr, 1 if n == 1 else 0, None)
        return out.to_numpy().reshape(n, H, nc)

    def oracle(self, qa, qr, c, r, gate):
        T = qa.shape[0]
        pos = np.arange(T)
        cn = R.rms_norm(c, self.cw, 1e-6)
        rr, qq = R.rotate_pairs(r, pos, self.dims, self.base), R.rotate_pairs(qr, pos, self.dims, self.base)
        out = np.zeros((T, self.H, self.nc))
        for h in range(self.H):
            s = (qa[:, h] @ cn.T + qq[:, h] @ rr.T) * self.scale
            out[:, h] = R.softmax_with_sink(s, R.window_mask(T, 0), self.sink[h]) @ cn
        return out * R.sigmoid(gate)[:, :, None]


@pytest.mark.parametrize("H,nc,Dr,dims,page", [(3, 20, 12, 12, 4), (6, 40, 6, 4, 3), (2, 264, 8, 8, 8), (33, 8, 4, 4, 4),
                                               (1, 30, 0, 0, 5), (4, 128, 32, 32, 8)])
def test_latent_attention_whole_portions_and_single_tokens_agree_with_the_oracle(H, nc, Dr, dims, page):
    rng = np.random.default_rng(H + nc)
    T = 45
    qa, qr = rng.standard_normal((T, H, nc)), rng.standard_normal((T, H, Dr))
    c, r, gate = rng.standard_normal((T, nc)), rng.standard_normal((T, Dr)), rng.standard_normal((T, H))
    h = LatentHarness(H, nc, Dr, dims, page=page)
    ref = h.oracle(qa, qr, c, r, gate)
    assert np.abs(h.run("w", qa, qr, c, r, gate) - ref).max() < 2e-5
    cuts = [0, 2, 5, 6, 19, 20, 31, 45]
    parts = np.concatenate([h.run("p", qa[a:b], qr[a:b], c[a:b], r[a:b], gate[a:b]) for a, b in zip(cuts, cuts[1:])])
    assert np.abs(parts - ref).max() < 2e-5
    h.cache.release("w")
    single = np.concatenate([h.run("s", qa[i:i + 1], qr[i:i + 1], c[i:i + 1], r[i:i + 1], gate[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < 2e-5


@pytest.mark.parametrize("splits", [1, 4])
def test_latent_far_keys_among_hundreds_across_page_borders_and_large_positions(splits):
    """Three far keys (early, first row of a page, last row of a page) are the only ones whose latent has weight on the
    coordinates the queries look at; every later query must find all of them, no earlier one any.  Random rotated parts
    at positions in the hundreds ride along and are held to the oracle."""
    H, nc, Dr, T = 2, 16, 8, 330
    rng = np.random.default_rng(5)
    h = LatentHarness(H, nc, Dr, Dr, base=50.0, scale=2.0, page=64, splits=splits)
    h.cw[:] = 1.0
    qa, c = np.zeros((T, H, nc)), np.zeros((T, nc))
    qa[:, :, 0:3] = 3.0
    c[np.arange(T), 3 + np.arange(T) % (nc - 3)] = 1.0                   # everybody else lives on the other coordinates
    stars = (3, 64, 127)
    for kk, star in enumerate(stars):
        c[star] = 0.0
        c[star, kk] = 1.0
    qr, r = 0.1 * rng.standard_normal((T, H, Dr)), rng.standard_normal((T, Dr))
    gate = np.full((T, H), 30.0)
    ref = h.oracle(qa, qr, c, r, gate)
    got = np.concatenate([h.run("a", qa[:290], qr[:290], c[:290], r[:290], gate[:290])] +
                         [h.run("a", qa[i:i + 1], qr[i:i + 1], c[i:i + 1], r[i:i + 1], gate[i:i + 1]) for i in range(290, T)])
    assert np.abs(got - ref).max() < 2e-5
    for i in (128, 289, 290, 329):                                       # in the prompt and decoded: all three count
        assert (got[i, :, 0:3] > 0.2).all(), i
    assert (got[100, :, 0:2] > 0.2).all() and (np.abs(got[100, :, 2]) < 1e-6).all()   # key 127 lies in the future of query 100
    assert (np.abs(got[2, :, 0:3]) < 1e-6).all()


# ================================================================ whole models
def variants():
    """Sizes that the mechanisms must not assume equal: key / rotated / value sizes of the latent mixer all different,
    fewer rotated dimensions than the rotated part, grouped key/value heads, one head, windows of 1 and beyond the
    sequence, loops that start late or cover everything, layers without feed-forward, no token input, odd widths."""
    yield "base", R.make_config([R.latent_layer(), R.windowed_layer(), R.windowed_layer(heads=2, kv_heads=1, dim=12, window=3, ff=20)],
                                loop=(0, 2, 2))
    yield "no_loop_no_side", R.make_config([R.windowed_layer(heads=6, kv_heads=2, dim=8, window=4), R.latent_layer(dims=8, limit=0.4)],
                                           side=0)
    yield "loop_late_odd_width", R.make_config(
        [R.windowed_layer(heads=3, kv_heads=3, dim=10, window=5, ff=0), R.latent_layer(heads=2, dim=6, rot_dim=4, vdim=14, kv_rank=11, q_rank=9, ff=18),
         R.windowed_layer(window=1, ff=30, limit=0.7), R.latent_layer(heads=5, ff=0)], vocab=61, width=52, side=1, loop=(1, 3, 3))
    yield "whole_stack_looped", R.make_config([R.windowed_layer(heads=1, kv_heads=1, dim=20, window=1000), R.latent_layer(heads=1)],
                                              side=3, loop=(0, 2, 2))
    yield "wide_latent", R.make_config([R.latent_layer(heads=2, dim=12, rot_dim=8, vdim=6, kv_rank=264, q_rank=16)], side=4)


VARIANTS = dict(variants())
# with a token input of ONE dimension the normalised side vector is sign(g) * const: a step function of g that bfloat16
# rounding can flip, so the bfloat16 comparison uses the same stack with five
VARIANTS["loop_late_odd_width_side5"] = dict(VARIANTS["loop_late_odd_width"], token_side={"dim": 5})


def make(name, dtype="float32", page=4, seed=1, tokens_hint=64):
    cfg = VARIANTS[name]
    P = R.random_params(cfg, seed=seed)
    m = llm.build_layered_model(layered_config_from_json(cfg), P, dtype)
    m.init_cache(tokens_hint, page_size=page, slots=2)
    return cfg, P, m


def tokens(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_and_every_layer_run_match_the_oracle_float32(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 29)
    ref, layers = R.forward(cfg, P, toks, True)
    seen = []
    m.trace_hook = lambda run, x: seen.append(x)
    got = m.step([("a", toks, list(range(len(toks))))])
    assert len(seen) == len(layers)
    for run, (a, b) in enumerate(zip(seen, layers)):
        assert np.abs(a - b).max() < F32_TOL, run
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "loop_late_odd_width", "whole_stack_looped"])
def test_prefill_then_token_by_token_decoding(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 40, seed=3)
    ref = R.forward(cfg, P, toks)
    got = [m.step([("a", toks[:9], list(range(9)))])]
    got += [m.step([("a", [t], [0])]) for t in toks[9:]]                 # the windows pass over decoded tokens
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "no_loop_no_side"])
def test_first_tokens_and_decoding_from_position_zero(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 12, seed=4)
    ref = R.forward(cfg, P, toks)
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks])
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("sizes", [[2] * 15, [3, 2, 7, 1, 11, 6], [16, 14], [1, 29]])
def test_prompt_portions(sizes):
    cfg, P, m = make("loop_late_odd_width")
    toks = tokens(cfg, sum(sizes), seed=5)
    ref = R.forward(cfg, P, toks)
    got, at = [], 0
    for n in sizes:
        got.append(m.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "loop_late_odd_width"])
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


def test_more_than_eight_decoding_requests():
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
    cfg, P, m = make("base", page=8)
    toks = tokens(cfg, 150, seed=6)
    ref = R.forward(cfg, P, toks)
    want = [0, 6, 7, 8, 30, 69]
    got = m.step([("a", toks[:70], want)])
    assert np.abs(got - ref[want]).max() < F32_TOL
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[70:]])
    assert np.abs(got - ref[70:]).max() < F32_TOL


def test_decoding_over_a_long_context_reads_the_latent_cache_in_slices():
    cfg, P, m = make("wide_latent", page=16, tokens_hint=512)
    toks = tokens(cfg, 300, seed=8)
    ref = R.forward(cfg, P, toks)
    m.step([("a", toks[:288], [])])
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[288:]])
    assert m._ws is not None                                             # the sliced path ran
    assert np.abs(got - ref[288:]).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "loop_late_odd_width_side5", "wide_latent", "no_loop_no_side"])
def test_bfloat16_mode_stays_within_bfloat16_rounding(name):
    cfg, P, m = make(name, dtype="bfloat16")
    toks = tokens(cfg, 33, seed=7)
    ref = R.forward(cfg, P, toks)
    whole = m.step([("a", toks, list(range(33)))])
    scale = np.abs(ref).max()
    assert np.abs(whole - ref).max() < 0.04 * scale
    got = np.concatenate([m.step([("b", toks[:20], list(range(20)))])] + [m.step([("b", [t], [0])]) for t in toks[20:]])
    assert np.abs(got - whole).max() < 0.04 * scale                      # the same sequence cut differently: rounding only


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


def _save(cfg, P, folder):
    tensors = {k: ((np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(v.shape), "BF16")
               for k, v in P.items()}
    llm.save_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return {k: (np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16 << 16).view(np.float32) for k, v in P.items()}


def test_loader_picks_the_family_from_config_json(tmp_path):
    cfg = VARIANTS["loop_late_odd_width"]
    P = _save(cfg, R.random_params(cfg, seed=8), str(tmp_path))
    m = llm.load_model_from_safetensors(str(tmp_path), dtype="float32")
    assert isinstance(m, llm.LayeredCausalModel) and m.config.architecture == "Turutar"
    toks = tokens(cfg, 10)
    assert np.abs(m.step([("a", toks, list(range(10)))]) - R.forward(cfg, P, toks)).max() < F32_TOL
    with pytest.raises(ValueError, match="shape"):
        bad = dict(P)
        bad["l1.mix.uk"] = P["l1.mix.uk"][:-1]
        llm.build_layered_model(layered_config_from_json(cfg), bad, "float32")


def test_trace_replay_command_line(tmp_path):
    cfg = VARIANTS["base"]
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    P = _save(cfg, R.random_params(cfg, seed=9), str(model_dir))
    a, b = tokens(cfg, 14, seed=1), tokens(cfg, 6, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": [0, 10]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[11]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[12]], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[13]], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                        "--out", str(out_dir), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = R.forward(cfg, P, a), R.forward(cfg, P, b)
    V = cfg["vocab"]
    got0 = np.fromfile(out_dir / "0.f32", "<f4").reshape(-1, V)
    assert np.abs(got0 - np.stack([ra[0], ra[10], rb[4]])).max() < F32_TOL
    assert np.abs(np.fromfile(out_dir / "1.f32", "<f4").reshape(-1, V) - rb[5:6]).max() < F32_TOL
    assert np.abs(np.fromfile(out_dir / "3.f32", "<f4").reshape(-1, V) - ra[13:14]).max() < F32_TOL
