"""Attention mixer of the token-major models on the paged cache (net-new; beside `Attention`, which serves one
sequence on a fixed cache).  One fused projection [q | k | v | gate], then two launches:

  pgk_seq_mixer_prep   RMS norm of q and k per head, value mixing, K / V rows into the cache pages
  pgk_seq_attention    scores with scale, tanh cap and per-head distance slopes, chunk mask, softmax, P.V, output gate

and the output projection.  Every constant comes from the `AttentionMixerSpec`; `v_role` says what the layer does
with its values: 0 nothing, 1 record them as the step's v_first, 2 mix them with the recorded ones.

Specs with `norm_scope == "all"` take the other preparation launch, pgk_seq_mixer_prep_all: projection biases, RMS norm of
q and of k over the whole projection, and (`values == "keys"`) the keys as projected written as the values.  A sliding
window, a sink (fixed at zero or learned per head) and a per-head gate are arguments of the attention launch.
"""
from __future__ import annotations

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.factory import from_numpy
from ...core.stream import current_stream_handle as _st
from ..config import AttentionMixerSpec
from .linear import LinearRows


def key_slices(ctx, heads: int, kv_heads: int, chunk: int, window: int, queries_per_tile: int, heads_per_block: int,
               decode_heads_per_block: int) -> int:
    """Few long tiles (decoding over a long context): the key range of every tile is cut into this many slices so that the
    whole GPU reads the cache.  A power of two, so that a decode step's launch shapes change rarely."""
    n_tiles = ctx.tiles(queries_per_tile)[1]
    rep = heads // kv_heads
    keys = ctx.max_keys(chunk, window)
    if ctx.decode_only:          # the decoding kernel: eight warps take 32 keys each per round
        blocks = n_tiles * kv_heads * -(-rep // decode_heads_per_block)
        want = max(1, min(64, -(-keys // 256), 592 // max(1, blocks)))
    else:
        blocks = n_tiles * kv_heads * -(-rep // heads_per_block)
        if blocks >= 148 or keys < 256:
            return 1
        want = max(1, min(64, -(-keys // 32), 592 // blocks))
    if n_tiles * kv_heads * rep > 4096:          # one arrival counter per (tile, head block)
        return 1
    return min(64, 1 << (want - 1).bit_length())


class PagedAttentionMixer:
    def __init__(self, spec: AttentionMixerSpec, layer: int, qkvg: LinearRows, o_proj: LinearRows, q_norm: GPUArray,
                 k_norm: GPUArray, eps: float, v_role: int = 0, v_lambda: float = 0.0, q_bias: GPUArray | None = None,
                 k_bias: GPUArray | None = None, sinks: GPUArray | None = None, norm_offset: float = 0.0):
        self.spec, self.layer = spec, layer
        self.qkvg, self.o_proj = qkvg, o_proj
        self.q_norm, self.k_norm, self.eps = q_norm, k_norm, float(eps)
        self.v_role, self.v_lambda = int(v_role), float(v_lambda)
        self.q_bias, self.k_bias, self.sinks, self.norm_offset = q_bias, k_bias, sinks, float(norm_offset)
        s = spec
        if s.norm_scope not in ("head", "all") or s.values not in ("own", "keys") or s.sink not in ("none", "zero", "learned"):
            raise ValueError(f"layer {layer}: unknown norm scope / value source / sink in {s}")
        if s.values == "keys" and (s.norm_scope != "all" or s.vdim != s.dim or v_role):
            raise ValueError(f"layer {layer}: values that are the keys need the whole-projection form and vdim == dim")
        if s.norm_scope == "all" and (s.values != "keys" or not s.qk_norm):
            raise ValueError(f"layer {layer}: the whole-projection norm is built for values that are the keys")
        if (s.sink == "learned") != (sinks is not None):
            raise ValueError(f"layer {layer}: sink {s.sink!r} and the sink vector do not agree")
        if s.sink == "zero":
            self.sinks = from_numpy(np.zeros((s.heads,), np.float32))
        self.q_cols, self.k_cols = s.heads * s.dim, s.kv_heads * s.dim
        self.v_cols = s.kv_heads * s.vdim if s.values == "own" else 0
        self.g_cols = s.gate_cols
        self.proj_cols = self.q_cols + self.k_cols + self.v_cols + self.g_cols
        if qkvg.out_features != self.proj_cols:
            raise ValueError(f"layer {layer}: fused projection has {qkvg.out_features} rows, the mixer needs {self.proj_cols}")
        sl = spec.slopes()
        self.slopes = from_numpy(np.asarray(sl, np.float32)) if sl else None
        self.queries_per_tile = int(api.seq_queries_per_tile(s.heads, s.kv_heads))
        self.heads_per_block = int(api.seq_heads_per_block(s.heads, s.kv_heads))
        self.decode_heads_per_block = int(api.seq_decode_heads_per_block())

    @property
    def weight_bytes(self) -> int:
        return self.qkvg.nbytes + self.o_proj.nbytes

    def key_slices(self, ctx) -> int:
        s = self.spec
        return key_slices(ctx, s.heads, s.kv_heads, s.chunk, s.window, self.queries_per_tile, self.heads_per_block,
                          self.decode_heads_per_block)

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None) -> None:
        """x [T, W] -> out [T, W] (the mixer's output before the block's norm); K / V of the T tokens enter the cache
        `cache_index` (default: the layer's own).  With out_scale (device pointer of [W] floats) the output projection
        adds out_scale * result to `out` instead of storing it."""
        s, T = self.spec, ctx.T
        W = self.qkvg.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        ld = self.proj_cols
        self.qkvg.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        cache = ctx.cache
        ci = self.layer if cache_index is None else cache_index
        kc, vc = cache.k[ci], cache.v[ci]
        if s.norm_scope == "all":
            api.seq_mixer_prep_all(proj.device_ptr, ld, T, s.heads, s.kv_heads, s.dim, self.q_cols,
                                   self.q_bias.device_ptr if self.q_bias is not None else None,
                                   self.k_bias.device_ptr if self.k_bias is not None else None, self.q_norm.device_ptr,
                                   self.k_norm.device_ptr, self.norm_offset, self.eps, kc.device_ptr, vc.device_ptr,
                                   cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size,
                                   ctx.slot_ptr, ctx.pos_ptr, _st())
        else:
            api.seq_mixer_prep(proj.device_ptr, ld, T, s.heads, s.kv_heads, s.dim, s.vdim, self.q_norm.device_ptr,
                               self.k_norm.device_ptr, self.eps, self.v_role, self.v_lambda,
                               ctx.buf.v_first.device_ptr if self.v_role else None, kc.device_ptr, vc.device_ptr,
                               cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size,
                               ctx.slot_ptr, ctx.pos_ptr, _st())
        tiles_ptr, n_tiles = ctx.tiles(self.queries_per_tile)
        ldo = s.heads * s.vdim
        splits, ws, tickets = self.key_slices(ctx), None, None
        if splits > 1:
            ws = ctx.workspace(T * s.heads * splits * (s.vdim + 2)).device_ptr
            tickets = ctx.buf.tickets.device_ptr
        gate_mode = 0 if not s.out_gate else (2 if s.gate_per_head else 1)
        api.seq_attention_ex(proj.device_ptr, ld, 0, proj.device_ptr, ld, self.q_cols + self.k_cols + self.v_cols, gate_mode,
                             attn.device_ptr, ldo, kc.device_ptr, vc.device_ptr, s.dim, s.vdim, cache.dtype_code,
                             cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size, tiles_ptr, n_tiles,
                             self.slopes.device_ptr if self.slopes is not None else None,
                             self.sinks.device_ptr if self.sinks is not None else None, s.heads, s.kv_heads, s.dim, s.vdim,
                             s.chunk, s.window, s.scale, s.softcap, splits, ws, tickets, 1 if ctx.decode_only else 0, _st())
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)


__all__ = ["PagedAttentionMixer", "key_slices"]
