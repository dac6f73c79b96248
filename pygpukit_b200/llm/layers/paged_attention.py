"""Attention mixer of the token-major models on the paged cache (net-new; beside `Attention`, which serves one
sequence on a fixed cache).  One fused projection [q | k | v | gate], then two launches:

  pgk_seq_mixer_prep   RMS norm of q and k per head, value mixing, K / V rows into the cache pages
  pgk_seq_attention    scores with scale, tanh cap and per-head distance slopes, chunk mask, softmax, P.V, output gate

and the output projection.  Every constant comes from the `AttentionMixerSpec`; `v_role` says what the layer does
with its values: 0 nothing, 1 record them as the step's v_first, 2 mix them with the recorded ones.
"""
from __future__ import annotations

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.factory import from_numpy
from ...core.stream import current_stream_handle as _st
from ..config import AttentionMixerSpec
from .linear import LinearRows


class PagedAttentionMixer:
    def __init__(self, spec: AttentionMixerSpec, layer: int, qkvg: LinearRows, o_proj: LinearRows, q_norm: GPUArray,
                 k_norm: GPUArray, eps: float, v_role: int = 0, v_lambda: float = 0.0):
        self.spec, self.layer = spec, layer
        self.qkvg, self.o_proj = qkvg, o_proj
        self.q_norm, self.k_norm, self.eps = q_norm, k_norm, float(eps)
        self.v_role, self.v_lambda = int(v_role), float(v_lambda)
        s = spec
        self.q_cols, self.k_cols, self.v_cols = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.g_cols = s.heads * s.vdim if s.out_gate else 0
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
        """Few long tiles (decoding over a long chunk): the key range of every tile is cut into this many slices so that
        the whole GPU reads the cache.  A power of two, so that a decode step's launch shapes change rarely."""
        s = self.spec
        n_tiles = ctx.tiles(self.queries_per_tile)[1]
        rep = s.heads // s.kv_heads
        keys = ctx.max_keys(s.chunk)
        if ctx.decode_only:          # the decoding kernel: eight warps take 32 keys each per round
            blocks = n_tiles * s.kv_heads * -(-rep // self.decode_heads_per_block)
            want = max(1, min(64, -(-keys // 256), 592 // max(1, blocks)))
        else:
            blocks = n_tiles * s.kv_heads * -(-rep // self.heads_per_block)
            if blocks >= 148 or keys < 256:
                return 1
            want = max(1, min(64, -(-keys // 32), 592 // blocks))
        return min(64, 1 << (want - 1).bit_length())

    def forward(self, ctx, x: GPUArray, out: GPUArray) -> None:
        """x [T, W] -> out [T, W] (the mixer's output before the block's norm); K / V of the T tokens enter the cache."""
        s, T = self.spec, ctx.T
        W = self.qkvg.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        ld = self.proj_cols
        self.qkvg.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        cache = ctx.cache
        kc, vc = cache.k[self.layer], cache.v[self.layer]
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
        api.seq_attention(proj.device_ptr, ld, 0, self.q_cols + self.k_cols + self.v_cols, attn.device_ptr, ldo,
                          kc.device_ptr, vc.device_ptr, cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages,
                          cache.page_size, tiles_ptr, n_tiles, self.slopes.device_ptr if self.slopes is not None else None,
                          s.heads, s.kv_heads, s.dim, s.vdim, s.chunk, s.scale, s.softcap, 1 if s.out_gate else 0,
                          splits, ws, tickets, 1 if ctx.decode_only else 0, _st())
        self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)


__all__ = ["PagedAttentionMixer"]
