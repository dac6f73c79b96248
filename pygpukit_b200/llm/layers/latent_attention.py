"""Latent attention of the token-major models on the paged cache (net-new; beside `PagedAttentionMixer`).

Per position the cache holds one row [c | r]: the RMS-normed key/value latent (kv_rank) and the rotated key part
(rot_dim) shared by all heads.  With per-head matrices Wuk_h, Wuv_h the key of head h is [Wuk_h c | r] and the value
Wuv_h c, so

    score_h(i, j) = scale (q_h^nope . Wuk_h c_j + q_h^rot . r_j) = scale ([Wuk_h^T q_h^nope | q_h^rot] . [c_j | r_j])
    out_h(i)      = Wuv_h sum_j p_ij c_j

and the attention kernel runs unchanged with ONE key/value head of row size kv_rank + rot_dim whose value rows are a
prefix of its key rows.  Launches: fused projection [query latent | c, r | gate], `pgk_seq_latent_prep` (norms, rotation
of r, cache write), query up-projection, per-head absorption q~_h = Wuk_h^T q_h^nope (one batched product),
`pgk_seq_rope_heads` (rotated query tails behind the absorbed queries), `pgk_seq_attention_ex` (sink, per-head gate),
per-head Wuv_h (batched), output projection.
"""
from __future__ import annotations

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.factory import from_numpy
from ...core.stream import current_stream_handle as _st
from ..config import LatentMixerSpec
from .linear import LinearRows


class LatentAttentionMixer:
    def __init__(self, spec: LatentMixerSpec, layer: int, down: LinearRows, q_up: LinearRows, k_absorb: LinearRows,
                 v_up: LinearRows, o_proj: LinearRows, q_norm: GPUArray | None, c_norm: GPUArray, eps: float,
                 sinks: GPUArray | None = None, norm_offset: float = 0.0):
        """down: [q_rank + kv_rank + rot_dim + gate, W]; q_up: [H (dim + rot_dim), q_rank]; k_absorb: the stack
        [H, kv_rank, dim] of Wuk_h^T; v_up: the stack [H, vdim, kv_rank]; o_proj: [W, H vdim]."""
        s = self.spec = spec
        self.layer = layer
        self.down, self.q_up, self.k_absorb, self.v_up, self.o_proj = down, q_up, k_absorb, v_up, o_proj
        self.q_norm, self.c_norm, self.eps, self.norm_offset = q_norm, c_norm, float(eps), float(norm_offset)
        self.sinks = sinks
        if s.q_rank <= 0:
            raise ValueError("LatentAttentionMixer: the query latent needs a positive rank")
        if down.out_features != s.proj_cols or q_up.out_features != s.heads * (s.dim + s.rot_dim) or q_up.in_features != s.q_rank:
            raise ValueError(f"layer {layer}: projections do not match the latent sizes")
        if (k_absorb.groups, k_absorb.out_features, k_absorb.in_features) != (s.heads, s.kv_rank, s.dim):
            raise ValueError(f"layer {layer}: absorbed key matrices must be [heads, kv_rank, dim]")
        if (v_up.groups, v_up.out_features, v_up.in_features) != (s.heads, s.vdim, s.kv_rank):
            raise ValueError(f"layer {layer}: value matrices must be [heads, vdim, kv_rank]")
        if s.sink not in ("none", "zero", "learned") or (s.sink == "learned") != (sinks is not None):
            raise ValueError(f"layer {layer}: sink {s.sink!r} and the sink vector do not agree")
        if s.sink == "zero":
            self.sinks = from_numpy(np.zeros((s.heads,), np.float32))
        self.inv_freq = from_numpy(np.asarray(s.inv_freq() or [0.0], np.float64))
        self.row = s.kv_rank + s.rot_dim                      # cache row = key row of the one key/value head
        self.queries_per_tile = int(api.seq_queries_per_tile(s.heads, 1))
        self.heads_per_block = int(api.seq_heads_per_block(s.heads, 1))
        self.decode_heads_per_block = 2 if s.kv_rank > 256 else int(api.seq_decode_heads_per_block())

    @property
    def weight_bytes(self) -> int:
        return self.down.nbytes + self.q_up.nbytes + self.k_absorb.nbytes + self.v_up.nbytes + self.o_proj.nbytes

    def key_slices(self, ctx) -> int:
        from .paged_attention import key_slices
        return key_slices(ctx, self.spec.heads, 1, 0, 0, self.queries_per_tile, self.heads_per_block, self.decode_heads_per_block)

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None) -> None:
        """x [T, W] (the block's normed rows) -> out [T, W]: stored, or out += out_scale * result when out_scale (device
        pointer of [W] floats) is given.  The T tokens' cache rows are written."""
        s, T, b = self.spec, ctx.T, ctx.buf
        W, H, R, row = self.down.in_features, s.heads, s.kv_rank, self.row
        proj, qup, qa, lat, vo = b.proj, b.q_up, b.q_abs, b.latent_out, b.head_out
        ld = s.proj_cols
        self.down.forward_seq(x.device_ptr, W, T, proj.device_ptr, ld, epilogue=0)
        cache = ctx.cache
        kc = cache.k[self.layer if cache_index is None else cache_index]
        api.seq_latent_prep(proj.device_ptr, ld, T, s.q_rank, s.q_rank, R, s.rot_dim, s.rot_dims,
                            self.q_norm.device_ptr if self.q_norm is not None else None, self.c_norm.device_ptr,
                            self.norm_offset, self.eps, self.inv_freq.device_ptr, kc.device_ptr, cache.dtype_code,
                            cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size, ctx.slot_ptr, ctx.pos_ptr, _st())
        hd = s.dim + s.rot_dim
        self.q_up.forward_seq(proj.device_ptr, ld, T, qup.device_ptr, H * hd, epilogue=0)
        # q~_h = Wuk_h^T q_h^nope for every head: product h reads columns h * hd .. of qup, writes columns h * row .. of qa
        self.k_absorb.forward_seq(qup.device_ptr, H * hd, T, qa.device_ptr, H * row, epilogue=0, batch=H, a_batch=hd, c_batch=row)
        api.seq_rope_heads(qup.device_ptr, H * hd, hd, s.dim, qa.device_ptr, H * row, row, R, T, H, s.rot_dim, s.rot_dims,
                           self.inv_freq.device_ptr, ctx.pos_ptr, _st())
        tiles_ptr, n_tiles = ctx.tiles(self.queries_per_tile)
        splits, ws, tickets = self.key_slices(ctx), None, None
        if splits > 1:
            ws = ctx.workspace(T * H * splits * (R + 2)).device_ptr
            tickets = b.tickets.device_ptr
        gate_mode = 0 if not s.out_gate else (2 if s.gate_per_head else 1)
        api.seq_attention_ex(qa.device_ptr, H * row, 0, proj.device_ptr, ld, s.q_rank + R + s.rot_dim, gate_mode,
                             lat.device_ptr, H * R, kc.device_ptr, kc.device_ptr, row, row, cache.dtype_code,
                             cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size, tiles_ptr, n_tiles, None,
                             self.sinks.device_ptr if self.sinks is not None else None, H, 1, row, R, 0, 0, s.scale, 0.0,
                             splits, ws, tickets, 1 if ctx.decode_only else 0, _st())
        self.v_up.forward_seq(lat.device_ptr, H * R, T, vo.device_ptr, H * s.vdim, epilogue=0, batch=H, a_batch=R, c_batch=s.vdim)
        if out_scale is None:
            self.o_proj.forward_seq(vo.device_ptr, H * s.vdim, T, out.device_ptr, self.o_proj.out_features, epilogue=0)
        else:
            self.o_proj.forward_seq(vo.device_ptr, H * s.vdim, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)


__all__ = ["LatentAttentionMixer"]
