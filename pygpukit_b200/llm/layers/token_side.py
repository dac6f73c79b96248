"""Per-layer token input of the token-major models (net-new): after a layer, every token adds a small vector that
depends on its id and on the residual stream,

    e = table[token, layer * dim : (layer + 1) * dim];  g = gelu_tanh(W_gate x) * e;  y = W_proj g;
    x <- x + y / rms(y) * w

Three launches: the gate product with the gelu and the gathered table entry in its epilogue, the projection, and the
RMS norm that accumulates into the residual stream -- which, when another pre-norm block follows, also applies that
block's norm to the updated row (one pass over the row instead of two launches).  The table is shared by all layers; `layer` picks the slice (a
layer that runs several times in a loop uses the same slice every time).
"""
from __future__ import annotations

from ...core.array import GPUArray
from .linear import LinearRows
from .norm import RowNorm


class TokenSideInput:
    def __init__(self, table: GPUArray, layer: int, dim: int, gate: LinearRows, proj: LinearRows, norm: RowNorm):
        if gate.out_features != dim or proj.in_features != dim or table.shape[1] < (layer + 1) * dim:
            raise ValueError(f"TokenSideInput: layer {layer} with slices of {dim} does not fit its matrices")
        self.table, self.layer, self.dim = table, layer, dim
        self.gate, self.proj, self.norm = gate, proj, norm
        self.table_dt = 2 if table.dtype.name == "bfloat16" else 0

    @property
    def weight_bytes(self) -> int:
        return self.gate.nbytes + self.proj.nbytes + self.norm.nbytes

    def forward(self, ctx, x: GPUArray, next_norm: RowNorm | None = None, next_add_ptr: int | None = None) -> bool:
        """Adds the token input to x.  With `next_norm` (the norm in front of the block that runs next) the last launch
        also writes that block's normed rows into ctx.buf.h -- after adding `next_add_ptr` rows to x when given -- and
        True is returned."""
        T, W, d = ctx.T, x.shape[1], self.dim
        g, y = ctx.buf.side, ctx.buf.y
        self.gate.forward_seq(x.device_ptr, W, T, g.device_ptr, d, epilogue=5,
                              aux=(self.table.device_ptr, self.table_dt, ctx.tok_ptr, self.table.shape[1], self.layer * d))
        self.proj.forward_seq(g.device_ptr, d, T, y.device_ptr, W, epilogue=0)
        if self.norm.fuses_with(next_norm) and ctx.buf.h is not None:
            self.norm.forward_seam(y.device_ptr, x.device_ptr, next_norm, ctx.buf.h.device_ptr, T, W, next_add_ptr)
            return True
        self.norm.forward(y.device_ptr, x.device_ptr, T, W, accumulate=True)
        return False


__all__ = ["TokenSideInput"]
