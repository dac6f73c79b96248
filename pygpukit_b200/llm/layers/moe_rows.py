"""Mixture of experts of the token-major models (net-new; beside `MoELayer`, whose router is top-k then softmax over
the chosen logits and whose experts are FP8 / NVF4 GEMVs on bfloat16 rows).

Router: float32 logits from the router GEMM (the router matrix is kept in float32 in both modes, so the logits are
FMAs on the unrounded residual stream), then pgk_moe_route_grouped:
softmax over ALL experts, optional group limit (only members of the best
`group_keep` of `group_count` groups of neighbours), the `top` largest scores, renormalised.  Experts: stacked
[E, 2 ff, W] gate/up pairs (SiLU * up in the GEMM epilogue) and [E, W, ff] down matrices.

  many tokens   rows (token, slot) are sorted by expert on the device (pgk_moe_row_lists) and the two grouped GEMMs
                gather their input rows through the permutation -- tokens are never copied;
  <= 8 tokens   rows stay in slot order and every row streams its own expert's matrices (few-row kernel).

The weighted sum of the expert outputs, the shared expert's output, the block's LayerNorm and the residual add are
ONE launch (pgk_combine_layernorm_f32), issued by the block with what `forward` returns.
"""
from __future__ import annotations

from ..._lib import api
from ...core.array import GPUArray
from ...core.stream import current_stream_handle as _st
from ..config import MoESpec
from .linear import LinearRows


class GroupedRouterMoE:
    def __init__(self, spec: MoESpec, router: GPUArray, gate_up: LinearRows, down: LinearRows,
                 shared_gate_up: LinearRows | None = None, shared_down: LinearRows | None = None):
        self.spec, self.router = spec, LinearRows(router)
        self.gate_up, self.down = gate_up, down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        if gate_up.groups != spec.experts or down.groups != spec.experts:
            raise ValueError("GroupedRouterMoE: expert stacks do not match the router")

    @property
    def weight_bytes(self) -> int:
        n = self.router.nbytes + self.gate_up.nbytes + self.down.nbytes
        if self.shared_gate_up is not None:
            n += self.shared_gate_up.nbytes + self.shared_down.nbytes
        return n

    def forward(self, ctx, x: GPUArray, shared_out: GPUArray):
        """Returns (base, parts, inv, weights, top) for the combine + norm launch: base = the shared expert's output
        rows (or None), parts [T * top, W] the routed experts' outputs, inv [T, top] their rows."""
        sp, T, b = self.spec, ctx.T, ctx.buf
        W, top, ff = self.gate_up.in_features, sp.top, sp.ff
        few = T <= LinearRows.FEW
        self.router.forward(x.device_ptr, W, T, b.moe_z.device_ptr, sp.experts)       # float32 logits [T, E]
        api.moe_route_grouped(b.moe_z.device_ptr, sp.experts, T, sp.experts, top,
                              sp.group_count, sp.group_keep, b.moe_idx.device_ptr, b.moe_w.device_ptr,
                              None if few else b.moe_rank.device_ptr, None if few else b.moe_counts.device_ptr, _st())
        if few:
            slot_tok, iota = ctx.slot_rows(top)
            self.gate_up.forward_per_row(x.device_ptr, W, T * top, b.moe_act.device_ptr, ff, slot_tok, b.moe_idx.device_ptr)
            self.down.forward_per_row(b.moe_act.device_ptr, ff, T * top, b.moe_parts.device_ptr, W, None, b.moe_idx.device_ptr)
            inv = iota
        else:
            api.moe_row_lists(b.moe_counts.device_ptr, b.moe_off.device_ptr, b.moe_idx.device_ptr, b.moe_rank.device_ptr,
                              b.moe_perm.device_ptr, b.moe_inv.device_ptr, sp.experts, T, top, _st())
            self.gate_up.forward_grouped(x.device_ptr, W, b.moe_act.device_ptr, ff, b.moe_perm.device_ptr,
                                         b.moe_off.device_ptr, T)
            self.down.forward_grouped(b.moe_act.device_ptr, ff, b.moe_parts.device_ptr, W, None, b.moe_off.device_ptr, T)
            inv = b.moe_inv.device_ptr
        base = None
        if self.shared_gate_up is not None:
            fs = self.shared_gate_up.out_cols
            self.shared_gate_up.forward(x.device_ptr, W, T, b.shared_act.device_ptr, fs)
            self.shared_down.forward(b.shared_act.device_ptr, fs, T, shared_out.device_ptr, W)
            base = shared_out.device_ptr
        return base, b.moe_parts.device_ptr, inv, b.moe_w.device_ptr, top


__all__ = ["GroupedRouterMoE"]
