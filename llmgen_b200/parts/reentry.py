"""A step on the residual stream between run items: the stream mixed with the embedding's output."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .linear import GEMM_MODULES, linear
from .spec import VECTOR, ReentrySpec, WeightDecl


class Reentry(Part):
    """x <- [x | x0] W^T + table[row]: W [hidden, 2 hidden] reads the stream's columns first and then those of x0, the
    embedding's output of the same token (kept in float32 by the model for every step that has such an item).

    The sum that the layer before left unfinished (its `delta`) is finished on the way: one kernel writes
    [resid + delta | x0] in the storage dtype, the product writes its float32 result over the residual rows, and the
    table's row is added there.  Items with the same `proj` and `table` share the device tensors."""

    @staticmethod
    def weight_decls(spec: ReentrySpec, hidden: int):
        return [WeightDecl(spec.proj, (hidden, 2 * hidden)), WeightDecl(spec.table, (spec.rows, hidden), VECTOR)]

    @staticmethod
    def kernel_modules(spec):
        return ("rowwise",) + GEMM_MODULES

    def __init__(self, spec: ReentrySpec, weights, dtype, device):
        if not 0 <= spec.row < spec.rows:
            raise ValueError(f"reentry: row {spec.row} outside a table of {spec.rows}")
        self.spec, self.dtype = spec, dtype
        self.w = weights.device_tensor(spec.proj, dtype, device)
        self.row = weights.device_tensor(spec.table, dtype, device)[spec.row].contiguous()

    def forward(self, ctx, resid: torch.Tensor, delta, x0: torch.Tensor) -> None:
        T, H = resid.shape
        both = ctx.workspace.buffer("reentry_in", T, 2 * H, self.dtype)
        ops.concat_stream(both, resid, delta, x0)
        linear(both, self.w, resid)
        ops.add_bias(resid, self.row)
