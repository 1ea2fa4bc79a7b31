"""Feed-forwards of layers other than the gated dense one: a dense one without a gate, and a mixture of experts."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import register_feed_forward
from .spec import ClampedExpertSpec, DenseMLPSpec, RoutedMLPSpec, WeightDecl


class DenseMLP(FeedForward):
    """down( act(x Wup^T) ), act = relu(.)^2: two products and one row-wise kernel between them, which also adds up the
    float32 slices when the first product was cut along K."""

    @staticmethod
    def weight_decls(spec: DenseMLPSpec):
        return [WeightDecl(spec.up_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.down_proj, (spec.hidden_size, spec.intermediate_size))]

    @staticmethod
    def kernel_modules(spec):
        return ("rowwise",) + GEMM_MODULES

    def __init__(self, spec: DenseMLPSpec, weights, dtype, device):
        if spec.activation not in ops.ACTIVATIONS or spec.activation == "clamped_glu":
            raise ValueError(f"dense feed-forward: activation {spec.activation!r} is not supported")
        self.spec, self.dtype = spec, dtype
        self.w_up = weights.device_tensor(spec.up_proj, dtype, device)
        self.w_down = weights.device_tensor(spec.down_proj, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (2 * self.spec.intermediate_size + self.spec.hidden_size) * elem + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x):
        T, F = x.shape[0], self.spec.intermediate_size
        ws = ctx.workspace
        up = linear_sliced(ws, "ffn_up", x, self.w_up, self.dtype)
        act = ws.buffer("ffn_act", T, F, self.dtype)
        ops.act_rows(act, up, self.spec.activation)
        return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype)


def _expert_decls(e: ClampedExpertSpec, hidden: int):
    return [WeightDecl(e.gate_proj, (e.intermediate_size, hidden)), WeightDecl(e.up_proj, (e.intermediate_size, hidden)),
            WeightDecl(e.down_proj, (hidden, e.intermediate_size))]


class RoutedMLP(FeedForward):
    """Mixture of experts whose every launch has a shape that follows from (tokens, experts, top) alone: no result is
    read back on the host, so a step holding it is recorded into a CUDA graph like any other.

    `moe_route` scores each token in float32 against the float32 router and keeps its `top` experts; `moe_plan` groups
    the (token, choice) slots by expert into tiles of 16 rows (a list of fixed length, padded); `moe_experts` runs the
    first product with the clamped gated activation and then the down product tile by tile, each tile reading its
    expert's matrices (stacked [experts, ...] at load); `moe_combine` adds a token's rows in slot order to the shared
    expert's output.  The shared expert is two of the framework's own products with the same activation between them.
    The routed products sum in float32 on the CUDA cores (csrc/moe.cu)."""

    step_arrays_follow_shapes = True

    @staticmethod
    def weight_decls(spec: RoutedMLPSpec):
        decls = [WeightDecl(spec.router, (len(spec.experts), spec.hidden_size))]
        for e in spec.experts:
            decls += _expert_decls(e, spec.hidden_size)
        if spec.shared is not None:
            decls += _expert_decls(spec.shared, spec.hidden_size)
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("moe", "rowwise") + GEMM_MODULES

    def __init__(self, spec: RoutedMLPSpec, weights, dtype, device):
        first = spec.experts[0]
        if any((e.intermediate_size, e.limit, e.alpha) != (first.intermediate_size, first.limit, first.alpha) for e in spec.experts):
            raise ValueError("routed feed-forward: all routed experts share one size, limit and alpha")
        if not 0 < spec.top_k <= len(spec.experts):
            raise ValueError(f"routed feed-forward: top {spec.top_k} of {len(spec.experts)} experts")
        if spec.scoring not in ops.ROUTER_SCORINGS:
            raise ValueError(f"routed feed-forward: scoring {spec.scoring!r} is not supported")
        self.spec, self.dtype = spec, dtype
        self.E, self.top, self.F = len(spec.experts), spec.top_k, first.intermediate_size
        self.router = weights.device_tensor(spec.router, torch.float32, device)      # routing is float32 in both dtypes
        stack = lambda names: torch.stack([weights.device_tensor(n, dtype, device, keep=False) for n in names]).contiguous()
        self.w_gate = stack([e.gate_proj for e in spec.experts])     # [E, F, H]
        self.w_up = stack([e.up_proj for e in spec.experts])         # [E, F, H]
        self.w_down = stack([e.down_proj for e in spec.experts])     # [E, H, F]
        self.shared_gate_up = self.shared_down = None
        if spec.shared is not None:
            self.shared_gate_up = torch.cat([weights.device_tensor(spec.shared.gate_proj, dtype, device, keep=False),
                                             weights.device_tensor(spec.shared.up_proj, dtype, device, keep=False)], dim=0).contiguous()
            self.shared_down = weights.device_tensor(spec.shared.down_proj, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        H = self.spec.hidden_size
        slots = tokens * self.top
        shared = tokens * (3 * self.spec.shared.intermediate_size + H) * elem if self.spec.shared is not None else 0
        return slots * (self.F + H) * 4 + tokens * H * 4 + shared + 16 * (slots + self.E) + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x):
        T, H = x.shape
        ws = ctx.workspace
        spec, top = self.spec, self.top
        n_slots = T * top
        tiles = ops.moe_max_tiles(n_slots, self.E)
        ints = ws.flat("moe_ints", 3 * n_slots + 3 * tiles, torch.int32)
        slot_expert, order, pos_of_slot = ints[:n_slots], ints[n_slots:2 * n_slots], ints[2 * n_slots:3 * n_slots]
        tile_expert, tile_start, tile_rows = (ints[3 * n_slots + i * tiles:3 * n_slots + (i + 1) * tiles] for i in range(3))
        slot_weight = ws.flat("moe_weights", n_slots, torch.float32)
        ops.moe_route(x, self.router, slot_expert, slot_weight, top, spec.scoring, spec.renormalize)
        ops.moe_plan(slot_expert, n_slots, self.E, order, pos_of_slot, tile_expert, tile_start, tile_rows)
        first = spec.experts[0]
        y = ws.buffer("moe_act", n_slots, self.F, torch.float32, capacity_rows=ws.default_rows * top)
        ops.moe_experts(y, x, self.w_gate, self.w_up, order, slot_weight, tile_expert, tile_start, tile_rows, n_slots, top,
                        first=True, weight_on_input=spec.weight_on_input, alpha=first.alpha, limit=first.limit)
        rows = ws.buffer("moe_rows", n_slots, H, torch.float32, capacity_rows=ws.default_rows * top)
        ops.moe_experts(rows, y, self.w_down, None, order, slot_weight, tile_expert, tile_start, tile_rows, n_slots, top,
                        first=False, weight_on_input=spec.weight_on_input)
        shared_out = None
        if spec.shared is not None:
            Fs = spec.shared.intermediate_size
            gate_up = linear_sliced(ws, "moe_shared_gate_up", x, self.shared_gate_up, self.dtype)
            act = ws.buffer("moe_shared_act", T, Fs, self.dtype)
            ops.act_rows(act, gate_up, "clamped_glu", alpha=spec.shared.alpha, limit=spec.shared.limit)
            shared_out = linear(act, self.shared_down, ws.buffer("moe_shared_out", T, H, self.dtype))
        out = ws.flat("moe_out", T * H, torch.float32).view(1, T, H)
        ops.moe_combine(out[0], rows, pos_of_slot, shared_out, top)
        return ops.Partials(out)


register_feed_forward("dense_mlp", DenseMLP)
register_feed_forward("routed_mlp", RoutedMLP)
