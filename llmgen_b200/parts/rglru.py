"""A recurrent block around a real-gated linear recurrent unit: a mixer whose state lives in the cache manager's slots."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import register_mixer
from .spec import VECTOR, RGLRUSpec, WeightDecl


class RGLRU(Mixer):
    """One packed projection [y | x] -> the short convolution of the x branch (float32 out; the sequence's last inputs
    come from and go to the state) -> the two gates of every block of channels and the recurrence's coefficients ->
    the scan S = a S + b over each sequence's new tokens, times gelu_tanh of the y branch -> output projection
    (csrc/recurrent.cu).  The projection leaves in the storage dtype; biases, the convolution's sum, gates, decays and
    the state are float32.

    State of a request, one float32 row of the cache manager's slots: [S (width) | the convolution's last taps - 1
    inputs, oldest first (taps - 1 rows of width)].  The kernels read the step's lengths and slots from the device
    arrays; sequences without tokens and rows that belong to none are skipped, so any step may be replayed from the
    graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: RGLRUSpec):
        C, H, n = spec.width, spec.hidden_size, spec.width // max(spec.blocks, 1)
        decls = [WeightDecl(spec.y_proj, (C, H)), WeightDecl(spec.x_proj, (C, H)), WeightDecl(spec.o_proj, (H, C)),
                 WeightDecl(spec.conv.weight, (C, spec.conv.taps), VECTOR),
                 WeightDecl(spec.a_gate, (spec.blocks, n, n)), WeightDecl(spec.i_gate, (spec.blocks, n, n)),
                 WeightDecl(spec.lam, (C,), VECTOR)]
        for name, shape in ((spec.y_bias, (C,)), (spec.x_bias, (C,)), (spec.conv.bias, (C,)),
                            (spec.a_gate_bias, (spec.blocks, n)), (spec.i_gate_bias, (spec.blocks, n))):
            if name:
                decls.append(WeightDecl(name, shape, VECTOR))
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("recurrent",) + GEMM_MODULES

    def __init__(self, spec: RGLRUSpec, weights, dtype, device):
        if spec.blocks <= 0 or spec.width % spec.blocks != 0:
            raise ValueError(f"rglru: {spec.width} channels are not cut evenly into {spec.blocks} blocks")
        if spec.conv.channels != spec.width or not 1 <= spec.conv.taps <= 8:
            raise ValueError("rglru: the convolution runs over the branch's channels with 1 to 8 taps")
        self.spec, self.dtype = spec, dtype
        self.C, self.taps = spec.width, spec.conv.taps

        def vec(name):
            return weights.device_tensor(name, dtype, device).contiguous().view(-1) if name else None

        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in (spec.y_proj, spec.x_proj)], dim=0).contiguous()
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.w_a = weights.device_tensor(spec.a_gate, dtype, device).contiguous()
        self.w_i = weights.device_tensor(spec.i_gate, dtype, device).contiguous()
        self.conv_w = weights.device_tensor(spec.conv.weight, dtype, device).contiguous()
        self.conv_b, self.y_b, self.x_b = vec(spec.conv.bias), vec(spec.y_bias), vec(spec.x_bias)
        self.b_a, self.b_i, self.lam = vec(spec.a_gate_bias), vec(spec.i_gate_bias), vec(spec.lam)

    def state_request(self) -> StateRequest:
        return StateRequest((self.taps * self.C,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (self.C * (3 * elem + 12) + self.spec.hidden_size * elem) + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T, C, ws = ctx.n_tokens, self.C, ctx.workspace
        packed = linear(x, self.w_in, ws.buffer("rglru_in", T, 2 * C, self.dtype))
        u = ws.buffer("rglru_u", T, C, torch.float32)
        ops.short_conv(u, packed[:, C:], self.conv_w, cache.state[:, C:], ctx.cu_q, ctx.state_slots, ctx.n_seqs,
                       in_bias=self.x_b, conv_bias=self.conv_b)
        out = ws.buffer("rglru_out", T, C, self.dtype)
        rows = ops.rglru_scratch_rows(T, ctx.n_seqs, self.dtype)
        scratch = ws.buffer("rglru_coeffs", rows, C, torch.float32,
                            capacity_rows=ops.rglru_scratch_rows(ws.default_rows, max(ctx.max_seqs_bound, ctx.n_seqs), self.dtype))
        ops.rglru(out, scratch, u, self.w_a, self.w_i, self.b_a, self.b_i, self.lam, packed[:, :C], self.y_b, cache.state,
                  ctx.cu_q, ctx.state_slots, ctx.n_seqs, self.spec.blocks, float(self.spec.decay_scale))
        return linear_sliced(ws, "mixer_out", out, self.w_o, self.dtype)


register_mixer("rglru", RGLRU)
