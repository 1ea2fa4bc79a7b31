"""Linear attention with a per-head decay: a recurrent mixer whose state lives in the cache manager's state slots."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import norm_class, register_mixer
from .spec import LinearAttentionSpec, WeightDecl


class LinearAttention(Mixer):
    """One packed projection [q | k | v | gate] -> the decayed outer-product recurrence over each sequence's new tokens,
    reading and writing the request's float32 state [heads, key_dim, value_dim] (csrc/linear_attention.cu: prompts in
    chunks, a decoded token as a chunk of one, the tokens of a long step in segments that run side by side) -> RMSNorm over the heads side by side times sigmoid(gate), one kernel
    -> output projection.  q, k and v leave the product in the storage dtype; their activation, the recurrence, the
    norm and the gate are float32.

    The kernel reads the step's lengths and state slots from the device arrays, one block per (sequence, head, 32
    value columns); sequences without tokens and rows that belong to none are skipped, so any step may be replayed
    from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: LinearAttentionSpec):
        kd, vd, H = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.hidden_size
        decls = [WeightDecl(spec.q_proj, (kd, H)), WeightDecl(spec.k_proj, (kd, H)), WeightDecl(spec.v_proj, (vd, H)),
                 WeightDecl(spec.o_proj, (H, vd))]
        if spec.gate_proj:
            decls.append(WeightDecl(spec.gate_proj, (vd, H)))
        if spec.out_norm is not None:
            decls += norm_class(spec.out_norm).weight_decls(spec.out_norm)
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("linear_attention", "rowwise") + GEMM_MODULES

    def __init__(self, spec: LinearAttentionSpec, weights, dtype, device):
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"linear attention: {len(spec.decay)} decay factors for {spec.num_heads} heads")
        if spec.activation not in ("silu", "none"):
            raise ValueError(f"linear attention: activation {spec.activation!r} is not supported")
        if spec.out_norm is not None and (spec.out_norm.kind != "rmsnorm" or spec.out_norm.dim != spec.num_heads * spec.value_dim
                                          or spec.out_norm.weight_offset != 0.0):
            raise ValueError("linear attention: the output norm is a plain RMSNorm over all heads' values")
        if spec.out_norm is not None and not spec.gate_proj:
            raise ValueError("linear attention: an output norm without a gate is not built")
        self.spec, self.dtype = spec, dtype
        self.heads, self.kd, self.vd = spec.num_heads, spec.key_dim, spec.value_dim
        names = [spec.q_proj, spec.k_proj, spec.v_proj] + ([spec.gate_proj] if spec.gate_proj else [])
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.decay = torch.tensor(list(spec.decay), dtype=torch.float32, device=device)
        self.norm_gain = weights.device_tensor(spec.out_norm.weight, dtype, device) if spec.out_norm is not None else None
        self.norm_eps = float(spec.out_norm.eps) if spec.out_norm is not None else 0.0
        self.k_off = self.heads * self.kd
        self.v_off = 2 * self.heads * self.kd
        self.g_off = self.v_off + self.heads * self.vd

    def state_request(self) -> StateRequest:
        return StateRequest((self.heads, self.kd, self.vd), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        wide = self.heads * self.vd
        return tokens * (self.w_in.shape[0] * elem + wide * (4 + elem) + self.spec.hidden_size * elem) + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T = ctx.n_tokens
        ws = ctx.workspace
        wide = self.heads * self.vd
        packed = linear(x, self.w_in, ws.buffer("linattn_in", T, self.w_in.shape[0], self.dtype))
        o = ws.buffer("linattn_o", T, wide, torch.float32)
        need = ops.linear_attention_scratch_floats(T, ctx.n_seqs, self.heads, self.kd, self.vd)
        scratch = ws.flat("linattn_segments", need, torch.float32) if need else None
        ops.linear_attention(o, packed, 0, self.k_off, self.v_off, cache.state, self.decay, ctx.cu_q, ctx.state_slots,
                             ctx.n_seqs, self.heads, self.kd, self.vd, silu=self.spec.activation == "silu", scratch=scratch)
        y = ws.buffer("linattn_y", T, wide, self.dtype)
        if self.spec.gate_proj:
            ops.gated_rmsnorm(y, o, packed[:, self.g_off:], self.norm_gain, self.norm_eps)
        else:
            ops.cast_rows(y, o)
        return linear_sliced(ws, "mixer_out", y, self.w_o, self.dtype)


register_mixer("linear_attention", LinearAttention)
