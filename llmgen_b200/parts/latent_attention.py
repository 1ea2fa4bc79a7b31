"""Attention over a cached latent vector per token (multi-head latent attention), as a mixer."""
from __future__ import annotations

import torch

from ..cache.manager import FULL
from ..kernels import ops
from .attention import add_query_tiles
from .base import KVRequest, LayerCache, Mixer
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import build_position, norm_class, register_mixer
from .spec import LatentAttentionSpec, WeightDecl


class LatentAttention(Mixer):
    """One packed projection [dq | dkv | gate] -> `latent_prep` (the query latent's norm; the key/value latent's norm,
    the rotation of the shared key part and the write of [c | rotated part] to the paged cache) -> the query in the
    latent space: one product with Wuk folded into Wuq at load and `latent_rotate` (or, `absorb_at_load=False`,
    q = cq Wuq^T and `latent_absorb`: each head's unrotated query through Wuk, its rotated part turned) ->
    `latent_attention` over the cached vectors, one shared entry per token for all heads -> Wuv per head and the gate:
    in bfloat16 with sizes the tensor-core attention takes, the attention leaves its result head-major in bfloat16, one
    grouped tcgen05 product (a group per head) applies Wuv and `latent_gate` multiplies by sigmoid(gate); otherwise
    `latent_expand` does both on the CUDA cores -> output projection.  Keys and values of the context are never expanded: a page holds
    kv_rank + rope_dim values per token whatever the number of heads.

    Scores, softmax weights and their sums with the latents are float32 (csrc/latent_attention.cu); a step of single
    tokens cuts long contexts into key parts (flash-decoding) in a fixed order."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: LatentAttentionSpec):
        H, n = spec.hidden_size, spec.num_heads
        decls = [WeightDecl(spec.dq_proj, (spec.q_rank, H)), WeightDecl(spec.uq_proj, (n * (spec.nope_dim + spec.rope_dim), spec.q_rank)),
                 WeightDecl(spec.dkv_proj, (spec.kv_rank + spec.rope_dim, H)), WeightDecl(spec.uk_proj, (n * spec.nope_dim, spec.kv_rank)),
                 WeightDecl(spec.uv_proj, (n * spec.value_dim, spec.kv_rank)), WeightDecl(spec.o_proj, (H, n * spec.value_dim))]
        if spec.gate_proj:
            decls.append(WeightDecl(spec.gate_proj, (n * spec.value_dim, H)))
        for norm in (spec.q_norm, spec.kv_norm):
            decls += norm_class(norm).weight_decls(norm)
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("latent_attention", "rowwise") + GEMM_MODULES

    def __init__(self, spec: LatentAttentionSpec, weights, dtype, device):
        for norm, dim in ((spec.q_norm, spec.q_rank), (spec.kv_norm, spec.kv_rank)):
            if norm.kind != "rmsnorm" or norm.dim != dim or norm.weight_offset != 0.0:
                raise ValueError("latent attention: the latents' norms are plain RMSNorms over the whole latent")
        if spec.q_norm.eps != spec.kv_norm.eps:
            raise ValueError("latent attention: both latent norms must share eps")
        if spec.rope_dim % 2 != 0 or (spec.position is not None and spec.position.rotary_dim != spec.rope_dim):
            raise ValueError("latent attention: the position encoding turns the whole rotated part, an even number of values")
        if spec.kv_rank > 512:
            raise ValueError(f"latent attention: kv_rank {spec.kv_rank} is more than 512")
        self.spec, self.dtype = spec, dtype
        self.heads, self.nope, self.rope, self.vd = spec.num_heads, spec.nope_dim, spec.rope_dim, spec.value_dim
        self.q_rank, self.kv_rank = spec.q_rank, spec.kv_rank
        names = [spec.dq_proj, spec.dkv_proj] + ([spec.gate_proj] if spec.gate_proj else [])
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.dkv_off = self.q_rank
        self.g_off = self.q_rank + self.kv_rank + self.rope
        self.w_uq = weights.device_tensor(spec.uq_proj, dtype, device, keep=not spec.absorb_at_load)
        self.w_uk = weights.device_tensor(spec.uk_proj, dtype, device, keep=not spec.absorb_at_load)
        self.w_qa = None
        if spec.absorb_at_load:
            # q' = [Wuk_h^T (Wuq_h,unrotated cq) | Wuq_h,rotated cq] = W_qa cq: the products of the two matrices in
            # float32, stacked head by head in the layout the attention reads, rounded once to the storage dtype
            n, d, r = self.heads, self.nope, self.rope
            uq = self.w_uq.float().view(n, d + r, self.q_rank)
            uk = self.w_uk.float().view(n, d, self.kv_rank)
            folded = torch.einsum("hdc,hdq->hcq", uk, uq[:, :d])
            self.w_qa = torch.cat([folded, uq[:, d:]], dim=1).reshape(n * (self.kv_rank + r), self.q_rank).to(dtype).contiguous()
            self.w_uq = self.w_uk = None
        self.w_uv = weights.device_tensor(spec.uv_proj, dtype, device)
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.q_gain = weights.device_tensor(spec.q_norm.weight, dtype, device)
        self.kv_gain = weights.device_tensor(spec.kv_norm.weight, dtype, device)
        self.eps = float(spec.q_norm.eps)
        self.position = build_position(spec.position, weights, dtype, device) if spec.position is not None and self.rope else None
        self.pairing = getattr(self.position, "pairing", "half") if self.position is not None else "half"
        self.bq = ops.latent_attention_tile_queries(self.heads)
        self.sm_count = ops.sm_count(device)
        # bfloat16 caches whose sizes fit leave the attention head-major in bfloat16, and Wuv runs as one grouped tensor-core
        # product over all heads (a group per head); the list of the tiles' heads is made once per padded token count
        self.grouped_expand = (ops.latent_attention_on_tensor_cores(dtype, self.kv_rank, self.rope) and self.vd % 8 == 0)
        self._head_of_tile = {}
        self.device = device

    def cache_request(self) -> KVRequest:
        return KVRequest(FULL, 0, 1, self.kv_rank + self.rope, values=False)

    def max_positions(self):
        return self.position.max_positions if self.position is not None else None

    def step_arrays_key(self):
        return ("attention_tiles", self.bq)

    def prepare_step(self, builder) -> None:
        add_query_tiles(builder, self.bq)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        n = self.heads
        per_token = (self.w_in.shape[0] + self.q_rank + n * (self.nope + self.rope) + n * self.vd + self.spec.hidden_size) * elem \
            + 4 * n * (2 * self.kv_rank + self.rope)
        return tokens * per_token + ops.SLICED_PRODUCT_BYTES

    def _parts(self, ctx) -> int:
        """Key parts of a step of single tokens: two blocks an SM, at least 128 keys a part (four tiles of the kernel), at
        most 32 parts; every sequence's own keys are cut evenly, so the bound of the step's context class decides."""
        if not ctx.pure_decode:
            return 1
        blocks = max(1, ctx.n_seqs * ((self.heads + 31) // 32))
        longest = max(ctx.max_ctx_bound, ctx.max_ctx, 1)
        return max(1, min((2 * self.sm_count) // blocks, longest // 128, 32))

    def forward(self, ctx, x, cache: LayerCache):
        T = ctx.n_tokens
        ws = ctx.workspace
        n, za = self.heads, self.kv_rank + self.rope
        group = ctx.groups[cache.group]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        packed = linear(x, self.w_in, ws.buffer("latent_in", T, self.w_in.shape[0], self.dtype))
        cq = ws.buffer("latent_cq", T, self.q_rank, self.dtype)
        ops.latent_prep(packed, 0, self.dkv_off, self.q_rank, self.kv_rank, self.rope, self.q_gain, self.kv_gain, self.eps, cq,
                        cache.k if cache.writes else None, ctx.positions, group.slots, cos, sin, self.pairing)
        qa = ws.buffer("latent_qa", T, n * za, torch.float32)
        if self.w_qa is not None:
            linear(cq, self.w_qa, qa)
            if self.rope:
                ops.latent_rotate(qa, ctx.positions, cos, sin, n, self.kv_rank, self.rope, self.pairing)
        else:
            q = linear(cq, self.w_uq, ws.buffer("latent_q", T, n * (self.nope + self.rope), self.dtype))
            ops.latent_absorb(qa, q, self.w_uk, ctx.positions, cos, sin, n, self.nope, self.rope, self.kv_rank, self.pairing)
        name = f"attention_tiles_bq{self.bq}"
        parts = self._parts(ctx)
        scratch = None
        if parts > 1:
            scratch = ws.flat("latent_split", ops.latent_attention_scratch_floats(T, n, self.kv_rank, parts), torch.float32)
        gate = packed[:, self.g_off:] if self.spec.gate_proj else None
        y = ws.buffer("latent_y", T, n * self.vd, self.dtype)
        if self.grouped_expand:
            t_pad = (T + ops.MOE_GROUPED_TILE - 1) // ops.MOE_GROUPED_TILE * ops.MOE_GROUPED_TILE
            cap = (ws.default_rows + ops.MOE_GROUPED_TILE - 1) // ops.MOE_GROUPED_TILE * ops.MOE_GROUPED_TILE * n
            oa_hm = ws.buffer("latent_oa_hm", n * t_pad, self.kv_rank, self.dtype, capacity_rows=cap)
            ops.latent_attention(None, qa, cache.k, group.block_tables, group.max_blocks, ctx.ctx_len, ctx.cu_q, ctx.array(name + "_seq"),
                                 ctx.array(name + "_q0"), T, n, self.kv_rank, self.rope, cache.page_size, float(self.spec.scale), parts,
                                 scratch, out_head_major=oa_hm.view(n, t_pad, self.kv_rank))
            o_hm = ws.buffer("latent_o_hm", n * t_pad, self.vd, torch.float32, capacity_rows=cap)
            ops.gemm_tc_grouped(o_hm, oa_hm, self.w_uv.view(n, self.vd, self.kv_rank), self._tile_heads(t_pad), real_rows=n * T)
            ops.latent_gate(y, o_hm, gate, n, self.vd, t_pad)
        else:
            oa = ws.buffer("latent_oa", T, n * self.kv_rank, torch.float32)
            ops.latent_attention(oa, qa, cache.k, group.block_tables, group.max_blocks, ctx.ctx_len, ctx.cu_q, ctx.array(name + "_seq"),
                                 ctx.array(name + "_q0"), T, n, self.kv_rank, self.rope, cache.page_size, float(self.spec.scale), parts,
                                 scratch)
            ops.latent_expand(y, oa, self.w_uv, gate, n, self.kv_rank, self.vd)
        return linear_sliced(ws, "mixer_out", y, self.w_o, self.dtype)

    def _tile_heads(self, t_pad: int) -> torch.Tensor:
        """int32 [heads * t_pad / 128] on the device: the head of every 128-row tile of the head-major rows."""
        tiles = self._head_of_tile.get(t_pad)
        if tiles is None:
            per_head = t_pad // ops.MOE_GROUPED_TILE
            tiles = torch.arange(self.heads, dtype=torch.int32).repeat_interleave(per_head).to(self.device)
            self._head_of_tile[t_pad] = tiles
        return tiles


register_mixer("latent_attention", LatentAttention)
