"""Derupel: from its typed configuration to a `ModelSpec`.

A decoder whose layers norm each sublayer's OUTPUT before it joins the residual stream (`PostNormBlockSpec`) and pick,
layer by layer, one of two mixers and one of three feed-forwards:

    mixer "lightning"          `LinearAttentionSpec`: silu on q, k, v; a decay per head; RMSNorm over the heads side by
                               side, times sigmoid(gate)
    mixer "latent_attention"   `LatentAttentionSpec`: queries and keys/values through normed latents, one rotated key
                               part shared by the heads (pairs (2i, 2i + 1)), an output gate
    mlp null | dense | moe     none | `DenseMLPSpec` (relu squared) | `RoutedMLPSpec` (sigmoid scores, the weight on the
                               expert's input, not renormalised, clamped gated experts, an optional shared expert)

Tensor names of a model folder (layer i):

    embed [vocab, width]; final.norm [width]; head [vocab, width]
    l<i>.norm1, l<i>.norm2 [width]
    l<i>.mix.{q,k,v,g,o,norm}                               lightning
    l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}         latent attention
    l<i>.mlp.{up,down}                                      dense
    l<i>.mlp.router, l<i>.mlp.e<j>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down}       moe

Fixed by the architecture, not by its config.json: the gated experts' alpha 1.702, causal attention without a window,
the embedding rows multiplied by `embedding.scale`, no biases, an untied output matrix.
"""
from __future__ import annotations

from ..config.derupel import DENSE, LIGHTNING, MOE, DerupelConfig
from ..parts.spec import (ClampedExpertSpec, DenseMLPSpec, LatentAttentionSpec, LinearAttentionSpec, ModelSpec,
                          PostNormBlockSpec, RMSNormSpec, RopeSpec, RoutedMLPSpec, default_run_order)
from ..registry import register_architecture

EXPERT_ALPHA = 1.702


def _expert(prefix: str, cfg) -> ClampedExpertSpec:
    return ClampedExpertSpec(cfg.ff, cfg.limit, prefix + "gate", prefix + "up", prefix + "down", alpha=EXPERT_ALPHA)


def build_derupel_spec(cfg: DerupelConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == LIGHTNING:
            mixer = LinearAttentionSpec(
                hidden_size=W, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, decay=m.decay,
                q_proj=p + "mix.q", k_proj=p + "mix.k", v_proj=p + "mix.v", o_proj=p + "mix.o", gate_proj=p + "mix.g",
                out_norm=RMSNormSpec(m.heads * m.vdim, eps, p + "mix.norm"), activation="silu")
        else:
            rope = RopeSpec(rotary_dim=m.rot_dims, theta=m.rot_base, max_positions=cfg.max_positions,
                            pairing="interleaved") if m.rot_dim else None
            mixer = LatentAttentionSpec(
                hidden_size=W, num_heads=m.heads, nope_dim=m.dim, rope_dim=m.rot_dim, value_dim=m.vdim, q_rank=m.q_rank,
                kv_rank=m.kv_rank, scale=m.scale, dq_proj=p + "mix.dq", uq_proj=p + "mix.uq", dkv_proj=p + "mix.dkv",
                uk_proj=p + "mix.uk", uv_proj=p + "mix.uv", o_proj=p + "mix.o",
                q_norm=RMSNormSpec(m.q_rank, eps, p + "mix.dq.norm"), kv_norm=RMSNormSpec(m.kv_rank, eps, p + "mix.dkv.norm"),
                position=rope, gate_proj=p + "mix.g")
        ffn = None
        if layer.mlp is not None and layer.mlp.kind == DENSE:
            ffn = DenseMLPSpec(W, layer.mlp.ff, p + "mlp.up", p + "mlp.down", activation="relu2")
        elif layer.mlp is not None and layer.mlp.kind == MOE:
            f = layer.mlp
            ffn = RoutedMLPSpec(
                hidden_size=W, router=p + "mlp.router",
                experts=tuple(_expert(f"{p}mlp.e{j}.", f.expert) for j in range(f.experts)), top_k=f.top,
                shared=_expert(p + "mlp.shared.", f.shared) if f.shared is not None else None,
                scoring="sigmoid", renormalize=False, weight_on_input=True)
        layers.append(PostNormBlockSpec(
            mixer_norm=RMSNormSpec(W, eps, p + "norm1"), mixer=mixer,
            ffn_norm=RMSNormSpec(W, eps, p + "norm2") if ffn is not None else None, ffn=ffn))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding="embed", layers=tuple(layers),
        run_order=default_run_order(len(layers)), final_norm=RMSNormSpec(W, eps, "final.norm"), lm_head="head",
        max_positions=cfg.max_positions, embedding_scale=cfg.embedding_scale,
        # a layer without a feed-forward has no use for a second norm; a folder may carry one all the same
        ignorable_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None))


register_architecture("Derupel", DerupelConfig, build_derupel_spec, aliases=("derupel",))
