"""A plain, slow implementation of the Derupel decoder: whole sequences, no cache, no state carried
between calls, one function per mechanism, float64 (or float32) on the CPU.  It shares no code with
`llmgen_b200`: tensors come in as a dict, the configuration as the parsed config.json.

Notation: h is a sublayer's input [T, width]; W_x is the tensor `<layer>.mix.x` or `<layer>.mlp.x`,
stored [out, in] and applied as h W^T.

    layer          x <- x + N1(mixer(x));  x <- x + N2(ff(x))    (the norm sits on the sublayer's output)
    N(y)           y / sqrt(mean(y^2) + eps) * gain
    lightning      q = silu(h Wq^T), k = silu(h Wk^T), v = silu(h Wv^T), per head
                   S_t = lambda_head S_(t-1) + k_t (x) v_t,  o_t = S_t^T q_t,  S_(-1) = 0
                   y = (N(concat heads o) * sigmoid(h Wg^T)) Wo^T
    latent         cq = N(h Wdq^T), q = cq Wuq^T  -> per head [dim | rot_dim]
                   (c_raw | kr) = h Wdkv^T, c = N(c_raw); per head kn = c Wuk^T, v = c Wuv^T
                   score_ij = (qn_i . kn_j + R(qr_i, i) . R(kr_j, j)) * scale, j <= i, softmax over j
                   y = (concat heads (sum_j p_ij v_j) * sigmoid(h Wg^T)) Wo^T
    R(u, p)        pairs (2i, 2i+1) turned by the angle p * base^(-2i / dims)
    dense ff       relu(h Wup^T)^2 Wdown^T
    expert(h)      g = min(h Wgate^T, L), u = clamp(h Wup^T, -L, L), (g sigmoid(1.702 g) (u + 1)) Wdown^T
    routed ff      s = sigmoid(h Wrouter^T); the `top` largest s choose experts; sum_e expert_e(s_e h) + shared(h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import torch


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """x [T, ..., >= dims]: the first `dims` values of the last axis turned pair by pair, (2i, 2i+1) by the angle
    position * base^(-2i / dims); the rest passes unchanged."""
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = float(p) * float(base) ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * c - v * s
            out[t, ..., 2 * i + 1] = v * c + u * s
    return out


def decayed_outer_product_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: Sequence[float],
                               state: torch.Tensor = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k [T, heads, dim], v [T, heads, vdim]; token by token S = decay_head * S + k (x) v, o = S^T q.
    Returns (o [T, heads, vdim], final S [heads, dim, vdim])."""
    T, H, D = q.shape
    E = v.shape[-1]
    S = torch.zeros(H, D, E, dtype=q.dtype) if state is None else state.clone()
    lam = torch.tensor(list(decay), dtype=q.dtype)[:, None, None]
    out = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        S = lam * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out, S


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].t()).view(T, H, D)
    k = silu(h @ w[p + "k"].t()).view(T, H, D)
    v = silu(h @ w[p + "v"].t()).view(T, H, E)
    o, _ = decayed_outer_product_scan(q, k, v, m["decay"])
    o = rms_norm(o.reshape(T, H * E), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def causal_softmax_attention(scores: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """scores [heads, T, T] (already scaled), v [T, heads, vdim]: row i sees columns j <= i."""
    H, T, _ = scores.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=v.dtype)
    for i in range(T):
        s = scores[:, i, : i + 1]
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        p = p / p.sum(dim=-1, keepdim=True)
        out[i] = torch.einsum("hj,jhe->he", p, v[: i + 1])
    return out


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                           positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, E, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    cq = rms_norm(h @ w[p + "dq"].t(), w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].t()).view(T, H, D + R)
    qn, qr = q[..., :D], rotate_pairs(q[..., D:], positions, rot["base"], rot["dims"])
    dkv = h @ w[p + "dkv"].t()
    c = rms_norm(dkv[:, :C], w[p + "dkv.norm"], eps)
    kr = rotate_pairs(dkv[:, C:], positions, rot["base"], rot["dims"])          # [T, R], one for all heads
    kn = (c @ w[p + "uk"].t()).view(T, H, D)
    v = (c @ w[p + "uv"].t()).view(T, H, E)
    scores = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    o = causal_softmax_attention(scores, v).reshape(T, H * E)
    o = o * sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    a = torch.relu(h @ w[p + "up"].t())
    return (a * a) @ w[p + "down"].t()


def clamped_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].t(), max=limit)
    u = torch.clamp(h @ w[p + "up"].t(), min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].t()


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    scores = sigmoid(h @ w[p + "router"].t())                    # [T, experts]
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(scores.shape[1]), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in chosen:
            out[t] += clamped_expert(scores[t, e] * h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64,
            start: int = 0) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """(logits [T, vocab], the residual stream after every layer) of one whole sequence whose first token sits at
    position `start` (with nothing before it)."""
    w = {k: v.to(dtype) for k, v in tensors.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    positions = list(range(start, start + len(ids)))
    x = w["embed"][torch.as_tensor(list(ids), dtype=torch.long)] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "lightning":
            y = lightning_mixer(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(x, w, p + "mix.", layer["mixer"], eps, positions)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + rms_norm(y, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, w, p + "mlp.", mlp)
            x = x + rms_norm(y, w[p + "norm2"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].t()
    return logits, after
