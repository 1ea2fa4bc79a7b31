"""A plain, slow implementation of the Sarulix decoder: whole sequences, no cache, no state carried between calls,
one function per mechanism, float64 (or float32) on the CPU.  It shares no code with `llmgen_b200`: tensors come in
as a dict, the configuration as the parsed config.json.

Notation: h is a sublayer's input [T, width]; W_x is the tensor `<layer>.mix.x` or `<layer>.mlp.x`, stored [out, in]
and applied as h W^T.  N(x, g) = x / sqrt(mean(x^2) + eps) * g.

    embedding      x0 = embed[id] * scale
    layer          x <- x + mixer(N(x, 1 + w1));  x <- x + ff(N(x, 1 + w2))  (the second only where the layer has a ff)
    loop           layers [start, stop) run `times` times with the same weights; before pass t:
                   x <- [x | x0] Win^T + step[t]
    attention      q, k, v with biases; per head N(q, gq), N(k, gk); the first `dims` values of a head turned, value i
                   with value i + dims/2, by the angle pos * base^(-2i/dims); s = cap tanh(q.k scale / cap);
                   p_j = exp(s_j) / (1 + sum_j' exp(s_j')) over j <= i; (concat heads * sigmoid(h Wg^T)) Wo^T + bo
    rglru          y = gelu(h Wy^T + by); u = conv(h Wx^T + bx) + bc; per block b of channels: r = sigmoid(Ra_b u_b + ba_b),
                   i = sigmoid(Ri_b u_b + bi_b); a = exp(-8 r softplus(lam)); S_t = a S_(t-1) + sqrt(1 - a^2) i u;
                   (S * y) Wo^T
    channel_delta  q, k, v = silu(conv(h W^T)); q, k unit vectors per head (q also / sqrt(dim)); beta = sigmoid(h Wb^T);
                   g = exp(-exp(A_log_head) softplus(h Wa1^T Wa2^T + dt_bias))  [heads, dim];
                   S <- diag(g) S; d = beta (v - S^T k); S <- S + k d^T; o = S^T q;
                   (N_head(o, gn) * sigmoid(h Wg1^T Wg2^T)) Wo^T
    ff             (gelu(h Wgate^T) * (h Wup^T)) Wdown^T
    logits         N(x, 1 + wf) head^T * logit_scale
    gelu(z)        0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

RGLRU_C = 8.0
UNIT_EPS = 1e-6


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half_pairs(x: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """x [T, heads, >= dims]: value i of a head turned together with value i + dims/2."""
    out = x.clone()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = float(p) * float(base) ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], taps [C, K]: out_t = sum_j taps[:, j] x_(t - (K-1) + j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1) + j
            if src >= 0:
                out[t] += taps[:, j] * x[src]
    if bias is not None:
        out = out + bias
    return out


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: float) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e]; causal; one more term of score 0 and no value in the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        for i in range(T):
            e = torch.exp(s[i, :i + 1])
            out[i, h] = (e / (1.0 + e.sum())) @ v[:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t() + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].t() + w[p + "k.b"]).view(T, G, D)
    v = (h @ w[p + "v"].t() + w[p + "v.b"]).view(T, G, E)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_half_pairs(q, positions, rot["base"], rot["dims"])
        k = rotate_half_pairs(k, positions, rot["base"], rot["dims"])
    o = sink_softmax_attention(q, k, v, m["scale"], float(m.get("softcap") or 0.0))
    o = o.reshape(T, H * E) * sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t() + w[p + "o.b"]


def rglru_scan(u: torch.Tensor, r: torch.Tensor, i: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-8 r_t softplus(lam)), S_(-1) = 0."""
    T, C = u.shape
    S = torch.zeros(C, dtype=u.dtype)
    out = torch.zeros_like(u)
    sp = softplus(lam)
    for t in range(T):
        a = torch.exp(-RGLRU_C * r[t] * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * i[t] * u[t]
        out[t] = S
    return out


def rglru_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].t() + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].t() + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.view(T, B, C // B)
    r = sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, C)
    i = sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, C)
    S = rglru_scan(u, r, i, w[p + "lam"])
    return (S * y) @ w[p + "o"].t()


def gated_delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """q, k [T, G, d] (unit vectors, q scaled), v [T, H, e], beta [T, H], g [T, H, d] -> o [T, H, e]."""
    T, H, E = v.shape
    G, D = k.shape[1], k.shape[2]
    out = torch.zeros(T, H, E, dtype=v.dtype)
    for h in range(H):
        kv = h // (H // G)
        S = torch.zeros(D, E, dtype=v.dtype)
        for t in range(T):
            S = g[t, h][:, None] * S
            d = beta[t, h] * (v[t, h] - S.t() @ k[t, kv])
            S = S + k[t, kv][:, None] * d[None, :]
            out[t, h] = S.t() @ q[t, kv]
    return out


def channel_delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].t(), w[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[p + "k"].t(), w[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[p + "v"].t(), w[p + "v.conv"])).view(T, H, E)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + UNIT_EPS) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + UNIT_EPS)
    beta = sigmoid(h @ w[p + "b"].t())
    dt = softplus((h @ w[p + "a1"].t()) @ w[p + "a2"].t() + w[p + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    o = gated_delta_scan(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps)
    gate = sigmoid((h @ w[p + "g1"].t()) @ w[p + "g2"].t()).view(T, H, E)
    return (o * gate).reshape(T, H * E) @ w[p + "o"].t()


def gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def layer_forward(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, layer: dict, eps: float, positions) -> torch.Tensor:
    p = f"l{i}."
    h = rms_norm(x, 1.0 + w[p + "norm1"], eps)
    kind = layer["type"]
    if kind == "attention":
        x = x + attention_mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
    elif kind == "rglru":
        x = x + rglru_mixer(h, w, p + "mix.", layer["mixer"])
    elif kind == "channel_delta":
        x = x + channel_delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
    else:
        raise ValueError(f"unknown layer type {kind!r}")
    if layer.get("mlp") is not None:
        x = x + gated_ff(rms_norm(x, 1.0 + w[p + "norm2"], eps), w, p + "mlp.")
    return x


def run_list(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, pass number if the layer is the first of a loop's pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64):
    """(logits [T, vocab], the residual stream after every layer run [runs, T, width])."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    positions = list(range(len(ids)))
    x0 = w["embed"][torch.as_tensor(list(ids), dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0
    after = []
    for i, first_of_pass in run_list(cfg):
        if first_of_pass is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].t() + w["loop.step"][first_of_pass]
        x = layer_forward(x, w, i, cfg["layers"][i], eps, positions)
        after.append(x)
    logits = rms_norm(x, 1.0 + w["final.norm"], eps) @ w["head"].t() * cfg.get("logit_scale", 1.0)
    return logits, torch.stack(after)
