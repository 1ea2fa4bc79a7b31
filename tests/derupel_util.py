"""Small Derupel configurations with random weights, for the tests: the engine's model and the tensors the plain
implementation reads, made from one seed."""
from __future__ import annotations

import copy
from typing import Dict, List, Sequence

import torch


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mlp):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def config(layers, width=64, vocab=97, scale=3.0, eps=1e-5) -> dict:
    return {"architecture": "Derupel", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": copy.deepcopy(list(layers))}


# Every kind of layer once, sizes that differ from one another wherever they can: heads 2 / 3, key width != value width,
# top 2 of 5 with a shared expert and top 1 of 3 without, a layer without a feed-forward, a head that never forgets
# (decay 1) beside one that forgets fast.
MIXED = config([
    lightning(2, 16, 24, (0.9, 1.0), dense(80)),
    latent(3, 16, 8, 24, 40, 32, 0.2, 100.0, moe(5, 2, 24, 0.8, shared=(32, 1.2))),
    latent(2, 8, 16, 16, 24, 48, 0.35, 5000.0, None),
    lightning(3, 40, 48, (0.5, 0.97, 0.999), moe(3, 1, 16, 2.0)),
])
# More heads than one block of the attention kernel takes rows (17 > 16), a key width that needs the widest state
# registers' next size, 3 value slices of which the last is partial.
WIDE = config([
    latent(17, 8, 4, 8, 24, 16, 0.3, 50.0, dense(48)),
    lightning(2, 72, 80, (0.99, 0.8), None),
], width=48, vocab=61, scale=1.0, eps=1e-6)
# Sizes that are multiples of nothing much (2 and 6): the products fall back from the TMA-fed kernels, the vector loads
# of the new kernels to their scalar paths, the routed experts in bfloat16 to the tiles of 16 rows.
ODD = config([
    latent(5, 6, 6, 10, 14, 18, 0.4, 77.0, moe(4, 3, 12, 0.5, shared=(10, 0.9))),
    lightning(1, 12, 20, (0.75,), dense(30)),
    lightning(3, 10, 6, (1.0, 0.3, 0.9), None),
], width=36, vocab=50, scale=0.5, eps=1e-4)
# One latent-attention layer whose weights `plant_needle` rewrites so that one token's query finds one other token's key.
NEEDLE = config([latent(2, 16, 8, 16, 24, 24, 1.0, 30.0, dense(64))], width=32, vocab=53, scale=2.0)
NEEDLE_ID, PROBE_ID, FILLER_ID = 5, 9, 11
# A state that keeps everything (decay 1) and nothing else to carry information: losing the state, or a token of it,
# shows at every later position.
KEEPING = config([lightning(2, 8, 8, (1.0, 1.0), None)], width=32, vocab=53, scale=2.0)


def build(cfg: dict, seed: int, dtype: str = "float32", sigma: float = 0.1, sigma_norm: float = 0.2, prepare=None):
    """(the engine's model on the GPU, tensors by name on the CPU)."""
    from llmgen_b200.engine.api import require_cuda, resolve_dtype
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.parts.registry import model_weight_decls
    from llmgen_b200.registry import config_from_dict
    from llmgen_b200.weights import random_tensors, weights_from_dict
    arch, typed = config_from_dict(cfg)
    spec = arch.build_spec(typed)
    decls = model_weight_decls(spec)
    tensors = random_tensors(decls, seed, sigma, sigma_norm, torch.bfloat16)     # stored as a model folder stores them
    if prepare is not None:
        prepare(cfg, tensors)
    model = DecoderModel(spec, weights_from_dict(tensors, decls), resolve_dtype(dtype), require_cuda())
    return model, tensors


def plant_needle(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Rewrites the tensors of the one-layer NEEDLE model in place so that the query of token PROBE_ID equals, in its
    unrotated part, the key of token NEEDLE_ID: the query's latent reads the first half of the residual row, the key's
    latent the second half, through the same matrix and gains; the probe's first half is the needle's second half; and
    every head's unrotated query rows are its key rows.  The score of that pair is then the squared length of the key
    (some tens), all others are those of random directions, and the probe's logits depend on the needle's value alone:
    a key or value that is not the one written for the needle shows far beyond rounding."""
    m = cfg["layers"][0]["mixer"]
    heads, dim, rot, rank, width = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], cfg["width"]
    assert m["q_rank"] == rank and width % 2 == 0
    half = width // 2
    dkv, dq = tensors["l0.mix.dkv"], tensors["l0.mix.dq"]
    dq[:, :half] = dkv[:rank, half:]
    dq[:, half:] = 0
    dkv[:rank, :half] = 0
    tensors["l0.mix.dq.norm"].copy_(tensors["l0.mix.dkv.norm"])
    uq, uk = tensors["l0.mix.uq"], tensors["l0.mix.uk"]
    for h in range(heads):
        uq[h * (dim + rot):h * (dim + rot) + dim] = uk[h * dim:(h + 1) * dim]
        uq[h * (dim + rot) + dim:(h + 1) * (dim + rot)] *= 0.1           # the rotated part decides nothing
    emb = tensors["embed"]
    emb[PROBE_ID, :half] = emb[NEEDLE_ID, half:]


def needle_ids(cfg: dict, n: int, needle_at: int, seed: int) -> List[int]:
    """`n` random ids with the needle token at `needle_at` only and the probe token last only."""
    ids = [t if t not in (NEEDLE_ID, PROBE_ID) else FILLER_ID for t in ids_for(cfg, n, seed)]
    ids[needle_at] = NEEDLE_ID
    ids[-1] = PROBE_ID
    return ids


def plain_logits(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    from tests.plain import derupel_plain
    return derupel_plain.forward(cfg, tensors, ids)[0]


def driver(model, dtype: str, pool_tokens: int = 512, page_size: int = 16, max_num_seqs: int = 4, eager: bool = True):
    from tests.util import Driver
    return Driver(None, dtype, pool_tokens, page_size=page_size, max_num_seqs=max_num_seqs, model=model, eager=eager)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Row-wise RMS difference (mean taken off) over the RMS of the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double() - want.double().mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / w.pow(2).mean(dim=-1).sqrt().mean()


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float(row_errors(got, want).max())


TOL = {"float32": 2e-5, "bfloat16": 6e-2}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what="") -> None:
    """float32: every row within TOL.  bfloat16: nine rows in ten within TOL and the median within a third of it; a
    router score that bfloat16 rounding moves across another (random weights have such close calls) sends one token to
    another expert, which is a large difference at that row and a small one after it, and says nothing about a kernel."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, float(e.max()))
    else:
        assert float(e.quantile(0.9)) < TOL[dtype] and float(e.median()) < TOL[dtype] / 3, (what, float(e.quantile(0.9)), float(e.median()))


def run_in_portions(drv, rid, ids: Sequence[int], portions: Sequence[int], end: bool = True) -> torch.Tensor:
    """Logits of every position of `ids`, fed in the given portions (the last one repeats until the end)."""
    out, pos, k = [], 0, 0
    while pos < len(ids):
        n = min(portions[min(k, len(portions) - 1)], len(ids) - pos)
        last = pos + n == len(ids)
        out.append(drv.step([(rid, ids[pos:pos + n], list(range(n)))], end=[rid] if last and end else []))
        pos += n
        k += 1
    return torch.cat(out)


def ids_for(cfg: dict, n: int, seed: int) -> List[int]:
    from tests.util import random_ids
    return random_ids(n, cfg["vocab"], seed)
