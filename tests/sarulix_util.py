"""Small Sarulix configurations with random weights, for the tests: the engine's model and the tensors the plain
implementation reads, made from one seed."""
from __future__ import annotations

import copy
from typing import Dict, List, Sequence

import torch

from tests.derupel_util import TOL, assert_close, driver, ids_for, relative_error, row_errors, run_in_portions  # noqa: F401


def attention(heads, kv_heads, dim, vdim, scale, mlp, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp, decay_rank=8, gate_rank=12):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(layers, width=64, vocab=97, scale=3.0, eps=1e-5, loop=None, logit_scale=None) -> dict:
    c = {"architecture": "Sarulix", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
         "layers": copy.deepcopy(list(layers))}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


# Every kind of layer, sizes that differ from one another wherever they can: a recurrent branch narrower than the stream,
# key width != value width, grouped heads, a rotation over half of a head, a loop that starts after the first layer and
# runs twice, a layer with and layers without a feed-forward.
MIXED = config([
    rglru(48, 3, 4, None),
    delta(4, 2, 16, 24, 3, None),
    attention(4, 2, 16, 24, 0.3, dense(80), softcap=15.0, rot=(5000.0, 8)),
    rglru(96, 4, 2, dense(40)),
], loop=(1, 3, 2), logit_scale=0.7)
# Sizes that are multiples of little (the products fall back from the TMA-fed kernels, vector loads to scalar ones),
# values that a usual model makes equal or one: one block, one head, as many key heads as heads, the whole head
# rotated, no bound on the scores, no loop, the logits as they are, two taps and five, key and value widths of the
# attention that are no multiples of 8 or of 4.
ODD = config([
    attention(3, 3, 12, 20, 0.4, None, rot=(77.0, 12)),
    rglru(36, 1, 2, dense(30)),
    delta(1, 1, 10, 6, 5, None, decay_rank=3, gate_rank=5),
    attention(2, 1, 10, 6, 0.2, dense(20), softcap=4.0),
], width=36, vocab=50, scale=0.5, eps=1e-4)
# A loop from the first layer on, three times; eight query heads on one key head; more value columns than one block of
# the delta rule's kernel takes (72 > 64), a key width that is no multiple of four times anything (40).
WIDE = config([
    attention(8, 1, 32, 16, 0.18, None, softcap=30.0, rot=(100.0, 32)),
    rglru(128, 4, 4, None),
    delta(6, 2, 40, 72, 4, dense(48)),
    rglru(48, 2, 3, None),
], width=48, vocab=61, scale=1.0, eps=1e-6, loop=(0, 3, 3), logit_scale=1.5)
# Key and value widths that the tensor-core attention of the bfloat16 engine takes (64 and 128, equal and not), beside a
# recurrent layer; prompts of a few hundred tokens then cross several tiles of keys and of queries.
TENSOR = config([
    attention(6, 3, 64, 64, 0.11, dense(64), softcap=25.0, rot=(10000.0, 32)),
    rglru(64, 2, 4, None),
    attention(2, 1, 128, 64, 0.09, None, rot=(500.0, 128)),
    attention(2, 2, 64, 128, 0.125, None, softcap=8.0),
], width=64, vocab=97, scale=2.0, loop=(0, 2, 2))
# One attention layer whose weights `plant_needle` rewrites so that one token's query finds one other token's key.
NEEDLE = config([attention(2, 1, 64, 16, 0.25, dense(64), softcap=24.0, rot=(30.0, 8))], width=32, vocab=53, scale=2.0)
NEEDLE_ID, PROBE_ID, FILLER_ID = 5, 9, 11
# States that keep (nearly) everything and nothing else to carry information: losing a state, or a token of it, shows
# at every later position.
KEEPING_LRU = config([rglru(32, 2, 4, None)], width=32, vocab=53, scale=2.0)
KEEPING_DELTA = config([delta(2, 1, 8, 8, 3, None)], width=32, vocab=53, scale=2.0)


def build(cfg: dict, seed: int, dtype: str = "float32", sigma: float = 0.1, sigma_norm: float = 0.2, prepare=None):
    """(the engine's model on the GPU, tensors by name on the CPU)."""
    from llmgen_b200.engine.api import require_cuda, resolve_dtype
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.weights import weights_from_dict
    spec, decls, tensors = draw(cfg, seed, sigma, sigma_norm)
    if prepare is not None:
        prepare(cfg, tensors)
    model = DecoderModel(spec, weights_from_dict(tensors, decls), resolve_dtype(dtype), require_cuda())
    return model, tensors


def draw(cfg: dict, seed: int, sigma: float = 0.1, sigma_norm: float = 0.2):
    from llmgen_b200.parts.registry import model_weight_decls
    from llmgen_b200.registry import config_from_dict
    from llmgen_b200.weights import random_tensors
    arch, typed = config_from_dict(cfg)
    spec = arch.build_spec(typed)
    decls = model_weight_decls(spec)
    return spec, decls, random_tensors(decls, seed, sigma, sigma_norm, torch.bfloat16)     # stored as a model folder stores them


def keep_long(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Makes the one-layer KEEPING models remember: the recurrent unit's decays lie just below one (lam far below zero),
    the delta rule's too (dt_bias far below zero) while its writes stay small (beta's matrix scaled down)."""
    if "l0.mix.lam" in tensors:
        tensors["l0.mix.lam"].fill_(-9.0)
    if "l0.mix.dt_bias" in tensors:
        tensors["l0.mix.dt_bias"].fill_(-7.0)
        tensors["l0.mix.a2"].mul_(0.1)


def plant_needle(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Rewrites the tensors of the one-layer NEEDLE model in place so that the query of token PROBE_ID points where the key
    of token NEEDLE_ID points: queries read the first half of the normed residual row, keys the second half, through the
    same matrix rows, with no biases and equal per-head gains; the first norm's gain is exactly one, so the two rows
    differ by a factor that the per-head norm removes; the probe's first half is the needle's second half.  The gains of
    the rotated values are small, so the position decides little.  The score of that pair is then scale * dim * gain^2
    (16, bounded to 14 by the softcap) against about 2 for random directions: the probe's output is the needle's value
    times exp(s) / (1 + sum exp(s)), and a key or value that is not the one written for the needle shows far beyond
    rounding."""
    m = cfg["layers"][0]["mixer"]
    heads, kv, dim, width = m["heads"], m["kv_heads"], m["dim"], cfg["width"]
    half = width // 2
    wq, wk = tensors["l0.mix.q"], tensors["l0.mix.k"]
    wk[:, :half] = 0
    for h in range(heads):
        g = h // (heads // kv)
        wq[h * dim:(h + 1) * dim, :half] = wk[g * dim:(g + 1) * dim, half:]
    wq[:, half:] = 0
    for n in ("l0.mix.q.b", "l0.mix.k.b", "l0.norm1"):
        tensors[n].zero_()
    gain = torch.ones(dim)
    gain[:m["rot"]["dims"]] = 0.1
    tensors["l0.mix.q.norm"].copy_(gain)
    tensors["l0.mix.k.norm"].copy_(gain)
    tensors["l0.mix.g"].mul_(0.1)
    emb = tensors["embed"]
    emb[PROBE_ID, :half] = emb[NEEDLE_ID, half:]


def needle_ids(cfg: dict, n: int, needle_at: int, seed: int) -> List[int]:
    """`n` random ids with the needle token at `needle_at` only and the probe token last only."""
    ids = [t if t not in (NEEDLE_ID, PROBE_ID) else FILLER_ID for t in ids_for(cfg, n, seed)]
    ids[needle_at] = NEEDLE_ID
    ids[-1] = PROBE_ID
    return ids


def plain_logits(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    from tests.plain import sarulix_plain
    return sarulix_plain.forward(cfg, tensors, ids)[0]
