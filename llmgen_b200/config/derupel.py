"""Typed configuration of the Derupel decoder, read from its config.json.

    architecture      "Derupel"
    vocab, width      sizes of the table of embeddings and of the residual stream
    embedding.scale   factor on the embedding rows
    norm.eps          eps of every RMSNorm
    layers[i]         type: "lightning" | "latent_attention"; mixer: that mixer's sizes and constants;
                      mlp: null, {kind: "dense", ff}, or {kind: "moe", expert: {ff, limit}, router: {experts, top},
                      shared: {ff, limit} (optional)}
    lightning mixer   heads, dim, vdim, decay (one factor per head)
    latent mixer      heads, dim (unrotated), rot_dim (rotated), vdim, q_rank, kv_rank, scale, rot: {base, dims}

Every size and constant comes from the file; `max_positions` (rows of the rotary tables) is optional.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader

LIGHTNING = "lightning"
LATENT_ATTENTION = "latent_attention"
DENSE = "dense"
MOE = "moe"
DEFAULT_MAX_POSITIONS = 1 << 17


@dataclass(frozen=True)
class LightningMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int = 0                              # dense
    experts: int = 0                         # moe
    top: int = 0
    expert: Optional[ExpertConfig] = None
    shared: Optional[ExpertConfig] = None


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


def _sub(r: ConfigReader, key: str, where: str, required: bool = True) -> Optional[ConfigReader]:
    v = r.raw(key)
    if v is None:
        if required:
            r.problem(f"missing object '{key}'")
        return None
    if not isinstance(v, dict):
        r.problem(f"'{key}' must be an object")
        return None
    sub = ConfigReader(v, f"{where}.{key}")
    sub.problems = r.problems          # one list for the whole file
    sub._prefix = f"{key}."
    return sub


def _expert(r: ConfigReader, key: str, where: str, required: bool) -> Optional[ExpertConfig]:
    e = _sub(r, key, where, required)
    if e is None:
        return None
    ff, limit = e.integer("ff"), e.number("limit")
    return ExpertConfig(ff, limit) if None not in (ff, limit) else None


def _layer(data, i: int, r: ConfigReader, where: str) -> Optional[LayerConfig]:
    if not isinstance(data, dict):
        r.problem(f"layers[{i}] must be an object")
        return None
    n0 = len(r.problems)
    lr = ConfigReader(data, f"{where}.layers[{i}]")
    lr.problems = r.problems
    kind = lr.string("type", choices=(LIGHTNING, LATENT_ATTENTION))
    m = _sub(lr, "mixer", lr.where)
    mixer = None
    if m is not None and kind == LIGHTNING:
        heads, dim, vdim = m.integer("heads"), m.integer("dim"), m.integer("vdim")
        decay = m.raw("decay")
        if not isinstance(decay, list) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            r.problem(f"layers[{i}].mixer.decay must be a list of numbers")
        elif heads is not None and len(decay) != heads:
            r.problem(f"layers[{i}].mixer.decay has {len(decay)} factors for {heads} heads")
        elif None not in (heads, dim, vdim):
            mixer = LightningMixerConfig(heads, dim, vdim, tuple(float(d) for d in decay))
    elif m is not None and kind == LATENT_ATTENTION:
        heads, dim, vdim = m.integer("heads"), m.integer("dim", minimum=0), m.integer("vdim")
        rot_dim, q_rank, kv_rank = m.integer("rot_dim", minimum=0), m.integer("q_rank"), m.integer("kv_rank")
        scale = m.number("scale")
        rot = _sub(m, "rot", m.where, required=bool(rot_dim))
        base = rot.number("base") if rot is not None else 1.0
        dims = rot.integer("dims", default=rot_dim, minimum=0) if rot is not None else 0
        if None not in (heads, dim, vdim, rot_dim, q_rank, kv_rank, scale, base, dims):
            r.check(dims == rot_dim, f"layers[{i}].mixer.rot.dims {dims} differs from rot_dim {rot_dim}")
            r.check(rot_dim % 2 == 0, f"layers[{i}].mixer.rot_dim {rot_dim} must be even")
            mixer = LatentMixerConfig(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims)
    mlp = None
    if data.get("mlp") is not None:
        f = _sub(lr, "mlp", lr.where)
        if f is not None:
            fk = f.string("kind", choices=(DENSE, MOE))
            if fk == DENSE:
                ff = f.integer("ff")
                mlp = MlpConfig(DENSE, ff=ff) if ff is not None else None
            elif fk == MOE:
                router = _sub(f, "router", f.where)
                experts = router.integer("experts") if router is not None else None
                top = router.integer("top") if router is not None else None
                expert = _expert(f, "expert", f.where, True)
                shared = _expert(f, "shared", f.where, False)
                if None not in (experts, top, expert):
                    r.check(top <= experts, f"layers[{i}].mlp.router.top {top} exceeds its {experts} experts")
                    mlp = MlpConfig(MOE, experts=experts, top=top, expert=expert, shared=shared)
    if len(r.problems) > n0 or kind is None or mixer is None:
        return None
    return LayerConfig(kind, mixer, mlp)


@dataclass(frozen=True)
class DerupelConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[LayerConfig, ...]
    max_positions: int
    raw: dict

    architecture = "Derupel"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "DerupelConfig":
        r = ConfigReader(data, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        emb = _sub(r, "embedding", where, required=False)
        scale = emb.number("scale", default=1.0) if emb is not None else 1.0
        norm = _sub(r, "norm", where)
        eps = norm.number("eps") if norm is not None else None
        max_positions = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS)
        layers = r.raw("layers")
        parsed = []
        if not isinstance(layers, list) or not layers:
            r.problem("'layers' must be a non-empty list")
        else:
            parsed = [_layer(d, i, r, where) for i, d in enumerate(layers)]
        r.finish()
        return cls(vocab, width, scale, eps, tuple(parsed), max_positions, dict(data))

    def to_dict(self) -> dict:
        return dict(self.raw)
