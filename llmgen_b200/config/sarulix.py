"""Typed configuration of the Sarulix decoder, read from its config.json.

    architecture      "Sarulix"
    vocab, width      sizes of the table of embeddings and of the residual stream
    embedding.scale   factor on the embedding rows
    norm.eps          eps of every RMSNorm
    logit_scale       factor on the logits
    loop              optional {start, stop, times}: layers [start, stop) run `times` times in a row with the same weights
    layers[i]         type: "attention" | "rglru" | "channel_delta"; mixer: that mixer's sizes and constants;
                      mlp: null or {kind: "dense", ff}
    attention mixer   heads, kv_heads, dim, vdim, scale, softcap (optional), rot: {base, dims} (optional)
    rglru mixer       width, blocks, conv (taps)
    channel_delta     heads, kv_heads, dim, vdim, conv (taps); optional decay_rank, gate_rank

Every size and constant comes from the file.  The ranks of the delta rule's two low-rank projections are sizes that a
model folder gives by the shapes of its tensors `l<i>.mix.a1` and `l<i>.mix.g1` alone: `fill_from_tensor_shapes` puts
them into the mixer's object as `decay_rank` and `gate_rank`, which a configuration written by hand (the random-weights
mode) may name itself (default 16).  `max_positions` (rows of the rotary tables) is optional.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .derupel import _sub

ATTENTION = "attention"
RGLRU = "rglru"
CHANNEL_DELTA = "channel_delta"
DENSE = "dense"
DEFAULT_MAX_POSITIONS = 1 << 17
DEFAULT_LOW_RANK = 16


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0: none
    rot_base: float
    rot_dims: int           # 0: no rotation


@dataclass(frozen=True)
class RGLRUMixerConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class ChannelDeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


def _layer(data, i: int, r: ConfigReader, where: str) -> Optional[LayerConfig]:
    if not isinstance(data, dict):
        r.problem(f"layers[{i}] must be an object")
        return None
    n0 = len(r.problems)
    lr = ConfigReader(data, f"{where}.layers[{i}]")
    lr.problems = r.problems
    kind = lr.string("type", choices=(ATTENTION, RGLRU, CHANNEL_DELTA))
    m = _sub(lr, "mixer", lr.where)
    mixer = None
    if m is not None and kind == ATTENTION:
        heads, kv_heads = m.integer("heads"), m.integer("kv_heads")
        dim, vdim, scale = m.integer("dim"), m.integer("vdim"), m.number("scale")
        softcap = m.number("softcap", default=0.0, positive=False)
        rot = _sub(m, "rot", m.where, required=False)
        base = rot.number("base") if rot is not None else 1.0
        dims = rot.integer("dims", minimum=0) if rot is not None else 0
        if None not in (heads, kv_heads, dim, vdim, scale, softcap, base, dims):
            r.check(heads % kv_heads == 0, f"layers[{i}].mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
            r.check(dims % 2 == 0 and dims <= dim, f"layers[{i}].mixer.rot.dims {dims} must be even and at most dim {dim}")
            r.check(softcap >= 0, f"layers[{i}].mixer.softcap must not be negative")
            mixer = AttentionMixerConfig(heads, kv_heads, dim, vdim, scale, softcap, base, dims)
    elif m is not None and kind == RGLRU:
        width, blocks, conv = m.integer("width"), m.integer("blocks"), m.integer("conv")
        if None not in (width, blocks, conv):
            r.check(width % blocks == 0, f"layers[{i}].mixer: width {width} is not cut evenly into {blocks} blocks")
            mixer = RGLRUMixerConfig(width, blocks, conv)
    elif m is not None and kind == CHANNEL_DELTA:
        heads, kv_heads = m.integer("heads"), m.integer("kv_heads")
        dim, vdim, conv = m.integer("dim"), m.integer("vdim"), m.integer("conv")
        decay_rank = m.integer("decay_rank", default=DEFAULT_LOW_RANK)
        gate_rank = m.integer("gate_rank", default=DEFAULT_LOW_RANK)
        if None not in (heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
            r.check(heads % kv_heads == 0, f"layers[{i}].mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
            mixer = ChannelDeltaMixerConfig(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank)
    mlp = None
    if data.get("mlp") is not None:
        f = _sub(lr, "mlp", lr.where)
        if f is not None:
            fk = f.string("kind", choices=(DENSE,))
            ff = f.integer("ff")
            mlp = MlpConfig(fk, ff) if None not in (fk, ff) else None
    if len(r.problems) > n0 or kind is None or mixer is None:
        return None
    return LayerConfig(kind, mixer, mlp)


@dataclass(frozen=True)
class SarulixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    layers: Tuple[LayerConfig, ...]
    loop: Optional[LoopConfig]
    max_positions: int
    raw: dict

    architecture = "Sarulix"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "SarulixConfig":
        r = ConfigReader(data, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        emb = _sub(r, "embedding", where, required=False)
        scale = emb.number("scale", default=1.0) if emb is not None else 1.0
        norm = _sub(r, "norm", where)
        eps = norm.number("eps") if norm is not None else None
        logit_scale = r.number("logit_scale", default=1.0)
        max_positions = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS)
        layers = r.raw("layers")
        parsed = []
        if not isinstance(layers, list) or not layers:
            r.problem("'layers' must be a non-empty list")
        else:
            parsed = [_layer(d, i, r, where) for i, d in enumerate(layers)]
        loop = None
        if data.get("loop") is not None:
            lp = _sub(r, "loop", where)
            if lp is not None:
                start, stop, times = lp.integer("start", minimum=0), lp.integer("stop"), lp.integer("times")
                if None not in (start, stop, times):
                    r.check(start < stop <= len(parsed), f"loop [{start}, {stop}) does not lie within the {len(parsed)} layers")
                    loop = LoopConfig(start, stop, times)
        r.finish()
        return cls(vocab, width, scale, eps, logit_scale, tuple(parsed), loop, max_positions, dict(data))

    def to_dict(self) -> dict:
        return dict(self.raw)

    @staticmethod
    def fill_from_tensor_shapes(data: dict, shapes: dict) -> dict:
        """`data` with `decay_rank` / `gate_rank` added to every channel_delta mixer that does not name them, from the
        shapes of the folder's tensors `l<i>.mix.a1` / `l<i>.mix.g1` ([rank, width])."""
        import copy
        layers = data.get("layers")
        if not isinstance(layers, list):
            return data
        out = copy.deepcopy(data)
        for i, layer in enumerate(out["layers"]):
            if isinstance(layer, dict) and layer.get("type") == CHANNEL_DELTA and isinstance(layer.get("mixer"), dict):
                for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if key not in layer["mixer"] and tensor in shapes and len(shapes[tensor]) == 2:
                        layer["mixer"][key] = int(shapes[tensor][0])
        return out
