"""Typed configuration of Biropel, read from the model's own config.json keys.

    architecture: "Biropel"        vocab, width, streams (optional: the residual stream kept as that many lanes)
    norm: {eps}
    layers: [{type, mixer: {...}, mlp: null | {kind: "dense", ff}}, ...]

A layer's `type` is "attention" (mixer: one softmax attention, optionally `kv_from`: an earlier attention layer
whose keys and values it reads), "parallel" (mixer: {left: a softmax attention, right: a state-space mixer: heads,
vdim, state, groups, conv, norm_groups}) or "parallel_2" (mixer: {left: a softmax attention, right: a matrix
memory: heads, dim, vdim, gate_cap}). A softmax attention has heads, kv_heads, dim, vdim, scale and, each
optional, mask: {size} (a sliding window; absent: every earlier token), rot: {base, dims, scaling: {factor,
original, fast, slow}} (absent: no rotation; no scaling: plain frequencies), softcap (absent: scores as they are)
and q_temp: {coef, every} (absent: queries as they are). `max_positions` is optional (the longest sequence the
position tables are built for; default 65,536). A missing or ill-typed key is INVALID_MANIFEST naming the key.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid_manifest, unsupported
from .gazezen import RotaryScaling
from .reader import ConfigReader

ATTENTION = "attention"
PARALLEL_STATE_SPACE = "parallel"
PARALLEL_MATRIX_MEMORY = "parallel_2"
DEFAULT_MAX_POSITIONS = 65536


@dataclasses.dataclass(frozen=True)
class SoftmaxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    rot_base: Optional[float] = None      # None: queries and keys are not rotated
    rot_dims: int = 0
    rot_scaling: Optional[RotaryScaling] = None
    softcap: Optional[float] = None
    q_temp: Optional[Tuple[float, int]] = None     # (coef, every)
    kv_from: Optional[int] = None

    @classmethod
    def read(cls, mixer: ConfigReader) -> "SoftmaxAttention":
        mask, rot, temp = mixer.child("mask"), mixer.child("rot"), mixer.child("q_temp")
        scaling = rot.child("scaling") if rot is not None else None
        return cls(
            heads=mixer.integer("heads"), kv_heads=mixer.integer("kv_heads"), dim=mixer.integer("dim"),
            vdim=mixer.integer("vdim"), scale=mixer.number("scale"),
            window=mask.integer("size") if mask is not None and mask.has("size") else None,
            rot_base=rot.number("base") if rot is not None else None,
            rot_dims=rot.integer("dims") if rot is not None else 0,
            rot_scaling=RotaryScaling(scaling.number("factor"), scaling.number("original"), scaling.number("fast"),
                                      scaling.number("slow")) if scaling is not None else None,
            softcap=mixer.number("softcap") if mixer.has("softcap") else None,
            q_temp=(temp.number("coef"), temp.integer("every")) if temp is not None else None,
            kv_from=mixer.integer("kv_from") if mixer.has("kv_from") else None)

    def to_dict(self) -> dict:
        values: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                        "scale": self.scale}
        if self.window is not None:
            values["mask"] = {"size": self.window}
        if self.rot_base is not None:
            values["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                values["rot"]["scaling"] = self.rot_scaling.to_dict()
        if self.softcap is not None:
            values["softcap"] = self.softcap
        if self.q_temp is not None:
            values["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        if self.kv_from is not None:
            values["kv_from"] = self.kv_from
        return values

    def validate(self, where: str) -> None:
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise invalid_manifest(f"{where}: sizes must be positive and heads a multiple of kv_heads")
        if self.window is not None and self.window <= 0:
            raise invalid_manifest(f"{where}: mask.size must be positive")
        if self.rot_base is not None:
            if self.rot_dims <= 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
                raise invalid_manifest(f"{where}: rot.dims must be even, positive and at most dim")
            if not self.rot_base > 0:
                raise invalid_manifest(f"{where}: rot.base must be positive")
            scaling = self.rot_scaling
            if scaling is not None and (min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0
                                        or not self.rot_base > 1):
                raise invalid_manifest(f"{where}: rot.scaling needs positive constants and a base above 1")
        if self.softcap is not None and not self.softcap > 0:
            raise invalid_manifest(f"{where}: softcap must be positive")
        if self.q_temp is not None and self.q_temp[1] <= 0:
            raise invalid_manifest(f"{where}: q_temp.every must be positive")


@dataclasses.dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def read(cls, mixer: ConfigReader) -> "StateSpace":
        return cls(heads=mixer.integer("heads"), vdim=mixer.integer("vdim"), state=mixer.integer("state"),
                   groups=mixer.integer("groups"), conv=mixer.integer("conv"), norm_groups=mixer.integer("norm_groups"))

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def validate(self, where: str) -> None:
        if min(self.heads, self.vdim, self.state, self.groups, self.conv, self.norm_groups) <= 0:
            raise invalid_manifest(f"{where}: every size must be positive")
        if self.heads % self.groups or (self.heads * self.vdim) % self.norm_groups:
            raise invalid_manifest(f"{where}: heads must be a multiple of groups and heads * vdim of norm_groups")


@dataclasses.dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def read(cls, mixer: ConfigReader) -> "MatrixMemory":
        return cls(heads=mixer.integer("heads"), dim=mixer.integer("dim"), vdim=mixer.integer("vdim"),
                   gate_cap=mixer.number("gate_cap"))

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def validate(self, where: str) -> None:
        if min(self.heads, self.dim, self.vdim) <= 0 or not self.gate_cap > 0:
            raise invalid_manifest(f"{where}: sizes and gate_cap must be positive")


@dataclasses.dataclass(frozen=True)
class BiropelLayer:
    type: str
    attention: SoftmaxAttention                    # the layer's mixer, or the left one of two
    right: Any = None                              # StateSpace or MatrixMemory; None for an attention layer
    ff: Optional[int] = None                       # None: the layer has no feed-forward

    def to_dict(self) -> dict:
        mixer = self.attention.to_dict() if self.right is None else {"left": self.attention.to_dict(),
                                                                     "right": self.right.to_dict()}
        return {"type": self.type, "mixer": mixer,
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff is not None else None}


@dataclasses.dataclass(frozen=True)
class BiropelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BiropelLayer, ...]
    streams: Optional[int] = None                  # None: one residual stream, added to as usual
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Biropel"

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "BiropelConfig":
        reader = ConfigReader(values)
        name = reader.string("architecture", cls.architecture)
        if name != cls.architecture:
            raise invalid_manifest(f"expected architecture '{cls.architecture}', found '{name}'")
        norm = reader.child("norm")
        if norm is None:
            raise invalid_manifest("config.json: 'norm' must be an object")
        raw_layers = reader.raw("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise invalid_manifest("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json:layers[{index}]"
            layer = ConfigReader(raw, where)
            kind = layer.string("type")
            mixer = layer.child("mixer")
            if mixer is None:
                raise invalid_manifest(f"{where}: 'mixer' must be an object")
            mlp = layer.child("mlp")
            if mlp is not None and mlp.string("kind") != "dense":
                raise unsupported(f"layers[{index}]: feed-forward kind '{mlp.string('kind')}' is not supported")
            ff = mlp.integer("ff") if mlp is not None else None
            if kind == ATTENTION:
                layers.append(BiropelLayer(kind, SoftmaxAttention.read(mixer), None, ff))
            elif kind in (PARALLEL_STATE_SPACE, PARALLEL_MATRIX_MEMORY):
                left, right = mixer.child("left"), mixer.child("right")
                if left is None or right is None:
                    raise invalid_manifest(f"{where}:mixer: 'left' and 'right' must be objects")
                other = StateSpace.read(right) if kind == PARALLEL_STATE_SPACE else MatrixMemory.read(right)
                layers.append(BiropelLayer(kind, SoftmaxAttention.read(left), other, ff))
            else:
                raise unsupported(f"layers[{index}]: layer type '{kind}' is not supported")
        eos = reader.raw("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise invalid_manifest("'eos_token_id' must be an integer or a list of integers")
        config = cls(vocab=reader.integer("vocab"), width=reader.integer("width"), norm_eps=norm.number("eps"),
                     layers=tuple(layers), streams=reader.integer("streams") if reader.has("streams") else None,
                     max_positions=reader.integer("max_positions", DEFAULT_MAX_POSITIONS), eos_token_ids=eos_ids)
        config.validate()
        return config

    def validate(self) -> None:
        if min(self.vocab, self.width, self.max_positions) <= 0:
            raise invalid_manifest("invalid Biropel dimensions: every size must be positive")
        if not self.norm_eps > 0:
            raise invalid_manifest("invalid Biropel configuration: norm.eps must be positive")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise unsupported("'streams' must lie between 1 and 8")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            layer.attention.validate(where)
            if layer.right is not None:
                layer.right.validate(where + ":right")
            if layer.ff is not None and layer.ff <= 0:
                raise invalid_manifest(f"{where}: mlp.ff must be positive")
            source = layer.attention.kv_from
            if source is None:
                continue
            if layer.type != ATTENTION:
                raise unsupported(f"{where}: kv_from belongs to attention layers")
            if not 0 <= source < index or self.layers[source].type != ATTENTION \
                    or self.layers[source].attention.kv_from is not None:
                raise invalid_manifest(f"{where}: kv_from must name an earlier attention layer with keys of its own")
            mine, other = layer.attention, self.layers[source].attention
            if (mine.kv_heads, mine.dim, mine.vdim, mine.rot_base, mine.rot_dims, mine.rot_scaling) != \
                    (other.kv_heads, other.dim, other.vdim, other.rot_base, other.rot_dims, other.rot_scaling):
                raise invalid_manifest(f"{where}: the layer named by kv_from has other key/value heads or rotation")
        if any(token < 0 or token >= self.vocab for token in self.eos_token_ids):
            raise invalid_manifest("eos_token_id lies outside the vocabulary")

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        values: dict = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                        "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.streams is not None:
            values["streams"] = self.streams
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            values["max_positions"] = self.max_positions
        if self.eos_token_ids:
            values["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return values
