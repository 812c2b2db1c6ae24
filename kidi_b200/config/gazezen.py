"""Typed configuration of Gazezen, read from the model's own config.json keys.

    architecture: "Gazezen"        vocab, width, logit_scale
    norm: {eps}
    loop: {start, stop, times}     optional: layers start .. stop-1 run `times` times in a row
    layers: [{type, mixer: {...}, mlp: null | {kind: "moe", expert: {ff}, router: {experts, top,
              groups: {count, keep}}, shared: {ff}}}, ...]

A layer's `type` is "attention" (mixer: heads, kv_heads, dim, vdim, scale, mask: {size}, rot: {base, dims}) or
"latent_attention" (mixer: heads, dim, rot_dim, vdim, kv_rank, scale, mask: {size}, rot: {base, dims, scaling:
{factor, original, fast, slow}}). `mask`, `rot` (of an attention layer), `rot.scaling`, `router.groups`, `shared`,
`loop` and `logit_scale` may be absent: no window, no rotation, no stretching, one group, no shared expert, every
layer once, logits as they are. `max_positions` is optional (the longest sequence the rotation tables are built
for; default 65,536). A missing or ill-typed key is INVALID_MANIFEST naming the key.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid_manifest, unsupported
from .reader import ConfigReader

ATTENTION = "attention"
LATENT_ATTENTION = "latent_attention"
DEFAULT_MAX_POSITIONS = 65536


@dataclasses.dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclasses.dataclass(frozen=True)
class GazezenFeedForward:
    expert_ff: int
    experts: int
    top: int
    groups: int = 1
    keep_groups: int = 1
    shared_ff: Optional[int] = None

    def to_dict(self) -> dict:
        router: dict = {"experts": self.experts, "top": self.top}
        if self.groups != 1 or self.keep_groups != 1:
            router["groups"] = {"count": self.groups, "keep": self.keep_groups}
        values: dict = {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": router}
        if self.shared_ff is not None:
            values["shared"] = {"ff": self.shared_ff}
        return values


@dataclasses.dataclass(frozen=True)
class GazezenLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    rot_base: Optional[float] = None      # None: the layer's queries and keys are not rotated
    rot_dims: int = 0
    rot_scaling: Optional[RotaryScaling] = None
    kv_heads: int = 0                     # attention only
    rot_dim: int = 0                      # latent attention only
    kv_rank: int = 0
    mlp: Optional[GazezenFeedForward] = None

    def to_dict(self) -> dict:
        mixer: dict = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.type == ATTENTION:
            mixer["kv_heads"] = self.kv_heads
        else:
            mixer.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank)
        if self.window is not None:
            mixer["mask"] = {"size": self.window}
        if self.rot_base is not None:
            mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                mixer["rot"]["scaling"] = self.rot_scaling.to_dict()
        return {"type": self.type, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclasses.dataclass(frozen=True)
class GazezenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[GazezenLayer, ...]
    logit_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Gazezen"

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "GazezenConfig":
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
            mask, rot = mixer.child("mask"), mixer.child("rot")
            scaling = rot.child("scaling") if rot is not None else None
            common = dict(
                type=kind, heads=mixer.integer("heads"), dim=mixer.integer("dim"), vdim=mixer.integer("vdim"),
                scale=mixer.number("scale"), window=mask.integer("size") if mask is not None and mask.has("size") else None,
                rot_base=rot.number("base") if rot is not None else None,
                rot_dims=rot.integer("dims") if rot is not None else 0,
                rot_scaling=RotaryScaling(scaling.number("factor"), scaling.number("original"), scaling.number("fast"),
                                          scaling.number("slow")) if scaling is not None else None,
                mlp=cls._feed_forward(layer.child("mlp"), index))
            if kind == ATTENTION:
                layers.append(GazezenLayer(**common, kv_heads=mixer.integer("kv_heads")))
            elif kind == LATENT_ATTENTION:
                layers.append(GazezenLayer(**common, rot_dim=mixer.integer("rot_dim"), kv_rank=mixer.integer("kv_rank")))
            else:
                raise unsupported(f"layers[{index}]: layer type '{kind}' is not supported")
        loop = reader.child("loop")
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
                     layers=tuple(layers), logit_scale=reader.number("logit_scale", 1.0),
                     loop=(loop.integer("start"), loop.integer("stop"), loop.integer("times")) if loop is not None else None,
                     max_positions=reader.integer("max_positions", DEFAULT_MAX_POSITIONS), eos_token_ids=eos_ids)
        config.validate()
        return config

    @staticmethod
    def _feed_forward(mlp: Optional[ConfigReader], index: int) -> Optional[GazezenFeedForward]:
        if mlp is None:
            return None
        if mlp.string("kind") != "moe":
            raise unsupported(f"layers[{index}]: feed-forward kind '{mlp.string('kind')}' is not supported")
        expert, router, shared = mlp.child("expert"), mlp.child("router"), mlp.child("shared")
        if expert is None or router is None:
            raise invalid_manifest(f"config.json:layers[{index}]:mlp: 'expert' and 'router' must be objects")
        groups = router.child("groups")
        return GazezenFeedForward(
            expert_ff=expert.integer("ff"), experts=router.integer("experts"), top=router.integer("top"),
            groups=groups.integer("count") if groups is not None else 1,
            keep_groups=groups.integer("keep") if groups is not None else 1,
            shared_ff=shared.integer("ff") if shared is not None else None)

    def validate(self) -> None:
        if min(self.vocab, self.width, self.max_positions) <= 0:
            raise invalid_manifest("invalid Gazezen dimensions: every size must be positive")
        if not self.norm_eps > 0:
            raise invalid_manifest("invalid Gazezen configuration: norm.eps must be positive")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start < stop <= len(self.layers) or times < 1:
                raise invalid_manifest("loop: start < stop must lie within the layers, and times must be at least 1")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if min(layer.heads, layer.dim, layer.vdim) <= 0:
                raise invalid_manifest(f"{where}: every size must be positive")
            if layer.window is not None and layer.window <= 0:
                raise invalid_manifest(f"{where}: mask.size must be positive")
            rotated = layer.dim if layer.type == ATTENTION else layer.rot_dim
            if layer.type == ATTENTION:
                if layer.kv_heads <= 0 or layer.heads % layer.kv_heads:
                    raise invalid_manifest(f"{where}: heads must be a multiple of kv_heads")
                if layer.rot_scaling is not None:
                    raise unsupported(f"{where}: rot.scaling belongs to latent-attention layers")
            else:
                if min(layer.rot_dim, layer.kv_rank) <= 0:
                    raise invalid_manifest(f"{where}: rot_dim and kv_rank must be positive")
                if layer.rot_base is None:
                    raise invalid_manifest(f"{where}: a latent-attention layer needs 'rot'")
            if layer.rot_base is not None:
                if layer.rot_dims <= 0 or layer.rot_dims % 2 or layer.rot_dims > rotated:
                    raise invalid_manifest(f"{where}: rot.dims must be even, positive and at most the rotated width")
                if not layer.rot_base > 0:
                    raise invalid_manifest(f"{where}: rot.base must be positive")
                scaling = layer.rot_scaling
                if scaling is not None and (min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0
                                            or not layer.rot_base > 1):
                    raise invalid_manifest(f"{where}: rot.scaling needs positive constants and a base above 1")
            mlp = layer.mlp
            if mlp is not None:
                if min(mlp.expert_ff, mlp.experts, mlp.top, mlp.groups, mlp.keep_groups) <= 0 or mlp.top > mlp.experts:
                    raise invalid_manifest(f"{where}: invalid feed-forward sizes")
                if mlp.experts % mlp.groups or mlp.keep_groups > mlp.groups \
                        or mlp.keep_groups * (mlp.experts // mlp.groups) < mlp.top:
                    raise invalid_manifest(f"{where}: the experts split into equal groups, and the kept groups hold "
                                           f"at least `top` experts")
                if mlp.shared_ff is not None and mlp.shared_ff <= 0:
                    raise invalid_manifest(f"{where}: shared.ff must be positive")
        if any(token < 0 or token >= self.vocab for token in self.eos_token_ids):
            raise invalid_manifest("eos_token_id lies outside the vocabulary")

    def run_order(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """(layer, pass) in the order the layers run; `pass` is the number of the pass at the first layer of
        each pass of the looped range, else None."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((index, None) for index in range(count))
        start, stop, times = self.loop
        order = [(index, None) for index in range(start)]
        for number in range(times):
            order += [(index, number if index == start else None) for index in range(start, stop)]
        return tuple(order + [(index, None) for index in range(stop, count)])

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        values: dict = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                        "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_scale != 1.0:
            values["logit_scale"] = self.logit_scale
        if self.loop is not None:
            values["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            values["max_positions"] = self.max_positions
        if self.eos_token_ids:
            values["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return values
