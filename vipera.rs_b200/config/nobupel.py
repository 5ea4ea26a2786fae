"""Typed configuration of the Nobupel decoder, read from the keys of its own config.json,
and its description in terms of parts.

The design: a stack of pre-norm layers, each with one of two mixers and, where config.json
gives one, a gated feed-forward (tanh form of gelu, biases).  The mixers: grouped-query
attention with q/k/v biases, rotary positions on the first values of each head (NeoX pairing,
YaRN scaling), a sliding window that keeps the first tokens of a request visible, and a
softmax with one added to its denominator; and the matrix-memory cell of xLSTM (mLSTM) with
capped log gates.  A range of layers may run several times in a row with the same weights,
each pass with a cache or state of its own.

config.json keys: ``architecture`` ("Nobupel"), ``vocab``, ``width``, ``norm.eps``, ``layers``
(a list of ``{type, mixer, mlp}``) and ``loop`` (``{start, stop, times}``).  Tensor names in
the weight file: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<name>``,
``l<i>.mlp.<name>``, biases with ``.b`` added, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import InvalidArgumentError, UnsupportedError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# Positions a model of this design may reach where config.json says nothing (key ``max_positions``).
DEFAULT_MAX_POSITIONS = 1 << 17


def _integer(where: str, value, least: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise InvalidArgumentError(f"{where} must be an integer of at least {least}, got {value!r}")
    return value


def _number(where: str, value, positive: bool = True) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or \
            (positive and not value > 0):
        raise InvalidArgumentError(f"{where} must be a {'positive ' if positive else ''}number, got {value!r}")
    return float(value)


def _need(where: str, data: Dict[str, Any], keys) -> None:
    if not isinstance(data, dict):
        raise InvalidArgumentError(f"{where} must be an object")
    for key in keys:
        if key not in data:
            raise UnsupportedError(f"config.json: {where} has no {key!r}")


@dataclass(frozen=True)
class NobupelLayer:
    kind: str                       # "attention" or "mlstm"
    mixer: Dict[str, Any]           # the mixer's sizes and constants, checked
    ff: Optional[int]               # the feed-forward's inner size, None for a layer without one


@dataclass(frozen=True)
class NobupelConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[NobupelLayer, ...]
    loop: Optional[Tuple[int, int, int]]   # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Nobupel"
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ---- reading -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "NobupelConfig":
        _need("the configuration", data, ("vocab", "width", "layers", "norm"))
        _need("norm", data["norm"], ("eps",))
        width = _integer("width", data["width"])
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise InvalidArgumentError("layers must be a list with at least one layer")
        layers = []
        for index, entry in enumerate(data["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, ("type", "mixer"))
            kind, mixer = entry["type"], entry["mixer"]
            if kind == "attention":
                checked = cls._attention(where, mixer)
            elif kind == "mlstm":
                checked = cls._mlstm(where, mixer)
            else:
                raise UnsupportedError(f"{where}: unknown mixer type {kind!r}; known: attention, mlstm")
            ff = None
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(f"{where}.mlp", mlp, ("kind", "ff"))
                if mlp["kind"] != "dense":
                    raise UnsupportedError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
                ff = _integer(f"{where}.mlp.ff", mlp["ff"])
            layers.append(NobupelLayer(kind, checked, ff))
        loop = None
        if data.get("loop") is not None:
            _need("loop", data["loop"], ("start", "stop", "times"))
            start = _integer("loop.start", data["loop"]["start"], 0)
            stop = _integer("loop.stop", data["loop"]["stop"], 0)
            times = _integer("loop.times", data["loop"]["times"], 1)
            if not start <= stop <= len(layers):
                raise InvalidArgumentError(f"loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(vocab=_integer("vocab", data["vocab"]), width=width, eps=_number("norm.eps", data["norm"]["eps"]),
                   layers=tuple(layers), loop=loop,
                   max_positions=_integer("max_positions", data.get("max_positions", DEFAULT_MAX_POSITIONS)),
                   eos_token_ids=eos_ids, raw=dict(data))

    @staticmethod
    def _attention(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(f"{where}.mixer", mixer, ("heads", "kv_heads", "dim", "vdim", "scale"))
        out = {
            "heads": _integer(f"{where}.mixer.heads", mixer["heads"]),
            "kv_heads": _integer(f"{where}.mixer.kv_heads", mixer["kv_heads"]),
            "dim": _integer(f"{where}.mixer.dim", mixer["dim"]),
            "vdim": _integer(f"{where}.mixer.vdim", mixer["vdim"]),
            "scale": _number(f"{where}.mixer.scale", mixer["scale"]),
            "mask": None, "rot": None,
        }
        if out["heads"] % out["kv_heads"]:
            raise InvalidArgumentError(f"{where}: heads {out['heads']} is not a multiple of kv_heads {out['kv_heads']}")
        mask = mixer.get("mask")
        if mask is not None:
            _need(f"{where}.mixer.mask", mask, ("size",))
            out["mask"] = {"size": _integer(f"{where}.mixer.mask.size", mask["size"]),
                           "keep_first": _integer(f"{where}.mixer.mask.keep_first", mask.get("keep_first", 0), 0)}
        rot = mixer.get("rot")
        if rot is not None:
            _need(f"{where}.mixer.rot", rot, ("dims", "base"))
            dims = _integer(f"{where}.mixer.rot.dims", rot["dims"], 0)
            if dims % 2 or dims > out["dim"]:
                raise InvalidArgumentError(f"{where}: rot.dims {dims} must be even and at most dim {out['dim']}")
            scaling = rot.get("scaling")
            if scaling is not None:
                _need(f"{where}.mixer.rot.scaling", scaling, ("factor", "original", "fast", "slow"))
                scaling = {key: _number(f"{where}.mixer.rot.scaling.{key}", scaling[key])
                           for key in ("factor", "original", "fast", "slow")}
            if dims:
                out["rot"] = {"dims": dims, "base": _number(f"{where}.mixer.rot.base", rot["base"]), "scaling": scaling}
        return out

    @staticmethod
    def _mlstm(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(f"{where}.mixer", mixer, ("heads", "dim", "vdim", "gate_cap"))
        return {
            "heads": _integer(f"{where}.mixer.heads", mixer["heads"]),
            "dim": _integer(f"{where}.mixer.dim", mixer["dim"]),
            "vdim": _integer(f"{where}.mixer.vdim", mixer["vdim"]),
            "gate_cap": _number(f"{where}.mixer.gate_cap", mixer["gate_cap"]),
        }

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            mixer = {k: v for k, v in layer.mixer.items() if v is not None}
            layers.append({"type": layer.kind, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "layers": layers,
                               "loop": None if self.loop is None else
                               {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    # ---- derived -----------------------------------------------------------------
    def layer_runs(self) -> List[int]:
        """The layers in the order they run: the looped range ``times`` times in a row, the rest once."""
        count = len(self.layers)
        if self.loop is None:
            return list(range(count))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


_NAMES_ATTENTION = ("q", "k", "v", "o")
_NAMES_FF = ("gate", "up", "down")


def nobupel_model_spec(config: NobupelConfig) -> ModelSpec:
    """Nobupel in parts.  Every run of a layer is a schedule entry with a cache slot of its own."""
    norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps})
    layers: List[LayerSpec] = []
    for index, layer in enumerate(config.layers):
        m = layer.mixer
        if layer.kind == "attention":
            mask, rot = m["mask"], m["rot"]
            if rot is None:
                position = PartSpec("none", {})
            else:
                position = PartSpec("rope_neox", {"head_dim": m["dim"], "rotary_dims": rot["dims"], "theta": rot["base"],
                                                  "scaling": rot["scaling"], "max_positions": config.max_positions})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": config.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                "head_dim": m["dim"], "value_dim": m["vdim"], "qkv_bias": True,
                "window": None if mask is None else mask["size"],
                "keep_first": 0 if mask is None else mask["keep_first"],
                "sink": True, "softmax_scale": m["scale"], "position": position,
                "projection_names": _NAMES_ATTENTION,
            })
        else:
            mixer = PartSpec("mlstm", {
                "hidden_size": config.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "gate_cap": m["gate_cap"], "norm_eps": config.eps, "denominator_eps": 1e-6,
            })
        parts = {"mixer_norm": norm, "mixer": mixer}
        names = {"mixer_norm": "norm1", "mixer": "mix"}
        block = "prenorm_mixer"
        if layer.ff is not None:
            block = "prenorm"
            parts.update(ffn_norm=norm, ffn=PartSpec("gated_mlp", {
                "hidden_size": config.width, "intermediate_size": layer.ff, "activation": "gelu_tanh", "bias": True,
                "projection_names": _NAMES_FF}))
            names.update(ffn_norm="norm2", ffn="mlp")
        layers.append(LayerSpec(block=block, prefix=f"l{index}", parts=parts, names=names))
    spec = ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        max_position_embeddings=config.max_positions,
        embedding_name="embed.weight",
        layers=layers,
        schedule=[ScheduleEntry(layer=layer, cache=run) for run, layer in enumerate(config.layer_runs())],
        final_norm=norm,
        final_norm_name="final.norm",
        head_name="head.weight",
    )
    spec.validate()
    return spec


def nobupel_tensor_alias(name: str) -> Optional[str]:
    """The weight file's names as the parts ask for them: a bias is ``<matrix>.b`` in the file and
    ``<matrix>.bias`` to a part; every other tensor gets ``.weight`` added."""
    if name.endswith((".weight", ".bias")):
        return None
    if name.endswith(".b"):
        return name[:-2] + ".bias"
    return name + ".weight"


def nobupel_stored_name(name: str) -> str:
    """The inverse: under which name the weight file stores the tensor a part calls `name`."""
    if name.endswith(".bias"):
        return name[:-len(".bias")] + ".b"
    if name.endswith(".weight"):
        return name[:-len(".weight")]
    return name


register_architecture("Nobupel", NobupelConfig.from_dict, nobupel_model_spec,
                      tensor_alias=nobupel_tensor_alias, stored_name=nobupel_stored_name)
