"""Typed configuration of the Gusolix decoder, read from the keys of its own config.json, and
its description in terms of parts.

The design: the embedding rows are scaled; every sublayer reads the residual stream itself
after a short causal convolution over time has been added to it (``h + conv(h)``, one filter
per channel), and its output is layer-normed before it joins the stream:
``x += LN1(mixer(c1(x)))``, then ``x += LN2(ff(c2(x)))``.  Three mixers: softmax attention
whose values are its keys as projected (RMS norm over the whole q and k rows, rotation of the
first values of a head with Llama-3.1 frequency scaling, a mask of chunks); Mamba's selective
scan; and two mixers side by side, softmax attention with mixed head weights beside gated
linear attention.  The feed-forward is a gated unit with silu; the model ends with a layer
norm and an output matrix of its own.

config.json keys: ``architecture`` ("Gusolix"), ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``canon.taps`` and ``layers`` (a list of ``{type, mixer, mlp}``).  Tensor
names in the weight file: ``embed``, ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.<name>``,
``l<i>.mlp.<name>``, biases with ``.b`` added, ``final.norm``, ``head``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import InvalidArgumentError, UnsupportedError
from .nobupel import DEFAULT_MAX_POSITIONS, _integer, _need, _number, nobupel_stored_name, nobupel_tensor_alias
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class GusolixLayer:
    kind: str                       # "attention", "mamba1" or "parallel"
    mixer: Dict[str, Any]           # the mixer's sizes and constants, checked
    ff: Optional[int]               # the feed-forward's inner size, None for a layer without one


def _softmax_heads(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
    _need(where, mixer, ("heads", "kv_heads", "dim", "vdim", "scale"))
    out = {
        "heads": _integer(f"{where}.heads", mixer["heads"]),
        "kv_heads": _integer(f"{where}.kv_heads", mixer["kv_heads"]),
        "dim": _integer(f"{where}.dim", mixer["dim"]),
        "vdim": _integer(f"{where}.vdim", mixer["vdim"]),
        "scale": _number(f"{where}.scale", mixer["scale"]),
    }
    if out["heads"] % out["kv_heads"]:
        raise InvalidArgumentError(f"{where}: heads {out['heads']} is not a multiple of kv_heads {out['kv_heads']}")
    return out


@dataclass(frozen=True)
class GusolixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    taps: int
    layers: Tuple[GusolixLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Gusolix"
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "GusolixConfig":
        _need("the configuration", data, ("vocab", "width", "layers", "norm", "embedding", "canon"))
        _need("norm", data["norm"], ("eps",))
        _need("embedding", data["embedding"], ("scale",))
        _need("canon", data["canon"], ("taps",))
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise InvalidArgumentError("layers must be a list with at least one layer")
        layers = []
        for index, entry in enumerate(data["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, ("type", "mixer"))
            kind, mixer = entry["type"], entry["mixer"]
            if kind == "attention":
                checked = cls._attention(f"{where}.mixer", mixer)
            elif kind == "mamba1":
                checked = cls._mamba(f"{where}.mixer", mixer)
            elif kind == "parallel":
                checked = cls._parallel(f"{where}.mixer", mixer)
            else:
                raise UnsupportedError(f"{where}: unknown mixer type {kind!r}; known: attention, mamba1, parallel")
            ff = None
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(f"{where}.mlp", mlp, ("kind", "ff"))
                if mlp["kind"] != "dense":
                    raise UnsupportedError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
                ff = _integer(f"{where}.mlp.ff", mlp["ff"])
            layers.append(GusolixLayer(kind, checked, ff))
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(vocab=_integer("vocab", data["vocab"]), width=_integer("width", data["width"]),
                   eps=_number("norm.eps", data["norm"]["eps"]),
                   embedding_scale=_number("embedding.scale", data["embedding"]["scale"]),
                   taps=_integer("canon.taps", data["canon"]["taps"]), layers=tuple(layers),
                   max_positions=_integer("max_positions", data.get("max_positions", DEFAULT_MAX_POSITIONS)),
                   eos_token_ids=eos_ids, raw=dict(data))

    @staticmethod
    def _attention(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        out = _softmax_heads(where, mixer)
        if out["vdim"] != out["dim"]:
            raise InvalidArgumentError(f"{where}: the values are the keys, so vdim {out['vdim']} must equal dim {out['dim']}")
        out.update(mask=None, rot=None)
        mask = mixer.get("mask")
        if mask is not None:
            _need(f"{where}.mask", mask, ("size",))
            out["mask"] = {"size": _integer(f"{where}.mask.size", mask["size"])}
        rot = mixer.get("rot")
        if rot is not None:
            _need(f"{where}.rot", rot, ("dims", "base"))
            dims = _integer(f"{where}.rot.dims", rot["dims"], 0)
            if dims % 2 or dims > out["dim"]:
                raise InvalidArgumentError(f"{where}: rot.dims {dims} must be even and at most dim {out['dim']}")
            scaling = rot.get("scaling")
            if scaling is not None:
                keys = ("factor", "low", "high", "original")
                _need(f"{where}.rot.scaling", scaling, keys)
                scaling = {key: _number(f"{where}.rot.scaling.{key}", scaling[key]) for key in keys}
                if not scaling["high"] > scaling["low"]:
                    raise InvalidArgumentError(f"{where}.rot.scaling: high must be above low")
            if dims:
                out["rot"] = {"dims": dims, "base": _number(f"{where}.rot.base", rot["base"]), "scaling": scaling}
        return out

    @staticmethod
    def _mamba(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mixer, ("inner", "state", "dt_rank", "conv"))
        return {key: _integer(f"{where}.{key}", mixer[key]) for key in ("inner", "state", "dt_rank", "conv")}

    @staticmethod
    def _parallel(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mixer, ("left", "right", "left_scale", "right_scale"))
        right = mixer["right"]
        _need(f"{where}.right", right, ("heads", "dim", "vdim", "tau"))
        return {
            "left": _softmax_heads(f"{where}.left", mixer["left"]),
            "right": {"heads": _integer(f"{where}.right.heads", right["heads"]),
                      "dim": _integer(f"{where}.right.dim", right["dim"]),
                      "vdim": _integer(f"{where}.right.vdim", right["vdim"]),
                      "tau": _number(f"{where}.right.tau", right["tau"]),
                      # the inner size of the decay's two matrices; where config.json is silent the
                      # stored tensors decide
                      "rank": None if right.get("rank") is None else _integer(f"{where}.right.rank", right["rank"])},
            "left_scale": _number(f"{where}.left_scale", mixer["left_scale"], positive=False),
            "right_scale": _number(f"{where}.right_scale", mixer["right_scale"], positive=False),
        }

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            mixer = {k: v for k, v in layer.mixer.items() if v is not None}
            for key in ("rot", "right"):
                if isinstance(mixer.get(key), dict):
                    mixer[key] = {k: v for k, v in mixer[key].items() if v is not None}
            layers.append({"type": layer.kind, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                               "canon": {"taps": self.taps}, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _attention_part(config: GusolixConfig, m: Dict[str, Any]) -> PartSpec:
    """The design's own attention: values are the raw keys, norm over whole rows, chunk mask."""
    rot = m["rot"]
    if rot is None:
        position = PartSpec("none", {})
    else:
        scaling = None if rot["scaling"] is None else {"kind": "llama3", **rot["scaling"]}
        position = PartSpec("rope_neox", {"head_dim": m["dim"], "rotary_dims": rot["dims"], "theta": rot["base"],
                                          "scaling": scaling, "max_positions": config.max_positions})
    return PartSpec("gqa_attention", {
        "hidden_size": config.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
        "head_dim": m["dim"], "value_dim": m["vdim"], "qkv_bias": False, "window": None,
        "chunk": None if m["mask"] is None else m["mask"]["size"], "values_from_keys": True,
        "row_norm": True, "norm_eps": config.eps,
        "softmax_scale": m["scale"], "position": position, "projection_names": ("q", "k", "v", "o"),
    })


def _parallel_part(config: GusolixConfig, m: Dict[str, Any]) -> PartSpec:
    left, right = m["left"], m["right"]
    softmax = PartSpec("gqa_attention", {
        "hidden_size": config.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
        "head_dim": left["dim"], "value_dim": left["vdim"], "qkv_bias": False, "window": None,
        "row_norm": True, "norm_eps": config.eps, "talking_heads": True,
        "softmax_scale": left["scale"], "position": PartSpec("none", {}), "projection_names": ("q", "k", "v", "o"),
    })
    linear = PartSpec("gla", {
        "hidden_size": config.width, "num_heads": right["heads"], "head_dim": right["dim"],
        "value_dim": right["vdim"], "tau": right["tau"], "norm_eps": config.eps,
        "decay_rank": right["rank"],
    })
    return PartSpec("parallel", {"branches": (("left", softmax, m["left_scale"]), ("right", linear, m["right_scale"]))})


def gusolix_model_spec(config: GusolixConfig) -> ModelSpec:
    """Gusolix in parts."""
    norm = PartSpec("layernorm", {"size": config.width, "eps": config.eps})
    layers: List[LayerSpec] = []
    for index, layer in enumerate(config.layers):
        m = layer.mixer
        if layer.kind == "attention":
            mixer = _attention_part(config, m)
        elif layer.kind == "mamba1":
            mixer = PartSpec("mamba1", {"hidden_size": config.width, "inner": m["inner"], "state": m["state"],
                                        "dt_rank": m["dt_rank"], "taps": m["conv"]})
        else:
            mixer = _parallel_part(config, m)
        parts = {"mixer": mixer, "mixer_norm": norm}
        names = {"mixer_norm": "norm1", "mixer": "mix", "mixer_conv": "canon1", "ffn_conv": "canon2"}
        if layer.ff is not None:
            parts.update(ffn_norm=norm, ffn=PartSpec("gated_mlp", {
                "hidden_size": config.width, "intermediate_size": layer.ff, "activation": "silu", "bias": False,
                "projection_names": ("gate", "up", "down")}))
            names.update(ffn_norm="norm2", ffn="mlp")
        layers.append(LayerSpec(block="outnorm_conv", prefix=f"l{index}", parts=parts, names=names,
                                params={"taps": config.taps, "hidden_size": config.width}))
    spec = ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        max_position_embeddings=config.max_positions,
        embedding_name="embed.weight",
        layers=layers,
        schedule=[ScheduleEntry(layer=index, cache=index) for index in range(len(layers))],
        final_norm=norm,
        final_norm_name="final.norm",
        head_name="head.weight",
        embedding_scale=config.embedding_scale,
    )
    spec.validate()
    return spec


_SECOND_SUBLAYER = re.compile(r"^l(\d+)\.(norm2\.(weight|bias)|canon2\.weight)$")


def gusolix_ignorable(config: GusolixConfig, name: str) -> bool:
    """A file may hold the second sublayer's norm and filter for a layer without a feed-forward;
    nothing reads them."""
    match = _SECOND_SUBLAYER.match(name)
    return bool(match) and int(match.group(1)) < len(config.layers) and config.layers[int(match.group(1))].ff is None


register_architecture("Gusolix", GusolixConfig.from_dict, gusolix_model_spec,
                      tensor_alias=nobupel_tensor_alias, stored_name=nobupel_stored_name, ignorable=gusolix_ignorable)
