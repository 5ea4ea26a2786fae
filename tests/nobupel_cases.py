"""Small Nobupel configurations and model folders for the tests, with weights scaled so that
the mechanisms show: sharp attention (one wrong key moves the logits), gates that open and
close, long memory."""
from __future__ import annotations

import functools
import os
import tempfile
from typing import Dict, Optional, Sequence

import numpy as np
import torch

import plain_nobupel as plain


def attention_layer(heads=3, kv_heads=1, dim=24, vdim=40, scale=0.35, size=24, keep_first=3, rot_dims=16,
                    scaling=True, base=5000.0, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        mixer["mask"] = {"size": size, "keep_first": keep_first}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            mixer["rot"]["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm_layer(heads=2, dim=20, vdim=36, gate_cap=9.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=96, vocab=301, eps=2e-6, loop=None):
    return {"architecture": "Nobupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
            "loop": loop}


# Sizes that share nothing: odd widths, one KV head, an inner size that is no multiple of 16, a loop.
MIXED = config([mlstm_layer(), attention_layer(ff=72), mlstm_layer(heads=3, dim=16, vdim=24, gate_cap=15.0, ff=40),
                attention_layer(heads=2, kv_heads=2, dim=32, vdim=16, scale=0.2, size=9, keep_first=0, rot_dims=32,
                                scaling=False)],
               loop={"start": 0, "stop": 2, "times": 2})
# The sizes the tensor-core kernels take: heads of 64, whole heads that turn, every key visible.
WIDE = config([attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=None, rot_dims=64, scaling=False,
                               ff=256),
               mlstm_layer(heads=2, dim=64, vdim=64, ff=128),
               attention_layer(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.11, size=48, keep_first=5, rot_dims=32,
                               ff=None),
               mlstm_layer(heads=1, dim=128, vdim=128, gate_cap=11.0)],
              width=256, vocab=512, eps=1e-5, loop={"start": 1, "stop": 3, "times": 3})
# One layer of each mechanism alone.
ONLY_ATTENTION = config([attention_layer()])
ONLY_ATTENTION_PLAIN = config([attention_layer(size=None, rot_dims=0, scaling=False)])
ONLY_MLSTM = config([mlstm_layer()])
ONLY_FF = config([mlstm_layer(ff=56)])

# Values that the other configurations make equal, even, or absent: a width that is no multiple of
# 8 (no tensor-core products), every key visible and no rotation at all, an odd head size, one head,
# a window longer than any request, kept tokens beyond a page, a looped range that is empty, a cell
# whose value size is no multiple of 4 with a q/k size the tensor-core form takes.
ODD = config([attention_layer(heads=2, kv_heads=2, dim=40, vdim=24, scale=0.3, size=None, rot_dims=0, scaling=False, ff=100),
              mlstm_layer(heads=1, dim=48, vdim=64, gate_cap=12.0),
              attention_layer(heads=1, kv_heads=1, dim=17, vdim=9, scale=0.5, size=1000, keep_first=0, rot_dims=0,
                              scaling=False),
              attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, size=7, keep_first=21, rot_dims=8,
                              scaling=True, ff=16)],
             width=100, vocab=97, eps=1e-4, loop={"start": 2, "stop": 2, "times": 5})
TENSOR = config([mlstm_layer(heads=2, dim=64, vdim=36, gate_cap=6.0, ff=48),
                 mlstm_layer(heads=1, dim=256, vdim=96, gate_cap=20.0),
                 attention_layer(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, size=100, keep_first=70, rot_dims=128,
                                 scaling=True, ff=None)],
                width=200, vocab=211, eps=1e-6, loop={"start": 0, "stop": 3, "times": 2})

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "tensor": TENSOR, "attention": ONLY_ATTENTION, "attention_plain": ONLY_ATTENTION_PLAIN,
           "mlstm": ONLY_MLSTM, "ff": ONLY_FF}
# How the stored tensors are scaled (by the end of their names) so that the mechanisms show.
SHARP = {".mix.q": 6.0, ".mix.k": 6.0, ".mix.i": 12.0, ".mix.f": 12.0, ".mix.v": 3.0, ".mlp.gate": 6.0}
# bfloat16 keeps 8 bits: softmaxes as sharp as above turn its rounding into other answers
MILD = {".mix.q": 2.5, ".mix.k": 2.5, ".mix.i": 4.0, ".mix.f": 4.0, ".mix.v": 2.0, ".mlp.gate": 3.0}
# forget gates held open (a large bias, weights left small): the state reaches hundreds of tokens back
LONG_MEMORY = dict(SHARP, **{".mix.f": 1.0, ".mix.f.b": ("add", 6.0), ".mix.i.b": ("add", -1.0)})


@functools.lru_cache(maxsize=None)
def folder(name: str, store_dtype: str = "float32", seed: int = 5, scaling: str = "sharp") -> str:
    """A model folder of configuration `name` with seeded random weights, scaled."""
    import vipera_rs_b200  # noqa: F401
    from safetensors.torch import load_file, save_file
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix=f"vipera_nobupel_{name}_{store_dtype}_{scaling}_")
    write_random_model(path, CONFIGS[name], seed, store_dtype)
    rules = {"sharp": SHARP, "mild": MILD, "long": LONG_MEMORY, "none": {}}[scaling]
    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for tensor_name in list(tensors):
        for ending, rule in rules.items():
            if tensor_name.endswith(ending):
                value = tensors[tensor_name].to(torch.float32)
                value = value + rule[1] if isinstance(rule, tuple) else value * rule
                tensors[tensor_name] = value.to(tensors[tensor_name].dtype)
    save_file(tensors, file)
    return path


_PLAIN: Dict[tuple, np.ndarray] = {}


def plain_logits(path: str, tokens: Sequence[int], round_to: Optional[torch.dtype] = None) -> np.ndarray:
    key = (path, tuple(tokens), round_to)
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(plain.read_config(path), plain.read_weights(path), list(tokens),
                                    round_to=round_to).numpy()
    return _PLAIN[key]
