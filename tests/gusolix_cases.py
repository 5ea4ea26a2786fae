"""Small Gusolix configurations and model folders for the tests, with weights scaled so that the
mechanisms show: sharp attention (one wrong key moves the logits), decays near one (a token
counts hundreds of tokens later), filters that matter."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, Sequence

import numpy as np
import torch

import plain_gusolix as plain


def ff_of(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def attention_layer(heads=4, kv_heads=2, dim=24, scale=0.4, size=13, rot_dims=16, base=5000.0, scaling=True, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if size is not None:
        mixer["mask"] = {"size": size}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            mixer["rot"]["scaling"] = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    return {"type": "attention", "mixer": mixer, "mlp": ff_of(ff)}


def mamba_layer(inner=80, state=5, dt_rank=3, conv=3, ff=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": ff_of(ff)}


def parallel_layer(heads=3, kv_heads=1, dim=16, vdim=24, scale=0.5, r_heads=3, r_dim=20, r_vdim=12, tau=7.0, rank=5,
                   left_scale=0.6, right_scale=1.3, ff=None):
    return {"type": "parallel", "mlp": ff_of(ff), "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale},
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau, "rank": rank},
        "left_scale": left_scale, "right_scale": right_scale}}


def config(layers, width=72, vocab=211, eps=3e-6, taps=3, scale=5.5):
    return {"architecture": "Gusolix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "canon": {"taps": taps}, "layers": layers}


# Sizes that share nothing with each other.
MIXED = config([mamba_layer(ff=56), attention_layer(), parallel_layer(ff=40),
                attention_layer(heads=2, kv_heads=2, dim=32, scale=0.3, size=None, rot_dims=32, scaling=False, ff=24)])
# Head sizes the tensor-core attention kernels take, a width the tensor-core products take.
WIDE = config([attention_layer(heads=4, kv_heads=1, dim=64, scale=0.2, size=40, rot_dims=64, base=10000.0, ff=256),
               parallel_layer(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, r_heads=2, r_dim=64, r_vdim=128, tau=12.0,
                              rank=16, ff=128),
               mamba_layer(inner=256, state=16, dt_rank=8, conv=4, ff=None),
               attention_layer(heads=2, kv_heads=2, dim=128, scale=0.1, size=100, rot_dims=32, scaling=True, ff=None)],
              width=256, vocab=512, eps=1e-5, taps=4, scale=11.0)
# Values the others make equal, even or absent: a width that is no multiple of 8, one tap (no
# filter state), two taps inside Mamba, one head, one state per channel, a rank of one, no rotation,
# a chunk longer than any request and a chunk of one, a state count that is no power of two.
ODD = config([attention_layer(heads=1, kv_heads=1, dim=18, scale=0.7, size=1000, rot_dims=0, ff=36),
              mamba_layer(inner=52, state=1, dt_rank=1, conv=2),
              parallel_layer(heads=2, kv_heads=2, dim=10, vdim=6, scale=0.9, r_heads=1, r_dim=7, r_vdim=40, tau=1.0, rank=1,
                             left_scale=1.0, right_scale=-0.5),
              attention_layer(heads=6, kv_heads=3, dim=8, scale=1.0, size=1, rot_dims=2, scaling=False, ff=20),
              mamba_layer(inner=24, state=37, dt_rank=9, conv=5, ff=16)],
             width=100, vocab=97, eps=1e-4, taps=1, scale=1.0)
LONG_TAPS = config([mamba_layer(inner=48, state=8, dt_rank=4, conv=7, ff=32), parallel_layer()], width=64, taps=11)
# Products with very few rows against inner sizes the tensor-core products take: a step-size rank and a
# decay rank of one, three states, single heads of eight values.
NARROW = config([mamba_layer(inner=64, state=3, dt_rank=1, conv=2, ff=16),
                 parallel_layer(heads=1, kv_heads=1, dim=8, vdim=8, scale=0.6, r_heads=1, r_dim=8, r_vdim=8, tau=3.0, rank=1),
                 attention_layer(heads=1, kv_heads=1, dim=8, scale=0.5, size=5, rot_dims=4, scaling=False)],
                width=64, vocab=50, taps=2)
ONLY_ATTENTION = config([attention_layer()])
ONLY_MAMBA = config([mamba_layer()])
ONLY_PARALLEL = config([parallel_layer()])
ONLY_FF = config([attention_layer(ff=56)])

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "long_taps": LONG_TAPS, "narrow": NARROW, "attention": ONLY_ATTENTION,
           "mamba": ONLY_MAMBA, "parallel": ONLY_PARALLEL, "ff": ONLY_FF}

# How stored tensors are changed (by the end of their names): ("mul", x) or ("add", x).
SHARP = {".q.norm": ("mul", 3.0), ".k.norm": ("mul", 3.0), ".mix.k": ("mul", 30.0), ".left.v": ("mul", 30.0),
         ".right.k": ("mul", 20.0), ".right.v": ("mul", 20.0), ".right.q": ("mul", 20.0), ".mix.in": ("mul", 20.0),
         ".mix.x": ("mul", 10.0), ".mlp.gate": ("mul", 20.0), ".mlp.up": ("mul", 20.0)}
MILD = {".q.norm": ("mul", 1.5), ".k.norm": ("mul", 1.5), ".mix.k": ("mul", 30.0), ".left.v": ("mul", 30.0),
        ".right.k": ("mul", 20.0), ".right.v": ("mul", 20.0), ".right.q": ("mul", 20.0), ".mix.in": ("mul", 20.0),
        ".mix.x": ("mul", 10.0), ".mlp.gate": ("mul", 20.0), ".mlp.up": ("mul", 20.0)}
# decays near one: the linear attention forgets 1 - sigmoid(7)^(1/tau) a token, Mamba's steps are small
LONG_MEMORY = dict(SHARP, **{".right.a2.b": ("add", 7.0), ".mix.dt.b": ("add", -5.0), ".mix.A_log": ("add", -1.0)})
RULES = {"sharp": SHARP, "mild": MILD, "long": LONG_MEMORY, "none": {}}


@functools.lru_cache(maxsize=None)
def folder(name: str, store_dtype: str = "float32", seed: int = 7, scaling: str = "sharp") -> str:
    """A model folder of configuration `name` with seeded random weights, scaled."""
    import vipera_rs_b200  # noqa: F401
    from safetensors.torch import load_file, save_file
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix=f"vipera_gusolix_{name}_{store_dtype}_{scaling}_")
    write_random_model(path, CONFIGS[name], seed, store_dtype)
    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for tensor_name in list(tensors):
        for ending, (how, amount) in RULES[scaling].items():
            if tensor_name.endswith(ending):
                value = tensors[tensor_name].to(torch.float32)
                value = value + amount if how == "add" else value * amount
                tensors[tensor_name] = value.to(tensors[tensor_name].dtype)
    save_file(tensors, file)
    return path


def read(path: str):
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as handle:
        return json.load(handle), load_file(os.path.join(path, "model.safetensors"))


_PLAIN: Dict[tuple, np.ndarray] = {}


def plain_logits(path: str, tokens: Sequence[int]) -> np.ndarray:
    key = (path, tuple(tokens))
    if key not in _PLAIN:
        config, weights = read(path)
        _PLAIN[key] = plain.forward(config, weights, list(tokens)).numpy()
    return _PLAIN[key]
