"""A plain, slow implementation of the Nobupel decoder for the tests to compare with.

Whole sequences, token by token where the design is recurrent, no cache, no batching, one
function for each mechanism.  It shares no code with the package under test: it reads
config.json and model.safetensors by itself and works on host tensors in float64 (angles of
the rotation in float32, as an engine computes them).

The design in short.  A stack of pre-norm layers, each ``x += mixer(norm1(x))`` and, where the
layer has a feed-forward, ``x += ff(norm2(x))``.  Two mixers: grouped-query attention with a
sliding window that keeps the first tokens, partial rotary positions with YaRN scaling and a
softmax whose denominator has one added; and the matrix-memory cell of xLSTM (mLSTM) with
capped gates.  A range of layers may run several times in a row with the same weights.

``round_to`` names a storage dtype (bfloat16) whose rounding is applied where a bfloat16
engine stores activations: the input of each matrix product, q, keys and values, and the
mixers' outputs in front of their output products.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        return json.load(handle)


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(os.path.join(model_dir, "model.safetensors"))


def _rounded(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


def layer_runs(config: dict) -> List[int]:
    """The layers in the order they run: the looped range ``times`` times, then the rest."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


# --------------------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """Each row divided by sqrt(mean of squares + eps), then scaled."""
    out = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return out if weight is None else out * weight.to(x.dtype)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot: dict):
    """(frequency per pair [dims/2], the factor on cos and sin).  Plain: base^(-2i/dims).  With
    YaRN scaling each frequency is blended between itself and itself / factor by a ramp over the
    pair index, whose ends are the pairs that turn ``fast`` and ``slow`` times within the
    original length; cos and sin are then stretched by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    index = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * index / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    high = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((index - low) / max(high - low, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x is [tokens, heads, d]; the first ``dims`` values of a head turn, value i with value
    i + dims/2; the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, stretch = rotary_frequencies(rot)
    angle = positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]   # 32-bit angles
    cos = (torch.cos(angle) * stretch).to(x.dtype)[:, None, :]
    sin = (torch.sin(angle) * stretch).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if not mask:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], mixer: dict, positions: torch.Tensor,
                    round_to=None) -> torch.Tensor:
    """Grouped-query attention.  p_j = exp(s_j) / (1 + sum_j exp(s_j)): a sink of score 0
    without a value."""
    heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
    d, dv = int(mixer["dim"]), int(mixer["vdim"])
    count = h.shape[0]
    hin = _rounded(h, round_to)
    q = (hin @ w["q"].T + w["q.b"]).view(count, heads, d)
    k = (hin @ w["k"].T + w["k.b"]).view(count, kv_heads, d)
    v = (hin @ w["v"].T + w["v.b"]).view(count, kv_heads, dv)
    if mixer.get("rot"):
        q, k = rotate(q, positions, mixer["rot"]), rotate(k, positions, mixer["rot"])
    q, k, v = _rounded(q, round_to), _rounded(k, round_to), _rounded(v, round_to)
    out = torch.zeros(count, heads, dv, dtype=h.dtype)
    group = heads // kv_heads
    scale = float(mixer["scale"])
    mask = mixer.get("mask")
    pos = [int(p) for p in positions]
    for head in range(heads):
        kv = head // group
        scores = (q[:, head] @ k[:, kv].T) * scale                      # [query, key]
        for i in range(count):
            seen = [j for j in range(count) if visible(pos[i], pos[j], mask)]
            s = scores[i, seen]
            top = max(float(s.max()), 0.0)
            e = torch.exp(s - top)
            p = e / (math.exp(-top) + e.sum())
            out[i, head] = p @ v[seen, kv]
    mixed = _rounded(out.reshape(count, heads * dv), round_to)
    return mixed @ w["o"].T


def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], mixer: dict, eps: float, state=None,
                round_to=None):
    """The mLSTM cell, one token after another.  Per head a matrix S [d, dv], a vector n [d]
    and a running maximum m, all zero at the start.  Returns (output [tokens, width], state)."""
    heads, d, dv = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    cap = float(mixer["gate_cap"])
    count = h.shape[0]
    hin = _rounded(h, round_to)
    q = _rounded((hin @ w["q"].T).view(count, heads, d), round_to) * d ** -0.5
    k = _rounded((hin @ w["k"].T).view(count, heads, d), round_to)
    v = _rounded((hin @ w["v"].T).view(count, heads, dv), round_to)
    gate_out = torch.sigmoid(_rounded(hin @ w["g"].T, round_to))
    log_in = cap * torch.tanh((hin @ w["i"].T + w["i.b"]) / cap)                       # [tokens, heads]
    log_forget = torch.nn.functional.logsigmoid(cap * torch.tanh((hin @ w["f"].T + w["f.b"]) / cap))
    if state is None:
        state = (torch.zeros(heads, d, dv, dtype=h.dtype), torch.zeros(heads, d, dtype=h.dtype),
                 torch.zeros(heads, dtype=h.dtype))
    S, n, m = (t.clone() for t in state)
    out = torch.zeros(count, heads, dv, dtype=h.dtype)
    for t in range(count):
        m_new = torch.maximum(log_forget[t] + m, log_in[t])
        keep = torch.exp(log_forget[t] + m - m_new)
        take = torch.exp(log_in[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        top = torch.einsum("hdv,hd->hv", S, q[t])
        bottom = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = top / bottom[:, None]
    normed = rms_norm(out, None, eps).reshape(count, heads * dv) * w["norm"].to(h.dtype)
    mixed = _rounded(normed * gate_out, round_to)
    return mixed @ w["o"].T, (S, n, m)


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], round_to=None) -> torch.Tensor:
    hin = _rounded(h, round_to)
    gate = hin @ w["gate"].T + w["gate.b"]
    up = hin @ w["up"].T + w["up.b"]
    act = _rounded(gelu_tanh(gate) * up, round_to)
    return act @ w["down"].T + w["down.b"]


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------
def _sub(weights: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {name[len(prefix):]: t.to(dtype) for name, t in weights.items() if name.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            round_to=None, return_layers: bool = False):
    """Logits [tokens, vocab] of one sequence from position 0 (and, where asked, the residual
    stream after every layer run, [runs, tokens, width])."""
    eps = float(config["norm"]["eps"])
    index = torch.as_tensor(list(tokens), dtype=torch.long)
    x = weights["embed"].to(dtype)[index]
    positions = torch.arange(len(tokens))
    streams = []
    for layer in layer_runs(config):
        spec = config["layers"][layer]
        name = f"l{layer}."
        h = rms_norm(x, weights[name + "norm1"].to(dtype), eps)
        mix = _sub(weights, name + "mix.", dtype)
        if spec["type"] == "attention":
            x = x + attention_mixer(h, mix, spec["mixer"], positions, round_to)
        elif spec["type"] == "mlstm":
            x = x + mlstm_mixer(h, mix, spec["mixer"], eps, None, round_to)[0]
        else:
            raise ValueError(f"unknown mixer {spec['type']!r}")
        if spec.get("mlp"):
            if spec["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward {spec['mlp']['kind']!r}")
            h = rms_norm(x, weights[name + "norm2"].to(dtype), eps)
            x = x + dense_ff(h, _sub(weights, name + "mlp.", dtype), round_to)
        streams.append(x)
    h = rms_norm(x, weights["final.norm"].to(dtype), eps)
    logits = _rounded(h, round_to) @ weights["head"].to(dtype).T
    if return_layers:
        return logits, torch.stack(streams)
    return logits
