"""A plain, slow implementation of the Gusolix decoder in float64: one function per mechanism,
whole sequences at once or token by token, no code shared with the package.

``weights`` maps the names of the design's own weight file (``embed``, ``l0.mix.q``,
``l0.norm1.b``, ...) to tensors; ``config`` is the design's config.json as a dict.

Notation.  A layer is ``x += LN1(mixer(c1(x)))`` then ``x += LN2(ff(c2(x)))`` with
``c(h) = h + conv(h)``, a causal convolution per channel.  Mixers: softmax attention whose
values are the raw keys (chunk mask, norm over the whole q and k rows, partial rotation with
Llama-3.1 frequency scaling); Mamba's selective scan; and a pair side by side of softmax
attention with mixed head weights and gated linear attention.
"""
import math

import torch

F = torch.float64


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(h, taps_weight, bias=None):
    """h [T, C], taps_weight [C, taps]: out_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before t = 0."""
    count, taps = h.shape[0], taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, h.shape[1], dtype=F), h])
    out = torch.zeros_like(h)
    for j in range(taps):
        out += padded[j:j + count] * taps_weight[:, j]
    if bias is not None:
        out = out + bias
    return out


def rotary_frequencies(dims, base, scaling):
    index = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * index / dims)
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for f in freq.tolist():
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                out.append(f)
            elif wavelength > original / low:
                out.append(f / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        freq = torch.tensor(out, dtype=F)
    return freq


def rotate(x, positions, freq, dims):
    """x [T, heads, d]: the first `dims` values of each head turn, value i with value i + dims/2."""
    half = dims // 2
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def visible(count, chunk=None):
    i = torch.arange(count)[:, None]
    j = torch.arange(count)[None, :]
    mask = j <= i
    if chunk:
        mask &= (i // chunk) == (j // chunk)
    return mask


def softmax_weights(q, k, scale, mask, group):
    """q [T, H, d], k [T, G, d] -> weights [H, T, T] (float64), query head h on kv head h // group."""
    heads = q.shape[1]
    out = []
    for h in range(heads):
        scores = (q[:, h] @ k[:, h // group].T) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(scores, dim=-1))
    return torch.stack(out)


def attention_mixer(w, prefix, m, h, eps):
    """Chunk-masked softmax attention whose values are the keys as projected."""
    heads, kv_heads, d = m["heads"], m["kv_heads"], m["dim"]
    count = h.shape[0]
    q = h @ w[prefix + "q"].T
    k = h @ w[prefix + "k"].T
    v = k.clone().view(count, kv_heads, d)
    q = (unit_rms(q, eps) * w[prefix + "q.norm"]).view(count, heads, d)
    k = (unit_rms(k, eps) * w[prefix + "k.norm"]).view(count, kv_heads, d)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        freq = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        positions = torch.arange(count)
        q, k = rotate(q, positions, freq, rot["dims"]), rotate(k, positions, freq, rot["dims"])
    mask = visible(count, (m.get("mask") or {}).get("size"))
    group = heads // kv_heads
    weights = softmax_weights(q, k, m["scale"], mask, group)
    out = torch.stack([weights[hd] @ v[:, hd // group] for hd in range(heads)], dim=1)
    return out.reshape(count, -1) @ w[prefix + "o"].T


def talking_attention(w, prefix, m, h, eps):
    """Causal softmax attention without positions whose head weights are mixed by a matrix."""
    heads, kv_heads, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    count = h.shape[0]
    q = h @ w[prefix + "q"].T
    k = h @ w[prefix + "k"].T
    v = (h @ w[prefix + "v"].T).view(count, kv_heads, dv)
    q = (unit_rms(q, eps) * w[prefix + "q.norm"]).view(count, heads, d)
    k = (unit_rms(k, eps) * w[prefix + "k.norm"]).view(count, kv_heads, d)
    group = heads // kv_heads
    weights = softmax_weights(q, k, m["scale"], visible(count), group)
    mixed = torch.einsum("hg,gij->hij", w[prefix + "talk"], weights)
    out = torch.stack([mixed[hd] @ v[:, hd // group] for hd in range(heads)], dim=1)
    return out.reshape(count, -1) @ w[prefix + "o"].T


def gated_linear_attention(w, prefix, m, h, eps):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    heads, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    count = h.shape[0]
    q = (h @ w[prefix + "q"].T).view(count, heads, d) * d ** -0.5
    k = (h @ w[prefix + "k"].T).view(count, heads, d)
    v = (h @ w[prefix + "v"].T).view(count, heads, dv)
    z = (h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / tau)).view(count, heads, d)
    state = torch.zeros(heads, d, dv, dtype=F)
    outs = []
    for t in range(count):
        state = alpha[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", state, q[t]))
    o = torch.stack(outs)
    o = unit_rms(o, eps) * w[prefix + "norm"]
    return (o.reshape(count, -1) * silu(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


def parallel_mixer(w, prefix, m, h, eps):
    left = talking_attention(w, prefix + "left.", m["left"], h, eps)
    right = gated_linear_attention(w, prefix + "right.", m["right"], h, eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mamba_mixer(w, prefix, m, h, eps):
    inner, state_size, rank = m["inner"], m["state"], m["dt_rank"]
    count = h.shape[0]
    xz = h @ w[prefix + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[prefix + "conv"], w[prefix + "conv.b"]))
    dbc = x @ w[prefix + "x"].T
    dt = softplus(dbc[:, :rank] @ w[prefix + "dt"].T + w[prefix + "dt.b"])
    b, c = dbc[:, rank:rank + state_size], dbc[:, rank + state_size:]
    a = -torch.exp(w[prefix + "A_log"])
    state = torch.zeros(inner, state_size, dtype=F)
    ys = []
    for t in range(count):
        state = torch.exp(dt[t][:, None] * a) * state + (dt[t] * x[t])[:, None] * b[t][None, :]
        ys.append(state @ c[t] + w[prefix + "D"] * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ w[prefix + "o"].T


def dense_ff(w, prefix, h):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


MIXERS = {"attention": attention_mixer, "mamba1": mamba_mixer, "parallel": parallel_mixer}


def forward(config, weights, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence (float64); with keep_layers also the residual stream
    after every layer."""
    w = {name: value.to(F) for name, value in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    kept = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = x + causal_conv(x, w[p + "canon1"])
        y = MIXERS[layer["type"]](w, p + "mix.", layer["mixer"], h, eps)
        x = x + layer_norm(y, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            h = x + causal_conv(x, w[p + "canon2"])
            y = dense_ff(w, p + "mlp.", h)
            x = x + layer_norm(y, w[p + "norm2"], w[p + "norm2.b"], eps)
        kept.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    return (logits, torch.stack(kept)) if keep_layers else logits
