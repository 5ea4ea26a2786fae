"""Gusolix without a GPU: configuration, tensor names, what a layer keeps between steps, the
frequency tables, and the plain implementation against other ways of writing its mechanisms."""
import json
import math
import os

import numpy as np
import pytest
import torch

import gusolix_cases as cases
import plain_gusolix as plain
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.cache.pools import plan_groups
from vipera_rs_b200.config import architecture_of
from vipera_rs_b200.engine.planner import plan_memory, spec_cache_requests
from vipera_rs_b200.parts.base import CacheBundle, FixedState, PagedKV, bundle_views, flatten_cache_requests
from vipera_rs_b200.parts.model import model_schema
from vipera_rs_b200.parts.rotary import rotary_tables


def spec_of(name):
    arch = architecture_of(cases.CONFIGS[name])
    return arch, arch.model_spec(arch.config_from_dict(cases.CONFIGS[name]))


def test_configuration_reads_back_and_refuses_what_it_does_not_know():
    arch, _ = spec_of("mixed")
    config = arch.config_from_dict(cases.MIXED)
    assert arch.config_from_dict(config.to_dict()) == config
    assert config.taps == 3 and config.embedding_scale == 5.5 and [l.kind for l in config.layers] == \
        ["mamba1", "attention", "parallel", "attention"]
    bad = json.loads(json.dumps(cases.MIXED))
    bad["layers"][0]["type"] = "lstm"
    with pytest.raises(errors.UnsupportedError):
        arch.config_from_dict(bad)
    bad = json.loads(json.dumps(cases.MIXED))
    bad["layers"][1]["mixer"]["vdim"] = 8        # the values are the keys
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)
    bad = json.loads(json.dumps(cases.MIXED))
    del bad["canon"]
    with pytest.raises(errors.UnsupportedError):
        arch.config_from_dict(bad)


def test_tensor_names_of_a_written_folder():
    path = cases.folder("mixed", "bfloat16", scaling="none")
    _, weights = cases.read(path)
    names = set(weights)
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.canon1", "l0.canon2", "l0.norm1.b", "l0.mix.in",
            "l0.mix.conv", "l0.mix.conv.b", "l0.mix.x", "l0.mix.dt", "l0.mix.dt.b", "l0.mix.A_log", "l0.mix.D",
            "l1.mix.q.norm", "l1.mix.k.norm", "l2.mix.left.talk", "l2.mix.right.a1", "l2.mix.right.a2.b",
            "l2.mix.right.norm"} <= names
    assert "l1.mix.v" not in names and "l1.canon2" not in names and "l1.norm2" not in names   # no value matrix, no feed-forward
    assert tuple(weights["l2.mix.right.a1"].shape) == (5, 72) and tuple(weights["l2.mix.right.a2"].shape) == (60, 5)
    assert tuple(weights["l0.mix.x"].shape) == (3 + 2 * 5, 80) and tuple(weights["l0.canon1"].shape) == (72, 3)


def test_the_decay_rank_comes_from_the_stored_tensors():
    arch, _ = spec_of("mixed")
    open_rank = json.loads(json.dumps(cases.MIXED))
    del open_rank["layers"][2]["mixer"]["right"]["rank"]
    schema = model_schema(arch.model_spec(arch.config_from_dict(open_rank)))
    assert schema["l2.mix.right.a1.weight"].shape == (None, 72) and schema["l2.mix.right.a2.weight"].shape == (60, None)


def test_what_layers_keep_between_steps():
    _, spec = spec_of("mixed")
    requests = spec_cache_requests(spec)
    conv = FixedState((2, 2, 72), torch.float32)
    assert requests[0] == CacheBundle((("conv", conv), ("mixer", CacheBundle(
        (("conv", FixedState((2, 80), torch.float32)), ("scan", FixedState((400,), torch.float32)))))))
    assert requests[1] == CacheBundle((("conv", FixedState((1, 2, 72), torch.float32)), ("mixer", PagedKV(2, 24, None))))
    assert dict(requests[2].members)["mixer"] == CacheBundle(
        (("left", PagedKV(1, 16, None, value_dim=24)), ("right", FixedState((3 * 20 * 12,), torch.float32))))
    flat = flatten_cache_requests(requests)
    assert set(flat) == {(0, "conv"), (0, "mixer.conv"), (0, "mixer.scan"), (1, "conv"), (1, "mixer"), (2, "conv"),
                         (2, "mixer.left"), (2, "mixer.right"), (3, "conv"), (3, "mixer")}
    groups, states = plan_groups(requests)
    assert len(groups) == 3 and len(states) == 7
    views = bundle_views(requests[2], 2, {key: key for key in flat})
    assert views == {"conv": (2, "conv"), "mixer": {"left": (2, "mixer.left"), "right": (2, "mixer.right")}}
    # one tap: nothing of the stream is kept
    _, odd = spec_of("odd")
    assert dict(spec_cache_requests(odd)[0].members).keys() == {"mixer"}
    plan = plan_memory(spec, 256, 4, "bfloat16", device_bytes=10**9)
    assert plan["feasible"] and plan["kv_bytes"] > 0


def test_frequency_tables_follow_the_wavelength_rule():
    scaling = {"kind": "llama3", "factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    cos, sin = rotary_tables(16, 5000.0, 50, "cpu", scaling).pair
    want = plain.rotary_frequencies(16, 5000.0, scaling)
    plain_freq = plain.rotary_frequencies(16, 5000.0, None)
    kinds = {"kept": 0, "slowed": 0, "blended": 0}
    for f, g in zip(plain_freq.tolist(), want.tolist()):
        kinds["kept" if g == f else "slowed" if abs(g - f / 8.0) < 1e-15 else "blended"] += 1
    assert min(kinds.values()) >= 1, kinds          # the constants reach all three branches
    angle = torch.arange(50, dtype=torch.float64)[:, None] * want[None, :]
    assert torch.allclose(cos.double(), torch.cos(angle), atol=2e-5) and torch.allclose(sin.double(), torch.sin(angle), atol=2e-5)


def test_plain_mechanisms_against_other_ways_of_writing_them():
    torch.manual_seed(3)
    # gated linear attention: the recurrence unrolled as a sum over earlier tokens
    config, weights = cases.read(cases.folder("parallel", "float32", scaling="sharp"))
    w = {k: v.double() for k, v in weights.items()}
    m = config["layers"][0]["mixer"]["right"]
    h = torch.randn(9, config["width"], dtype=torch.float64)
    got = plain.gated_linear_attention(w, "l0.mix.right.", m, h, 3e-6)
    heads, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["l0.mix.right.q"].T).view(9, heads, d) * d ** -0.5
    k = (h @ w["l0.mix.right.k"].T).view(9, heads, d)
    v = (h @ w["l0.mix.right.v"].T).view(9, heads, dv)
    log_alpha = torch.nn.functional.logsigmoid((h @ w["l0.mix.right.a1"].T) @ w["l0.mix.right.a2"].T + w["l0.mix.right.a2.b"]) / m["tau"]
    log_alpha = log_alpha.view(9, heads, d)
    o = torch.zeros(9, heads, dv, dtype=torch.float64)
    for t in range(9):
        for s in range(t + 1):
            decay = torch.exp(log_alpha[s + 1:t + 1].sum(0))            # [heads, d]
            o[t] += torch.einsum("hd,hd,hv->hv", q[t] * decay, k[s], v[s])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 3e-6) * w["l0.mix.right.norm"]
    want = (o.reshape(9, -1) * plain.silu(h @ w["l0.mix.right.g"].T)) @ w["l0.mix.right.o"].T
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-9)
    # mixed head weights with the identity are plain attention heads
    left = config["layers"][0]["mixer"]["left"]
    w2 = dict(w)
    w2["l0.mix.left.talk"] = torch.eye(left["heads"], dtype=torch.float64)
    got = plain.talking_attention(w2, "l0.mix.left.", left, h, 3e-6)
    count = 9
    qn = (plain.unit_rms(h @ w["l0.mix.left.q"].T, 3e-6) * w["l0.mix.left.q.norm"]).view(count, left["heads"], left["dim"])
    kn = (plain.unit_rms(h @ w["l0.mix.left.k"].T, 3e-6) * w["l0.mix.left.k.norm"]).view(count, left["kv_heads"], left["dim"])
    vv = (h @ w["l0.mix.left.v"].T).view(count, left["kv_heads"], left["vdim"])
    rows = []
    for t in range(count):
        heads_out = []
        for hd in range(left["heads"]):
            kv = hd // (left["heads"] // left["kv_heads"])
            scores = torch.stack([(qn[t, hd] * kn[s, kv]).sum() * left["scale"] for s in range(t + 1)])
            p = torch.exp(scores - scores.max())
            heads_out.append((p / p.sum()) @ vv[:t + 1, kv])
        rows.append(torch.cat(heads_out))
    assert torch.allclose(got, torch.stack(rows) @ w["l0.mix.left.o"].T, rtol=1e-9, atol=1e-9)
    # the convolution against an explicit loop; the chunk mask against its definition
    x = torch.randn(7, 3, dtype=torch.float64)
    taps = torch.randn(3, 4, dtype=torch.float64)
    loop = torch.zeros_like(x)
    for t in range(7):
        for j in range(4):
            if t - 3 + j >= 0:
                loop[t] += taps[:, j] * x[t - 3 + j]
    assert torch.allclose(plain.causal_conv(x, taps), loop)
    mask = plain.visible(11, 4)
    assert all(bool(mask[i, j]) == (j <= i and i // 4 == j // 4) for i in range(11) for j in range(11))


def test_the_plain_model_depends_on_every_edge_the_gpu_tests_rely_on():
    """A chunk that is one token longer or shorter, and a token far back, move the plain logits."""
    path = cases.folder("attention", "float32", scaling="sharp")
    config, weights = cases.read(path)
    tokens = [int(t) for t in np.random.default_rng(5).integers(0, config["vocab"], 60)]
    base = plain.forward(config, weights, tokens).numpy()
    for size in (12, 14):
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = size
        assert np.abs(plain.forward(other, weights, tokens).numpy() - base).max() / np.abs(base).max() > 0.05
    path = cases.folder("mixed", "float32", scaling="long")
    config, weights = cases.read(path)
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, config["vocab"], 300)]
    base = plain.forward(config, weights, tokens).numpy()
    changed = list(tokens)
    changed[3] = (changed[3] + 1) % config["vocab"]
    moved = plain.forward(config, weights, changed).numpy()
    assert np.abs(moved[-20:] - base[-20:]).max() / np.abs(base).max() > 1e-3


def test_a_file_may_hold_the_second_sublayer_of_a_layer_without_feed_forward():
    from vipera_rs_b200.config.gusolix import gusolix_ignorable

    arch, _ = spec_of("mixed")
    config = arch.config_from_dict(cases.MIXED)
    assert gusolix_ignorable(config, "l1.norm2.weight") and gusolix_ignorable(config, "l1.canon2.weight")
    assert gusolix_ignorable(config, "l1.norm2.bias")
    assert not gusolix_ignorable(config, "l0.norm2.weight") and not gusolix_ignorable(config, "l1.norm1.weight")
    assert not gusolix_ignorable(config, "l9.norm2.weight") and not gusolix_ignorable(config, "l1.mix.q.weight")


def test_the_cut_of_the_mixed_weights_attention_covers_every_history():
    from vipera_rs_b200.kernels import ops

    for tokens in (1, 2, 7, 8, 64, 300, 5000):
        for max_keys in (1, 31, 32, 33, 64, 65, 1000, 2048, 2049, 100000):
            keys, splits = ops.talk_splits(tokens, max_keys, 148)
            assert keys % 32 == 0 and keys >= 32 and splits >= 1
            assert keys * splits >= max_keys > keys * (splits - 1)
            if tokens >= 296:
                assert splits == 1
    # chunks of a step: an entry more than whole chunks of all tokens bounds them
    for tokens, entries in ((1, 1), (64, 1), (65, 2), (2048, 5)):
        assert ops.scan_jobs(tokens, entries) >= sum(-(-n // ops.SCAN_CHUNK) for n in [tokens - entries + 1] + [1] * (entries - 1))
