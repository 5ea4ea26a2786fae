"""Nobupel without a GPU: configuration, tensor names, the order of layer runs, the cache
manager's kept first pages, and the plain implementation held to direct formulas."""
import json
import math
import os

import pytest
import torch

import nobupel_cases as cases
import plain_nobupel as plain

import vipera_rs_b200  # noqa: F401
from vipera_rs_b200.build import runtime_module
from vipera_rs_b200.config import NobupelConfig, architecture_of, load_config, nobupel_model_spec
from vipera_rs_b200.errors import InvalidArgumentError, UnsupportedError
from vipera_rs_b200.parts import FixedState, PagedKV
from vipera_rs_b200.parts.model import model_schema
from vipera_rs_b200.parts.rotary import rotary_tables


def test_config_reads_back_and_orders_layer_runs():
    config = NobupelConfig.from_dict(cases.MIXED)
    assert config.layer_runs() == [0, 1, 0, 1, 2, 3]
    assert NobupelConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    assert architecture_of(cases.MIXED).name == "Nobupel"
    spec = nobupel_model_spec(config)
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (0, 2), (1, 3), (2, 4), (3, 5)]
    assert [layer.block for layer in spec.layers] == ["prenorm_mixer", "prenorm", "prenorm", "prenorm_mixer"]
    no_loop = NobupelConfig.from_dict(dict(cases.MIXED, loop=None))
    assert no_loop.layer_runs() == [0, 1, 2, 3]
    once = NobupelConfig.from_dict(dict(cases.MIXED, loop={"start": 1, "stop": 4, "times": 1}))
    assert once.layer_runs() == [0, 1, 2, 3]
    assert plain.layer_runs(cases.WIDE) == NobupelConfig.from_dict(cases.WIDE).layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3]


def test_config_refuses_what_it_does_not_know():
    with pytest.raises(UnsupportedError):
        NobupelConfig.from_dict(dict(cases.MIXED, layers=[{"type": "conv", "mixer": {}}]))
    bad = json.loads(json.dumps(cases.MIXED))
    bad["layers"][1]["mixer"]["kv_heads"] = 2
    with pytest.raises(InvalidArgumentError):
        NobupelConfig.from_dict(bad)
    bad = json.loads(json.dumps(cases.MIXED))
    bad["layers"][1]["mlp"]["kind"] = "routed"
    with pytest.raises(UnsupportedError):
        NobupelConfig.from_dict(bad)
    with pytest.raises(InvalidArgumentError):
        NobupelConfig.from_dict(dict(cases.MIXED, loop={"start": 3, "stop": 9, "times": 2}))
    with pytest.raises(UnsupportedError):
        NobupelConfig.from_dict({k: v for k, v in cases.MIXED.items() if k != "norm"})


def test_cache_requests_and_tensor_names_of_a_written_folder():
    path = cases.folder("mixed", "bfloat16")
    arch, config = load_config(path)
    spec = arch.model_spec(config)
    from safetensors import safe_open

    with safe_open(os.path.join(path, "model.safetensors"), "pt") as handle:
        stored = set(handle.keys())
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.i.b", "l0.mix.norm", "l1.mix.q.b",
            "l1.mlp.gate.b", "l1.mlp.down", "l1.norm2", "l3.mix.o"} <= stored
    assert not any(name.endswith((".weight", ".bias")) for name in stored)
    assert {arch.tensor_alias(name) or name for name in stored} == set(model_schema(spec))
    assert "l0.norm2" not in stored and "l0.mlp.up" not in stored      # a layer without a feed-forward
    from vipera_rs_b200.config.registry import BLOCKS

    requests = [BLOCKS.find(spec.layers[e.layer].block).cache_request_for(spec.layers[e.layer]) for e in spec.schedule]
    assert isinstance(requests[0], FixedState) and requests[0].shape == ((2 * (20 * 36 + 20 + 1) + 3) // 4 * 4,)
    assert requests[1] == PagedKV(1, 24, 24, value_dim=40, keep_first=3)
    assert requests[5] == PagedKV(2, 32, 9, value_dim=16, keep_first=0)


def test_kept_first_pages_stay_when_the_window_moves_on():
    manager = runtime_module().CacheManager([(8, 12, 20, 10), (8, 12, 20, 0)], 2)
    assert manager.group(0) == (8, 12, 20, 10)
    manager.open(7)
    done = 0
    for portion in (5, 30, 2, 1, 1, 17, 9):
        manager.reserve(7, done + portion)
        done += portion
        manager.commit(7, done)
        kept, plain_window = manager.tables([7], 0, 16)[0], manager.tables([7], 1, 16)[0]
        oldest = max(0, done - 20 + 1) // 8
        for page in range((done + 7) // 8):
            assert (plain_window[page] >= 0) == (page >= oldest)
            assert (kept[page] >= 0) == (page >= oldest or page < 2), (done, page)   # 10 kept tokens: two pages
        assert manager.audit() == ""
    manager.close(7)
    assert manager.stats(0)["free_pages"] == 12 and manager.audit() == ""


def test_yarn_tables_against_the_plain_frequencies():
    rot = {"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}}
    cos, sin = rotary_tables(16, 5000.0, 300, "cpu", rot["scaling"]).pair
    freq, stretch = plain.rotary_frequencies(rot)
    angle = torch.arange(300, dtype=torch.float64)[:, None] * freq[None, :]
    assert stretch == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert float((cos.double() - torch.cos(angle) * stretch).abs().max()) < 2e-4
    assert float((sin.double() - torch.sin(angle) * stretch).abs().max()) < 2e-4
    # the fastest pair keeps its frequency, the slowest is slowed by the factor
    assert float(freq[0]) == pytest.approx(1.0) and float(freq[-1]) == pytest.approx(5000.0 ** (-14 / 16) / 4.0)
    same, one = plain.rotary_frequencies({"dims": 16, "base": 5000.0, "scaling": dict(rot["scaling"], factor=1.0)})
    assert one == 1.0 and torch.allclose(same, plain.rotary_frequencies({"dims": 16, "base": 5000.0})[0])


def test_plain_cell_against_the_unstabilised_recurrence():
    """With gates small enough nothing overflows, and the cell can be written without its running
    maximum: C_t = f C + i k v^T, o = C^T q / (max(|n . q|, 1) + eps e^{m_t})."""
    torch.manual_seed(3)
    mixer = {"heads": 2, "dim": 5, "vdim": 7, "gate_cap": 2.5}
    width, count, eps = 12, 40, 1e-6
    w = {"q": torch.randn(10, width), "k": torch.randn(10, width), "v": torch.randn(14, width), "g": torch.randn(14, width),
         "i": torch.randn(2, width), "i.b": torch.randn(2), "f": torch.randn(2, width), "f.b": torch.randn(2),
         "norm": torch.rand(14) + 0.5, "o": torch.randn(width, 14)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(count, width, dtype=torch.float64)
    got, state = plain.mlstm_mixer(h, w, mixer, eps)
    cap = mixer["gate_cap"]
    li = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    q = (h @ w["q"].T).view(count, 2, 5) * 5 ** -0.5
    k, v = (h @ w["k"].T).view(count, 2, 5), (h @ w["v"].T).view(count, 2, 7)
    C, n, m = torch.zeros(2, 5, 7, dtype=torch.float64), torch.zeros(2, 5, dtype=torch.float64), torch.zeros(2, dtype=torch.float64)
    rows = []
    for t in range(count):
        m = torch.maximum(lf[t] + m, li[t])
        C = torch.exp(lf[t])[:, None, None] * C + torch.exp(li[t])[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = torch.exp(lf[t])[:, None] * n + torch.exp(li[t])[:, None] * k[t]
        bottom = torch.maximum((n * q[t]).sum(-1).abs(), torch.ones(2, dtype=torch.float64)) + 1e-6 * torch.exp(m)
        rows.append(torch.einsum("hdv,hd->hv", C, q[t]) / bottom[:, None])
    o = torch.stack(rows)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    want = (o.reshape(count, 14) * w["norm"] * torch.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert float((got - want).abs().max()) < 1e-9 * float(want.abs().max())
    # the state carries: two halves give what the whole gives
    first, carried = plain.mlstm_mixer(h[:17], w, mixer, eps)
    second, _ = plain.mlstm_mixer(h[17:], w, mixer, eps, carried)
    assert float((torch.cat([first, second]) - got).abs().max()) < 1e-12


def test_plain_attention_sink_window_and_kept_keys():
    torch.manual_seed(4)
    mixer = cases.attention_layer(heads=2, kv_heads=1, dim=8, vdim=6, scale=0.9, size=5, keep_first=2, rot_dims=0)["mixer"]
    width, count = 10, 14
    w = {"q": torch.randn(16, width), "q.b": torch.randn(16), "k": torch.randn(8, width), "k.b": torch.randn(8),
         "v": torch.randn(6, width), "v.b": torch.randn(6), "o": torch.randn(width, 12)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(count, width, dtype=torch.float64)
    got = plain.attention_mixer(h, w, mixer, torch.arange(count))
    q = (h @ w["q"].T + w["q.b"]).view(count, 2, 8)
    k, v = h @ w["k"].T + w["k.b"], h @ w["v"].T + w["v.b"]
    out = torch.zeros(count, 2, 6, dtype=torch.float64)
    for i in range(count):
        seen = [j for j in range(i + 1) if i - j < 5 or j < 2]
        assert plain.visible(i, 0, mixer["mask"]) and plain.visible(i, 1, mixer["mask"]) == (i >= 1)
        assert plain.visible(i, 2, mixer["mask"]) == (2 <= i < 7) and not plain.visible(i, i + 1, mixer["mask"])
        for head in range(2):
            scores = torch.cat([(k[seen] @ q[i, head]) * 0.9, torch.zeros(1, dtype=torch.float64)])   # the sink last
            out[i, head] = torch.softmax(scores, 0)[:-1] @ v[seen]
    assert float((got - out.reshape(count, 12) @ w["o"].T).abs().max()) < 1e-12


def test_command_line_on_a_nobupel_folder():
    """model-info and plan as a process, on a folder in the design's own file names."""
    import subprocess
    import sys

    path = cases.folder("mixed", "bfloat16")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    info = subprocess.run([sys.executable, os.path.join(root, "bin", "vipera"), "model-info", path, "--json"],
                          capture_output=True, text=True, timeout=300)
    assert info.returncode == 0, info.stderr
    report = json.loads(info.stdout)
    assert report["architecture"] == "Nobupel" and report["layer_count"] == 4 and report["scheduled_layers"] == 6
    assert report["vocab_size"] == 301 and report["hidden_size"] == 96 and not report["tied_output"]
    # keys and values of one token: the attention runs (layer 1 twice, layer 3 once), bfloat16
    assert report["kv_bytes_per_token_bf16"] == 2 * (2 * 1 * (24 + 40) + 2 * (32 + 16))
    plan = subprocess.run([sys.executable, os.path.join(root, "bin", "vipera"), "plan", path, "--ctx", "512", "--batch", "3"],
                          capture_output=True, text=True, timeout=300)
    assert plan.returncode == 0 and "feasible                 True" in plan.stdout, plan.stdout + plan.stderr
