"""CPU-side checks of the Falerax family: config.json (+ checkpoint header) -> engine specs, the parameter list, presets, and
properties of the plain oracle that the GPU tests lean on (causality, the query temperature, the soft cap, state carried
token by token, grouped key/value heads)."""
import json
import math
import struct

import pytest
import torch

from oracle import falerax_oracle as O
from vllm_tgis_adapter_b200.engine import _lib
from vllm_tgis_adapter_b200.engine.falerax import (PRESETS, checkpoint_shapes, config_json, model_config_from_json, model_spec,
                                                   synthetic_weights, tensor_shapes)

CFG = {
    "architecture": "Falerax", "width": 24, "vocab": 50, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 5}, "mlp": None},
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.3, "softcap": 7.0,
                            "q_temp": {"coef": 0.25, "every": 4}},
                   "right": {"heads": 3, "dim": 4, "vdim": 5, "gate_cap": 6.0}},
         "mlp": {"kind": "dense", "ff": 14}},
        {"type": "mamba1", "mixer": {"inner": 10, "state": 3, "dt_rank": 2, "conv": 3}, "mlp": {"kind": "dense", "ff": 9}},
    ],
}
SHAPES = {"l0.mix.w1": (7, 24)}


def test_config_json_to_specs():
    mc = model_config_from_json(CFG, 256, "float32", SHAPES)
    assert (mc.arch, mc.hidden, mc.vocab, mc.n_layers, mc.max_model_len, mc.rms_eps, mc.dtype) == ("falerax", 24, 50, 3, 256, 1e-3, "float32")
    a, b, c = mc.layers
    assert (a.kind, a.heads, a.dim, a.decay_rank, a.ff) == ("wkv", 2, 5, 7, 0)
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.scale, b.softcap, b.qt_coef, b.qt_every) == (4, 2, 6, 3, 0.3, 7.0, 0.25, 4)
    assert (b.mm_heads, b.mm_dim, b.mm_vdim, b.gate_cap, b.ff) == (3, 4, 5, 6.0, 14)
    assert (c.inner, c.state, c.dt_rank, c.conv, c.ff) == (10, 3, 2, 3, 9)
    spec, keep = model_spec(mc)
    assert spec.n_layers == 3 and spec.dtype == _lib.DTYPE_F32 and spec.style == _lib.STYLE_POST_NORM | _lib.STYLE_TIED_HEAD
    assert [k.mixer for k in keep] == [_lib.MIXER_WKV, _lib.MIXER_PARALLEL, _lib.MIXER_SELECTIVE_SCAN]
    assert [k.mlp for k in keep] == [_lib.MLP_NONE, _lib.MLP_DENSE_GELU, _lib.MLP_DENSE_GELU] and keep[0].decay_rank == 7
    assert model_config_from_json(config_json(mc), 256, "float32").layers == mc.layers      # round trip
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][0], "type": "something_else"}]}, None, shapes=SHAPES)
    with pytest.raises(ValueError):
        model_config_from_json(CFG, None)                                                    # the decay rank is nowhere
    # optional parts: no cap, no temperature, kv_heads defaults to heads
    left = {"heads": 2, "dim": 4, "vdim": 4, "scale": 0.5}
    l = model_config_from_json({**CFG, "layers": [{"type": "parallel", "mixer": {"left": left, "right": CFG["layers"][1]["mixer"]["right"]},
                                                   "mlp": None}]}, None).layers[0]
    assert (l.kv_heads, l.softcap, l.qt_every) == (2, 0.0, 0)


def test_loader_reads_family_and_decay_rank_from_the_checkpoint(tmp_path):
    from vllm_tgis_adapter_b200.engine.loader import model_config_from_hf

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    header = json.dumps({"l0.mix.w1": {"dtype": "BF16", "shape": [5, 24], "data_offsets": [0, 240]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + bytes(240))
    assert checkpoint_shapes(tmp_path) == {"l0.mix.w1": (5, 24)}
    mc = model_config_from_hf(tmp_path, 128, "bfloat16")
    assert mc.arch == "falerax" and mc.max_model_len == 128 and mc.layers[0].decay_rank == 5


def test_parameter_list_and_presets():
    mc = model_config_from_json(CFG, None, shapes=SHAPES)
    shapes = tensor_shapes(mc)
    assert shapes["l0.mix.w2"] == (10, 7) and shapes["l0.mix.u"] == (2, 5) and shapes["l1.mix.left.v"] == (6, 24)
    assert shapes["l1.mix.left.g"] == (12, 24) and shapes["l1.mix.right.i"] == (3, 24) and shapes["l2.mix.x"] == (8, 10)
    assert "head" not in shapes and "l0.norm2" not in shapes and shapes["l2.mlp.down"] == (24, 9)
    assert len(shapes) == 2 + (1 + 15) + (1 + 19 + 4) + (1 + 9 + 4)
    w = synthetic_weights(mc, 1)
    assert set(w) == set(shapes) and all(tuple(w[k].shape) == shapes[k] and w[k].dtype == torch.bfloat16 for k in w)
    for name, p in PRESETS.items():
        assert p.arch == "falerax" and {l.kind for l in p.layers} == {"wkv", "parallel", "mamba1"}, name


def test_oracle_is_causal_and_carries_state():
    mc = model_config_from_json(CFG, None, shapes=SHAPES)
    w = synthetic_weights(mc, 2)
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(0)).tolist()
    full = O.forward(CFG, w, toks)
    assert torch.allclose(O.forward(CFG, w, toks[:17]), full[:17], atol=1e-12)     # later tokens change nothing earlier
    other = list(toks)
    other[0] = (other[0] + 1) % 50
    assert not torch.allclose(O.forward(CFG, w, other)[29], full[29], atol=1e-9)   # ... and the first token reaches the last


def test_oracle_mechanisms():
    f = torch.float64
    assert torch.allclose(O.query_temperature(9, 0.5, 4), torch.tensor([1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 2, dtype=f))
    # one token: attention returns its own value times the gate, whatever cap and temperature say
    m = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 2, "scale": 1.0, "softcap": 0.5, "q_temp": {"coef": 1.0, "every": 1}}
    g = torch.Generator().manual_seed(1)
    w = {k: torch.randn(s, generator=g, dtype=f) for k, s in
         {"q": (6, 5), "k": (3, 5), "v": (2, 5), "g": (4, 5), "o": (5, 4), "q.norm": (3,), "k.norm": (3,)}.items()}
    h = torch.randn(1, 5, generator=g, dtype=f)
    v = h @ w["v"].T
    assert torch.allclose(O.capped_attention(h, w, m, 1e-5), (torch.cat([v, v], -1) * torch.sigmoid(h @ w["g"].T)) @ w["o"].T)
    # the cap bounds what one key can win by: with a tiny cap the weights are near uniform
    h3 = torch.randn(6, 5, generator=g, dtype=f)
    tiny = O.capped_attention(h3, w, {**m, "softcap": 1e-6}, 1e-5)
    mean_v = torch.cumsum(h3 @ w["v"].T, 0) / torch.arange(1, 7, dtype=f)[:, None]
    assert torch.allclose(tiny, (torch.cat([mean_v, mean_v], -1) * torch.sigmoid(h3 @ w["g"].T)) @ w["o"].T, atol=1e-5)
    # selective scan with zero step size passes D x only; gelu's tanh form at a known point
    mm = {"inner": 2, "state": 2, "dt_rank": 1, "conv": 1}
    ws = {"in": torch.eye(4, dtype=f), "conv": torch.ones(2, 1, dtype=f), "conv.b": torch.zeros(2, dtype=f),
          "x": torch.zeros(5, 2, dtype=f), "dt": torch.zeros(2, 1, dtype=f), "dt.b": torch.full((2,), -1e9, dtype=f),
          "A_log": torch.zeros(2, 2, dtype=f), "D": torch.tensor([2.0, 3.0], dtype=f), "o": torch.eye(2, dtype=f)}
    hs = torch.randn(4, 4, generator=g, dtype=f)
    x = O.silu(hs[:, :2])
    assert torch.allclose(O.selective_scan(hs, ws, mm), ws["D"] * x * O.silu(hs[:, 2:]))
    assert abs(float(O.gelu_tanh(torch.tensor(1.0, dtype=f))) - 0.8411919906082768) < 1e-12
