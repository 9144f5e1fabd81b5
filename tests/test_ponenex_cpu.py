"""CPU-side checks of the Ponenex family: config.json -> engine specs, the parameter list, the command-line switches, and
properties of the plain oracle that the GPU tests lean on (causality, window, rotation, router)."""
import json

import pytest
import torch

from oracle import ponenex_oracle as O
from vllm_tgis_adapter_b200.engine import _lib
from vllm_tgis_adapter_b200.engine.ponenex import (LayerSpec, model_config_from_json, model_spec, synthetic_weights,
                                                   tensor_shapes)

CFG = {
    "architecture": "Ponenex", "width": 24, "vocab": 50, "residual_mult": 0.5, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-3},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 8, "q_rank": 7, "scale": 0.3,
                   "mask": {"size": 5}, "rot": {"base": 100.0, "dims": 4}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 9}, "shared": {"ff": 4}}},
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 4, "rot_dim": 6, "vdim": 3, "kv_rank": 10, "q_rank": 5, "scale": 0.4,
                   "mask": {"size": 9}, "rot": {"base": 50.0, "dims": 2}},
         "mlp": None},
    ],
}


def test_config_json_to_specs():
    mc = model_config_from_json(CFG, 256, "float32")
    assert (mc.arch, mc.hidden, mc.vocab, mc.n_layers, mc.max_model_len) == ("ponenex", 24, 50, 2, 256)
    assert (mc.embed_scale, mc.residual_mult, mc.rms_eps, mc.dtype) == (2.0, 0.5, 1e-3, "float32")
    a, b = mc.layers
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank, a.window, a.rot_dims) == (2, 6, 4, 5, 8, 7, 5, 4)
    assert (a.experts, a.top, a.expert_ff, a.shared_ff) == (3, 2, 9, 4)
    assert (b.rot_dims, b.rot_base, b.experts, b.shared_ff) == (2, 50.0, 0, 0)
    spec, keep = model_spec(mc)
    assert spec.n_layers == 2 and spec.dtype == _lib.DTYPE_F32 and abs(spec.residual_mult - 0.5) < 1e-7
    assert keep[0].mlp == _lib.MLP_MOE and keep[1].mlp == _lib.MLP_NONE and keep[1].window == 9
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][0], "type": "something_else"}]}, None)


def test_loader_picks_the_family_from_config_json(tmp_path):
    from vllm_tgis_adapter_b200.engine.loader import model_config_from_hf

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    mc = model_config_from_hf(tmp_path, 128, "bfloat16")
    assert mc.arch == "ponenex" and mc.max_model_len == 128 and len(mc.layers) == 2


def test_parameter_list():
    mc = model_config_from_json(CFG, None)
    shapes = tensor_shapes(mc)
    assert shapes["l0.mix.dkv"] == (12, 24) and shapes["l0.mix.uq"] == (20, 7) and shapes["l1.mix.g"] == (3, 24)
    assert shapes["l0.mlp.shared.sg"] == (1, 24) and "l1.norm2" not in shapes and "l1.mlp.router" not in shapes
    assert len(shapes) == 3 + (11 + 4 + 9 + 4) + 11
    w = synthetic_weights(mc, 1)
    assert set(w) == set(shapes) and all(tuple(w[k].shape) == shapes[k] and w[k].dtype == torch.bfloat16 for k in w)


def test_command_line_accepts_float32():
    from vllm_tgis_adapter_b200.tgis_utils.args import parse_args

    args = parse_args(["--model", "x", "--dtype", "float32"])
    assert args.dtype == "float32"


def test_oracle_is_causal_and_windowed():
    mc = model_config_from_json(CFG, None)
    w = synthetic_weights(mc, 2)
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(0)).tolist()
    full = O.forward(mc, w, toks)
    assert torch.allclose(O.forward(mc, w, toks[:17]), full[:17], atol=1e-12)     # later tokens change nothing earlier
    # windows of 5 and 9 over two layers: position 29 depends on nothing before 29 - 4 - 8 = 17
    other = list(toks)
    other[16] = (other[16] + 1) % 50
    changed = O.forward(mc, w, other)
    assert torch.allclose(changed[29], full[29], atol=1e-12) and not torch.allclose(changed[28], full[28], atol=1e-9)
    ok = O.visible(6, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True] and ok[1].tolist() == [True, True] + [False] * 4


def test_oracle_rotation_and_router():
    v = torch.randn(5, 3, 10, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    r = O.rotate(v, pos, 100.0, 6)
    assert torch.allclose(r[0], v[0]) and torch.equal(r[..., 6:], v[..., 6:])                 # position 0; dims that pass
    assert torch.allclose(r[..., :6].norm(dim=-1), v[..., :6].norm(dim=-1))
    # pair (i, i + 3) of position 7 turns by 7 * 100^(-2 i / 6)
    a = 7 * 100.0 ** (-2 * 1 / 6)
    assert torch.allclose(r[2, :, 1], v[2, :, 1] * torch.cos(torch.tensor(a)) - v[2, :, 4] * torch.sin(torch.tensor(a)))
    h = torch.randn(4, 8, dtype=torch.float64)
    ids, wt = O.route(h, torch.randn(6, 8, dtype=torch.float64), torch.zeros(6, dtype=torch.float64), 3)
    assert ids.shape == (4, 3) and torch.allclose(wt.sum(-1), torch.ones(4, dtype=torch.float64)) and bool((wt[:, 0] >= wt[:, 1]).all())
