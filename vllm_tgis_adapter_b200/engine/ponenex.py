"""Ponenex: a decoder whose config.json lists its layers one by one.

Every layer has a latent-attention mixer (low-rank query and key/value latents, one rotary key part shared by all heads,
sliding window, sigmoid output gate per head) and optionally a mixture-of-experts feed-forward (biased top-k router,
softmax over the chosen logits, gated shared expert), both wrapped in a pre- and a post-norm and added to an fp32 residual
stream scaled by `residual_mult`.  This module only reads the configuration: sizes and constants go to the native engine as
`tgis_model_spec` / `tgis_layer_spec` (include/tgis_engine.h), the arithmetic is csrc/engine.cu `pnx_forward`.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

from . import _lib
from .core import ModelConfig


@dataclasses.dataclass
class LayerSpec:
    heads: int
    dim: int            # unrotated query/key dims per head
    rot_dim: int        # rotated query/key dims per head (the key part is shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    window: int         # i sees j with 0 <= i - j < window (0: no window)
    rot_dims: int       # how many of the rot_dim dims turn
    rot_base: float
    scale: float
    experts: int = 0    # 0: the layer has no feed-forward
    top: int = 0
    expert_ff: int = 0
    shared_ff: int = 0  # 0: no shared expert


def layer_from_json(i: int, entry: dict) -> LayerSpec:
    if entry.get("type") != "latent_attention":
        raise ValueError(f"layer {i}: unknown mixer type {entry.get('type')!r}")
    m = entry["mixer"]
    rot = m.get("rot") or {}
    rot_dim = int(m["rot_dim"])
    spec = LayerSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rot_dim, vdim=int(m["vdim"]),
                     kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), window=int((m.get("mask") or {}).get("size", 0)),
                     rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
                     scale=float(m["scale"]))
    mlp = entry.get("mlp")
    if mlp is not None:
        if mlp.get("kind") != "moe":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        spec.experts, spec.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        spec.expert_ff = int(mlp["expert"]["ff"])
        spec.shared_ff = int((mlp.get("shared") or {}).get("ff", 0))
    return spec


def model_config_from_json(cfg: dict, max_model_len: int | None, dtype: str = "bfloat16") -> ModelConfig:
    layers = [layer_from_json(i, e) for i, e in enumerate(cfg["layers"])]
    if not layers:
        raise ValueError("config.json lists no layers")
    return ModelConfig(n_layers=len(layers), hidden=int(cfg["width"]), n_q_heads=1, n_kv_heads=1, ffn=64,
                       vocab=int(cfg["vocab"]), rms_eps=float(cfg["norm"]["eps"]), max_model_len=max_model_len or 4096,
                       arch="ponenex", layers=layers, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                       residual_mult=float(cfg.get("residual_mult", 1.0)), dtype=dtype)


def model_spec(mc: ModelConfig):
    """(TgisModelSpec, the ctypes array it points into)."""
    if mc.dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {mc.dtype!r}: bfloat16 or float32")
    arr = (_lib.TgisLayerSpec * len(mc.layers))()
    for a, l in zip(arr, mc.layers):
        a.mixer = _lib.MIXER_LATENT_ATTENTION
        a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank = l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.q_rank
        a.window, a.rot_dims, a.rot_base, a.scale = l.window, l.rot_dims, l.rot_base, l.scale
        a.mlp = _lib.MLP_MOE if l.experts > 0 else _lib.MLP_NONE
        a.experts, a.top, a.expert_ff, a.shared_ff = l.experts, l.top, l.expert_ff, l.shared_ff
    spec = _lib.TgisModelSpec()
    spec.n_layers = len(mc.layers)
    spec.dtype = _lib.DTYPE_F32 if mc.dtype == "float32" else _lib.DTYPE_BF16
    spec.embed_scale, spec.residual_mult, spec.norm_eps = mc.embed_scale, mc.residual_mult, mc.rms_eps
    spec.layers = C.cast(arr, C.POINTER(_lib.TgisLayerSpec))
    return spec, arr


def tensor_shapes(mc: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Every parameter of the checkpoint with its shape ([out, in] for matrices)."""
    w, out = mc.hidden, {}
    out["embed"] = (mc.vocab, w)
    out["head"] = (mc.vocab, w)
    out["final.norm"] = (w,)
    for i, l in enumerate(mc.layers):
        p = f"l{i}."
        out[p + "norm1"] = out[p + "norm1b"] = (w,)
        out[p + "mix.dq"] = (l.q_rank, w)
        out[p + "mix.dq.norm"] = (l.q_rank,)
        out[p + "mix.uq"] = (l.heads * (l.dim + l.rot_dim), l.q_rank)
        out[p + "mix.dkv"] = (l.kv_rank + l.rot_dim, w)
        out[p + "mix.dkv.norm"] = (l.kv_rank,)
        out[p + "mix.uk"] = (l.heads * l.dim, l.kv_rank)
        out[p + "mix.uv"] = (l.heads * l.vdim, l.kv_rank)
        out[p + "mix.g"] = (l.heads, w)
        out[p + "mix.o"] = (w, l.heads * l.vdim)
        if l.experts > 0:
            out[p + "norm2"] = out[p + "norm2b"] = (w,)
            out[p + "mlp.router"] = (l.experts, w)
            out[p + "mlp.router.b"] = (l.experts,)
            for j in range(l.experts):
                out[p + f"mlp.e{j}.gate"] = out[p + f"mlp.e{j}.up"] = (l.expert_ff, w)
                out[p + f"mlp.e{j}.down"] = (w, l.expert_ff)
            if l.shared_ff > 0:
                out[p + "mlp.shared.gate"] = out[p + "mlp.shared.up"] = (l.shared_ff, w)
                out[p + "mlp.shared.down"] = (w, l.shared_ff)
                out[p + "mlp.shared.sg"] = (1, w)
    return out


def iter_synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu"):
    """Seeded random bf16 weights of the architecture, one (name, tensor) at a time, drawn on `device` (norm weights around
    zero, the latents' plain norm weights around one, matrices ~ N(0, 1 / fan_in))."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)
    for name, shape in tensor_shapes(mc).items():
        if len(shape) == 1:
            t = torch.randn(shape, generator=gen, device=device) * (0.5 if name.endswith("router.b") else 0.1)
            if name.endswith(".norm") and name != "final.norm":
                t = t + 1.0
        else:
            t = torch.randn(shape, generator=gen, device=device) * (1.0 if name == "embed" else shape[1] ** -0.5)
        yield name, t.to(torch.bfloat16)


def synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu") -> dict:
    return dict(iter_synthetic_weights(mc, seed, device))


def _uniform(n_layers: int, hidden: int, vocab: int, **layer) -> ModelConfig:
    return ModelConfig(n_layers=n_layers, hidden=hidden, n_q_heads=1, n_kv_heads=1, ffn=64, vocab=vocab, rms_eps=1e-5,
                       max_model_len=4096, arch="ponenex", layers=[LayerSpec(**layer) for _ in range(n_layers)],
                       embed_scale=1.0, residual_mult=1.0)


# Sizes that resemble the layers of real latent-attention / mixture-of-experts models (random weights; `--model <name>
# --synthetic-weights`, bench.py --arch-compare)
PRESETS: dict[str, ModelConfig] = {
    "ponenex-tiny": _uniform(2, 256, 1024, heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=128, window=128,
                             rot_dims=16, rot_base=10000.0, scale=48 ** -0.5, experts=8, top=2, expert_ff=128, shared_ff=128),
    "ponenex-1k": _uniform(4, 1024, 32768, heads=8, dim=128, rot_dim=64, vdim=128, kv_rank=256, q_rank=768, window=2048,
                           rot_dims=64, rot_base=10000.0, scale=192 ** -0.5, experts=16, top=2, expert_ff=1024, shared_ff=1024),
    "ponenex-2k": _uniform(4, 2048, 32768, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, window=4096,
                           rot_dims=64, rot_base=10000.0, scale=192 ** -0.5, experts=64, top=6, expert_ff=1408, shared_ff=2816),
}
