"""Falerax: a decoder whose config.json lists its layers one by one, each with one of three mixers and optionally a dense
gated feed-forward.  The sublayers read the fp32 residual stream itself and only their outputs are normed
(x <- x + rmsnorm(sublayer(x)) * w); the logits come from the embedding table.

  "parallel"  softcapped grouped-query attention (normed queries and keys, query temperature, sigmoid output gate, no
              rotation) beside a gated matrix memory (mLSTM); the two outputs are normed and averaged
  "mamba1"    short causal convolution + selective scan
  "wkv"       token shift + per-channel decayed outer-product memory with a bonus for the current token

This module only reads the configuration: sizes and constants go to the native engine as `tgis_model_spec` /
`tgis_layer_spec` (include/tgis_engine.h), the arithmetic is csrc/engine.cu `stream_layer`, the recurrent state lives in the
engine's sequence slots (csrc/recurrent.cu).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import struct
from pathlib import Path

from . import _lib
from .core import ModelConfig


@dataclasses.dataclass
class LayerSpec:
    kind: str                 # "parallel" | "mamba1" | "wkv"
    ff: int = 0               # 0: no feed-forward
    # parallel, attention side
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 1.0
    softcap: float = 0.0      # 0: no cap
    qt_coef: float = 0.0
    qt_every: int = 0         # 0: no query temperature
    # parallel, matrix-memory side
    mm_heads: int = 0
    mm_dim: int = 0
    mm_vdim: int = 0
    gate_cap: float = 0.0
    # mamba1
    inner: int = 0
    state: int = 0
    dt_rank: int = 0
    conv: int = 0
    # wkv (heads, dim above)
    decay_rank: int = 0


def layer_from_json(i: int, entry: dict, decay_rank: int | None = None) -> LayerSpec:
    kind, m = entry.get("type"), entry["mixer"]
    if kind == "parallel":
        a, b = m["left"], m["right"]
        qt = a.get("q_temp") or {}
        spec = LayerSpec(kind, heads=int(a["heads"]), kv_heads=int(a.get("kv_heads", a["heads"])), dim=int(a["dim"]),
                         vdim=int(a["vdim"]), scale=float(a["scale"]), softcap=float(a.get("softcap") or 0.0),
                         qt_coef=float(qt.get("coef", 0.0)), qt_every=int(qt.get("every", 0)),
                         mm_heads=int(b["heads"]), mm_dim=int(b["dim"]), mm_vdim=int(b["vdim"]), gate_cap=float(b["gate_cap"]))
    elif kind == "mamba1":
        spec = LayerSpec(kind, inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m["conv"]))
    elif kind == "wkv":
        rank = m.get("decay_rank", decay_rank)
        if rank is None:
            raise ValueError(f"layer {i}: the decay map's rank is given neither by the config nor by the checkpoint")
        spec = LayerSpec(kind, heads=int(m["heads"]), dim=int(m["dim"]), decay_rank=int(rank))
    else:
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
    mlp = entry.get("mlp")
    if mlp is not None:
        if mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        spec.ff = int(mlp["ff"])
    return spec


def checkpoint_shapes(path: Path) -> dict[str, tuple[int, ...]]:
    """name -> shape from the headers of the directory's *.safetensors files (8-byte length, then JSON)."""
    out: dict[str, tuple[int, ...]] = {}
    for f in sorted(Path(path).glob("*.safetensors")):
        with open(f, "rb") as fh:
            (n,) = struct.unpack("<Q", fh.read(8))
            for name, meta in json.loads(fh.read(n)).items():
                if name != "__metadata__":
                    out[name] = tuple(meta["shape"])
    return out


def model_config_from_json(cfg: dict, max_model_len: int | None, dtype: str = "bfloat16",
                           shapes: dict | None = None) -> ModelConfig:
    """`shapes`: the checkpoint's tensor shapes; the rank of a wkv layer's decay map is the first extent of its `mix.w1`."""
    layers = []
    for i, e in enumerate(cfg["layers"]):
        w1 = (shapes or {}).get(f"l{i}.mix.w1")
        layers.append(layer_from_json(i, e, w1[0] if w1 else None))
    if not layers:
        raise ValueError("config.json lists no layers")
    return ModelConfig(n_layers=len(layers), hidden=int(cfg["width"]), n_q_heads=1, n_kv_heads=1, ffn=64,
                       vocab=int(cfg["vocab"]), rms_eps=float(cfg["norm"]["eps"]), max_model_len=max_model_len or 4096,
                       arch="falerax", layers=layers, dtype=dtype)


def config_json(mc: ModelConfig) -> dict:
    """The config.json of `mc` (what model_config_from_json reads back)."""
    out = []
    for l in mc.layers:
        if l.kind == "parallel":
            left = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale}
            if l.softcap > 0:
                left["softcap"] = l.softcap
            if l.qt_every > 0:
                left["q_temp"] = {"coef": l.qt_coef, "every": l.qt_every}
            m = {"left": left, "right": {"heads": l.mm_heads, "dim": l.mm_dim, "vdim": l.mm_vdim, "gate_cap": l.gate_cap}}
        elif l.kind == "mamba1":
            m = {"inner": l.inner, "state": l.state, "dt_rank": l.dt_rank, "conv": l.conv}
        else:
            m = {"heads": l.heads, "dim": l.dim, "decay_rank": l.decay_rank}
        out.append({"type": l.kind, "mixer": m, "mlp": {"kind": "dense", "ff": l.ff} if l.ff > 0 else None})
    return {"architecture": "Falerax", "width": mc.hidden, "vocab": mc.vocab, "norm": {"eps": mc.rms_eps}, "layers": out}


_MIXER = {"parallel": _lib.MIXER_PARALLEL, "mamba1": _lib.MIXER_SELECTIVE_SCAN, "wkv": _lib.MIXER_WKV}


def model_spec(mc: ModelConfig):
    """(TgisModelSpec, the ctypes array it points into)."""
    if mc.dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {mc.dtype!r}: bfloat16 or float32")
    arr = (_lib.TgisLayerSpec * len(mc.layers))()
    for a, l in zip(arr, mc.layers):
        a.mixer = _MIXER[l.kind]
        a.mlp, a.ff = (_lib.MLP_DENSE_GELU, l.ff) if l.ff > 0 else (_lib.MLP_NONE, 0)
        a.heads, a.kv_heads, a.dim, a.vdim, a.scale = l.heads, l.kv_heads, l.dim, l.vdim, l.scale
        a.softcap, a.qt_coef, a.qt_every = l.softcap, l.qt_coef, l.qt_every
        a.mm_heads, a.mm_dim, a.mm_vdim, a.gate_cap = l.mm_heads, l.mm_dim, l.mm_vdim, l.gate_cap
        a.inner, a.state, a.dt_rank, a.conv, a.decay_rank = l.inner, l.state, l.dt_rank, l.conv, l.decay_rank
    spec = _lib.TgisModelSpec()
    spec.n_layers = len(mc.layers)
    spec.dtype = _lib.DTYPE_F32 if mc.dtype == "float32" else _lib.DTYPE_BF16
    spec.embed_scale, spec.residual_mult, spec.norm_eps = 1.0, 1.0, mc.rms_eps
    spec.style = _lib.STYLE_POST_NORM | _lib.STYLE_TIED_HEAD
    spec.layers = C.cast(arr, C.POINTER(_lib.TgisLayerSpec))
    return spec, arr


def cache_row_elems(mc: ModelConfig) -> int:
    """Cache elements one token takes over all layers (only the attention sides are cached per token)."""
    return sum(l.kv_heads * (l.dim + l.vdim) for l in mc.layers if l.kind == "parallel")


def tensor_shapes(mc: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Every parameter of the checkpoint with its shape ([out, in] for matrices)."""
    w, out = mc.hidden, {}
    out["embed"] = (mc.vocab, w)
    out["final.norm"] = (w,)
    for i, l in enumerate(mc.layers):
        p = f"l{i}."
        out[p + "norm1"] = (w,)
        if l.kind == "parallel":
            a, b = p + "mix.left.", p + "mix.right."
            out[a + "q"] = (l.heads * l.dim, w)
            out[a + "k"] = (l.kv_heads * l.dim, w)
            out[a + "v"] = (l.kv_heads * l.vdim, w)
            out[a + "g"] = (l.heads * l.vdim, w)
            out[a + "o"] = (w, l.heads * l.vdim)
            out[a + "q.norm"] = out[a + "k.norm"] = (l.dim,)
            out[a + "out"] = out[b + "out"] = (w,)
            out[b + "q"] = out[b + "k"] = (l.mm_heads * l.mm_dim, w)
            out[b + "v"] = out[b + "g"] = (l.mm_heads * l.mm_vdim, w)
            out[b + "o"] = (w, l.mm_heads * l.mm_vdim)
            out[b + "norm"] = (l.mm_heads * l.mm_vdim,)
            out[b + "i"] = out[b + "f"] = (l.mm_heads, w)
            out[b + "i.b"] = out[b + "f.b"] = (l.mm_heads,)
        elif l.kind == "mamba1":
            m = p + "mix."
            out[m + "in"] = (2 * l.inner, w)
            out[m + "conv"] = (l.inner, l.conv)
            out[m + "conv.b"] = out[m + "dt.b"] = out[m + "D"] = (l.inner,)
            out[m + "x"] = (l.dt_rank + 2 * l.state, l.inner)
            out[m + "dt"] = (l.inner, l.dt_rank)
            out[m + "A_log"] = (l.inner, l.state)
            out[m + "o"] = (w, l.inner)
        else:
            m, a = p + "mix.", l.heads * l.dim
            for s in "rkvgw":
                out[m + "mu." + s] = (w,)
            for s in "rkvg":
                out[m + s] = (a, w)
            out[m + "w1"] = (l.decay_rank, w)
            out[m + "w2"] = (a, l.decay_rank)
            out[m + "w0"] = out[m + "norm"] = (a,)
            out[m + "u"] = (l.heads, l.dim)
            out[m + "o"] = (w, a)
        if l.ff > 0:
            out[p + "norm2"] = (w,)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (l.ff, w)
            out[p + "mlp.down"] = (w, l.ff)
    return out


def iter_synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu"):
    """Seeded random bf16 weights of the architecture, one (name, tensor) at a time, drawn on `device`: matrices
    ~ N(0, 1 / fan_in), norm weights around one, token-shift blends in (0, 1), decays and step sizes in a range where the
    states neither vanish nor blow up."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)

    def randn(shape):
        return torch.randn(shape, generator=gen, device=device)

    for name, shape in tensor_shapes(mc).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(".mu." + leaf):
            t = torch.rand(shape, generator=gen, device=device)
        elif leaf == "A_log":
            t = torch.log(torch.arange(1, shape[1] + 1, device=device, dtype=torch.float32)).repeat(shape[0], 1)
        elif name.endswith("dt.b"):
            t = randn(shape) * 0.5 - 3.0
        elif leaf == "w0":
            t = randn(shape) * 0.5 - 1.0
        elif leaf in ("u", "D"):
            t = randn(shape) * 0.5
        elif name.endswith("f.b"):
            t = randn(shape) * 0.5 + 3.0
        elif name.endswith(("i.b", "conv.b")):
            t = randn(shape) * 0.1
        elif len(shape) == 1:
            t = 1.0 + randn(shape) * 0.1
        elif leaf == "conv":
            t = randn(shape) * shape[1] ** -0.5
        else:
            t = randn(shape) * (1.0 if name == "embed" else shape[1] ** -0.5)
        yield name, t.to(torch.bfloat16)


def synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu") -> dict:
    return dict(iter_synthetic_weights(mc, seed, device))


def _attn(width: int, heads: int, kv_heads: int, dim: int, vdim: int, mm_heads: int, mm_dim: int, mm_vdim: int, ff: int):
    return LayerSpec("parallel", ff=ff, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5, softcap=30.0,
                     qt_coef=0.1, qt_every=256, mm_heads=mm_heads, mm_dim=mm_dim, mm_vdim=mm_vdim, gate_cap=15.0)


def _stack(hidden: int, vocab: int, layers: list[LayerSpec]) -> ModelConfig:
    return ModelConfig(n_layers=len(layers), hidden=hidden, n_q_heads=1, n_kv_heads=1, ffn=64, vocab=vocab, rms_eps=1e-5,
                       max_model_len=4096, arch="falerax", layers=layers)


# Sizes that resemble the layers of real hybrid models (random weights; `--model <name> --synthetic-weights`,
# bench.py --arch-compare): one layer of each recurrent kind around two attention + matrix-memory layers
PRESETS: dict[str, ModelConfig] = {
    "falerax-tiny": _stack(128, 512, [
        LayerSpec("wkv", heads=2, dim=32, decay_rank=8),
        _attn(128, 4, 2, 32, 48, 2, 16, 32, 192),
        LayerSpec("mamba1", ff=160, inner=192, state=8, dt_rank=6, conv=3)]),
    "falerax-1k": _stack(1024, 32768, [
        LayerSpec("wkv", ff=3072, heads=16, dim=64, decay_rank=64),
        _attn(1024, 8, 2, 128, 128, 4, 128, 256, 3072),
        _attn(1024, 8, 2, 128, 128, 4, 128, 256, 3072),
        LayerSpec("mamba1", ff=3072, inner=2048, state=16, dt_rank=64, conv=4)]),
    "falerax-2k": _stack(2048, 32768, [
        LayerSpec("wkv", ff=11264, heads=32, dim=64, decay_rank=64),
        _attn(2048, 16, 4, 128, 128, 8, 128, 256, 11264),
        _attn(2048, 16, 4, 128, 128, 8, 128, 256, 11264),
        LayerSpec("mamba1", ff=11264, inner=4096, state=16, dt_rank=128, conv=4)]),
}
