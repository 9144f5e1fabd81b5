"""Plain, slow restatement of the Ponenex decoder in float64 torch on the CPU: one function per mechanism, whole
sequences only (no cache, no batching, no chunking), dense [T, T] masks.  It shares no code with the engine; the GPU tests
compare the engine's kernels and steps with it.

Notation.  x_t: residual stream at position t (positions count from 0).  rms(v) = v / sqrt(mean(v^2) + eps).
A layer is   x <- x + m * rms(mixer(rms(x) * (1 + n1))) * (1 + n1b),   x <- x + m * rms(ff(rms(x) * (1 + n2))) * (1 + n2b).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def norm_around_zero(v, w, eps):
    """The sublayer norms: weight stored as a deviation from one."""
    return rms(v, eps) * (1.0 + w)


def norm_plain(v, w, eps):
    """The latents' norms: plain weight."""
    return rms(v, eps) * w


def rotate(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, ..., d]: entry i < dims / 2 pairs with entry i + dims / 2 and the pair turns by the angle
    positions[t] * base^(-2 i / dims); entries from `dims` on pass unchanged."""
    out = v.clone()
    half = dims // 2
    for i in range(half):
        ang = positions.to(F64) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang), torch.sin(ang)
        while c.dim() < v.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


def visible(T: int, window: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff 0 <= i - j < window (window <= 0: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok &= (i - j) < window
    return ok


def latent_attention(h: torch.Tensor, w: dict, l, eps: float, positions: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, width] -> mixer output [T, width].  w: the layer's 'mix.*' tensors (float64), l: LayerSpec-like."""
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, l.heads, l.dim + l.rot_dim)
    q_plain, q_rot = q[..., : l.dim], rotate(q[..., l.dim:], pos, l.rot_base, l.rot_dims)
    kv = h @ w["dkv"].T
    c = norm_plain(kv[:, : l.kv_rank], w["dkv.norm"], eps)
    k_rot = rotate(kv[:, l.kv_rank:], pos, l.rot_base, l.rot_dims)          # one rotated key part for all heads
    k_plain = (c @ w["uk"].T).view(T, l.heads, l.dim)
    v = (c @ w["uv"].T).view(T, l.heads, l.vdim)
    gate = torch.sigmoid(h @ w["g"].T)                                       # [T, heads]
    ok = visible(T, l.window)
    heads_out = []
    for hd in range(l.heads):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * l.scale
        s = s.masked_fill(~ok, -math.inf)
        p = torch.softmax(s, -1)
        heads_out.append((p @ v[:, hd]) * gate[:, hd: hd + 1])
    return torch.cat(heads_out, -1) @ w["o"].T


def expert(h, gate_w, up_w, down_w):
    a = h @ gate_w.T
    return ((a * torch.sigmoid(a)) * (h @ up_w.T)) @ down_w.T


def route(h, router_w, router_b, top: int):
    """(ids [T, top], weights [T, top]): the `top` largest of W h + b, softmax over just those."""
    z = h @ router_w.T + router_b
    val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    val, idx = val[:, :top], idx[:, :top]
    return idx, torch.softmax(val, -1)


def mixture_of_experts(h: torch.Tensor, w: dict, l) -> torch.Tensor:
    ids, wt = route(h, w["router"], w["router.b"], l.top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(l.top):
            e = int(ids[t, k])
            out[t] += wt[t, k] * expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    if l.shared_ff > 0:
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(mc, weights: dict, tokens: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of every position of one sequence.  mc: ModelConfig(arch="ponenex")."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, m = mc.rms_eps, mc.residual_mult
    x = w["embed"][torch.tensor(tokens)] * mc.embed_scale
    for i, l in enumerate(mc.layers):
        lw = sub(w, f"l{i}.")
        x = x + m * norm_around_zero(latent_attention(norm_around_zero(x, lw["norm1"], eps), sub(lw, "mix."), l, eps),
                                     lw["norm1b"], eps)
        if l.experts > 0:
            x = x + m * norm_around_zero(mixture_of_experts(norm_around_zero(x, lw["norm2"], eps), sub(lw, "mlp."), l),
                                         lw["norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T


def greedy(mc, weights: dict, prompt: list[int], n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(mc, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
