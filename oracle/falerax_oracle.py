"""Plain, slow restatement of the Falerax decoder in float64 torch on the CPU: one function per mechanism, whole sequences
only (no cache, no state slots, no batching, no chunking), token-by-token loops for every recurrence.  It shares no code
with the engine; the GPU tests compare the engine's kernels and steps with it.

`cfg` is the model's config.json as a dict, `weights` maps checkpoint names to tensors.

Notation.  x_t: residual stream at position t (positions count from 0).  rms(v) = v / sqrt(mean(v^2) + eps).
A layer is   x <- x + rms(mixer(x)) * n1,   x <- x + rms(ff(x)) * n2   (the second line only with a feed-forward): the
sublayers read the stream itself, only their outputs are normed.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def logsigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


# ------------------------------------------------------------------------------------------------ softcapped attention
def query_temperature(T: int, coef: float, every: int) -> torch.Tensor:
    """[T]: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T)
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").to(F64) + 1.0)


def capped_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Causal grouped-query attention without rotation: per-head RMS norm of queries and keys (one weight for all heads),
    position-dependent query temperature, tanh soft cap on the scores, sigmoid output gate read from the same input."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ w["q"].T).view(T, H, d), eps) * w["q.norm"]
    k = rms((h @ w["k"].T).view(T, G, d), eps) * w["k.norm"]
    v = (h @ w["v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(T, float(qt["coef"]), int(qt["every"]))[:, None, None]
    cap = float(m.get("softcap") or 0.0)
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~causal, -math.inf)
        out.append(torch.softmax(s, -1) @ v[:, g])
    o = torch.cat(out, -1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ------------------------------------------------------------------------------------------------ matrix memory (mLSTM)
def matrix_memory(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Per head a matrix S [dim, vdim], a vector n [dim] and a running maximum mx (all start at 0).  With log gates
    i_t, f_t:  mx' = max(f + mx, i);  S' = e^(f + mx - mx') S + e^(i - mx') k v^T;  n' likewise with k;
    o = S'^T q / (max(|n' . q|, e^(-mx')) + 1e-6)."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                       # [T, H]
    fg = logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        mx = 0.0
        for t in range(T):
            f, i = float(fg[t, hd]), float(ig[t, hd])
            mn = max(f + mx, i)
            a, b = math.exp(f + mx - mn), math.exp(i - mn)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = mn
            den = max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = rms(out, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Softcapped attention and the matrix memory side by side on the same input: each output is normed over the model
    width with its own weight, the result is half their sum."""
    left = capped_attention(h, sub(w, "left."), m["left"], eps)
    right = matrix_memory(h, sub(w, "right."), m["right"], eps)
    return 0.5 * (rms(left, eps) * w["left.out"] + rms(right, eps) * w["right.out"])


# ------------------------------------------------------------------------------------------------ selective scan
def selective_scan(h: torch.Tensor, w: dict, m: dict) -> torch.Tensor:
    """W_in h = [x | z]; x <- silu(causal conv over the last `conv` inputs); W_x x = [dt | B | C];
    dt <- softplus(W_dt dt + b); S[c, n] <- e^(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = S[c] . C + D_c x_c; y silu(z)."""
    T = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ w["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    xp = torch.cat([torch.zeros(taps - 1, inner, dtype=F64), x], 0)
    xc = torch.stack([(xp[t: t + taps] * w["conv"].T).sum(0) for t in range(T)]) + w["conv.b"]
    x = silu(xc)
    p = x @ w["x"].T
    dt = softplus(p[:, :R] @ w["dt"].T + w["dt.b"])                              # [T, inner]
    B, C = p[:, R: R + N], p[:, R + N: R + 2 * N]
    A = -torch.exp(w["A_log"])                                                   # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w["D"] * x[t]
    return (y * silu(z)) @ w["o"].T


# ------------------------------------------------------------------------------------------------ decayed outer-product memory
def wkv_mixer(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Every projection reads its own blend of the token and its predecessor, h + (h_prev - h) mu_s.  Per head a matrix
    S [dim, dim]:  o_t = (S + diag(u) k v^T)^T r,  then  S <- diag(w_t) S + k v^T,  w_t = e^(-e^(W_w2 tanh(W_w1 .) + w0))."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=F64), h[:-1]], 0)
    mix = {s: h + (prev - h) * w["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].T).view(T, H, d)
    k = (mix["k"] @ w["k"].T).view(T, H, d)
    v = (mix["v"] @ w["v"].T).view(T, H, d)
    gate = silu(mix["g"] @ w["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).view(T, H, d)
    out = torch.zeros(T, H, d, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, d, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = (S + w["u"][hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    o = rms(out, eps).reshape(T, H * d) * w["norm"] * gate
    return o @ w["o"].T


# ------------------------------------------------------------------------------------------------ feed-forward, model
def dense_ff(h: torch.Tensor, w: dict) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(kind: str, h, w, m, eps):
    if kind == "parallel":
        return parallel_mixer(h, w, m, eps)
    if kind == "mamba1":
        return selective_scan(h, w, m)
    if kind == "wkv":
        return wkv_mixer(h, w, m, eps)
    raise ValueError(kind)


def forward(cfg: dict, weights: dict, tokens: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of every position of one sequence."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        lw = sub(w, f"l{i}.")
        x = x + rms(mixer(layer["type"], x, sub(lw, "mix."), layer["mixer"], eps), eps) * lw["norm1"]
        if layer.get("mlp") is not None:
            x = x + rms(dense_ff(x, sub(lw, "mlp.")), eps) * lw["norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T


def greedy(cfg: dict, weights: dict, prompt: list[int], n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
