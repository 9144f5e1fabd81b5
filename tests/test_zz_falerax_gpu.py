"""-m gpu parity of the Falerax architecture against oracle/falerax_oracle.py.

Kernel level (include/tgis_kernels.h hooks), each mechanism alone and run in portions through its state slot or paged cache:
softcapped grouped-query attention (with inputs built so that ONE key decides: far away, on both sides of a cache block's
border, the first token), the gated matrix memory, token shift + decayed outer-product memory, short convolution + selective
scan, the averaged pair tail and the GeGLU epilogue.
Engine level (trace replay = the engine's own step function, sequence slots and block manager): whole prompts in fp32 and
bf16, portions down to two tokens, token-by-token decoding, mixed batches against each request alone with blocks and state
slots that are used again, long decoding across block borders, other sizes and layer orders (values equal to 1, parts
absent), and greedy generation through add_request + the step loop with and without CUDA-graph replay."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 1
KV_BLOCK = 32
F64 = torch.float64


def _lib():
    from vllm_tgis_adapter_b200.engine import _lib as L

    return L.load_library()


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _ok(rc):
    assert rc == 0, (_lib().tgis_k_last_error() or b"").decode()


_KEEP = []   # device tensors whose pointers went into a C call stay alive until the test ends


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    _KEEP.clear()


def _dev(t, dt=torch.float32):
    d = t.to(dt).cuda().contiguous()
    _KEEP.append(d)
    return d


def _ints(v):
    return (C.c_int32 * len(v))(*v)


def _i32(v):
    d = torch.tensor(v, dtype=torch.int32).cuda()
    _KEEP.append(d)
    return d


def _close(got, ref, tol):
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    err = float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err < tol, err


def _eye_rows(width, start, n):
    """[n, width]: the projection that copies columns [start, start + n) of the input."""
    w = torch.zeros(n, width, dtype=F64)
    w[torch.arange(n), start + torch.arange(n)] = 1.0
    return w


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n))
        at += n
        i += 1
    return out


# ====================================================================================================== attention
def _cap_geom(m):
    from vllm_tgis_adapter_b200.engine._lib import TgisKCapAttnGeom

    qt = m.get("q_temp") or {}
    return TgisKCapAttnGeom(m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m.get("softcap") or 0.0,
                            qt.get("coef", 0.0), qt.get("every", 0))


def _run_capattn(h, m, wq, wk, dt, sizes, pool_blocks=24, seed=0):
    """h [T, width] whose columns are [q | k | v | gate logits]: the sequence goes through the kernels in portions of the given
    sizes over a paged cache whose blocks are scattered through the pool.  Returns the gated heads [T, heads * vdim]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    tdt = torch.bfloat16 if dt == BF16 else torch.float32
    geom = _cap_geom(m)
    n_blocks = (T + KV_BLOCK - 1) // KV_BLOCK
    blocks = torch.randperm(pool_blocks, generator=torch.Generator().manual_seed(seed))[:n_blocks].tolist()
    kc = torch.zeros(pool_blocks * KV_BLOCK, G * d, dtype=tdt, device="cuda")
    vc = torch.zeros(pool_blocks * KV_BLOCK, G * dv, dtype=tdt, device="cuda")
    y = _dev(h)
    out = torch.full((T, H * dv), float("nan"), dtype=tdt, device="cuda")
    wq_d, wk_d = _dev(wq), _dev(wk)
    c_q, c_k, c_v, c_g = 0, H * d, H * d + G * d, H * d + G * d + G * dv
    for at, n in _portions(T, sizes):
        pos = list(range(at, at + n))
        slots = [blocks[p // KV_BLOCK] * KV_BLOCK + p % KV_BLOCK for p in pos]
        q = torch.zeros(n, H * d, dtype=tdt, device="cuda")
        yp = y[at:at + n].contiguous()
        _ok(_lib().tgis_k_capattn_prep(_p(yp), y.shape[1], c_q, c_k, c_v, C.byref(geom), _p(wq_d), _p(wk_d), 1e-5, _p(_i32(pos)),
                                       _p(_i32(slots)), _p(q), _p(kc), _p(vc), dt, n))
        gate = yp[:, c_g:].contiguous()
        o = torch.full((n, H * dv), float("nan"), dtype=tdt, device="cuda")
        _ok(_lib().tgis_k_capattn(_p(q), _p(kc), _p(vc), dt, _ints([0, n, at + n, 0]), 1, _ints(blocks), 1, len(blocks), _p(gate),
                                  H * dv, _p(o), C.byref(geom)))
        out[at:at + n] = o
    return out


def _cap_weights(m, wq, wk):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width = H * d + G * d + G * dv + H * dv
    return width, {"q": _eye_rows(width, 0, H * d), "k": _eye_rows(width, H * d, G * d), "v": _eye_rows(width, H * d + G * d, G * dv),
                   "g": _eye_rows(width, H * d + G * d + G * dv, H * dv), "q.norm": wq.double(), "k.norm": wk.double(),
                   "o": torch.eye(H * dv, dtype=F64)}


@pytest.mark.parametrize("m", [
    dict(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.4, softcap=5.0, q_temp=dict(coef=0.4, every=7)),
    dict(heads=3, kv_heads=1, dim=40, vdim=33, scale=0.2, softcap=0.0),
    dict(heads=2, kv_heads=2, dim=5, vdim=140, scale=0.5, softcap=50.0, q_temp=dict(coef=1.5, every=1)),
    dict(heads=1, kv_heads=1, dim=64, vdim=64, scale=0.125, softcap=2.0, q_temp=dict(coef=0.1, every=64)),
    # sizes the tensor-core kernels take in bf16: one head per CTA, and the heads of a key/value head grouped in one CTA
    dict(heads=2, kv_heads=2, dim=96, vdim=200, scale=0.1, softcap=15.0, q_temp=dict(coef=0.3, every=50)),
    dict(heads=4, kv_heads=2, dim=32, vdim=48, scale=0.2, softcap=8.0, q_temp=dict(coef=0.3, every=20)),
    dict(heads=8, kv_heads=1, dim=16, vdim=128, scale=0.3, softcap=0.0),
    dict(heads=6, kv_heads=2, dim=128, vdim=8, scale=0.09, softcap=25.0),
])
@pytest.mark.parametrize("dt", [F32, BF16])
def test_capped_attention_in_portions_matches_oracle(m, dt):
    from oracle import falerax_oracle as O

    g = torch.Generator().manual_seed(m["dim"])
    T = 150
    wq, wk = 1.0 + 0.2 * torch.randn(m["dim"], generator=g), 1.0 + 0.2 * torch.randn(m["dim"], generator=g)
    width, w = _cap_weights(m, wq, wk)
    h = torch.randn(T, width, generator=g)
    ref = O.capped_attention(h.double(), w, m, 1e-5)
    for sizes in ([T], [1], [2, 33, 1, 17, 64]):
        got = _run_capattn(h, m, wq, wk, dt, sizes, seed=len(sizes))
        _close(got, ref, 1e-5 if dt == F32 else 3e-2)


def test_capped_attention_grouped_heads_kernel_matches_oracle(monkeypatch):
    """The variant that runs the query heads of one key/value head in one CTA (an experiment switch, off by default)."""
    from oracle import falerax_oracle as O

    monkeypatch.setenv("TGIS_CAPATTN_GROUP", "1")
    for m in (dict(heads=4, kv_heads=2, dim=32, vdim=48, scale=0.2, softcap=8.0, q_temp=dict(coef=0.3, every=20)),
              dict(heads=8, kv_heads=1, dim=16, vdim=128, scale=0.3, softcap=0.0),
              dict(heads=6, kv_heads=2, dim=128, vdim=8, scale=0.09, softcap=25.0)):
        g = torch.Generator().manual_seed(m["vdim"])
        T = 150
        wq, wk = 1.0 + 0.2 * torch.randn(m["dim"], generator=g), 1.0 + 0.2 * torch.randn(m["dim"], generator=g)
        width, w = _cap_weights(m, wq, wk)
        h = torch.randn(T, width, generator=g)
        ref = O.capped_attention(h.double(), w, m, 1e-5)
        for sizes in ([T], [1], [2, 33, 1, 17, 64]):
            _close(_run_capattn(h, m, wq, wk, BF16, sizes, seed=len(sizes)), ref, 3e-2)


@pytest.mark.parametrize("key", [0, 31, 32, 63, 64, 200, 399])
@pytest.mark.parametrize("shape", ["prompt", "decode"])
def test_capped_attention_one_key_decides(key, shape):
    """Query 399 and key `key` point the same way and are long before the norm's weight; every other key is orthogonal to
    the query: the output must be that key's value -- far away, at a block's last and first rows, the first token."""
    from oracle import falerax_oracle as O

    m = dict(heads=2, kv_heads=1, dim=8, vdim=12, scale=4.0, softcap=30.0)
    T = 400
    g = torch.Generator().manual_seed(key)
    wq = wk = torch.ones(8)
    width, w = _cap_weights(m, wq, wk)
    h = torch.zeros(T, width)
    H, G, d, dv = 2, 1, 8, 12
    kcols = slice(H * d, H * d + d)
    h[:, kcols] = torch.randn(T, d, generator=g)
    h[:, kcols.start] = 0.0                      # all keys orthogonal to e0 ...
    h[key, kcols] = 0.0
    h[key, kcols.start] = 1.0                    # ... but one
    h[T - 1, 0], h[T - 1, d] = 1.0, 1.0          # the last query of both heads is e0
    h[:, H * d + d: H * d + d + dv] = torch.randn(T, dv, generator=g)
    h[:, H * d + d + dv:] = 20.0                 # gates open
    ref = O.capped_attention(h.double(), w, m, 1e-5)
    assert torch.allclose(ref[T - 1, :dv], h[key, H * d + d: H * d + d + dv].double(), atol=1e-3)   # the oracle agrees with the construction
    sizes = [T] if shape == "prompt" else [T - 1, 1]
    got = _run_capattn(h, m, wq, wk, F32, sizes, seed=key)
    _close(got[T - 1], ref[T - 1], 1e-5)


# ====================================================================================================== recurrences
def _seq_meta(at, n, row0=0):
    return [row0, n, at + n, 0]


def test_gated_matrix_memory_in_portions_and_two_slots_matches_oracle():
    from oracle import falerax_oracle as O

    for m, T in ((dict(heads=3, dim=5, vdim=7, gate_cap=4.0), 90), (dict(heads=1, dim=70, vdim=40, gate_cap=15.0), 40),
                 (dict(heads=2, dim=130, vdim=33, gate_cap=8.0), 20)):
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        g = torch.Generator().manual_seed(d)
        cols = [H * d, H * d, H * dv, H * dv, H, H]
        width = sum(cols)
        offs = np.concatenate([[0], np.cumsum(cols)]).tolist()
        names = ["q", "k", "v", "g", "i", "f"]
        w = {n: _eye_rows(width, offs[j], cols[j]) for j, n in enumerate(names)}
        w["i.b"], w["f.b"] = torch.randn(H, generator=g).double(), (1.0 + torch.randn(H, generator=g)).double()
        w["norm"] = (1.0 + 0.1 * torch.randn(H * dv, generator=g)).double()
        w["o"] = torch.eye(H * dv, dtype=F64)
        seqs = [torch.randn(T, width, generator=g) * 1.5, torch.randn(T - 7, width, generator=g) * 1.5]
        refs = [O.matrix_memory(s.double(), w, m, 1e-5) for s in seqs]
        slots_n = 3
        S = torch.full((slots_n, H, d, dv), 7.0, device="cuda")       # stale state of an earlier owner: must be ignored
        nst, mst = torch.full((slots_n, H, d), 7.0, device="cuda"), torch.full((slots_n, H), 7.0, device="cuda")
        ib, fb, nw = _dev(w["i.b"]), _dev(w["f.b"]), _dev(w["norm"])
        for sizes in ([1000], [1], [2, 9, 1, 30]):
            got = [[], []]
            plans = [_portions(len(s), sizes) for s in seqs]
            for step in range(max(len(p) for p in plans)):
                # both sequences in one launch when both still have portions: slots 2 and 0
                live = [(i, plans[i][step]) for i in range(2) if step < len(plans[i])]
                rows = torch.cat([seqs[i][at:at + n] for i, (at, n) in live])
                y = _dev(rows)
                meta, tokslot, r0 = [], [], 0
                for i, (at, n) in live:
                    meta += _seq_meta(at, n, r0)
                    tokslot += [2 - 2 * i] * n
                    r0 += n
                o = torch.full((r0, H * dv), float("nan"), device="cuda")
                _ok(_lib().tgis_k_outer_scan(1, _p(y[:, offs[0]:]), _p(y[:, offs[1]:]), _p(y[:, offs[2]:]), width, width, width,
                                             d ** -0.5, None, 0, None, None, _p(y[:, offs[4]:]), _p(y[:, offs[5]:]), width, _p(ib),
                                             _p(fb), m["gate_cap"], _p(S), _p(nst), _p(mst), _p(o), H * dv, H, d, dv, None, None, 0,
                                             _ints(meta), len(live), _p(_i32(tokslot))))
                out = torch.full((r0, H * dv), float("nan"), device="cuda")
                _ok(_lib().tgis_k_head_norm_gate(_p(o), H * dv, H, dv, _p(nw), _p(y[:, offs[3]:]), width, 0, 1e-5, _p(out), F32, r0))
                r0 = 0
                for i, (at, n) in live:
                    got[i].append(out[r0:r0 + n].cpu())
                    r0 += n
            for i in range(2):
                _close(torch.cat(got[i]), refs[i], 2e-5)


def test_token_shift_and_decayed_memory_in_portions_matches_oracle():
    from oracle import falerax_oracle as O

    for m, W, rank, T in ((dict(heads=2, dim=12), 20, 3, 80), (dict(heads=1, dim=100), 36, 1, 30), (dict(heads=5, dim=4), 24, 6, 50)):
        H, d = m["heads"], m["dim"]
        A = H * d
        g = torch.Generator().manual_seed(A)
        w = {f"mu.{s}": torch.rand(W, generator=g).double() for s in "rkvgw"}
        for s in "rkvg":
            w[s] = (torch.randn(A, W, generator=g) * W ** -0.5).double()
        w["w1"], w["w2"] = (torch.randn(rank, W, generator=g) * W ** -0.5).double(), torch.randn(A, rank, generator=g).double()
        w["w0"], w["u"] = (torch.randn(A, generator=g) * 0.5 - 1.0).double(), torch.randn(H, d, generator=g).double()
        w["norm"], w["o"] = (1.0 + 0.1 * torch.randn(A, generator=g)).double(), torch.eye(A, dtype=F64)
        x = torch.randn(T, W, generator=g)
        ref = O.wkv_mixer(x.double(), w, m, 1e-5)
        mu = _dev(torch.stack([w[f"mu.{s}"] for s in "rkvgw"]))
        w0, u, nw = _dev(w["w0"]), _dev(w["u"].reshape(-1)), _dev(w["norm"])
        for sizes in ([T], [1], [2, 1, 13, 40]):
            prev = torch.full((2, W), 9.0, device="cuda")             # stale: position 0 must not read it
            S = torch.full((2, H, d, d), 9.0, device="cuda")
            got = []
            for at, n in _portions(T, sizes):
                xs = _dev(x[at:at + n])
                mixes = torch.empty(5, n, W, device="cuda")
                tokslot = _i32([1] * n)
                _ok(_lib().tgis_k_token_shift(_p(xs), W, _p(mu), 5, _p(_i32(list(range(at, at + n)))), _p(tokslot), _p(prev),
                                              _p(mixes), F32, n * W, n))
                mx = mixes.double().cpu()
                r, k, v, gl = (_dev(mx[j] @ w[s].T) for j, s in enumerate("rkvg"))
                draw = _dev(torch.tanh(mx[4] @ w["w1"].T) @ w["w2"].T)
                o = torch.full((n, A), float("nan"), device="cuda")
                _ok(_lib().tgis_k_outer_scan(0, _p(r), _p(k), _p(v), A, A, A, 1.0, _p(draw), A, _p(w0), _p(u), None, None, 0, None,
                                             None, 0.0, _p(S), None, None, _p(o), A, H, d, d, _p(xs), _p(prev), W,
                                             _ints(_seq_meta(at, n)), 1, _p(tokslot)))
                out = torch.empty(n, A, device="cuda")
                _ok(_lib().tgis_k_head_norm_gate(_p(o), A, H, d, _p(nw), _p(gl), A, 1, 1e-5, _p(out), F32, n))
                got.append(out.cpu())
            _close(torch.cat(got), ref, 2e-5)


def test_short_convolution_and_selective_scan_in_portions_matches_oracle():
    from oracle import falerax_oracle as O

    for m, W, T in ((dict(inner=24, state=5, dt_rank=3, conv=3), 16, 70), (dict(inner=70, state=1, dt_rank=1, conv=1), 8, 20),
                    (dict(inner=9, state=40, dt_rank=4, conv=6), 12, 45), (dict(inner=130, state=16, dt_rank=8, conv=2), 10, 33)):
        I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
        g = torch.Generator().manual_seed(I)
        w = {"in": torch.randn(2 * I, W, generator=g) * W ** -0.5, "conv": torch.randn(I, K, generator=g) * 0.6,
             "conv.b": torch.randn(I, generator=g) * 0.1, "x": torch.randn(R + 2 * N, I, generator=g) * I ** -0.5,
             "dt": torch.randn(I, R, generator=g), "dt.b": torch.randn(I, generator=g) - 2.0,
             "A_log": torch.log(torch.arange(1, N + 1).float()).repeat(I, 1), "D": torch.randn(I, generator=g),
             "o": torch.eye(I)}
        w = {k: v.double() for k, v in w.items()}
        h = torch.randn(T, W, generator=g)
        ref = O.selective_scan(h.double(), w, m)
        dev = {k: _dev(v) for k, v in w.items()}
        for sizes in ([T], [1], [2, 1, 5, 31]):
            cst = torch.full((2, max(K - 1, 1), I), 9.0, device="cuda")
            S = torch.full((2, I, N), 9.0, device="cuda")
            got = []
            for at, n in _portions(T, sizes):
                xz = _dev(h[at:at + n].double() @ w["in"].T)
                tokslot, pos = _i32([1] * n), _i32(list(range(at, at + n)))
                xc = torch.empty(n, I, device="cuda")
                _ok(_lib().tgis_k_short_conv(_p(xz), 2 * I, I, _p(dev["conv"]), _p(dev["conv.b"]), K, _p(pos), _p(tokslot), _p(cst),
                                             _p(xc), None, F32, n))
                proj = _dev(xc.double().cpu() @ w["x"].T)
                dtraw = _dev(proj.double().cpu()[:, :R] @ w["dt"].T)
                out = torch.full((n, I), float("nan"), device="cuda")
                _ok(_lib().tgis_k_selective_scan(_p(xc), _p(xz), 2 * I, _p(proj), R + 2 * N, R, _p(dtraw), _p(dev["dt.b"]),
                                                 _p(dev["A_log"]), _p(dev["D"]), _p(S), _p(cst), _p(out), F32, I, N, K,
                                                 _ints(_seq_meta(at, n)), 1, _p(tokslot)))
                got.append(out.cpu())
            _close(torch.cat(got), ref, 2e-5)


def test_pair_tail_and_geglu_epilogue_match_oracle():
    from oracle import falerax_oracle as O

    T, W, eps = 9, 50, 1e-3
    g = torch.Generator().manual_seed(3)
    ya, yb, x = (torch.randn(T, W, generator=g) * s for s in (3.0, 0.2, 1.0))
    wa, wb, wp, wn = (1.0 + 0.3 * torch.randn(W, generator=g) for _ in range(4))
    y = 0.5 * (O.rms(ya.double(), eps) * wa.double() + O.rms(yb.double(), eps) * wb.double())
    ref = x.double() + O.rms(y, eps) * wp.double()
    for w_pre, dt in ((None, F32), (None, BF16), (wn, F32)):
        resid = _dev(x)
        out = torch.zeros(T, W, device="cuda", dtype=torch.bfloat16 if dt == BF16 else torch.float32)
        _ok(_lib().tgis_k_resid_tail_pair(_p(_dev(ya)), _p(_dev(yb)), _p(_dev(wa)), _p(_dev(wb)), _p(_dev(wp)),
                                          _p(_dev(w_pre)) if w_pre is not None else None, _p(resid), _p(out), dt, 1, eps, T, W))
        _close(resid, ref, 1e-5)
        _close(out, ref if w_pre is None else O.rms(ref, eps) * wn.double(), 1e-5 if dt == F32 else 1e-2)
    # GeGLU: gate / up rows interleaved, the gated activation in the product's epilogue
    K, ff = 24, 11
    h = torch.randn(T, K, generator=g)
    gate, up, down = torch.randn(ff, K, generator=g), torch.randn(ff, K, generator=g), torch.eye(ff)
    wi = torch.empty(2 * ff, K)
    wi[0::2], wi[1::2] = gate, up
    for tdt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        hx, wx = _dev(h, tdt), _dev(wi, tdt)
        yv = torch.zeros(T, ff, device="cuda", dtype=tdt)
        code = BF16 if tdt == torch.bfloat16 else F32
        _ok(_lib().tgis_k_gemm_any(_p(hx), _p(wx), _p(yv), code, code, code, T, 2 * ff, K, K, K, ff, 1, 0, 0, 0, None, 0, 0, None, 1,
                                   3, None, 0))
        ref = O.dense_ff(hx.double().cpu(), {"gate": wx[0::2].double().cpu(), "up": wx[1::2].double().cpu(), "down": down.double()})
        _close(yv, ref, tol)


# ====================================================================================================== engine
def _cfg(layers=None, width=40, vocab=97):
    layers = layers or [
        {"type": "mamba1", "mixer": {"inner": 24, "state": 5, "dt_rank": 3, "conv": 3}, "mlp": {"kind": "dense", "ff": 28}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.3, "softcap": 5.0, "q_temp": {"coef": 0.4, "every": 7}},
            "right": {"heads": 3, "dim": 5, "vdim": 7, "gate_cap": 4.0}}, "mlp": None},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 12}, "mlp": {"kind": "dense", "ff": 20}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.25, "softcap": 12.0, "q_temp": {"coef": 0.2, "every": 32}},
            "right": {"heads": 1, "dim": 9, "vdim": 20, "gate_cap": 10.0}}, "mlp": {"kind": "dense", "ff": 33}},
    ]
    return {"architecture": "Falerax", "width": width, "vocab": vocab, "norm": {"eps": 1e-4}, "layers": layers}


def _model(cfg, dtype="float32", max_model_len=512, decay_rank=4):
    from vllm_tgis_adapter_b200.engine.falerax import model_config_from_json

    shapes = {f"l{i}.mix.w1": (decay_rank, cfg["width"]) for i, l in enumerate(cfg["layers"]) if l["type"] == "wkv"}
    return model_config_from_json(cfg, max_model_len, dtype, shapes)


def _engine(mc, weights, *, blocks=16, seqs=4, graphs=False, tokens=512):
    from vllm_tgis_adapter_b200.engine.core import NativeEngine, cache_block_bytes

    eng = NativeEngine(mc, max_num_seqs=seqs, max_batched_tokens=tokens, kv_cache_bytes=cache_block_bytes(mc) * blocks,
                       use_cuda_graphs=graphs)
    eng.load_weights(weights)
    return eng


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rel(got, ref):
    """Error of logit rows the way a user sees it: mean removed, root mean square, relative to the rows' own spread."""
    d = torch.as_tensor(got).double() - ref
    d = d - d.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / ref.std(-1)).max())


def _bf16_close(got, ref):
    """bf16 operands on widths this small: rounding alone moves single rows by several percent of their spread, so the bound
    is on the typical row and on the tail (the sharp comparison is the float32 one)."""
    rows = sorted(_rel(got[t:t + 1], ref[t:t + 1]) for t in range(len(ref)))
    return rows[len(rows) // 2] < 3e-2 and rows[int(0.95 * len(rows))] < 0.1 and rows[-1] < 0.3


def _whole(eng, toks, rid="w"):
    return eng.trace_step([(rid, toks, list(range(len(toks))))], [rid])


def test_whole_prompt_matches_oracle_fp32_and_bf16():
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    toks = _tokens(150, 97, 1)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", None)):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 11)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        got = _whole(eng, toks)
        if dtype == "float32":
            for n in (1, 2):    # the first tokens of a sequence on their own
                assert _rel(_whole(eng, toks[:n]), O.forward(cfg, weights, toks[:n])) < tol
        eng.close()
        assert _rel(got, ref) < tol if tol else _bf16_close(got, ref), dtype


def _variants():
    par = lambda left, right, mlp=None: {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}  # noqa: E731
    ff = lambda n: {"kind": "dense", "ff": n}  # noqa: E731
    return {
        "ones": _cfg([par({"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0, "softcap": 1.0, "q_temp": {"coef": 1.0, "every": 1}},
                          {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 1.0}, ff(1)),
                      {"type": "mamba1", "mixer": {"inner": 1, "state": 1, "dt_rank": 1, "conv": 1}, "mlp": None},
                      {"type": "wkv", "mixer": {"heads": 1, "dim": 1}, "mlp": None}], width=6, vocab=11),
        "no_cap_no_temperature_no_ff": _cfg([par({"heads": 6, "kv_heads": 3, "dim": 7, "vdim": 7, "scale": 0.4},
                                                 {"heads": 2, "dim": 6, "vdim": 6, "gate_cap": 30.0})], width=22),
        "only_recurrent": _cfg([{"type": "wkv", "mixer": {"heads": 3, "dim": 5}, "mlp": ff(17)},
                                {"type": "mamba1", "mixer": {"inner": 50, "state": 9, "dt_rank": 2, "conv": 5}, "mlp": None},
                                {"type": "wkv", "mixer": {"heads": 1, "dim": 70}, "mlp": None}], width=30),
        "attention_first_equal_sizes": _cfg([par({"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18, "softcap": 3.0,
                                                  "q_temp": {"coef": 0.7, "every": 3}},
                                                 {"heads": 2, "dim": 32, "vdim": 32, "gate_cap": 2.0}, ff(64)),
                                             {"type": "mamba1", "mixer": {"inner": 64, "state": 16, "dt_rank": 4, "conv": 4}, "mlp": ff(64)}],
                                            width=64, vocab=130),
        "tensor_core_sizes": _cfg([{"type": "wkv", "mixer": {"heads": 5, "dim": 64}, "mlp": ff(512)},
                                   par({"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 96, "scale": 0.125, "softcap": 20.0},
                                       {"heads": 2, "dim": 64, "vdim": 128, "gate_cap": 15.0}, ff(256)),
                                   {"type": "mamba1", "mixer": {"inner": 512, "state": 8, "dt_rank": 16, "conv": 4}, "mlp": None}],
                                  width=320, vocab=300),
    }


@pytest.mark.parametrize("name", list(_variants()))
def test_other_sizes_orders_and_absent_parts(name):
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _variants()[name]
    toks = _tokens(70, cfg["vocab"], 7)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", None)):
        mc = _model(cfg, dtype, decay_rank=1 if name == "ones" else 5)
        weights = synthetic_weights(mc, 23)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        whole = _whole(eng, toks)
        parts = [eng.trace_step([("p", toks[a:a + n], list(range(n)))], ["p"] if a + n == len(toks) else [])
                 for a, n in _portions(len(toks), [3, 1, 40, 2])]
        eng.close()
        parts = np.concatenate(parts)
        if tol:
            assert _rel(whole, ref) < tol and _rel(parts, ref) < tol, (name, dtype)
        elif name != "ones":    # (single-entry heads in bf16: a norm of one rounded number is a sign, nothing to bound)
            assert _bf16_close(whole, ref) and _bf16_close(parts, ref), (name, dtype)


def test_prefill_portions_and_token_by_token_agree_with_whole_prompt():
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 31)
    toks = _tokens(131, 97, 3)
    ref = O.forward(cfg, weights, toks)
    eng = _engine(mc, weights)
    for sizes in ([2], [1], [31, 33, 2, 64, 1], [64, 1, 1, 1, 1, 1, 1]):
        got = [eng.trace_step([("s", toks[a:a + n], list(range(n)))], ["s"] if a + n == len(toks) else [])
               for a, n in _portions(len(toks), sizes)]
        assert _rel(np.concatenate(got), ref) < 3e-5, sizes
    eng.close()


def test_long_decoding_crosses_block_borders_bf16_stays_close():
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    toks = _tokens(300, 97, 9)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", None)):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 37)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        got = [eng.trace_step([("d", toks[:40], list(range(40)))], [])]
        for t in range(40, 300):
            got.append(eng.trace_step([("d", [toks[t]], [0])], ["d"] if t == 299 else []))
        eng.close()
        got = np.concatenate(got)
        assert _rel(got, ref) < tol if tol else _bf16_close(got, ref), dtype


def test_mixed_batches_of_unequal_requests_match_each_alone_and_reuse_blocks_and_slots():
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 41)
    reqs = {f"q{i}": _tokens(n, 97, 50 + i) for i, n in enumerate([97, 40, 3, 130, 64, 33, 71, 1, 90])}
    ref = {k: O.forward(cfg, weights, v) for k, v in reqs.items()}
    # 3 slots and a pool of 10 blocks: the requests only fit because finished ones give their state slot and blocks back
    eng = _engine(mc, weights, blocks=10, seqs=3)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    nb = lambda k: (len(reqs[k]) + KV_BLOCK - 1) // KV_BLOCK  # noqa: E731
    waiting, live, step = list(reqs), [], 0
    while waiting or live:
        while waiting and len(live) < 3 and sum(nb(k) for k in live) + nb(waiting[0]) <= 10:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            if (step + j) % 5 == 4:
                continue                                        # a request may sit a step out
            n = min(len(reqs[k]) - at[k], [1, 7, 2, 29, 1, 33][(step + 2 * j) % 6])   # single tokens beside portions
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                ends.append(k)
        if entries:
            out = eng.trace_step(entries, ends)
            o = 0
            for k, t, _ in entries:
                got[k].append(out[o:o + len(t)])
                o += len(t)
        live = [k for k in live if k not in ends]
        step += 1
    st = eng.status()
    eng.close()
    assert st.free_blocks == st.total_blocks == 10
    for k in reqs:
        assert _rel(np.concatenate(got[k]), ref[k]) < 3e-5, k


def test_greedy_generation_through_the_scheduler_matches_oracle():
    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.core import make_sampling_params
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 61)
    prompts = [_tokens(45, 97, 70), _tokens(3, 97, 71), _tokens(80, 97, 72)]
    n_new = 40
    for graphs in (False, True):
        eng = _engine(mc, weights, graphs=graphs, tokens=64)     # 64-token steps: the prompts are prefilled in portions
        sp = make_sampling_params(greedy=True, max_tokens=n_new, min_tokens=n_new, eos_token_id=-1, num_logprobs=1)
        outs = eng.generate_sync(prompts, sp)
        st = eng.status()
        eng.close()
        assert st.errored == 0 and (st.graph_launches > 0) == graphs
        for p, recs in zip(prompts, outs):
            toks = [r.new_token for r in recs if r.new_token is not None]
            assert toks == O.greedy(cfg, weights, p, n_new), graphs
            lp = torch.log_softmax(O.forward(cfg, weights, p + toks[:-1])[len(p) - 1:], -1)
            for i, r in enumerate([r for r in recs if r.new_token is not None]):
                assert abs(r.logprob - float(lp[i, r.new_token])) < 1e-3


def test_trace_runner_command_line_on_a_model_directory(tmp_path):
    """bin/trace_run on a directory with config.json + model.safetensors: the family and the decay map's rank come from the
    files, a mixed schedule with a reused slot goes through standard input, the logits land in the output folder."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import save_file

    from oracle import falerax_oracle as O
    from vllm_tgis_adapter_b200.engine.falerax import synthetic_weights

    cfg = _cfg()
    weights = synthetic_weights(_model(cfg, decay_rank=3), 71)
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(model / "model.safetensors"))
    a, b, c = _tokens(70, 97, 1), _tokens(9, 97, 2), _tokens(40, 97, 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}, {"id": "a", "tokens": a[33:69], "want": []}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}, {"id": "c", "tokens": c, "want": [39]}], "end": ["a", "c"]},
    ]
    root = Path(__file__).resolve().parent.parent
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 0.1)):
        out = tmp_path / f"out_{dtype}"
        p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                           text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        ra, rb, rc = (O.forward(cfg, weights, t) for t in (a, b, c))
        want = {0: torch.stack([ra[0], ra[32], rb[1]]), 1: rb[8:9], 2: torch.stack([ra[69], rc[39]])}
        for n, ref in want.items():
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 97)
            assert _rel(got, ref) < tol, (dtype, n)
