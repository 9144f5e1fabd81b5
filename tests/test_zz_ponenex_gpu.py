"""-m gpu parity of the Ponenex architecture (latent attention with a sliding window, mixture of experts with a gated
shared expert, pre- and post-normed sublayers on an fp32 residual stream) against oracle/ponenex_oracle.py.

Kernel level (include/tgis_kernels.h hooks): the general matrix product in its three geometries and epilogues, the fp32
norms and the sublayer tail, the latent preparation (norms, rotary key, cache write, gates), the query rotation, the
windowed attention over the paged latent cache with inputs built so that ONE key decides the result, router and row lists.
Engine level (trace replay = the engine's own step function, scheduler slots and block manager): whole prompts, portions
down to two tokens, token-by-token decoding, mixed batches against each request alone, blocks and slots that are used
again, windows and block borders crossed while decoding, sizes where heads / top / experts are 1 or where parts are absent,
and greedy generation through add_request + the step loop."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 1
KV_BLOCK = 32


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


def _tdt(code):
    return torch.bfloat16 if code == BF16 else torch.float32


# ====================================================================================================== kernels
def _gemm_any(x, w, y, T, N, K, *, ldx=None, ldw=None, ldy=None, batch=1, x_bs=0, w_bs=0, y_bs=0, seg_off=None, n_groups=0,
              w_gs=0, gather=None, gather_div=1, mode=0, row_scale=None, scale_ld=0):
    code = lambda t: BF16 if t.dtype == torch.bfloat16 else F32  # noqa: E731
    _ok(_lib().tgis_k_gemm_any(_p(x), _p(w), _p(y), code(x), code(w), code(y), T, N, K, ldx or K, ldw or K, ldy or N, batch,
                               x_bs, w_bs, y_bs, _p(seg_off), n_groups, w_gs, _p(gather), gather_div, mode, _p(row_scale),
                               scale_ld))
    torch.cuda.synchronize()


@pytest.mark.parametrize("T,N,K", [(1, 5, 200), (5, 17, 33), (70, 130, 88), (200, 64, 100), (3, 440, 7), (7, 65, 2048), (1, 17, 264),
                                   (3, 9, 301)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gemm_any_dense_any_shape(T, N, K, dt):
    g = torch.Generator().manual_seed(T * 1000 + N)
    x, w = _dev(torch.randn(T, K, generator=g), dt), _dev(torch.randn(N, K, generator=g), dt)
    y = torch.full((T, N), float("nan"), device="cuda")
    _gemm_any(x, w, y, T, N, K)
    ref = x.double() @ w.double().T
    assert torch.allclose(y.double(), ref, rtol=1e-5, atol=1e-4 * math.sqrt(K))


def test_gemm_any_batched_heads_with_row_scale_and_mixed_types():
    T, H, K, N = 9, 3, 20, 11
    g = torch.Generator().manual_seed(1)
    x = _dev(torch.randn(T, H * K, generator=g))                       # fp32 activations
    w = _dev(torch.randn(H, N, K, generator=g), torch.bfloat16)        # bf16 weights, one matrix per head
    scale = _dev(torch.rand(T, H, generator=g))
    y = torch.zeros(T, H * N, device="cuda", dtype=torch.bfloat16)
    _gemm_any(x, w, y, T, N, K, ldx=H * K, ldw=K, ldy=H * N, batch=H, x_bs=K, w_bs=N * K, y_bs=N, mode=2, row_scale=scale,
              scale_ld=H)
    ref = torch.einsum("thk,hnk->thn", x.view(T, H, K).double(), w.double()) * scale.double()[:, :, None]
    assert torch.allclose(y.double().view(T, H, N), ref, rtol=1e-2, atol=2e-2)


def test_gemm_any_tensor_core_variant_batched_and_long_k():
    """bf16 operands with 16-byte aligned rows take the mma.sync kernel: several k-blocks with a ragged tail, several row and
    column tiles, one problem per head, bf16 and fp32 outputs."""
    T, H, K, N = 150, 3, 104, 136
    g = torch.Generator().manual_seed(2)
    x = _dev(torch.randn(T, H * K, generator=g), torch.bfloat16)
    w = _dev(torch.randn(H, N, K, generator=g), torch.bfloat16)
    scale = _dev(torch.rand(T, H, generator=g))
    ref = torch.einsum("thk,hnk->thn", x.view(T, H, K).double(), w.double())
    y = torch.full((T, H * N), float("nan"), device="cuda")
    _gemm_any(x, w, y, T, N, K, ldx=H * K, ldw=K, ldy=H * N, batch=H, x_bs=K, w_bs=N * K, y_bs=N)
    assert torch.allclose(y.double().view(T, H, N), ref, rtol=1e-5, atol=1e-3)
    yb = torch.zeros(T, H * N, device="cuda", dtype=torch.bfloat16)
    _gemm_any(x, w, yb, T, N, K, ldx=H * K, ldw=K, ldy=H * N, batch=H, x_bs=K, w_bs=N * K, y_bs=N, mode=2, row_scale=scale,
              scale_ld=H)
    assert torch.allclose(yb.double().view(T, H, N), ref * scale.double()[:, :, None], rtol=1e-2, atol=5e-2)


@pytest.mark.parametrize("counts", [[0, 3, 0, 70, 1], [17], [1, 1, 1, 1]])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gemm_any_grouped_gather_swiglu(counts, dt):
    E, K, ff, top = len(counts), 24, 10, 2
    n = sum(counts)
    g = torch.Generator().manual_seed(n)
    tokens = (n + top - 1) // top
    x = _dev(torch.randn(tokens, K, generator=g), dt)
    gate, up = torch.randn(E, ff, K, generator=g).to(dt).float(), torch.randn(E, ff, K, generator=g).to(dt).float()
    w = torch.empty(E, 2 * ff, K)
    w[:, 0::2], w[:, 1::2] = gate, up                                  # interleaved rows: (gate_j, up_j)
    w = _dev(w, dt)
    seg = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32).cuda()
    order = torch.randperm(tokens * top, generator=g)[:n].to(torch.int32).cuda()   # position p reads token order[p] // top
    y = torch.full((n, ff), float("nan"), device="cuda")
    _gemm_any(x, w, y, n, 2 * ff, K, ldy=ff, seg_off=seg, n_groups=E, w_gs=2 * ff * K, gather=order, gather_div=top, mode=1)
    p = 0
    for e, c in enumerate(counts):
        for _ in range(c):
            h = x[int(order[p]) // top].double().cpu()
            a = gate[e].double() @ h
            ref = a * torch.sigmoid(a) * (up[e].double() @ h)
            assert torch.allclose(y[p].double().cpu(), ref, rtol=1e-4, atol=1e-4), (e, p)
            p += 1


def test_rmsnorm_f32_and_sublayer_tail():
    from oracle import ponenex_oracle as O

    T, Wd, top, eps, mult = 7, 50, 3, 1e-3, 0.6
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, Wd, generator=g) * 3
    wn = torch.randn(Wd, generator=g) * 0.2
    out = torch.zeros(T, Wd, device="cuda")
    _ok(_lib().tgis_k_rmsnorm_f32(_p(_dev(x)), Wd, _p(_dev(wn)), 1.0, _p(out), F32, Wd, T, Wd, eps))
    assert torch.allclose(out.cpu().double(), O.norm_around_zero(x.double(), wn.double(), eps), rtol=1e-5, atol=1e-5)
    # tail with a plain input
    resid = torch.randn(T, Wd, generator=g)
    y, w_post, w_pre = torch.randn(T, Wd, generator=g), torch.randn(Wd, generator=g) * 0.1, torch.randn(Wd, generator=g) * 0.1
    r_dev, o_dev = _dev(resid), torch.zeros(T, Wd, device="cuda", dtype=torch.bfloat16)
    _ok(_lib().tgis_k_resid_tail(_p(_dev(y)), None, None, None, 0, None, None, _p(_dev(w_post)), _p(_dev(w_pre)), _p(r_dev),
                                 _p(o_dev), BF16, mult, 1.0, eps, T, Wd))
    r_ref = resid.double() + mult * O.norm_around_zero(y.double(), w_post.double(), eps)
    assert torch.allclose(r_dev.cpu().double(), r_ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(o_dev.cpu().double(), O.norm_around_zero(r_ref, w_pre.double(), eps), rtol=1e-2, atol=1e-2)
    # tail over a mixture: rows picked through inv, weighted, plus a gated side term; no following norm
    rows = torch.randn(T * top, Wd, generator=g)
    inv = torch.randperm(T * top, generator=g).to(torch.int32)
    mw, side, sg = torch.rand(T, top, generator=g), torch.randn(T, Wd, generator=g), torch.rand(T, generator=g)
    r_dev = _dev(resid)
    _ok(_lib().tgis_k_resid_tail(None, _p(_dev(rows)), _p(_dev(inv, torch.int32)), _p(_dev(mw)), top, _p(_dev(side)), _p(_dev(sg)),
                                 _p(_dev(w_post)), None, _p(r_dev), None, F32, mult, 1.0, eps, T, Wd))
    mix = torch.stack([sum(mw[t, k].double() * rows[int(inv[t * top + k])].double() for k in range(top)) for t in range(T)])
    mix = mix + sg.double()[:, None] * side.double()
    assert torch.allclose(r_dev.cpu().double(), resid.double() + mult * O.norm_around_zero(mix, w_post.double(), eps),
                          rtol=1e-5, atol=1e-5)


def _geom(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, rot_dims, scale):
    from vllm_tgis_adapter_b200.engine._lib import TgisKLatentGeom

    return TgisKLatentGeom(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, rot_dims, scale)


def _cos_sin(n_pos, base, dims):
    half = dims // 2
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    return _dev(torch.cat([ang.cos(), ang.sin()], -1))


@pytest.mark.parametrize("rot_dim,rot_dims", [(8, 8), (12, 8), (6, 2)])
def test_latent_prep_norms_rotary_cache_and_gates(rot_dim, rot_dims):
    from oracle import ponenex_oracle as O

    heads, dim, vdim, kv_rank, q_rank, eps, base = 3, 5, 7, 20, 9, 1e-4, 50.0
    T, n_pos = 6, 300
    geom = _geom(heads, dim, rot_dim, vdim, kv_rank, q_rank, 0, rot_dims, 1.0)
    g = torch.Generator().manual_seed(rot_dim)
    ld = q_rank + kv_rank + rot_dim + heads
    y = torch.randn(T, ld, generator=g) * 2
    wq, wkv = torch.randn(q_rank, generator=g), torch.randn(kv_rank, generator=g)
    pos = torch.tensor([0, 1, 33, 255, 64, 299], dtype=torch.int32)
    slots = torch.tensor([5, 0, 70, -1, 31, 32], dtype=torch.int32)       # -1: not cached
    row = kv_rank + rot_dim
    cache = torch.full((3 * KV_BLOCK, row), 7.0, device="cuda")
    cq, gate = torch.zeros(T, q_rank, device="cuda"), torch.zeros(T, heads, device="cuda")
    _ok(_lib().tgis_k_latent_prep(_p(_dev(y)), ld, C.byref(geom), _p(_dev(wq)), _p(_dev(wkv)), eps, _p(_dev(pos, torch.int32)),
                                  _p(_dev(slots, torch.int32)), _p(_cos_sin(n_pos, base, rot_dims)), _p(cq), _p(cache), F32, _p(gate), T))
    yd = y.double()
    assert torch.allclose(cq.cpu().double(), O.norm_plain(yd[:, :q_rank], wq.double(), eps), rtol=1e-5, atol=1e-5)
    assert torch.allclose(gate.cpu().double(), torch.sigmoid(yd[:, -heads:]), rtol=1e-5, atol=1e-6)
    c_ref = O.norm_plain(yd[:, q_rank:q_rank + kv_rank], wkv.double(), eps)
    k_ref = O.rotate(yd[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim], pos, base, rot_dims)
    cache = cache.cpu().double()
    touched = set()
    for t in range(T):
        if slots[t] < 0:
            continue
        touched.add(int(slots[t]))
        assert torch.allclose(cache[slots[t], :kv_rank], c_ref[t], rtol=1e-5, atol=1e-5)
        assert torch.allclose(cache[slots[t], kv_rank:], k_ref[t], rtol=1e-5, atol=1e-5), t
    untouched = [s for s in range(cache.shape[0]) if s not in touched]
    assert bool((cache[untouched] == 7.0).all())
    # the query's rotated part lands behind the kv_rank absorbed entries of every head
    q = torch.randn(T, heads * (dim + rot_dim), generator=g)
    q_abs = torch.zeros(T, heads, row, device="cuda")
    _ok(_lib().tgis_k_latent_q_rope(_p(_dev(q)), F32, C.byref(geom), _p(_dev(pos, torch.int32)), _p(_cos_sin(n_pos, base, rot_dims)), _p(q_abs), T))
    q_ref = O.rotate(q.double().view(T, heads, dim + rot_dim)[..., dim:], pos, base, rot_dims)
    assert torch.allclose(q_abs.cpu().double()[..., kv_rank:], q_ref, rtol=1e-5, atol=1e-5)
    assert bool((q_abs[..., :kv_rank] == 0).all())


def _attn_ref(q_abs, rows, positions_q, window, scale, kv_rank):
    """q_abs [Tq, H, D], rows [n_keys, D] (key j at position j) -> [Tq, H, kv_rank] in float64."""
    out = torch.zeros(q_abs.shape[0], q_abs.shape[1], kv_rank, dtype=torch.float64)
    for t, pq in enumerate(positions_q):
        lo = max(0, pq - window + 1) if window > 0 else 0
        keys = rows[lo:pq + 1].double()
        for h in range(q_abs.shape[1]):
            p = torch.softmax(keys @ q_abs[t, h].double() * scale, 0)
            out[t, h] = p @ keys[:, :kv_rank]
    return out


def _paged(rows, n_blocks_pool, seed, dt):
    """Scatter `rows` (one sequence) over shuffled blocks of a larger pool; returns (cache, block table row)."""
    n_blk = (rows.shape[0] + KV_BLOCK - 1) // KV_BLOCK
    g = torch.Generator().manual_seed(seed)
    blocks = torch.randperm(n_blocks_pool, generator=g)[:n_blk]
    cache = torch.randn(n_blocks_pool * KV_BLOCK, rows.shape[1], generator=g) * 5   # other sequences' rows: finite garbage
    for j in range(rows.shape[0]):
        cache[int(blocks[j // KV_BLOCK]) * KV_BLOCK + j % KV_BLOCK] = rows[j]
    return cache.to(dt).cuda().contiguous(), blocks.to(torch.int32)


@pytest.mark.parametrize("heads,kv_rank,rot_dim", [(6, 24, 8), (1, 130, 2), (20, 40, 6), (3, 300, 4), (16, 512, 64), (5, 72, 8),
                                                   (2, 128, 32)])
@pytest.mark.parametrize("dt", [F32, BF16])
def test_latent_attention_prompt_portion_and_decode_match_dense_softmax(heads, kv_rank, rot_dim, dt):
    window, kv_len = 45, 150
    D = kv_rank + rot_dim
    scale = 2.0 / math.sqrt(D)                 # scores of spread 2 whatever the row length
    g = torch.Generator().manual_seed(heads)
    rows = torch.randn(kv_len, D, generator=g)
    cache, blocks = _paged(rows, 9, heads, _tdt(dt))
    rows_seen = cache.view(-1, D)[[int(blocks[j // KV_BLOCK]) * KV_BLOCK + j % KV_BLOCK for j in range(kv_len)]].float().cpu()
    geom = _geom(heads, 4, rot_dim, 4, kv_rank, 4, window, rot_dim, scale)
    # a portion of 37 queries ending at the last position, and a single decoded token, as two "sequences" over the same rows
    for q_len in (37, 1, kv_len):
        q_abs = torch.randn(q_len, heads, D, generator=g)
        o = torch.full((q_len, heads, kv_rank), float("nan"), device="cuda")
        seqs = (C.c_int32 * 4)(0, q_len, kv_len, 0)
        bt = (C.c_int32 * len(blocks))(*blocks.tolist())
        _ok(_lib().tgis_k_latent_attn(_p(_dev(q_abs)), _p(cache), dt, seqs, 1, bt, 1, len(blocks), _p(o), F32, C.byref(geom)))
        ref = _attn_ref(q_abs, rows_seen, list(range(kv_len - q_len, kv_len)), window, scale, kv_rank)
        tol = 2e-4 if dt == F32 else 3e-2    # bf16 rows with aligned sizes run on the tensor cores: Q and P rounded to bf16
        assert torch.allclose(o.cpu().double(), ref, rtol=tol, atol=tol), q_len


@pytest.mark.parametrize("q_len", [1, 5, 64])
@pytest.mark.parametrize("dt,window,kv_len", [(F32, 70, 200), (BF16, 70, 200), (BF16, 300, 500), (BF16, 0, 500)])
def test_latent_attention_one_key_decides_at_window_and_block_edges(q_len, dt, window, kv_len):
    """Every key row carries its own position as a one-hot code in c; the query is built so that ONE chosen key outweighs
    all others by e^40.  If that key is visible the output is its code, otherwise the weight spreads evenly over what is
    visible: a window that is one token off, or a block (or a split of blocks) that is skipped or read twice, flips the
    answer.  bf16 rows run on the tensor cores; long key ranges of few queries are cut into splits and merged."""
    heads, rot_dim = 2, 8
    kv_rank = (kv_len + 7) // 8 * 8
    D = kv_rank + rot_dim
    rows = torch.zeros(kv_len, D)
    for j in range(kv_len):
        rows[j, j] = 1.0                                   # code of position j (kv_rank >= kv_len)
    cache, blocks = _paged(rows, (kv_len + KV_BLOCK - 1) // KV_BLOCK + 3, q_len, _tdt(dt))
    geom = _geom(heads, 4, rot_dim, 4, kv_rank, 4, window, rot_dim, 1.0)
    bt = (C.c_int32 * len(blocks))(*blocks.tolist())
    last = kv_len - 1
    first_q = kv_len - q_len
    w_eff = window if window > 0 else 10 ** 9
    # distances from the LAST query: itself, neighbours, block borders, split borders, the window's two sides, far away
    dists = {0, 1, last % KV_BLOCK, last % KV_BLOCK + 1, last % 128, last % 128 + 1, 150, last}
    if window > 0:
        dists |= {window - 2, window - 1, window, window + 1}
    for dist in sorted(d for d in dists if 0 <= d <= last):
        target = last - dist
        q_abs = torch.zeros(q_len, heads, D)
        q_abs[:, :, target] = 40.0
        o = torch.zeros(q_len, heads, kv_rank, device="cuda")
        seqs = (C.c_int32 * 4)(0, q_len, kv_len, 0)
        _ok(_lib().tgis_k_latent_attn(_p(_dev(q_abs)), _p(cache), dt, seqs, 1, bt, 1, len(blocks), _p(o), F32, C.byref(geom)))
        o = o.cpu()
        for t in range(q_len):
            pq = first_q + t
            sees = 0 <= pq - target < w_eff
            got = float(o[t, 1, target])
            assert (got > 0.99) == sees, (dist, t, got)
            if not sees:   # then the weight is spread evenly over what IS visible
                n_vis = min(w_eff, pq + 1)
                assert abs(float(o[t, 0, pq]) - 1.0 / n_vis) < 1e-5, (dist, t)


def test_router_picks_top_and_normalises_over_chosen_only():
    from oracle import ponenex_oracle as O

    T, E, top = 37, 19, 3
    g = torch.Generator().manual_seed(3)
    logits, bias = torch.randn(T, E + 1, generator=g) * 2, torch.randn(E, generator=g)
    ids, w = torch.zeros(T, top, dtype=torch.int32, device="cuda"), torch.zeros(T, top, device="cuda")
    sg = torch.zeros(T, device="cuda")
    _ok(_lib().tgis_k_moe_route(_p(_dev(logits)), E + 1, _p(_dev(bias)), E, top, _p(ids), _p(w), _p(sg), T))
    z = logits[:, :E].double() + bias.double()
    val, idx = torch.sort(z, -1, descending=True)
    assert torch.equal(ids.cpu().long(), idx[:, :top])
    assert torch.allclose(w.cpu().double(), torch.softmax(val[:, :top], -1), rtol=1e-5, atol=1e-6)
    assert torch.allclose(sg.cpu().double(), torch.sigmoid(logits[:, E].double()), rtol=1e-5, atol=1e-6)
    # bias alone can decide: expert 4 wins everywhere once its bias is large; top = 1 gives weight exactly 1
    bias2 = bias.clone()
    bias2[4] = 100.0
    ids1, w1 = torch.zeros(T, 1, dtype=torch.int32, device="cuda"), torch.zeros(T, 1, device="cuda")
    _ok(_lib().tgis_k_moe_route(_p(_dev(logits)), E + 1, _p(_dev(bias2)), E, 1, _p(ids1), _p(w1), None, T))
    assert bool((ids1 == 4).all()) and bool((w1 == 1.0).all())
    # row lists: every (token, k) lands exactly once in its expert's segment
    seg = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    order, inv = torch.zeros(T * top, dtype=torch.int32, device="cuda"), torch.zeros(T * top, dtype=torch.int32, device="cuda")
    _ok(_lib().tgis_k_moe_align(_p(ids), T, top, E, _p(seg), _p(order), _p(inv)))
    seg, order, inv, flat = seg.cpu(), order.cpu().long(), inv.cpu().long(), ids.cpu().view(-1).long()
    assert int(seg[E]) == T * top and sorted(order.tolist()) == list(range(T * top))
    for e in range(E):
        assert bool((flat[order[int(seg[e]):int(seg[e + 1])]] == e).all())
    assert torch.equal(order[inv], torch.arange(T * top))


# ====================================================================================================== engine
def _config(**kw):
    from vllm_tgis_adapter_b200.engine.core import ModelConfig
    from vllm_tgis_adapter_b200.engine.ponenex import LayerSpec

    base = dict(heads=3, dim=10, rot_dim=6, vdim=9, kv_rank=20, q_rank=14, window=11, rot_dims=6, rot_base=300.0, scale=0.22,
                experts=5, top=2, expert_ff=18, shared_ff=12)
    layers = kw.pop("layers", None) or [LayerSpec(**base), LayerSpec(**{**base, "window": 40, "heads": 2, "top": 1})]
    return ModelConfig(n_layers=len(layers), hidden=kw.pop("hidden", 44), n_q_heads=1, n_kv_heads=1, ffn=64,
                       vocab=kw.pop("vocab", 101), rms_eps=1e-4, max_model_len=kw.pop("max_model_len", 512), arch="ponenex",
                       layers=layers, embed_scale=2.5, residual_mult=0.8, dtype=kw.pop("dtype", "float32"))


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


def _whole(eng, toks, rid="w"):
    return eng.trace_step([(rid, toks, list(range(len(toks))))], [rid])


def test_whole_prompt_matches_oracle_fp32_and_bf16():
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    toks = _tokens(150, 101, 1)
    for dtype in ("float32", "bfloat16"):
        mc = _config(dtype=dtype)
        weights = synthetic_weights(mc, 11)
        ref = O.forward(mc, weights, toks)
        eng = _engine(mc, weights)
        got = _whole(eng, toks)
        eng.close()
        if dtype == "float32":
            assert _rel(got, ref) < 2e-5
        else:
            # bf16 operands: rounding can flip a close router call of these random weights, which moves that row by far
            # more than rounding does -- so the bound is on the typical row, with few rows allowed to stray
            rows = sorted(_rel(got[t:t + 1], ref[t:t + 1]) for t in range(len(toks)))
            assert rows[len(rows) // 2] < 2e-2 and rows[int(0.8 * len(rows))] < 5e-2, (rows[len(rows) // 2], rows[-1])
    # the first tokens of a sequence on their own: lengths 1 and 2
    mc = _config()
    weights = synthetic_weights(mc, 11)
    eng = _engine(mc, weights)
    for n in (1, 2):
        assert _rel(_whole(eng, toks[:n]), O.forward(mc, weights, toks[:n])) < 2e-5
    eng.close()


def _variants():
    from vllm_tgis_adapter_b200.engine.ponenex import LayerSpec

    b = dict(heads=3, dim=10, rot_dim=6, vdim=9, kv_rank=20, q_rank=14, window=11, rot_dims=6, rot_base=300.0, scale=0.22,
             experts=5, top=2, expert_ff=18, shared_ff=12)
    return {
        "one head, one expert, top 1": [LayerSpec(**{**b, "heads": 1, "experts": 1, "top": 1})],
        "no shared expert, then no feed-forward at all": [LayerSpec(**{**b, "shared_ff": 0}),
                                                          LayerSpec(**{**b, "experts": 0, "top": 0, "expert_ff": 0, "shared_ff": 0}),
                                                          LayerSpec(**b)],
        "rot.dims smaller than rot_dim, window 1, window wider than the prompt": [
            LayerSpec(**{**b, "rot_dim": 8, "rot_dims": 4}), LayerSpec(**{**b, "window": 1}), LayerSpec(**{**b, "window": 4000})],
        "many heads (more pairs than a tile), odd sizes, top = experts": [
            LayerSpec(**{**b, "heads": 19, "dim": 3, "vdim": 5, "kv_rank": 33, "q_rank": 7, "experts": 3, "top": 3, "expert_ff": 7,
                         "shared_ff": 5, "rot_dim": 2, "rot_dims": 2})],
        "equal dims everywhere": [LayerSpec(**{**b, "dim": 8, "rot_dim": 8, "rot_dims": 8, "vdim": 8, "kv_rank": 8, "q_rank": 8,
                                               "expert_ff": 8, "shared_ff": 8})],
    }


@pytest.mark.parametrize("name", list(_variants()))
def test_other_sizes_and_absent_parts(name):
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    mc = _config(layers=_variants()[name], hidden=40 if "equal" not in name else 8, vocab=77)
    weights = synthetic_weights(mc, 5)
    toks = _tokens(70, 77, 2)
    ref = O.forward(mc, weights, toks)
    eng = _engine(mc, weights)
    got_whole = _whole(eng, toks)
    # and again in portions of 33, 2, 1, 1, 30, 3 tokens through the cache
    got, at = [], 0
    for n in (33, 2, 1, 1, 30, 3):
        got.append(eng.trace_step([("p", toks[at:at + n], list(range(n)))], ["p"] if at + n == len(toks) else []))
        at += n
    eng.close()
    assert _rel(got_whole, ref) < 3e-5
    assert _rel(np.concatenate(got), ref) < 3e-5


def test_tensor_core_paths_agree_with_the_general_kernels(monkeypatch):
    """Sizes that fit the tcgen05 kernel's operand layout (dense projections, shared expert, lm_head) and the mma.sync kernel
    (per-head and per-expert products): the bf16 engine with and without the tcgen05 route, against the oracle."""
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import LayerSpec, synthetic_weights

    b = dict(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=128, window=50, rot_dims=16, rot_base=1000.0, scale=0.15,
             experts=4, top=2, expert_ff=64, shared_ff=128)
    mc = _config(layers=[LayerSpec(**b), LayerSpec(**{**b, "window": 200})], hidden=256, vocab=384, dtype="bfloat16")
    weights = synthetic_weights(mc, 7)
    toks = _tokens(300, 384, 8)
    ref = O.forward(mc, weights, toks)
    got = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("TGIS_PNX_TC", tc)
        eng = _engine(mc, weights, blocks=12)
        whole = _whole(eng, toks)
        parts, at = [], 0
        for n in (257, 1, 1, 30, 2, 9):                       # a 257-token portion (two token tiles), then small steps
            parts.append(eng.trace_step([("p", toks[at:at + n], list(range(n)))], ["p"] if at + n == len(toks) else []))
            at += n
        launches = eng.status().kernel_launches
        eng.close()
        got[tc] = (whole, np.concatenate(parts), launches)
    for tc, (whole, parts, _) in got.items():
        for out in (whole, parts):
            rows = sorted(_rel(out[t:t + 1], ref[t:t + 1]) for t in range(len(toks)))
            assert rows[len(rows) // 2] < 2e-2 and rows[int(0.8 * len(rows))] < 6e-2, (tc, rows[len(rows) // 2], rows[-1])
    rows = sorted(_rel(got["1"][0][t:t + 1], torch.as_tensor(got["0"][0][t:t + 1]).double()) for t in range(len(toks)))
    assert rows[len(rows) // 2] < 2e-2


def test_prefill_portions_and_token_by_token_agree_with_whole_prompt():
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    mc = _config()
    weights = synthetic_weights(mc, 21)
    toks = _tokens(131, 101, 3)
    ref = O.forward(mc, weights, toks)
    eng = _engine(mc, weights)
    for sizes in ([131], [1] * 131, [2] * 65 + [1], [31, 1, 33, 2, 64], [64, 67], [5, 7, 11, 13, 17, 19, 23, 29, 7]):
        assert sum(sizes) == len(toks)
        got, at = [], 0
        for n in sizes:
            got.append(eng.trace_step([("r", toks[at:at + n], list(range(n)))], ["r"] if at + n == len(toks) else []))
            at += n
        assert _rel(np.concatenate(got), ref) < 3e-5, sizes[:4]
    eng.close()


def test_long_decoding_crosses_windows_and_block_borders():
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    mc = _config()                               # windows 11 and 40, blocks of 32 tokens
    weights = synthetic_weights(mc, 31)
    toks = _tokens(9 + 200, 101, 4)
    ref = O.forward(mc, weights, toks)
    eng = _engine(mc, weights)
    got = [eng.trace_step([("d", toks[:9], list(range(9)))])]
    for t in range(9, len(toks)):
        got.append(eng.trace_step([("d", [toks[t]], [0])]))
    eng.close()
    assert _rel(np.concatenate(got), ref) < 3e-5


def test_mixed_batches_of_unequal_requests_match_each_alone_and_reuse_blocks_and_slots():
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    mc = _config()
    weights = synthetic_weights(mc, 41)
    reqs = {f"q{i}": _tokens(n, 101, 50 + i) for i, n in enumerate([97, 40, 3, 130, 64, 33, 71])}
    ref = {k: O.forward(mc, weights, v) for k, v in reqs.items()}
    # 4 slots and a pool of 10 blocks (320 tokens): the seven requests (438 tokens, 17 blocks) only fit because finished
    # ones give their slot and blocks back
    eng = _engine(mc, weights, blocks=10, seqs=4)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live, step = list(reqs), [], 0
    while waiting or live:
        blocks_live = sum((len(reqs[k]) + KV_BLOCK - 1) // KV_BLOCK for k in live)
        while waiting and len(live) < 4 and blocks_live + (len(reqs[waiting[0]]) + KV_BLOCK - 1) // KV_BLOCK <= 10:
            blocks_live += (len(reqs[waiting[0]]) + KV_BLOCK - 1) // KV_BLOCK
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            if (step + j) % 5 == 4:
                continue                                        # a request may sit a step out
            left = len(reqs[k]) - at[k]
            n = min(left, [1, 7, 2, 29, 1, 33][(step + 2 * j) % 6])   # single tokens beside portions of changing size
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
    from oracle import ponenex_oracle as O
    from vllm_tgis_adapter_b200.engine.core import make_sampling_params
    from vllm_tgis_adapter_b200.engine.ponenex import synthetic_weights

    mc = _config()
    weights = synthetic_weights(mc, 61)
    prompts = [_tokens(45, 101, 70), _tokens(3, 101, 71), _tokens(80, 101, 72)]
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
            assert toks == O.greedy(mc, weights, p, n_new), graphs
            # the reported logprob is the oracle's log-softmax of the chosen token
            lp = torch.log_softmax(O.forward(mc, weights, p + toks[:-1])[len(p) - 1:], -1)
            for i, r in enumerate([r for r in recs if r.new_token is not None]):
                assert abs(r.logprob - float(lp[i, r.new_token])) < 1e-3
