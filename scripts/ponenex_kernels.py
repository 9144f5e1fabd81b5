"""Stand-alone timing of the two heaviest Ponenex kernels at the `ponenex-2k` layer sizes, through the C test hooks:
the grouped expert product (gate/up with the SwiGLU epilogue; 2048 tokens x top 6 over 64 experts) and the latent attention
(a 2048-token prefill step of four 512-token prompts; a decode step of 32 sequences).  CUDA events around each launch,
inputs larger than L2.  `--once`: one launch of each and no timing loop (the small case for an ncu capture)."""
import ctypes as C
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from vllm_tgis_adapter_b200.engine import _lib  # noqa: E402

lib = _lib.load_library()
ONCE = "--once" in sys.argv
KEEP = []


def p(t):
    KEEP.append(t)
    return C.c_void_p(t.data_ptr())


def timed(fn, n=5):
    fn()
    if ONCE:
        return 0.0
    best = 1e9
    for _ in range(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def ok(rc):
    assert rc == 0, (lib.tgis_k_last_error() or b"").decode()


def grouped():
    T, top, E, K, ff = 2048, 6, 64, 2048, 1408
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.stack([torch.randperm(E, generator=g, device="cuda")[:top] for _ in range(T)]).to(torch.int32).contiguous()
    seg = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    order, inv = torch.zeros(T * top, dtype=torch.int32, device="cuda"), torch.zeros(T * top, dtype=torch.int32, device="cuda")
    ok(lib.tgis_k_moe_align(p(ids), T, top, E, p(seg), p(order), p(inv)))
    x = (torch.randn(T, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(E, 2 * ff, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    y = torch.zeros(T * top, ff, dtype=torch.bfloat16, device="cuda")
    ms = timed(lambda: ok(lib.tgis_k_gemm_any(p(x), p(w), p(y), 1, 1, 1, T * top, 2 * ff, K, K, K, ff, 1, 0, 0, 0, p(seg), E,
                                              2 * ff * K, p(order), top, 1, None, 0)))
    flops = 2.0 * T * top * 2 * ff * K
    print(f"grouped gate/up product: {ms * 1e3:.0f} us, {flops / (ms * 1e-3) / 1e12 if ms else 0:.0f} TFLOP/s")


def attention(name, n_seqs, q_len, kv_len):
    heads, kv_rank, rot = 16, 512, 64
    D = kv_rank + rot
    geom = _lib.TgisKLatentGeom(heads, 128, rot, 128, kv_rank, 1536, 4096, rot, D ** -0.5)
    nb = (kv_len + 31) // 32
    g = torch.Generator(device="cuda").manual_seed(1)
    cache = (torch.randn(n_seqs * nb * 32, D, generator=g, device="cuda")).to(torch.bfloat16)
    q = torch.randn(n_seqs * q_len, heads, D, generator=g, device="cuda")
    o = torch.zeros(n_seqs * q_len, heads, kv_rank, dtype=torch.bfloat16, device="cuda")
    seqs = (C.c_int32 * (4 * n_seqs))(*[v for i in range(n_seqs) for v in (i * q_len, q_len, kv_len, i)])
    bt = (C.c_int32 * (n_seqs * nb))(*range(n_seqs * nb))
    ms = timed(lambda: ok(lib.tgis_k_latent_attn(p(q), p(cache), 1, seqs, n_seqs, bt, n_seqs, nb, p(o), 1, C.byref(geom))))
    print(f"latent attention, {name}: {ms * 1e3:.0f} us (includes the hook's staging copies)")


if __name__ == "__main__":
    grouped()
    attention("prefill 4 x 512", 4, 512, 512)
    attention("decode 32 x 544", 32, 1, 544)
