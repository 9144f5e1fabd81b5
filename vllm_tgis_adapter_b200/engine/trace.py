"""Trace replay: given token ids go through the engine's own step function, one step per input line, and the logits at
the asked positions are written out.  Nothing is sampled.

    python -m vllm_tgis_adapter_b200.engine.trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: for each request its next tokens and the places among them whose logits are wanted; all entries of a step run
as ONE batch (portions of prompts beside single tokens).  A request is admitted at its first entry, may pause, and gives
its sequence slot and cache blocks back when it is listed under `end`.  A step with wanted places writes OUT/<step>.f32
(little-endian fp32 [wanted, vocab], entry order then `want` order); every step prints `done <step>`.

The model class comes from config.json (engine/loader.py `model_config_from_hf`), the weights through the engine's loader,
the cache pool is sized for --max-tokens tokens (each request rounded up to whole cache blocks) and four sequence slots.
--dtype float32 exits with code 3 for architectures that only run in bfloat16."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

SEQ_SLOTS = 4
ROUND_TO = 64   # requests are accounted in multiples of this many tokens (a multiple of the engine's 32-token blocks)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)

    from .core import KV_BLOCK_TOKENS, LAYER_LIST_ARCHS, NativeEngine, cache_block_bytes
    from .loader import load_safetensors_dir, model_config_from_hf

    path = Path(args.model)
    pool_tokens = (args.max_tokens + ROUND_TO - 1) // ROUND_TO * ROUND_TO
    mc = model_config_from_hf(path, pool_tokens, args.dtype)
    if args.dtype == "float32" and mc.arch not in LAYER_LIST_ARCHS:
        print(f"the {mc.arch} architecture runs in bfloat16 only", file=sys.stderr)
        return 3
    eng = NativeEngine(mc, max_num_seqs=SEQ_SLOTS, max_batched_tokens=max(pool_tokens, 16),
                       kv_cache_bytes=cache_block_bytes(mc) * (pool_tokens // KV_BLOCK_TOKENS), use_cuda_graphs=False)
    load_safetensors_dir(eng, path)
    if mc.arch == "llama":
        from .loader import rope_cos_sin

        eng.load_weight("tgis.rope_cos_sin", rope_cos_sin(mc))
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in step.get("entries", [])]
        logits = eng.trace_step(entries, [str(x) for x in step.get("end", [])])
        if logits.shape[0]:
            tmp = out_dir / f".{step['step']}.f32.part"
            logits.astype("<f4").tofile(tmp)
            tmp.replace(out_dir / f"{step['step']}.f32")
        print(f"done {step['step']}", flush=True)
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
