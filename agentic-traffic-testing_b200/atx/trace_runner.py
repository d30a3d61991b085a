"""Step-by-step replay of a recorded schedule through the engine (`bin/trace_run`).

The runner reads steps from standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry brings the next tokens of a request (admitted at its first entry; it may skip steps) and the offsets among
them whose logits are wanted; all entries of a line run as ONE engine step (prompt portions beside single tokens), from
the pages and states earlier steps left. Requests named in `end` give their pages and state slot back after the step.
For a step that wants something, `<out>/<step>.f32` receives the logits [wanted, vocab] as little-endian fp32 in the
order of the entries; after every step the line `done <step>` is printed.

It builds an ordinary LLMEngine (model class chosen from config.json by the registry) and calls LLMEngine.feed(): the
scheduler's structures, the block allocator, the state-slot pool, ModelRunner.launch and the kernels are the ones
generation uses. The page pool holds `--max-tokens` tokens (in 16-token pages) and there are four sequence slots, so
pages and slots are reused as requests end. Nothing is sampled."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="tokens the live requests hold at most (each rounded up to the page size)")
    ap.add_argument("--max-seqs", type=int, default=4, help="sequence (state) slots")
    a = ap.parse_args(argv)

    import numpy as np

    from .config import EngineConfig, resolve_model
    from .engine import LLMEngine

    source = resolve_model(a.model)
    if a.dtype == "float32" and getattr(source.config, "architecture", "llama") == "llama":
        print("float32 is not available for this model family", file=sys.stderr)
        return 3
    bs = 16
    tokens = max(bs, (a.max_tokens + bs - 1) // bs * bs)
    ecfg = EngineConfig(max_model_len=tokens, max_num_seqs=a.max_seqs, max_num_batched_tokens=tokens,
                        block_size=bs, num_gpu_blocks=tokens // bs, enable_prefix_caching=False,
                        enable_cuda_graphs=False, async_scheduling=False, dtype=a.dtype,
                        max_logit_rows=min(tokens, 8192))
    eng = LLMEngine(source, ecfg)
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want") or []) for e in step.get("entries", [])]
        if entries:
            logits = eng.feed(entries, step.get("end") or ())
        else:
            logits = eng.feed([], step.get("end") or ()) if step.get("end") else np.zeros((0, 0), np.float32)
        if any(w for _, _, w in entries):
            np.ascontiguousarray(logits, dtype="<f4").tofile(out / f"{step['step']}.f32")
        print(f"done {step['step']}", flush=True)
    eng.runner.close()
    return 0
