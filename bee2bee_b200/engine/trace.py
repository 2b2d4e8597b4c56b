"""Trace replay: given token ids go through the serving engine step by step and the logits of chosen positions are
written to files.  Nothing is sampled.  Command line: ``bin/trace_run`` or ``python -m bee2bee_b200 trace-run``.

    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

One JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

Every step is ONE batch of the engine (``Engine.replay_step``: prompt portions of some sequences beside single tokens of
others, on the scheduler's batch slots, the page allocator's KV pages and the chunk path of the GPU runner).  For a step
that wants logits, ``<out>/<step>.f32`` holds them as little-endian float32 ``[wanted, vocab]`` in entry order; after
every step a line ``done <step>`` is printed.  ``--max-tokens``: tokens that live sequences hold at most (each rounded up
to the 64-token KV page); the page pool is sized for exactly that, with ``--slots`` batch slots, so pages and slots are
used again as sequences end.  Exit code 3: ``--dtype float32`` for a model family whose kernels are bf16 only.
The native extension is built in-tree at the first call if it is missing.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="preset name or a directory with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, default=4096)
    ap.add_argument("--slots", type=int, default=4, help="batch slots = sequences that can be live at once")
    a = ap.parse_args(argv)

    from ..models.config import resolve_config

    cfg = resolve_config(a.model)
    if a.dtype == "float32" and not cfg.hybrid:
        sys.stderr.write(f"{cfg.family}: this family is served in bf16 only\n")
        return 3

    from .._build import build, ext_path

    if not ext_path().exists() or os.environ.get("B2B_REBUILD") == "1":
        build(verbose=False)
    import numpy as np
    import torch

    from .core import Engine
    from .kv import PAGE

    torch.backends.cuda.matmul.allow_tf32 = False          # float32 means float32
    torch.backends.cudnn.allow_tf32 = False
    pages = (max(a.max_tokens, PAGE) + PAGE - 1) // PAGE
    chunk = 64
    while chunk < min(pages * PAGE, 8192):
        chunk *= 2
    eng = Engine(a.model, cfg=cfg, device="cuda:0", max_batch=a.slots, max_seq_len=pages * PAGE, max_prefill_tokens=chunk,
                 num_pages=pages + 1, dtype=torch.float32 if a.dtype == "float32" else torch.bfloat16,
                 max_logit_rows=chunk, prefix_cache=False)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want") or []) for e in step.get("entries", [])]
        logits = eng.replay_step(entries, step.get("end") or [])
        if logits is not None:
            tmp = os.path.join(a.out, f".{step['step']}.part")
            np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
