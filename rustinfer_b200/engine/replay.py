"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
same `ModelRunner.step` that generation uses.  Steps come on standard input, one JSON
object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, `<out>/<step>.f32` holds them as little-endian fp32
[wanted, vocab] in the order of the entries and of `want`.  After every step a line
`done <step>` is printed and flushed.  RustInfer has nothing of the kind; the nearest is a
hidden-state tap (crates/infer-worker/src/application/runtime/mod.rs:1310-1348).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

PAGE_SIZE = 16                      # divides 64, the unit --max-tokens is counted in
MAX_LIVE = 8


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if 64 % args.page_size:
        ap.error("--page-size must divide 64")

    print(f"[trace_run] loading {args.model} ({args.dtype}); kernels are compiled at first use",
          file=sys.stderr, flush=True)
    from .runner import ModelRunner, StepEntry

    capacity = (args.max_tokens + 63) // 64 * 64
    os.makedirs(args.out, exist_ok=True)
    runner = ModelRunner(args.model, dtype=args.dtype, max_model_len=capacity, page_size=args.page_size,
                         num_pages=capacity // args.page_size, max_batch_seqs=MAX_LIVE,
                         max_batch_tokens=capacity)
    import torch

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if not runner.cache.is_open(e["id"]):
                runner.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step_no}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step_no}.f32"))
            else:
                torch.cuda.synchronize()
            runner.check_kernel_errors()
        for rid in rec.get("end", []):
            if runner.cache.is_open(rid):
                runner.close(rid)
        print(f"done {step_no}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
