"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it opens
requests in the engine's cache, calls the engine's step function and closes them.

Input (standard input, one JSON object a line)::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step with wanted places, ``<out>/<step>.f32`` holds the logits at those
places in the order of the entries and of ``want``, little-endian 32-bit floats,
``[wanted, vocab]``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a page); sizes the pool")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import numpy as np
    import torch  # noqa: F401

    from .engine import Engine

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    num_pages = max(1, -(-args.max_tokens // page))
    eng = Engine.from_pretrained(args.model, dtype=args.dtype, device=args.device, page_size=page,
                                 num_pages=num_pages, max_requests=16, max_context=max(args.max_tokens, page))
    slots: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        items = []
        for ent in rec.get("entries", []):
            rid = str(ent["id"])
            if rid not in slots:
                s = eng.cache.open()
                if s < 0:
                    raise RuntimeError("more live requests than state slots")
                slots[rid] = s
            items.append((slots[rid], [int(t) for t in ent["tokens"]], [int(w) for w in ent.get("want", [])]))
        if items:
            logits = eng.step(items)
            if logits.shape[0] > 0:
                arr = logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
            elif eng.rt.device.type == "cuda":
                torch.cuda.synchronize()
            eng.rt.ops.check_errors()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                eng.cache.close(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
