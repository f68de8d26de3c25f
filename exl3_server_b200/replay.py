"""Trace replay: feeds given token ids through the model step by step and
writes logits.  It samples nothing and has no forward pass, cache or loader of
its own: it opens slots, calls ``Engine.step`` and closes slots.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request id seen for the first time gets a fresh slot; ``end`` lists the
requests that are finished after the step.  For a step that wants logits,
``<out>/<step>.f32`` holds them as little-endian float32 ``[wanted, vocab]``,
in the order of the entries and of their ``want`` lists.  After every step a
line ``done <step>`` is printed and flushed.

The reference has no such tool; the nearest are the hand-driven loops of
tests/glm5_forward_test.cpp:103-131 and tests/glm5_batch_test.cpp:172-293.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


class TraceRunner:
    """Applies trace steps to an engine: the request-id -> slot table and
    nothing else."""

    def __init__(self, engine):
        self.engine = engine
        self.slots: Dict[str, int] = {}

    def run_step(self, msg: dict):
        """Runs one step object; returns the float32 logits ``[wanted, vocab]``
        as a device tensor, or None when nothing was wanted."""
        from .engine import StepEntry
        entries = []
        for e in msg["entries"]:
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = self.engine.open()
            entries.append(StepEntry(self.slots[rid], e["tokens"], list(e.get("want", []))))
        logits = self.engine.step(entries) if entries else None
        for rid in msg.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.engine.close(self.slots.pop(rid))
        return logits


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    os.makedirs(args.out, exist_ok=True)
    print("trace_run: loading the model and the kernels ...", file=sys.stderr, flush=True)
    import torch

    from .engine import Engine

    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens, device=args.device)
    print("trace_run: ready", file=sys.stderr, flush=True)
    runner = TraceRunner(engine)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        logits = runner.run_step(msg)
        if logits is not None:
            arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            with open(tmp, "wb") as f:
                f.write(np.ascontiguousarray(arr).tobytes())
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        engine.check_kernels()
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
