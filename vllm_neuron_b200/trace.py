"""Trace replay: teacher-forced stepping of the stand-alone engine, logits to files.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl

Standard input carries one engine step per line, as a JSON object such as
    {"step": 7, "entries": [{"id": "r1", "tokens": [40, 2], "want": [1]}, {"id": "r2", "tokens": [9], "want": []}], "end": ["r2"]}
`entries` names the requests that take part in the step, each with the tokens it continues with and the offsets (into
that list) of the positions to report; an id not seen before starts a new request, and a live request may be absent from a
step.  `end` lists ids to retire when the step is over.  The line's entries form ONE ragged engine batch, prompt portions
next to single tokens; the engine appends exactly the listed tokens and samples nothing.  When a step reports anything,
OUT/<step>.f32 receives those logit rows (entry order, then offset order) as little-endian fp32 [rows, vocab]; every step,
reporting or not, is acknowledged with `done <step>` on standard output.  --max-tokens sizes the KV pool (tokens of live
requests, each request rounded up to whole pages) and --max-seqs the rows / state slots, so both are recycled as requests
come and go.  --dtype float32 serves the model in true 32-bit arithmetic; a family without such a mode exits with code 3.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-seqs", type=int, default=4)
    a = ap.parse_args(argv)

    import torch

    from . import build
    from .registry import load_config

    _, entry, config = load_config(a.model)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
    if dt not in entry.dtypes:
        print(f"this model family is not served in {a.dtype}", file=sys.stderr)
        return 3
    build.build()  # compiles the kernel library on first use (in-tree); a no-op afterwards
    from .engine import B200Engine

    eng = B200Engine(config, entry.open_weights(a.model, config), entry=entry, dtype=a.dtype, max_num_seqs=a.max_seqs,
                     max_pool_tokens=a.max_tokens, max_num_batched_tokens=1 << 30)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want") or []) for e in step.get("entries", [])]
        taps = eng.replay_step(entries, step.get("end") or [])
        rows = [taps[rid] for rid, _, want in entries if want]
        if rows:
            data = torch.cat(rows).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(a.out, f".{step['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
