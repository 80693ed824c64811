"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
:class:`Engine` that generation uses and calls :meth:`Engine.step` with the entries of each
line.  The reference has nothing equivalent (the closest is its raw-completion smoke test,
``ft ctl generate``, docs/cli.md:104).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 ``[wanted, vocab]``.
After every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

PAGE_SIZE = 16  # divides 64: a request's pages never exceed its token count rounded up to 64
MAX_LIVE = 8


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens that live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE, help=argparse.SUPPRESS)
    p.add_argument("--no-cuda-graph", action="store_true", help=argparse.SUPPRESS)
    p.add_argument("--device", default="cuda:0", help=argparse.SUPPRESS)
    return p


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens < 1:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    print("[trace_run] loading the engine (kernels are compiled at the first call)", file=sys.stderr, flush=True)
    import numpy as np
    import torch

    from .config.engine_config import EngineConfig
    from .config.reader import read_config_json
    from .engine.engine import Engine, StepEntry
    from .errors import FreeTokenError
    from .registry import architecture_of

    page = args.page_size
    n_pages = -(-args.max_tokens // page)
    try:
        raw = read_config_json(args.model)
        arch = architecture_of(raw)  # the architecture says how long its sequences may get
        seq = min(int(arch.build_spec(arch.parse_config(raw)).max_position), n_pages * page)
        engine = Engine(EngineConfig(
            model_path=args.model, dtype=args.dtype, device=args.device, page_size=page, num_page_override=n_pages,
            max_running_req=MAX_LIVE, max_seq_len_override=seq, max_extend_tokens=seq,
            max_step_tokens=max(seq, MAX_LIVE), cuda_graph=not args.no_cuda_graph))
    except FreeTokenError as e:
        print(f"trace_run: {e}", file=sys.stderr)
        return 1
    print("[trace_run] ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                       for e in rec.get("entries", [])]
        except (ValueError, KeyError, TypeError) as e:
            print(f"trace_run: bad input line ({e}): {line[:200]}", file=sys.stderr)
            return 1
        try:
            if entries:
                out = engine.step(entries)
                if out.rows:
                    arr = out.logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f".{step}.f32.tmp")
                    arr.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
                    engine.check_kernels()  # the logits were just read: the device is idle anyway
            for rid in rec.get("end", []):
                if engine.is_open(rid):
                    engine.close(rid)
        except FreeTokenError as e:
            print(f"trace_run: step {step}: {e}", file=sys.stderr)
            return 1
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
