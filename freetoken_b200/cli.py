"""Command line: ``python -m freetoken_b200 <command>`` (console scripts ``freetoken`` and ``ft``).

Commands are looked up in a name -> function table and imported lazily, like the reference's
dispatcher (python/freetoken/cli.py:93-126).  Engine options carry the reference's names
(python/freetoken/server/args.py:200-365): ``--model-path/--model``, ``--dtype``,
``--max-running-requests``, ``--max-seq-len-override``, ``--memory-ratio``, ``--dummy-weight``,
``--max-prefill-length/--max-extend-length``, ``--num-pages``, ``--num-tokens``, ``--page-size``,
``--cuda-graph-max-bs``.  ``generate`` is the raw completion smoke test (``ft ctl generate``,
python/freetoken/control_cli.py:294-297) run in-process on token ids; ``replay`` is the trace
replay; ``make-model`` writes a random-weights model folder; ``bench`` runs the benchmark.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Callable, Dict, List, Optional


def add_engine_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model-path", "--model", dest="model_path", required=True,
                   help="folder with config.json and the safetensors files")
    p.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    p.add_argument("--device", default="cuda:0", help="the CUDA device the engine runs on")
    p.add_argument("--max-running-requests", type=int, default=4)
    p.add_argument("--max-seq-len-override", type=int, default=None)
    p.add_argument("--memory-ratio", type=float, default=0.9)
    p.add_argument("--dummy-weight", action="store_true", help="random weights made on the device")
    p.add_argument("--max-prefill-length", "--max-extend-length", dest="max_extend_tokens", type=int,
                   default=8192, help="most prompt tokens of one request in one step")
    p.add_argument("--max-step-tokens", type=int, default=None, help="token budget of one step")
    p.add_argument("--num-pages", type=int, default=None)
    p.add_argument("--num-tokens", type=int, default=None)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--num-layers", type=int, default=None, help="run only the first N layers")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--cuda-graph-max-bs", type=int, default=None)
    p.add_argument("--disable-cuda-graph", action="store_true")
    p.add_argument("--decode-log-interval", type=int, default=0,
                   help="log a status line every so many decode steps (0: none)")


def engine_kwargs(a: argparse.Namespace) -> Dict:
    return dict(dtype=a.dtype, device=a.device, max_running_req=a.max_running_requests,
                max_seq_len_override=a.max_seq_len_override, memory_ratio=a.memory_ratio,
                use_dummy_weight=a.dummy_weight, max_extend_tokens=a.max_extend_tokens,
                max_step_tokens=a.max_step_tokens, num_page_override=a.num_pages,
                num_token_override=a.num_tokens, page_size=a.page_size, num_layers=a.num_layers,
                seed=a.seed, cuda_graph=not a.disable_cuda_graph, cuda_graph_max_bs=a.cuda_graph_max_bs,
                decode_log_interval=a.decode_log_interval)


def cmd_generate(argv: List[str]) -> int:
    p = argparse.ArgumentParser(prog="ft generate", description="generate from prompts of token ids")
    add_engine_args(p)
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="comma-separated token ids; repeat for several prompts")
    p.add_argument("--prompt-file", default=None, help="JSON file: a list of lists of token ids")
    p.add_argument("--max-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    a = p.parse_args(argv)
    prompts = [[int(x) for x in s.split(",") if x.strip()] for s in a.prompt_ids]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += json.load(f)
    if not prompts:
        p.error("give --prompt-ids or --prompt-file")
    from .engine.llm import LLM
    from .sampling.params import SamplingParams

    kw = engine_kwargs(a)
    if a.decode_log_interval > 0:
        import logging

        logging.basicConfig(level=logging.INFO, format="[%(asctime)s] %(message)s", stream=sys.stderr)
    dtype = kw.pop("dtype")
    llm = LLM(a.model_path, dtype=dtype, **kw)
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                        ignore_eos=a.ignore_eos, max_tokens=a.max_tokens, seed=a.seed)
    for r in llm.generate(prompts, sp):
        print(json.dumps(r))
    return 0


def cmd_replay(argv: List[str]) -> int:
    from .replay import main

    return main(argv)


def cmd_make_model(argv: List[str]) -> int:
    p = argparse.ArgumentParser(prog="ft make-model",
                                description="write a model folder with seeded random weights")
    p.add_argument("--config", required=True, help="a config.json to take the sizes from")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--fused-names", action="store_true",
                   help="write the engine's fused tensor names instead of the checkpoint's")
    a = p.parse_args(argv)
    from .weights.random_init import write_model_folder

    with open(a.config) as f:
        cfg = json.load(f)
    print(write_model_folder(cfg, a.out, a.seed, fused_names=a.fused_names))
    return 0


def cmd_bench(argv: List[str]) -> int:
    import os
    import runpy

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.argv = ["bench.py"] + list(argv)
    runpy.run_path(os.path.join(root, "bench.py"), run_name="__main__")
    return 0


COMMANDS: Dict[str, Callable[[List[str]], int]] = {
    "generate": cmd_generate,
    "replay": cmd_replay,
    "make-model": cmd_make_model,
    "bench": cmd_bench,
}


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: ft <command> [options]\n\ncommands: " + ", ".join(COMMANDS))
        return 0 if argv else 2
    if argv[0] not in COMMANDS:
        print(f"ft: unknown command '{argv[0]}' (commands: {', '.join(COMMANDS)})", file=sys.stderr)
        return 2
    from .errors import FreeTokenError

    try:
        return COMMANDS[argv[0]](argv[1:])
    except FreeTokenError as e:
        print(f"ft {argv[0]}: {e}", file=sys.stderr)
        return 1
