"""Two larger workloads beside the headline benchmark, on the same layer sizes and random weights.

``long_contexts``: several requests with prompts of very different lengths (thousands to tens of
thousands of tokens) go through the scheduler, the prompts in portions beside the decoding of the
others, then every request decodes a few hundred tokens greedily.  Reported: prefill and decode
tokens a second, the high-water mark of the page pool.

``chunked_prefill``: one very long prompt is read in portions of a few hundred tokens, every step
beside one decoded token of many other requests.  Reported: tokens a second of the mixed steps, the
time of a step at the start and at the end of the prompt.

    python bench.py --workload long_contexts [--layers 16] [--requests 8] [--max-prompt 24576] [--new-tokens 512]
    python bench.py --workload chunked_prefill [--layers 4] [--prompt 131072] [--chunk 512] [--decoders 63]

Each prints one JSON line.  The reference times whole generations of this kind in
benchmarks/bench_decode_moe.py:8-24 (tokens after the first / time between first and last).
"""

from __future__ import annotations

import json
import time
from typing import Any, Dict

import numpy as np
import torch

from .config.engine_config import EngineConfig
from .engine.engine import Engine, StepEntry
from .engine.scheduler import Scheduler
from .sampling import Sampler, SamplingParams


def _engine(raw: Dict[str, Any], layers: int, max_seq: int, max_tokens: int, reqs: int, step_tokens: int) -> Engine:
    cfg = dict(raw, num_hidden_layers=layers, max_position_embeddings=max_seq)
    return Engine(EngineConfig(model_path="", dtype="bfloat16", use_dummy_weight=True, seed=0, page_size=16,
                               max_running_req=reqs, num_token_override=max_tokens, max_seq_len_override=max_seq,
                               max_extend_tokens=step_tokens, max_step_tokens=step_tokens), raw_config=cfg)


def long_contexts(raw: Dict[str, Any], layers: int = 16, requests: int = 8, min_prompt: int = 1024,
                  max_prompt: int = 24576, new_tokens: int = 512, seed: int = 0) -> Dict[str, Any]:
    rng = np.random.default_rng(seed)
    lengths = [int(x) for x in rng.integers(min_prompt, max_prompt + 1, requests)]
    max_seq = max_prompt + new_tokens + 16
    pool_tokens = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths) + 16 * requests
    eng = _engine(raw, layers, max_seq, pool_tokens, requests, 8192)
    V = eng.spec.vocab_size
    sched = Scheduler(eng, Sampler(eng.device, V, requests), ())
    for i, n in enumerate(lengths):
        sched.add_request(rng.integers(0, V, n).tolist(), SamplingParams(max_tokens=new_tokens, ignore_eos=True), rid=i)
    pool = eng.cache.paged[0].pool
    high = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_prefill_done = None
    decoded_at_prefill_done = 0
    steps = 0
    while not sched.idle:
        sched.step_overlapped()
        steps += 1
        high = max(high, pool.num_pages - pool.free_count)
        if t_prefill_done is None and all(r.decoding for r in sched.running) and not sched.waiting:
            torch.cuda.synchronize()
            t_prefill_done = time.perf_counter()
            decoded_at_prefill_done = sum(len(r.output) + r.in_flight for r in sched.running)
    sched.drain()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    total_new = sum(len(sched.done[i].output) for i in range(requests))
    assert total_new == requests * new_tokens, (total_new, requests, new_tokens)
    t_mid = t_prefill_done if t_prefill_done is not None else t1
    decode_tokens = total_new - decoded_at_prefill_done
    return {
        "workload": "long_contexts", "layers": layers, "requests": requests, "prompt_lengths": lengths,
        "new_tokens": new_tokens, "steps": steps,
        "prefill_tokens_per_s": round(sum(lengths) / (t_mid - t0), 1), "prefill_s": round(t_mid - t0, 3),
        "decode_tokens_per_s": round(decode_tokens / max(t1 - t_mid, 1e-9), 1), "decode_s": round(t1 - t_mid, 3),
        "pages_high_water": int(high), "pages": int(pool.num_pages), "page_size": 16,
    }


def chunked_prefill(raw: Dict[str, Any], layers: int = 4, prompt: int = 131072, chunk: int = 512, decoders: int = 63,
                    seed: int = 0) -> Dict[str, Any]:
    rng = np.random.default_rng(seed)
    n_steps = -(-prompt // chunk)
    dec_prompts = [int(x) for x in rng.integers(128, 4097, decoders)]
    max_seq = max(prompt, max(dec_prompts) + n_steps) + 16
    pool_tokens = -(-prompt // 16) * 16 + sum(-(-(n + n_steps) // 16) * 16 for n in dec_prompts) + 16 * (decoders + 1)
    eng = _engine(raw, layers, max_seq, pool_tokens, decoders + 1, max(8192, chunk + decoders))
    V = eng.spec.vocab_size
    for i, n in enumerate(dec_prompts):  # the others' prompts first
        eng.step([StepEntry(("d", i), rng.integers(0, V, n).tolist(), [])])
    long_prompt = rng.integers(0, V, prompt).tolist()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ev[0].record()
    fed = 0
    for s in range(n_steps):
        part = long_prompt[fed:fed + chunk]
        fed += len(part)
        entries = [StepEntry("long", part, [len(part) - 1] if fed == prompt else [])]
        entries += [StepEntry(("d", i), [int(rng.integers(0, V))], [0]) for i in range(decoders)]
        eng.step(entries)
        ev[s + 1].record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(n_steps)]
    tokens = prompt + decoders * n_steps
    return {
        "workload": "chunked_prefill", "layers": layers, "prompt": prompt, "chunk": chunk, "decoders": decoders,
        "decoder_prompts": [min(dec_prompts), max(dec_prompts)], "steps": n_steps,
        "tokens_per_s": round(tokens / (t1 - t0), 1), "seconds": round(t1 - t0, 3),
        "ms_first_steps": round(float(np.median(ms[: max(1, n_steps // 16)])), 3),
        "ms_last_steps": round(float(np.median(ms[-max(1, n_steps // 16):])), 3),
    }


def run(name: str, raw: Dict[str, Any], **kw: Any) -> int:
    fn = {"long_contexts": long_contexts, "chunked_prefill": chunked_prefill}[name]
    print(json.dumps(fn(raw, **{k: v for k, v in kw.items() if v is not None})))
    return 0
