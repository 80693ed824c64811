"""Benchmark: MiniMax-M3 decode throughput on one B200 (and prefill, and the decode roofline).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--impl ours|reference]

The default run builds the 12-layer model of the headline configuration (hidden 3072, 48 query /
8 KV heads of 128, rotary 64, 256 experts top-8 of width 1536, vocabulary 200064) with random
bfloat16 weights made on the device, gives 8 requests a 2048-token prompt each (context length
4096 = 2048 prompt + up to 2048 decoded), and times K decode steps.  A "step" is one decode step
of the whole batch.  It prints ONE JSON line:

* ``value``: decoded tokens per second, timed on the device with CUDA events around K steps;
* ``e2e``: the same through the Python entry point's scheduler loop, wall clock, host token ids in
  and sampled token ids out every step (pinned host-to-device and device-to-host copies included);
* ``prefill``: one 2048-token prompt in one step: tokens/s, ms, and flops / time / bf16 peak;
* ``roofline``: bytes the decode step has to read (every weight it uses once, plus the cache of the
  live requests) / its time, against the measured HBM copy bandwidth;
* ``points``: decode tokens/s at batch 1 and 64, at longer contexts (batch 8 at 8k and 32k tokens, batch 64
  at 8k), and the two larger workloads of freetoken_b200/workloads.py (``--no-long-points`` and
  ``--no-workloads`` leave them out); ``points_hbm_frac``: bytes read / time / HBM peak of the decode points;
* ``clocks``: SM clock and throttle reasons sampled during the timed region.

``--workload long_contexts | chunked_prefill`` runs one of the larger workloads of
freetoken_b200/workloads.py instead and prints that workload's own JSON line.

Peaks come from MEASURED_PEAKS.json when the driver wrote it, else 6.65 TB/s and 1.59 PFLOP/s.
More than one GPU is outside this engine: ``--gpus N`` with N > 1 prints one line and exits 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADLINE = {
    "architectures": ["MiniMaxM3SparseForCausalLM"], "model_type": "minimax_m3",
    "vocab_size": 200064, "hidden_size": 3072, "num_hidden_layers": 12,
    "num_attention_heads": 48, "num_key_value_heads": 8, "head_dim": 128, "rotary_dim": 64,
    "rope_theta": 5000000.0, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6,
    "use_qk_norm": True, "use_gemma_norm": True, "tie_word_embeddings": False,
    "hidden_act": "silu", "num_local_experts": 256, "num_experts_per_tok": 8,
    "intermediate_size": 1536, "scoring_func": "sigmoid", "use_routing_bias": True,
    "routed_scaling_factor": 1.0, "n_shared_experts": 0, "torch_dtype": "bfloat16",
}
PROMPT = 2048
CONTEXT = 4096
# further decode points on the same engine: (batch, context) with their own roofline fractions
LONG_POINTS = ((8, 8192), (8, 32768), (64, 8192))
MAX_POSITION = 32768 + 256


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            with open(path) as f:
                m = json.load(f)
            if "hbm_gbs" in m:
                out["hbm_gbs"] = float(m["hbm_gbs"])
            if "bf16_tflops" in m:
                out["bf16_tflops"] = float(m["bf16_tflops"])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while active."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.index = index

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:6]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def reference_arm():
    """The unmodified reference through its own entry point, where it can run at all."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "freetoken")):
        why = ("baseline/_ref is absent: the reference installs offline only with --no-deps, its package then fails to "
               "import (flashlib is not installable offline), its MiniMax-M3 loader takes NVFP4 expert banks only, and "
               "its installed tree names a CUDA call that is closed on this pool, so it was taken out again")
    else:
        p = subprocess.run([sys.executable, "-c",
                            f"import sys; sys.path.insert(0, {ref!r}); import freetoken.layers"],
                           capture_output=True, text=True)
        if p.returncode != 0:
            last = (p.stderr.strip().splitlines() or ["import failed"])[-1]
            why = ("the reference's MiniMax-M3 path cannot start here: " + last +
                   " (flashlib is not installable offline; its M3 loader also requires NVFP4 expert banks)")
        else:
            why = ("the reference's MiniMax-M3 loader only accepts NVFP4 expert banks behind its CPU offload cache "
                   "(python/freetoken/models/minimax_m3/weight.py:154-158); bfloat16 random weights cannot be served")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def expert_bytes_read(engine, entries_fn, n_steps=1):
    """Distinct (layer, expert) pairs one decode step touches, counted on a real step."""
    import torch

    counts = []
    engine.env.shared["record_expert_counts"] = counts
    was = engine.use_graphs
    engine.use_graphs = False
    try:
        for _ in range(n_steps):
            engine.step(entries_fn())
        torch.cuda.synchronize()
    finally:
        engine.use_graphs = was
        engine.env.shared.pop("record_expert_counts", None)
    per_step = len(counts) // max(n_steps, 1)
    distinct = sum(int((c > 0).sum()) for c in counts[-per_step:]) if per_step else 0
    return distinct


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=HEADLINE["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-long-points", action="store_true", help="skip the decode points at 8k and 32k tokens of context")
    ap.add_argument("--no-workloads", action="store_true", help="skip the long_contexts and chunked_prefill workloads")
    ap.add_argument("--profile", choices=["decode", "prefill"], default=None,
                    help="run only that phase and bracket `--steps` steps of it with cudaProfilerStart/Stop "
                         "(for ncu --profile-from-start off); prints no bench line")
    ap.add_argument("--workload", choices=["long_contexts", "chunked_prefill"], default=None,
                    help="run one of the larger workloads of freetoken_b200/workloads.py instead (its own JSON line)")
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--max-prompt", type=int, default=None)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--decoders", type=int, default=None)
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is outside its scope")
        return 2
    if args.impl == "reference":
        return reference_arm()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload:
        from freetoken_b200 import workloads

        layers = args.layers if "--layers" in sys.argv else None
        if args.workload == "long_contexts":
            return workloads.run("long_contexts", HEADLINE, layers=layers, requests=args.requests,
                                 max_prompt=args.max_prompt, new_tokens=args.new_tokens)
        return workloads.run("chunked_prefill", HEADLINE, layers=layers, prompt=args.prompt, chunk=args.chunk,
                             decoders=args.decoders)

    import numpy as np
    import torch

    from freetoken_b200.config.engine_config import EngineConfig
    from freetoken_b200.engine.engine import Engine, StepEntry
    from freetoken_b200.engine.scheduler import Scheduler
    from freetoken_b200.kernels import ops
    from freetoken_b200.sampling import Sampler, SamplingParams

    pk = peaks()
    long_points = [] if (args.no_points or args.no_long_points) else list(LONG_POINTS)
    raw = dict(HEADLINE, num_hidden_layers=args.layers,
               max_position_embeddings=MAX_POSITION if long_points else HEADLINE["max_position_embeddings"])
    max_b = max(args.batch, 1 if args.no_points else 64)
    pool_tokens = max([max_b * CONTEXT] + [b * (ctx + 256) for b, ctx in long_points])
    max_seq = max([CONTEXT] + [ctx + 256 for _, ctx in long_points])
    t0 = time.time()
    engine = Engine(EngineConfig(model_path="", dtype="bfloat16", use_dummy_weight=True, seed=0, page_size=16,
                                 max_running_req=max_b, num_token_override=pool_tokens,
                                 max_seq_len_override=max_seq, max_extend_tokens=PROMPT, max_step_tokens=PROMPT),
                    raw_config=raw)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    sampler = Sampler(engine.device, engine.spec.vocab_size, max_b)
    V = engine.spec.vocab_size
    rng = np.random.default_rng(0)
    cfg = engine.typed
    L, H, E, k, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size
    qdim, kvdim = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim

    def ev():
        return torch.cuda.Event(enable_timing=True)

    if args.profile:
        if args.profile == "prefill":
            for i in range(args.warmup + args.steps):
                if i == args.warmup:
                    torch.cuda.synchronize()
                    torch.cuda.profiler.start()
                engine.step([StepEntry(("p", i), rng.integers(0, V, PROMPT).tolist(), [PROMPT - 1])])
                engine.close(("p", i))
        else:
            rids = [("d", i) for i in range(args.batch)]
            for r in rids:
                engine.step([StepEntry(r, rng.integers(0, V, PROMPT).tolist(), [])])
            for i in range(args.warmup + args.steps):
                if i == args.warmup:
                    torch.cuda.synchronize()
                    torch.cuda.profiler.start()
                out = engine.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rids])
                sampler.sample(out.logits, [SamplingParams()] * len(rids), rids, [i] * len(rids))
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"profiled {args.steps} {args.profile} step(s)")
        return 0

    # ------------------------------------------------------------------ prefill of one 2048-token prompt
    prefill = None
    if not args.no_prefill:
        times = []
        for i in range(3 + 3):
            toks = rng.integers(0, V, PROMPT).tolist()
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            engine.step([StepEntry(("p", i), toks, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            engine.close(("p", i))
            if i >= 3:
                times.append(a.elapsed_time(b))
        ms = statistics.median(times)
        T = PROMPT
        flops = L * (2 * T * H * (qdim + 2 * kvdim) + 2 * T * qdim * H + 4 * (T * (T + 1) // 2) * qdim
                     + 2 * T * H * E + k * T * (2 * H * 2 * I + 2 * I * H)) + 2 * H * V
        # what the step has to read at least: every expert's weights once (2 048 tokens x top-k reach all of
        # them), the attention weights, the router and the head
        pre_bytes = L * (2 * (H * (qdim + 2 * kvdim) + qdim * H) + 4 * E * H + E * 2 * (2 * I * H + H * I)) + 2 * H * V
        prefill = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                   "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "hbm_frac": round(pre_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}

    # ------------------------------------------------------------------ decode
    def fill(batch, tag, context=PROMPT, rids=None):
        """Give `batch` requests a real prompt of `context` tokens each (in portions of 2048 tokens, a
        request's next portion at a time; requests in `rids` are grown to that length); return their ids."""
        rids = rids or [(tag, i) for i in range(batch)]
        for r in rids:
            have = engine.length(r) if engine.is_open(r) else 0
            while have < context:
                n = min(PROMPT, context - have)
                engine.step([StepEntry(r, rng.integers(0, V, n).tolist(), [])])
                have += n
        return rids

    def step_bytes_of(rids):
        """Bytes a decode step of these requests has to read: every weight it uses once (the experts it
        touches counted on a real step) and the cache of the live requests."""
        distinct = expert_bytes_read(engine, lambda: [StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rids])
        kv = sum(engine.length(r) for r in rids) * L * 2 * kvdim * 2
        weights = L * 2 * (H * (qdim + 2 * kvdim) + qdim * H) + L * 4 * E * H + distinct * 2 * (2 * I * H + H * I) + 2 * H * V
        return weights + kv, distinct

    def decode_tokens_per_s(rids, steps, warmup, sample=True):
        B = len(rids)
        params = [SamplingParams()] * B

        def one(i):
            out = engine.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in rids])
            if sample:  # the tokens stay on the device here; the end-to-end loop below reads them
                sampler.launch(out.logits, params, rids, [i] * B)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        before = ops.launch_count()
        a.record()
        for i in range(steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        return B / (ms / 1e3), ms, (ops.launch_count() - before)

    rids = fill(args.batch, "d")
    with ClockSampler() as clocks:
        value, ms_step, launches = decode_tokens_per_s(rids, args.steps, args.warmup)
    # bytes the step had to read
    step_bytes, distinct = step_bytes_of(rids)
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes),
                "distinct_experts": distinct, "peak_source": pk["source"]}

    # ------------------------------------------------------------------ end to end through the scheduler
    for r in rids:
        engine.close(r)
    sched = Scheduler(engine, sampler, ())
    n_e2e = args.warmup + args.steps
    for i in range(args.batch):
        sched.add_request(rng.integers(0, V, PROMPT).tolist(),
                          SamplingParams(max_tokens=n_e2e + 4 * args.batch + 8, ignore_eos=True), rid=("e", i))
    while any(not r.decoding for r in sched.running) or sched.waiting:
        sched.step()
    # the entry point's own loop (LLM.generate -> Scheduler.run): step N+1 is launched before step
    # N's tokens are read; every timed call uploads one step's metadata from pinned memory and
    # brings one step's tokens back to host lists
    for _ in range(args.warmup):
        sched.step_overlapped()
    sched.drain()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    got = 0
    for _ in range(args.steps):
        got += len(sched.step_overlapped().sampled)
    last = sched.drain()
    got += len(last.sampled) if last is not None else 0
    torch.cuda.synchronize()
    assert got == args.steps * args.batch, (got, args.steps, args.batch)
    e2e_ms = (time.perf_counter() - t1) * 1e3 / args.steps
    h2d = engine.buffers.last_upload_bytes + 16 * sampler.max_rows
    e2e = {"value": round(args.batch / (e2e_ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 3),
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * args.batch}
    for r in list(sched.running):
        sched.abort(r.rid)

    # ------------------------------------------------------------------ batch 1 and 64
    points, fracs = {}, {}
    if not args.no_points:
        n_steps = max(8, args.steps // 2)

        def point(name, rr):
            v, ms, _ = decode_tokens_per_s(rr, n_steps, args.warmup)
            nbytes, _ = step_bytes_of(rr)
            points[name] = round(v, 1)
            fracs[name] = round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

        for B in (1, 64):
            rr = fill(B, f"b{B}")
            point(f"decode_b{B}", rr)
            for r in rr:
                engine.close(r)
        rr, last_b = [], None
        for B, ctx in long_points:  # (batch 8 grows from 8k to 32k tokens: the same requests go on)
            if B != last_b:
                for r in rr:
                    engine.close(r)
                rr = None
            rr = fill(B, f"c{B}", context=ctx, rids=rr)
            last_b = B
            point(f"decode_b{B}_ctx{ctx // 1024}k", rr)
        for r in rr or []:
            engine.close(r)

    line = {
        "metric": "decode tok/s at batch 8, context 4096 (2048 prompt + decode), MiniMax-M3 layer sizes",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random N(0,0.02) weights made on the device",
        "config": {"model": "MiniMax-M3 layer sizes", "layers": L, "layers_of_config": HEADLINE["num_hidden_layers"],
                   "hidden": H, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "rotary_dim": cfg.rotary_dim, "experts": E, "top_k": k,
                   "expert_width": I, "vocab": V, "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT, "page_size": 16, "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (a step reads >20 GB of weights)", "cuda_graph": engine.use_graphs},
        "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline, "points": points,
        "points_hbm_frac": fracs, "clocks": clocks.summary(), "build_seconds": round(build_s, 1),
    }
    if not (args.no_points or args.no_workloads):
        # the two larger workloads need engines of their own (16 and 4 layers): this one goes first
        import gc

        from freetoken_b200 import workloads

        del sched, sampler, engine
        gc.collect()
        torch.cuda.empty_cache()
        with ClockSampler() as wl_clocks:
            for name, keys in (("long_contexts", ("prefill_tokens_per_s", "decode_tokens_per_s")),
                               ("chunked_prefill", ("tokens_per_s",))):
                try:
                    res = getattr(workloads, name)(HEADLINE)
                    for key in keys:
                        points[f"{name}_{key}"] = res[key]
                except Exception as e:  # a workload that does not fit must not cost the headline its line
                    points[f"{name}_error"] = f"{type(e).__name__}: {e}"[:200]
                gc.collect()
                torch.cuda.empty_cache()
        line["workload_clocks"] = wl_clocks.summary()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
