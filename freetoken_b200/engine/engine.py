"""The engine: owns the model, the cache manager and the step function.

``Engine.step`` takes a batch of (request, its next tokens, the places among them whose
logits are wanted).  Portions of prompts and single decoded tokens may stand side by side,
cut anywhere; the step runs only the tokens it is given, reads everything earlier from the
cache, and returns float32 logits at the wanted places.  Sampling is a separate call, so
that the replay tool can take the logits as they are.

The reference's ``Engine.forward_batch`` (python/freetoken/engine/engine.py:863-883) runs a
batch that is either all prompt portions or all decode tokens
(python/freetoken/core.py:115, python/freetoken/scheduler/scheduler.py:828-833), samples inside
and exposes logits only for each request's last token
(python/freetoken/layers/embedding.py:107-110).  Construction follows its order
(engine.py:292-423): resolve config, build and fill the model, size the cache from the
memory that is left, then the sampler and the CUDA graphs of decode steps
(python/freetoken/engine/graph.py:94-217).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager, PagedCacheView
from ..config.engine_config import EngineConfig, normalize_dtype
from ..config.reader import read_config_json
from ..config.spec import ModelSpec, PagedKVNeed
from ..errors import CacheError, ConfigError, SchedulerError
from ..kernels import ops
from ..parts import BuildEnv, PositionEncoding, Segment, StepState, Workspace
from ..registry import architecture_of
from .build import build_model, load_weights, random_weights
from .step import StepBuffers, StepBuilder

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}
STATUS_CHECK_EVERY = 1024  # steps between two looks at the kernels' status words (a look waits for the device)


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()  # indices into ``tokens`` whose logits are wanted
    # (int32 device tensor, index): the entry's single token is still on the device (sampled by a
    # step whose result the host has not read yet); ``tokens`` then holds a placeholder
    device_token: Optional[Tuple[torch.Tensor, int]] = None


@dataclass
class StepOutput:
    logits: torch.Tensor  # [n_rows, vocab] float32 on the device (valid until the next step)
    rows: List[Tuple[Hashable, int]]  # (request, index into its tokens of this step) per row


class Engine:
    def __init__(self, config: EngineConfig, spec: Optional[ModelSpec] = None,
                 raw_config: Optional[dict] = None):
        """``spec`` replaces the model description that the architecture would build from
        config.json (another schedule, toy parts); with ``config.use_dummy_weight`` no folder is
        needed at all."""
        self.config = config
        self.device = torch.device(config.device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            torch.backends.cuda.matmul.allow_tf32 = False  # the 32-bit path is true 32-bit
            torch.backends.cudnn.allow_tf32 = False
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.arch = self.typed = None
        raw = raw_config
        if raw is None and os.path.isfile(os.path.join(config.model_path, "config.json")):
            raw = read_config_json(config.model_path)
        if raw is not None:
            self.arch = architecture_of(raw)
            self.typed = self.arch.parse_config(raw, num_layers=config.num_layers)
        if spec is None:
            if self.arch is None:
                raise ConfigError(f"{config.model_path}: no config.json in the model folder")
            spec = self.arch.build_spec(self.typed)
        file_dtype = getattr(self.typed, "torch_dtype", None)
        dtype = config.dtype
        if dtype == "auto":  # python/freetoken/server/args.py:660-679
            try:
                dtype = normalize_dtype(file_dtype) if file_dtype else "bfloat16"
            except ConfigError:
                dtype = "bfloat16"
        self.dtype_name = dtype
        self.dtype = _TORCH_DTYPE[dtype]
        self.spec = spec

        self.sm_count = (torch.cuda.get_device_properties(self.device).multi_processor_count
                         if self.device.type == "cuda" else 148)
        free_before = self._free_memory()
        # longest sequence: the override, else the model's own limit (engine/config.py:94-98)
        limit = config.max_seq_len_override or spec.max_position
        if config.max_seq_len_override and config.max_seq_len_override > spec.max_position:
            raise ConfigError(
                f"max_seq_len_override={config.max_seq_len_override} exceeds the model's "
                f"max_position_embeddings={spec.max_position}")
        self.max_step_tokens = int(config.max_step_tokens)
        self.workspace = Workspace(self.device)
        self.env = BuildEnv(dtype=self.dtype, device=self.device, max_seq_len=limit,
                            max_step_tokens=self.max_step_tokens, workspace=self.workspace,
                            max_decode_rows=config.max_running_req)
        self.model = build_model(spec, self.env)
        needs = self.model.cache_needs()
        # a cache given in pages bounds the longest sequence, unless every mixer that keeps pages has
        # a window (then a sequence never holds more than its window and a step's tokens)
        keeps_all = any(isinstance(n, PagedKVNeed) and n.window is None for _, n in needs)
        if config.num_page_override is not None and keeps_all:
            limit = min(limit, config.num_page_override * config.page_size)
        self.max_seq_len = self.env.max_seq_len = limit
        if config.use_dummy_weight:
            random_weights(self.model, config.seed)
        else:
            load_weights(self.model, self.arch, self.typed, config.model_path)
        for part in self.model.parts():  # position tables: made now, so that the cache is sized after them
            table = getattr(part, "table", None)
            if callable(table) and isinstance(part, PositionEncoding):
                table()

        itemsize = 4 if self.dtype == torch.float32 else 2
        if config.num_page_override is not None:
            num_pages = config.num_page_override
        else:  # python/freetoken/engine/engine.py:65-69,340-346, python/freetoken/kvcache/base.py:62-76
            per_token = CacheManager.bytes_per_token(needs, itemsize)
            used = free_before - self._free_memory()
            budget = int(config.memory_ratio * free_before) - used - self._activation_reserve()
            if per_token == 0:
                num_pages = 1
            else:
                num_pages = budget // (per_token * config.page_size)
                num_pages = min(num_pages, config.max_running_req * -(-self.max_seq_len // config.page_size))
            if num_pages < 1:
                raise ConfigError("no memory left for the cache after loading the model")
        self.num_pages = int(num_pages)
        self.cache = CacheManager(needs, config.page_size, self.num_pages, config.max_running_req,
                                  self.max_seq_len, self.dtype, self.device,
                                  max_step_tokens=self.max_step_tokens)
        self._views: List[Any] = []
        for i, e in enumerate(spec.schedule):
            owner = i if e.cache_from is None else e.cache_from
            self._views.append(self.cache.view(owner))
        self.buffers = StepBuffers(self.device, self._metadata_capacity())
        self.graphs: Dict[Any, Any] = {}
        self.graph_logits: Dict[Any, torch.Tensor] = {}
        self.graph_launches: Dict[Any, int] = {}
        # a graph's warm-up runs the step once more, so only mixers whose step can be repeated
        # without changing the result (they say so with ``graph_safe``) may be replayed
        self.use_graphs = (bool(config.cuda_graph) and self.device.type == "cuda"
                           and all(getattr(m, "graph_safe", False) for m in self.model.mixers()))
        self.steps_run = 0
        self.kernel_launches = 0

    # ------------------------------------------------------------------ sizing helpers
    def _free_memory(self) -> int:
        if self.device.type != "cuda":
            return 1 << 40
        torch.cuda.synchronize(self.device)
        return torch.cuda.mem_get_info(self.device)[0]

    def _activation_reserve(self) -> int:
        """Room for the step's work buffers, which are allocated at the first steps: what the model
        and its parts report for the largest step (:meth:`Part.workspace_bytes`), and some slack for
        the library's own work areas."""
        return self.model.workspace_bytes(self.max_step_tokens) + (1 << 28)

    def _metadata_capacity(self) -> int:
        """int32 elements the packed metadata of the largest step can take."""
        T = self.max_step_tokens
        S = self.config.max_running_req
        n_groups = max(1, len(self.cache.paged))
        core = 3 * T + 8 * S + 64
        per_group = T + 2 * (T // self.config.page_size + 2 * S + 4)
        n_plans = max(1, 2 * len({m.plan_key() for m in self.model.mixers() if hasattr(m, "plan_key")}))
        items = 8 * (T + S + 2 * self.sm_count * 32)
        return core + n_groups * per_group + n_plans * items + 4096

    # ------------------------------------------------------------------ requests
    def open(self, rid: Hashable) -> None:
        self.cache.open(rid)

    def close(self, rid: Hashable) -> None:
        """The request is finished: its pages and state slot go back to the free lists."""
        self.cache.close(rid)
        if self.config.check_cache:
            self.cache.check()

    def length(self, rid: Hashable) -> int:
        return self.cache.length(rid)

    def is_open(self, rid: Hashable) -> bool:
        return self.cache.is_open(rid)

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> StepOutput:
        if not entries:
            raise SchedulerError("a step needs at least one entry")
        total = sum(len(e.tokens) for e in entries)
        if total > self.max_step_tokens:
            raise SchedulerError(f"the step carries {total} tokens, max_step_tokens is {self.max_step_tokens}")
        if len(entries) > self.config.max_running_req:
            raise SchedulerError(
                f"the step carries {len(entries)} requests, max_running_req is {self.config.max_running_req}")
        vocab = self.spec.vocab_size
        token_ids = np.empty(total, dtype=np.int32)
        t0 = 0
        rows: List[Tuple[Hashable, int]] = []
        logit_rows: List[int] = []
        for e in entries:
            n = len(e.tokens)
            if n < 1:
                raise SchedulerError(f"request {e.request_id!r}: an entry needs at least one token")
            ids = np.asarray(e.tokens, dtype=np.int64)
            if e.device_token is not None:
                if n != 1:
                    raise SchedulerError(f"request {e.request_id!r}: a token taken from the device stands alone")
                ids = np.zeros(1, dtype=np.int64)
            if ids.min() < 0 or ids.max() >= vocab:
                raise SchedulerError(f"request {e.request_id!r}: token id outside [0, {vocab})")
            token_ids[t0:t0 + n] = ids
            for w in e.want:
                if not 0 <= w < n:
                    raise SchedulerError(f"request {e.request_id!r}: wanted place {w} outside its {n} tokens")
                rows.append((e.request_id, int(w)))
                logit_rows.append(t0 + int(w))
            t0 += n
        opened: List[Hashable] = []  # requests this call opened: closed again if the step is refused
        try:
            for e in entries:
                if not self.cache.is_open(e.request_id) and e.request_id not in opened:
                    self.cache.open(e.request_id)
                    opened.append(e.request_id)
            plan = self.cache.begin_step([(e.request_id, len(e.tokens)) for e in entries])
        except Exception:
            for rid in opened:
                self.cache.close(rid)
            raise
        try:
            logits = self._run(entries, plan, token_ids, logit_rows)
        except Exception:
            self.cache.abort_step()
            for rid in opened:
                self.cache.close(rid)
            raise
        self.cache.end_step()
        if self.config.check_cache:
            self.cache.check()
        self.steps_run += 1
        if self.steps_run == 1 or self.steps_run % STATUS_CHECK_EVERY == 0:
            self.check_kernels()
        return StepOutput(logits=logits, rows=rows)

    def check_kernels(self) -> None:
        """Raise if a kernel gave up a bounded wait since the last check (its results are not valid).
        Reading the status words waits for the device, so steps do it only now and then; whoever reads a
        result on the host anyway (trace replay, the end of a generation) calls this as well."""
        if self.device.type == "cuda":
            ops.check_status()

    def _run(self, entries, plan, token_ids: np.ndarray, logit_rows: List[int]) -> torch.Tensor:
        S = len(entries)
        T = token_ids.shape[0]
        decode_only = all(len(e.tokens) == 1 for e in entries)
        graphable = (self.use_graphs and decode_only and len(logit_rows) == S
                     and logit_rows == list(range(S)))
        segments: List[Segment] = []
        seg_info = np.empty((S, 4), dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        q0 = 0
        for i, e in enumerate(entries):
            n = len(e.tokens)
            kv = plan.kv_lens[i]
            segments.append(Segment(e.request_id, q0, n, kv, plan.state_slots[i], plan.fresh[i]))
            seg_info[i] = (q0, n, kv, plan.rows[i])
            positions[q0:q0 + n] = np.arange(kv - n, kv)
            q0 += n
        builder = StepBuilder(self, [(s.q_len, s.kv_len) for s in segments], fixed=graphable,
                              sm_count=self.sm_count)
        builder.add("token_ids", token_ids)
        builder.add("positions", positions)
        builder.add("seg_info", seg_info)
        builder.add("state_slots", np.asarray(plan.state_slots, dtype=np.int32))
        builder.add("logit_rows", np.asarray(logit_rows, dtype=np.int32))
        # tokens that are still on the device: (place among this step's tokens, index in the source)
        pending = np.full((S, 2), -1, dtype=np.int32)
        pending_src = None
        for i, e in enumerate(entries):
            if e.device_token is not None:
                src, idx = e.device_token
                if pending_src is not None and src is not pending_src:
                    raise SchedulerError("tokens taken from the device must come from one tensor per step")
                pending_src = src
                pending[i] = (segments[i].q_start, idx)
        builder.add("pending", pending)
        n_updates = []
        for g in self.cache.paged:
            builder.add(f"slot_map.{g.index}", plan.slot_maps[g.index])
            ups = self.cache.take_updates(g.index)
            n_up = len(ups)
            if graphable:
                cap = S + 1  # a decode step adds at most one page per request
                if n_up > cap:
                    graphable = False
                    builder.fixed = False
                else:
                    n_up = cap
            arr = np.full((max(n_up, 1), 2), -1, dtype=np.int32)
            if ups:
                arr[:len(ups)] = np.asarray(ups, dtype=np.int32)
            builder.add(f"table_updates.{g.index}", arr)
            n_updates.append(arr.shape[0])
        for mixer in self.model.mixers():
            prep = getattr(mixer, "prepare", None)
            if prep is not None:
                prep(builder)
        tensors, plans = builder.finish(self.buffers, self.workspace)
        step = StepState(
            n_tokens=T, segments=segments, token_ids=tensors["token_ids"],
            positions=tensors["positions"], seg_info=tensors["seg_info"],
            state_slots=tensors["state_slots"], logit_rows=tensors["logit_rows"],
            n_logit_rows=len(logit_rows), attention_plans=plans, decode_only=decode_only)
        step.extras["tensors"] = tensors
        views = self._step_views(tensors)

        if pending_src is not None:  # before the step (and outside its graph): fill in the device tokens
            ops.copy_tokens(tensors["token_ids"], tensors["pending"], pending_src, S, self.spec.vocab_size)

        def body() -> torch.Tensor:
            for g, n_up in zip(self.cache.paged, n_updates):
                ops.table_update(g.table_dev, tensors[f"table_updates.{g.index}"], n_up)
            return self.model.forward(step, views)

        if not graphable:
            return body()
        # one graph per batch size and metadata layout (the attention split count moves with the
        # longest request, which changes the size of the work list a few times over a long decode)
        key = (S, tuple(arr.size for _, arr in builder.sections), tuple(sorted(map(repr, builder.plans))),
               builder.longest_span())
        if key not in self.graphs:
            body()  # warm-up: allocates work buffers and library workspaces outside the capture
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            step.capturing = True
            with torch.cuda.graph(graph):
                out = body()
            step.capturing = False
            self.graphs[key] = graph
            self.graph_logits[key] = out
            self.graph_launches[key] = ops.launch_count() - before
        # (after a capture the warm-up has already run this step; the replay repeats it, which
        # graph_safe mixers allow, so that every result comes from the same code path)
        self.graphs[key].replay()
        ops.count_launches(self.graph_launches[key])
        return self.graph_logits[key]

    def _step_views(self, tensors: Dict[str, torch.Tensor]) -> List[Any]:
        out = []
        for v in self._views:
            if isinstance(v, PagedCacheView):
                v = PagedCacheView(v.slabs, v.block_table, tensors[f"slot_map.{v.group.index}"],
                                   v.page_size, v.window, v.group)
            out.append(v)
        return out
