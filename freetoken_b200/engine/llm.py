"""Python entry point for offline generation, in the manner of the reference's ``LLM``
(python/freetoken/llm/llm.py:30-43,105-142): ``LLM(model_path, dtype, **engine options)`` and
``generate(prompts, sampling_params) -> [{"text", "token_ids"}]``.  Prompts are lists of token
ids; strings are accepted when the model folder has a ``tokenizer.json`` and the ``tokenizers``
package is importable.  An EOS token that ends a request is not part of its output (llm.py:94-103).
"""

from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..errors import ConfigError
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .engine import Engine
from .scheduler import Scheduler
from .status import StatusLine


class LLM:
    def __init__(self, model_path: str, dtype: Union[str, torch.dtype] = torch.bfloat16, **kwargs: Any):
        self.config = EngineConfig(model_path=model_path, dtype=str(dtype).replace("torch.", ""), **kwargs)
        self.engine = Engine(self.config)
        self.sampler = Sampler(self.engine.device, self.engine.spec.vocab_size,
                               max(self.config.max_running_req, 1), default_seed=self.config.seed)
        self.eos_token_ids = tuple(self.engine.spec.eos_token_ids)
        self.tokenizer = None
        tok = os.path.join(model_path, "tokenizer.json")
        if os.path.isfile(tok):
            try:
                from tokenizers import Tokenizer

                self.tokenizer = Tokenizer.from_file(tok)
            except Exception:  # a missing package only disables text prompts
                self.tokenizer = None

    def _ids(self, prompt: Union[str, Sequence[int]]) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ConfigError("text prompts need a tokenizer.json in the model folder; "
                                  "pass lists of token ids instead")
            return list(self.tokenizer.encode(prompt).ids)
        return [int(t) for t in prompt]

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams]]) -> List[Dict[str, Any]]:
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ConfigError("one SamplingParams per prompt, or a single one for all")
        status = StatusLine(self.config.decode_log_interval) if self.config.decode_log_interval > 0 else None
        sched = Scheduler(self.engine, self.sampler, self.eos_token_ids, status=status)
        for i, (p, sp) in enumerate(zip(prompts, sampling_params)):
            sched.add_request(self._ids(p), sp, rid=i)
        off = os.environ.get("FREETOKEN_DISABLE_OVERLAP_SCHEDULING", "").lower() in ("1", "true", "yes", "on")
        sched.run(overlap=self.config.overlap_scheduling and not off)
        self.engine.check_kernels()
        results = []
        for i in range(len(prompts)):
            req = sched.done[i]
            ids = list(req.output)
            if req.finish_reason == "stop" and ids and ids[-1] in sched.eos:
                ids = ids[:-1]
            text = self.tokenizer.decode(ids) if self.tokenizer is not None else ""
            item = {"text": text, "token_ids": ids, "finish_reason": req.finish_reason}
            if req.error:
                item["error"] = req.error
            results.append(item)
        return results
