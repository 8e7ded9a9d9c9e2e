"""The Python entry point: a resident session that loads a model once and generates from token ids.

Option names and meanings are the reference's (src/opts.c:30-76): ``ctx_max``, ``batch`` (prefill tokens per
step), ``temp``, ``top_k``, ``top_p``, ``min_p``, ``seed``, ``max_tokens``, ``n`` (completions decoded together, seeds
seed, seed+1, ...), ``logprobs``, ``timeout``.  The reference's programming interface is its C API
(src/model.h:49-79: load, context, forward); a session here plays the part of its resident model and
context (src/ops.c:468-482).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Union

import torch

from .engine import Engine, FinishEvent, Request, Scheduler, TokenEvent
from .models import Model, load_model
from .sampling import SamplingParams

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class Completion:
    tokens: List[int] = field(default_factory=list)
    stop: str = ""
    error: Optional[str] = None
    logprobs: List[float] = field(default_factory=list)
    top_logprobs: List[list] = field(default_factory=list)


class Session:
    def __init__(self, model: Union[str, Model], dtype: str = "bfloat16", device: str = "cuda:0", ctx_max: int = 0,
                 batch: int = 0, kv_block: int = 16, kv_pages: int = 0, kv_mem: int = 0, max_seqs: int = 64,
                 max_batched_tokens: int = 2048, eos_ids: Optional[Sequence[int]] = None):
        if isinstance(model, str):
            if dtype not in _DTYPES:
                raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
            model = load_model(model, _DTYPES[dtype], device)
        self.model = model
        ctx_max = min(ctx_max or model.plan.max_positions, model.plan.max_positions)
        if not kv_pages:
            kv_pages = self._default_pages(model, kv_block, kv_mem, max_seqs, ctx_max)
        self.engine = Engine(model, block_size=kv_block, num_pages=kv_pages, max_requests=max_seqs, ctx_max=ctx_max)
        self.scheduler = Scheduler(self.engine, max_num_seqs=max_seqs, max_num_batched_tokens=max_batched_tokens,
                                   prefill_chunk=batch)
        self.eos_ids = list(eos_ids) if eos_ids is not None else list(model.plan.eos_token_ids)
        self._serial = 0

    @staticmethod
    def _default_pages(model: Model, block: int, kv_mem: int, max_seqs: int, ctx_max: int) -> int:
        """Pages for every slot at full context, bounded by ``kv_mem`` bytes or by most of the free memory."""
        per_token = 0
        for i, e in enumerate(model.plan.schedule):
            spec = model.layers[e.layer].mixer.cache_spec()
            if e.cache_of is None and spec is not None:
                per_token += 2 * spec.num_kv_heads * spec.head_dim * (2 if model.run_dtype == torch.bfloat16 else 4)
        want = max_seqs * ((ctx_max + block - 1) // block)
        if model.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(model.device)
            limit = kv_mem or int(free * 0.8)
        else:
            limit = kv_mem or 1 << 30
        if per_token:
            want = min(want, max(1, limit // (per_token * block)))
        return max(want, 1)

    def generate(self, prompt_ids: Union[Sequence[int], Sequence[Sequence[int]]], *, temp: float = 0.8,
                 top_k: int = 40, top_p: float = 0.95, min_p: float = 0.05, seed: int = 0, max_tokens: int = 512,
                 n: int = 1, logprobs: int = 0, timeout: float = 0.0, eos_ids: Optional[Sequence[int]] = None,
                 on_event: Optional[Callable] = None, keep_cache: bool = False,
                 prefix_cache: bool = True) -> Union[List[Completion], List[List[Completion]]]:
        """Generate ``n`` completions for one prompt (a list of ids) or for each of several prompts.

        Returns a list of ``n`` completions for one prompt, or one such list per prompt.  All run together
        through the scheduler; requests with the same first tokens share the cache pages of those tokens.
        ``keep_cache`` keeps the pages of the last prompt's first completion after it has ended, so that the next
        call can start on them where its first tokens are the same (a conversation's next turn), which
        ``prefix_cache=False`` forbids.  ``on_event`` sees every TokenEvent / FinishEvent as it happens; event
        request ids are ``(serial, prompt index, sequence index)``."""
        single = len(prompt_ids) > 0 and not isinstance(prompt_ids[0], (list, tuple))
        prompts = [list(prompt_ids)] if single else [list(p) for p in prompt_ids]
        eos = list(eos_ids) if eos_ids is not None else self.eos_ids
        self._serial += 1
        results: Dict[tuple, Completion] = {}
        for pi, prompt in enumerate(prompts):
            for si in range(n):
                rid = (self._serial, pi, si)
                results[rid] = Completion()
                params = SamplingParams(temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, seed=seed + si,
                                        max_tokens=max_tokens, logprobs=logprobs)
                self.scheduler.submit(Request(rid, prompt, params, eos_ids=eos, timeout=timeout, reuse_cache=prefix_cache,
                                              keep_cache=keep_cache and si == 0 and pi == len(prompts) - 1))

        def handle(ev):
            c = results[ev.req]
            if isinstance(ev, TokenEvent):
                c.tokens.append(ev.token)
                if ev.logprob is not None:
                    c.logprobs.append(ev.logprob)
                    c.top_logprobs.append(ev.top)
            else:
                c.stop, c.error = ev.stop, ev.error
            if on_event:
                on_event(ev)
        try:
            self.scheduler.run(handle)
        except BaseException:
            # nothing of a failed call stays behind to be scheduled with the next one
            self.scheduler.abort(list(results))
            self.scheduler.drop_retained()
            raise
        out = [[results[(self._serial, pi, si)] for si in range(n)] for pi in range(len(prompts))]
        return out[0] if single else out


def generate(model: str, prompt_ids, dtype: str = "bfloat16", **options):
    """One-shot form: load ``model`` (a folder), generate, return the completions."""
    session_keys = ("device", "ctx_max", "batch", "kv_block", "kv_pages", "kv_mem", "max_seqs", "max_batched_tokens")
    sess = Session(model, dtype=dtype, **{k: options.pop(k) for k in session_keys if k in options})
    return sess.generate(prompt_ids, **options)
