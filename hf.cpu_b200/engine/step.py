"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere, runs only the
tokens it is given as one flat batch, and returns float32 logits at the wanted places.  The
reference's forward takes either one sequence of n consecutive tokens or n sequences of one
token, never both (src/model.c:542-545), reserves cache blocks before any compute
(src/model.c:555-564) and advances the position only after the layers ran (src/model.c:626-627);
the same order holds here: reserve, run, advance.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import KVCacheManager, OutOfPages, StateSlots
from ..models import Model


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits are wanted."""
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class GroupMeta:
    """What kernels need to find one cache group's pages for this step's tokens."""
    __slots__ = ("group", "slots", "block_table", "block_size", "max_blocks")

    def __init__(self, group, slots, block_table, block_size, max_blocks):
        self.group, self.slots, self.block_table = group, slots, block_table
        self.block_size, self.max_blocks = block_size, max_blocks


class Workspace:
    """Named scratch buffers that live across steps (a buffer grows when a larger one is asked for)."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}  # (name, dtype, shape) -> the view handed out (asked for at every call of every step)
        self._retired: List[torch.Tensor] = []      # outgrown buffers stay alive: captured graphs may point at them

    def get(self, name, shape, dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        vkey = (name, dtype, shape)
        v = self._views.get(vkey)
        if v is not None:
            return v
        n = 1
        for s in shape:
            n *= s
        key = (name, dtype)
        b = self._bufs.get(key)
        if b is None or b.numel() < n:
            if b is not None:
                self._retired.append(b)
                self._views = {k: w for k, w in self._views.items() if k[:2] != key}      # they showed the old buffer
            b = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = b
        if len(self._views) > 4096:
            self._views.clear()
        v = self._views[vkey] = b[:n].view(*shape)
        return v


@dataclass
class StepBatch:
    """The host's view of a step, handed to the mixers that build index arrays of their own for it."""
    q_lens: List[int]                  # tokens each request brings
    kv_lens: List[int]                 # tokens each request holds after the step
    starts: List[int]                  # position of each request's first token of the step
    block_size: int

    @property
    def num_seqs(self) -> int:
        return len(self.q_lens)

    @property
    def num_tokens(self) -> int:
        return sum(self.q_lens)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens)


class StepContext:
    """Per-step batch description handed to every part."""

    def __init__(self, engine: "Engine"):
        self.engine = engine
        self.run_dtype = engine.model.run_dtype
        self.device = engine.device
        self.num_tokens = self.num_seqs = self.num_logit_rows = 0
        self.logits_for_all = False
        self.max_q_len = self.max_kv_len = 0
        self.token_ids = self.positions = self.token_seq = None
        self.cu_tokens = self.kv_lens = self.seq_slots = self.logit_rows = None
        self.h_cu_tokens: List[int] = []
        self.h_kv_lens: List[int] = []
        self.h_seq_slots: List[int] = []
        self._groups: List[GroupMeta] = []
        self._arrays: Dict[Hashable, Dict[str, torch.Tensor]] = {}

    def buf(self, name, shape, dtype) -> torch.Tensor:
        return self.engine.workspace.get(name, shape, dtype)

    def group_meta(self, group: int) -> GroupMeta:
        return self._groups[group]

    def entry_cache(self, entry: int):
        return self.engine.cache.entry_cache(entry)

    def entry_state(self, entry: int):
        return self.engine.slots.entry_state(entry)

    def arrays(self, key: Hashable) -> Dict[str, torch.Tensor]:
        """The int32 device arrays a mixer asked for under ``key`` (``Mixer.step_arrays``), by name."""
        return self._arrays.get(key, {})


class Engine:
    """Model + cache + slots + the step function.

    ``num_pages`` pages of ``block_size`` tokens are made for every cache group.  ``ctx_max`` bounds
    one request's length; ``max_requests`` bounds how many are live at once.
    """

    def __init__(self, model: Model, *, block_size: int = 16, num_pages: int = 0, max_tokens: int = 0,
                 max_requests: int = 64, ctx_max: int = 0):
        if not model.bound:
            raise ValueError("the model has no weights bound")
        self.model, self.device = model, model.device
        plan = model.plan
        self.ctx_max = int(ctx_max) if ctx_max else plan.max_positions
        if self.ctx_max > plan.max_positions:
            raise ValueError(f"ctx_max {self.ctx_max} exceeds the model's {plan.max_positions} positions")
        if not num_pages:
            if not max_tokens:
                raise ValueError("give num_pages or max_tokens")
            num_pages = (int(max_tokens) + block_size - 1) // block_size
        self.block_size, self.num_pages, self.max_requests = int(block_size), int(num_pages), int(max_requests)
        self.max_blocks = (self.ctx_max + block_size - 1) // block_size
        cache_specs, state_specs = {}, {}
        for i, e in enumerate(plan.schedule):
            mixer = model.layers[e.layer].mixer
            if e.cache_of is None and mixer.cache_spec() is not None:
                cache_specs[i] = mixer.cache_spec()
            if mixer.state_spec() is not None:
                state_specs[i] = mixer.state_spec()
        for i, e in enumerate(plan.schedule):
            if e.cache_of is not None and e.cache_of not in cache_specs:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which keeps none")
        # index arrays the mixers want built per step (tile lists of their kernels and the like): one owner per key,
        # so that layers with the same needs share one set
        self._array_owners: Dict[Hashable, object] = {}
        for l in model.layers:
            key = l.mixer.step_arrays_key()
            if key is not None:
                self._array_owners.setdefault(key, l.mixer)
        self.cache = KVCacheManager(cache_specs, self.block_size, self.num_pages, model.run_dtype,
                                    self.device, self.max_blocks)
        self.slots = StateSlots(state_specs, self.max_requests, self.device)
        self.workspace = Workspace(self.device)
        self._pinned = self.device.type == "cuda"
        # pure decode steps are captured once per (batch size, key-split bucket) as a CUDA graph and replayed
        self.use_graphs = (self._pinned and os.environ.get("HFB_GRAPHS", "1") != "0"
                           and all(getattr(p, "graph_safe", False) for p in model.all_parts()))
        self._graphs: Dict[tuple, tuple] = {}
        self._static_meta: Dict[int, torch.Tensor] = {}
        self._meta_ring = []            # [host buffer, device buffer, event of its last copy]
        self._meta_next = 0
        self.steps_run = 0

    # ---- requests -----------------------------------------------------------------------------
    def add_request(self, req: Hashable) -> int:
        slot = self.slots.acquire(req)
        self.cache.add(req)
        return slot

    def fork_request(self, src: Hashable, dst: Hashable, n_tokens: int) -> int:
        """``dst`` (just added) starts on the cache pages of ``src``'s first ``n_tokens`` tokens, which must be
        the same tokens; returns how many tokens ``dst`` holds afterwards.  0 when some mixer keeps state of fixed
        size per request: its state behind the shared tokens is not to be had from ``src``, which has moved on."""
        if not self.can_fork:
            return 0
        return self.cache.fork(src, dst, n_tokens)

    @property
    def can_fork(self) -> bool:
        return not self.slots.tensors

    def finish_request(self, req: Hashable) -> None:
        self.cache.release(req)
        self.slots.release(req)

    def has_request(self, req) -> bool:
        return req in self.slots.slot_of

    def length(self, req) -> int:
        return self.cache.length(req)

    def live_requests(self):
        return list(self.slots.slot_of)

    # ---- the step -----------------------------------------------------------------------------
    def _meta_buffers(self, n: int):
        """A pinned host buffer and its device twin from a small ring: a host buffer is rewritten only
        after the copy that last read it has finished, and the device twin only after the steps that
        read it were queued behind it on the same stream."""
        if len(self._meta_ring) < 4:
            self._meta_ring.append([None, None, None])
        slot = self._meta_ring[self._meta_next % len(self._meta_ring)]
        self._meta_next += 1
        if slot[2] is not None:
            slot[2].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            cap = max(n, 4096) * 2
            slot[0] = torch.empty(cap, dtype=torch.int32, pin_memory=self._pinned)
            slot[1] = torch.empty(cap, dtype=torch.int32, device=self.device)
        return slot

    def prepare(self, entries: Sequence[StepEntry], static: bool = False) -> StepContext:
        """Check the entries, reserve their pages (all or nothing) and build the step's batch arrays.  With
        ``static`` the arrays have a layout and device addresses that depend on the number of entries only
        (block tables at full width, one device buffer per entry count), as graph replay needs."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        V = self.model.plan.vocab_size
        seen = set()
        for e in entries:
            if e.req in seen:
                raise ValueError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            if not self.has_request(e.req):
                raise KeyError(f"request {e.req!r} is not live")
            if len(e.tokens) < 1:
                raise ValueError(f"request {e.req!r} brings no tokens")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise ValueError(f"token id {t} of request {e.req!r} is outside the vocabulary of {V}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.req!r} wants logits at place {w} of {len(e.tokens)} tokens")
            if self.cache.length(e.req) + len(e.tokens) > self.ctx_max:
                raise OutOfPages(f"request {e.req!r} would exceed the context limit of {self.ctx_max} tokens")
        wants = [(e.req, self.cache.length(e.req) + len(e.tokens)) for e in entries]
        if not self.cache.can_reserve(wants):
            raise OutOfPages(f"the step needs more pages than are free {self.cache.free_pages()}")
        for req, new_len in wants:
            self.cache.reserve(req, new_len)

        ctx = StepContext(self)
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        M = sum(len(e.want) for e in entries)
        groups = self.cache.groups
        bs = self.block_size
        starts = [self.cache.length(e.req) for e in entries]
        kv_lens = [w[1] for w in wants]
        max_q = max(q_lens)
        MB = self.max_blocks if static else max(1, (max(kv_lens) + bs - 1) // bs)
        batch = StepBatch(q_lens, kv_lens, starts, bs)
        extras = [(key, {n: np.ascontiguousarray(v, dtype=np.int32) for n, v in mixer.step_arrays(batch).items()})
                  for key, mixer in self._array_owners.items()]
        total = 3 * T + (S + 1) + 2 * S + M + len(groups) * (T + S * MB) + sum(len(v) for _, arrs in extras for v in arrs.values())
        # one flat int32 buffer, filled through its numpy view: a single host-to-device copy per step
        ring_slot = self._meta_buffers(total)
        h, d = ring_slot[0], ring_slot[1]
        if static:
            d = self._static_meta.get(S)
            if d is None or d.numel() < total:
                d = self._static_meta[S] = torch.empty(total, dtype=torch.int32, device=self.device)
        hn = h.numpy()
        cu = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        if max_q == 1:
            tok = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=S)
            pos = np.asarray(starts, dtype=np.int32)
            seq = np.arange(S, dtype=np.int32)
        else:
            tok = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
            pos = np.concatenate([np.arange(st, st + n, dtype=np.int32) for st, n in zip(starts, q_lens)])
            seq = np.repeat(np.arange(S, dtype=np.int32), q_lens)
        rows = [int(cu[s]) + int(w) for s, e in enumerate(entries) for w in e.want]
        seq_slots = [self.slots.slot_of[e.req] for e in entries]
        o = 0

        def put(arr):
            nonlocal o
            n = len(arr)
            hn[o:o + n] = arr
            o += n

        put(tok), put(pos), put(seq), put(cu), put(kv_lens), put(seq_slots), put(rows)
        for g in groups:
            tables = np.stack([g.np_tables[e.req][:MB] for e in entries])          # [S, MB]
            blk = pos // bs
            put(tables[seq, blk] * bs + pos % bs)                                  # cache slot of every token
            put(tables.reshape(-1))
        for _, arrs in extras:
            for v in arrs.values():
                put(v)
        assert o == total
        d[:total].copy_(h[:total], non_blocking=True)
        if self._pinned:
            ring_slot[2] = torch.cuda.Event()
            ring_slot[2].record()
        cu = cu.tolist()
        o = 0

        def take(n, shape=None):
            nonlocal o
            v = d[o:o + n]
            o += n
            return v if shape is None else v.view(*shape)

        ctx.token_ids, ctx.positions, ctx.token_seq = take(T), take(T), take(T)
        ctx.cu_tokens, ctx.kv_lens, ctx.seq_slots, ctx.logit_rows = take(S + 1), take(S), take(S), take(M)
        for g in groups:
            ctx._groups.append(GroupMeta(g.index, take(T), take(S * MB, (S, MB)), bs, MB))
        for key, arrs in extras:
            ctx._arrays[key] = {n: take(len(v)) for n, v in arrs.items()}
        ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows = T, S, M
        ctx.logits_for_all = rows == list(range(T))      # every token's logits, in order: the last block may run the final norm
        ctx.h_cu_tokens, ctx.h_kv_lens, ctx.h_seq_slots = cu, kv_lens, seq_slots
        ctx.max_q_len = max_q
        ctx.max_kv_len = max(kv_lens)
        # how finely decode attention may split a request's keys: a power of two, so that few graphs exist
        hint = max(1, ((ctx.max_kv_len + 63) // 64) // 2)
        ctx.decode_split_hint = 1 << (min(hint, 64).bit_length() - 1)
        return ctx

    def _replay(self, ctx: StepContext) -> torch.Tensor:
        """A decode step through its CUDA graph: the first step of a kind runs eagerly (it sizes the scratch
        buffers), the second is captured, later ones are replayed on the arrays ``prepare`` has just refreshed."""
        key = (ctx.num_seqs, ctx.decode_split_hint)
        state = self._graphs.get(key)
        if state is None:
            self._graphs[key] = ("warm", None, None)
            return self.model.forward(ctx)
        if state[0] == "warm":
            torch.cuda.synchronize(self.device)
            from .. import kernels
            backend = kernels.backend()
            before = getattr(backend, "launches", 0)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
            captured = getattr(backend, "launches", 0) - before        # kernels one replay launches
            self._graphs[key] = ("ready", graph, logits, captured)
            backend.launches = before
        state = self._graphs[key]
        state[1].replay()
        from .. import kernels
        backend = kernels.backend()
        if hasattr(backend, "launches"):
            backend.launches += state[3]
        return state[2]

    def step(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits ``[wanted, vocab]`` (device), in the order of the entries and
        of their ``want`` lists, or None when nothing is wanted.  The returned tensor is scratch that the
        next step overwrites.

        ``token_source`` (int32 on the device, one id per token of the step) replaces the entries' token ids:
        the ids a sampling kernel has just written can be fed back without the host having seen them."""
        entries = list(entries)
        from .. import kernels
        # (a step that is being profiled phase by phase runs kernel by kernel, not as a graph)
        graphable = (self.use_graphs and not kernels.profile.enabled
                     and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries))
        ctx = self.prepare(entries, static=graphable)
        if token_source is not None:
            if token_source.dtype != torch.int32 or token_source.numel() != ctx.num_tokens:
                raise ValueError("token_source must hold one int32 id per token of the step")
            ctx.token_ids[:ctx.num_tokens].copy_(token_source.reshape(-1), non_blocking=True)
        if graphable:
            logits = self._replay(ctx)
        else:
            logits = self.model.forward(ctx)
        for e in entries:
            self.cache.advance(e.req, self.cache.length(e.req) + len(e.tokens))
        self.steps_run += 1
        return logits
