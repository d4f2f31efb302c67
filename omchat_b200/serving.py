"""Continuous batching over the paged KV cache (the reference has no serving loop - cli.py serves one
request at a time through generate()).

A fixed number of decode SLOTS share one page pool: up to 4 slots decode with the persistent kernel (one launch per token
for all slots), 5..64 slots with the batched step on the weight-streaming GEMMs (csrc/gemm_stream.cu; one CUDA graph
replay per token). A request is admitted into a free slot as soon as one exists: its prompt is spliced (image features in place of the
-200 placeholders, omchat_arch.py:115-195) and prefilled into pages taken from a free list, its first token is sampled from
the prefill logits, and from the next step on it decodes together with whatever the other slots hold. A finished request
(EOS or max_new_tokens) gives its pages back and frees its slot at the next chunk boundary. Idle slots point at one
scratch page and are reset every chunk, so the kernel always runs the same batch shape.

Every request produces exactly the tokens a stand-alone greedy generate() of the same prompt produces (up to bf16-level
near-ties: the split of the keys over CTAs depends on the batch size) - tests/test_serving_gpu.py checks that against the
oracle.

`StepScheduler` is the token-level loop for models that expose `step()` over (slot, position)-addressed rows (model/voduzen.py,
model/tifisun.py):
every step is ONE packed batch in which portions of prompts run beside the single decode rows of other requests; pages are
taken one by one as a request grows and go back to the free list when it ends, slots likewise.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from . import lib
from .model.decoder import PagedKVCache
from .model.paged_cache import PageAllocator

MAX_SLOTS = 64  # rows of the batched decode step (csrc/gemm_stream.cu)


@dataclass
class _Request:
    rid: int
    input_ids: torch.Tensor          # [1, S] int64 with -200 placeholders
    images: Optional[torch.Tensor]   # [n, 3, S, S] or None
    max_new: int
    eos: Optional[int]
    out: List[int] = field(default_factory=list)
    pages: List[int] = field(default_factory=list)
    done: bool = False


class ContinuousBatcher:
    """model: OmChatQwen2ForCausalLM (single GPU). slots: decode batch (1..64). max_ctx: longest prompt + generation a slot
    can hold. total_pages: size of the shared page pool (default: enough for every slot at max_ctx). chunk: decode steps
    between two looks at the host side (admission, EOS, release)."""

    def __init__(self, model, slots: int = 4, max_ctx: int = 4096, total_pages: Optional[int] = None, chunk: int = 8):
        if not 1 <= slots <= MAX_SLOTS:
            raise ValueError(f"slots must be 1..{MAX_SLOTS}")
        self.model, self.dec = model, model.model.decoder
        self.slots, self.chunk = slots, chunk
        ps = model.config.kv_page_size
        # one page more per slot than max_ctx needs: the pool then holds every slot at full length PLUS the scratch page
        self.cache: PagedKVCache = self.dec.new_cache(slots, max_ctx + ps, shuffle_pages=False)
        self.max_pages = self.cache.max_pages
        n_pool = self.cache.pool.shape[1]
        total = n_pool if total_pages is None else min(total_pages, n_pool)
        if total < 2:
            raise ValueError("the page pool needs at least a scratch page and one data page")
        # page 0 = scratch page of the idle slots; the others are handed out from a free list (LIFO: freed pages are
        # reused first, so block tables become non-contiguous as soon as requests of different lengths come and go)
        self.scratch = 0
        self.pages = PageAllocator(total - 1, first=1)
        self.page_size = ps
        self.table_host = torch.zeros(slots, self.max_pages, dtype=torch.int32)
        self.cache.block_table.copy_(self.table_host)
        self.cache.host_lens = [0] * slots
        self.cache.ctx_lens.zero_()
        self.active: List[Optional[_Request]] = [None] * slots
        self.cur = torch.zeros(slots, device=model.device, dtype=torch.int64)  # token each slot feeds next
        self.queue: deque = deque()
        self.results: Dict[int, torch.Tensor] = {}
        self._next_id = 0
        self.steps_run = 0

    @property
    def free_pages(self) -> List[int]:
        """Page ids currently free (the allocator's list, most recently freed last)."""
        return self.pages._free

    # ------------------------------------------------------------------------------------------------ public
    def submit(self, input_ids: torch.Tensor, images: Optional[torch.Tensor] = None, max_new_tokens: int = 64,
               eos_token_id: Optional[int] = None) -> int:
        """Queue one request ([1, S] or [S] ids with -200 where an image goes). Returns its id."""
        ids = input_ids.view(1, -1).to(torch.int64).cpu()
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        rid = self._next_id
        self._next_id += 1
        eos = eos_token_id if eos_token_id is not None and eos_token_id >= 0 else None
        self.queue.append(_Request(rid, ids, images, max_new_tokens, eos))
        return rid

    def run(self) -> Dict[int, torch.Tensor]:
        """Serve until the queue and the slots are empty. Returns {request id: generated ids (LongTensor)}."""
        while self.queue or any(r is not None for r in self.active):
            self.step()
        return self.results

    @torch.no_grad()
    def step(self):
        """Admit what fits, then one chunk of decode steps for all slots, then retire what finished."""
        self._admit()
        live = [r for r in self.active if r is not None]
        if not live:
            if self.queue:
                raise RuntimeError("a queued request does not fit the page pool even when it is empty")
            return
        n = min(self.chunk, min(r.max_new - len(r.out) for r in live))
        if n > 0:
            toks = self.dec.generate_greedy(self.cur, self.cache, n).cpu()  # [slots, n]
            self.steps_run += n
            self.cur = toks[:, -1].to(self.model.device)
            for s, r in enumerate(self.active):
                if r is None:
                    continue
                for t in toks[s].tolist():
                    r.out.append(t)
                    if (r.eos is not None and t == r.eos) or len(r.out) >= r.max_new:
                        r.done = True
                        break
        self._retire()

    # ------------------------------------------------------------------------------------------------ internals
    def _admit(self):
        for s in range(self.slots):
            if self.active[s] is not None or not self.queue:
                continue
            r: _Request = self.queue[0]
            embeds, pos, seq, offsets = self.model._splice_packed(r.input_ids.to(self.model.device), None, r.images)
            T = offsets[-1]
            need = (T + r.max_new + self.page_size - 1) // self.page_size
            if need > self.max_pages:
                raise ValueError(f"request {r.rid}: {T} prompt + {r.max_new} new tokens exceed the slot capacity")
            if need > self.pages.available():
                break  # wait for pages (FIFO admission: later requests do not overtake)
            self.queue.popleft()
            r.pages = self.pages.take(need)
            self.table_host[s].fill_(self.scratch)
            self.table_host[s, :need] = torch.tensor(r.pages, dtype=torch.int32)
            self.cache.block_table.copy_(self.table_host)
            seq.fill_(s)  # the packed rows of this request belong to cache row s
            logits = self.dec.prefill(embeds, pos, seq, offsets, self.cache, logits="last", slots=[s])
            first = lib.argmax(logits)
            t0 = int(first[0])
            r.out.append(t0)
            if (r.eos is not None and t0 == r.eos) or r.max_new == 1:
                r.done = True
            self.cur[s] = first[0]
            self.active[s] = r
        self._retire()

    def _retire(self):
        changed = False
        for s, r in enumerate(self.active):
            if r is not None and r.done:
                self.results[r.rid] = torch.tensor(r.out, dtype=torch.int64)
                self.pages.give(r.pages)
                r.pages = []
                self.active[s] = None
                self.table_host[s].fill_(self.scratch)
                changed = True
        # idle slots: scratch page, context 0 (the kernel still runs them: it appends to the scratch page and its
        # samples are ignored); live slots keep their lengths
        for s, r in enumerate(self.active):
            if r is None and self.cache.host_lens[s] != 0:
                self.cache.host_lens[s] = 0
                changed = True
        if changed:
            self.cache.block_table.copy_(self.table_host)
            self.cache.ctx_lens.copy_(torch.tensor(self.cache.host_lens, dtype=torch.int32))
            self.cur = torch.where(torch.tensor([r is not None for r in self.active], device=self.cur.device), self.cur,
                                   torch.zeros_like(self.cur))


# ---------------------------------------------------------------------------------------------------------------------------
@dataclass
class _Live:
    """A request that holds a slot: `length` tokens of it are in the cache, on `pages`."""
    slot: int
    length: int = 0
    pages: List[int] = field(default_factory=list)


@dataclass
class _GenRequest:
    rid: int
    prompt: List[int]
    max_new: int
    eos: Optional[int]
    fed: int = 0                     # prompt tokens already given to a step
    out: List[int] = field(default_factory=list)
    key: str = ""


class StepScheduler:
    """Token-level continuous batching over a PagedLatentCache (or a PagedStateCache: the slot a request holds is also where its
    recurrent states live; the model's kernels start from zero at position 0, so nothing is cleared when a slot changes hands).

    model: exposes `decoder.new_cache(n_pages, n_slots)`, `config.kv_page_size` and
    `step(tokens, pos, slot, cache, want_rows) -> fp32 logits`. max_tokens: the most tokens live requests hold at any time,
    each request rounded up to whole pages - the pool has exactly that many pages (plus the scratch page idle table entries
    point at), so pages are reused as requests come and go. slots: requests live at the same time.

    Two levels: `run_step(entries, end)` executes one given batch (trace replay; also what `run()` is built on), and
    `submit()` / `run()` is greedy generation with chunked prefill: every iteration feeds each prefilling request its next
    `chunk` tokens and each generating request its last sampled token, all in one batch."""

    def __init__(self, model, max_tokens: int, slots: int = 4, chunk: int = 512):
        self.model = model
        self.page_size = ps = model.config.kv_page_size
        n_pages = max(1, -(-max_tokens // ps))
        self.cache = model.decoder.new_cache(n_pages + 1, slots)   # page 0: scratch
        self.pages = PageAllocator(n_pages, first=1)
        self.free_slots: List[int] = list(range(slots - 1, -1, -1))
        self.live: Dict[str, _Live] = {}
        self.chunk = chunk
        self.queue: deque = deque()
        self.results: Dict[int, List[int]] = {}
        self._gen: Dict[str, _GenRequest] = {}
        self._pinned = None   # host staging of a decode-only step's (tokens, positions, slots)
        self._pin_event = None
        self._next_id = 0
        self.steps_run = 0

    # ------------------------------------------------------------------------------------------------ one given batch
    def _admit(self, key: str) -> _Live:
        if not self.free_slots:
            raise RuntimeError(f"no free slot for request {key!r}: {len(self.live)} requests are live")
        r = _Live(slot=self.free_slots.pop())
        self.cache.clear_slot(r.slot)
        self.live[key] = r
        return r

    def _grow(self, r: _Live, n: int):
        have = len(r.pages)
        need = -(-(r.length + n) // self.page_size)
        if need > self.cache.max_pages:
            raise RuntimeError("request longer than a slot can hold")
        if need > have:
            new = self.pages.take(need - have)
            self.cache.set_pages(r.slot, have, new)
            r.pages += new

    def release(self, key: str):
        """The request's pages and slot go back to the free lists (its cache rows are simply overwritten later)."""
        r = self.live.pop(key, None)
        if r is None:
            return
        self.pages.give(r.pages)
        self.cache.clear_slot(r.slot)
        self.free_slots.append(r.slot)

    @torch.no_grad()
    def run_step(self, entries, end=()) -> Optional[torch.Tensor]:
        """entries: [(request key, token ids, wanted offsets among these tokens)]; a key seen for the first time is admitted.
        Runs them as one batch and returns fp32 logits [total wanted, vocab] in the order of the entries (None if nothing is
        wanted); then releases the requests named in `end`."""
        toks: List[int] = []
        pos: List[int] = []
        slot: List[int] = []
        want: List[int] = []
        portions = []
        for key, ids, wanted in entries:
            ids = list(ids)
            if not ids:
                continue
            r = self.live.get(key) or self._admit(key)
            self._grow(r, len(ids))
            base = len(toks)
            portions.append((base, len(ids), r.slot, r.length))
            toks += ids
            pos += range(r.length, r.length + len(ids))
            slot += [r.slot] * len(ids)
            want += [base + int(o) for o in wanted]
            r.length += len(ids)
            self.cache.host_lens[r.slot] = r.length
        logits = None
        if toks:
            dev = self.model.device
            self.cache.sync()
            meta = torch.tensor([toks, pos, slot], dtype=torch.int32)
            decode_only = all(n == 1 for _, n, _, _ in portions) and hasattr(self.model, "decode_step")
            if decode_only and torch.device(dev).type == "cuda":
                # one token per request: the model's captured decode step (CUDA graph) computes the logits of every row
                if self._pin_event is not None:
                    self._pin_event.synchronize()      # the previous step's copy out of the staging buffer has been done
                if self._pinned is None or self._pinned.shape[1] != len(toks):
                    self._pinned = torch.empty(3, len(toks), dtype=torch.int32).pin_memory()
                self._pinned.copy_(meta)
                logits = self.model.decode_step(self._pinned, self.cache, max(pos) + 1)
                self._pin_event = torch.cuda.Event()
                self._pin_event.record()
                if len(want) != len(toks):
                    logits = logits[torch.tensor(want, dtype=torch.int64).to(dev)] if want else None
            else:
                if torch.device(dev).type == "cuda":
                    meta = meta.pin_memory().to(dev, non_blocking=True)
                wr = torch.tensor(want, dtype=torch.int64).to(dev) if want else None
                logits = self.model.step(meta[0], meta[1], meta[2], self.cache, wr, portions=portions)
            self.steps_run += 1
        for key in end:
            self.release(key)
        return logits

    # ------------------------------------------------------------------------------------------------ greedy generation
    def submit(self, prompt: Sequence[int], max_new_tokens: int = 32, eos_token_id: Optional[int] = None) -> int:
        if max_new_tokens < 1 or len(prompt) < 1:
            raise ValueError("a request needs at least one prompt token and max_new_tokens >= 1")
        rid = self._next_id
        self._next_id += 1
        eos = eos_token_id if eos_token_id is not None and eos_token_id >= 0 else None
        self.queue.append(_GenRequest(rid, [int(t) for t in prompt], max_new_tokens, eos, key=f"g{rid}"))
        return rid

    def _pages_for(self, g: _GenRequest) -> int:
        return -(-(len(g.prompt) + g.max_new) // self.page_size)

    def run(self) -> Dict[int, List[int]]:
        """Serve until the queue and the slots are empty. Returns {request id: generated ids}."""
        while self.queue or self._gen:
            # admission: a free slot, and pages for the whole request once the promises to the running ones are kept
            while self.queue and self.free_slots:
                g = self.queue[0]
                promised = sum(self._pages_for(x) - len(self.live[x.key].pages) if x.key in self.live else self._pages_for(x)
                               for x in self._gen.values())
                if self._pages_for(g) > self.cache.max_pages:
                    raise ValueError(f"request {g.rid} does not fit the page pool even when it is empty")
                if self._pages_for(g) + promised > self.pages.available():
                    break
                self.queue.popleft()
                self._gen[g.key] = g
                self._admit(g.key)
            if not self._gen:
                raise RuntimeError("a queued request cannot be admitted although nothing is running")
            entries, order = [], []
            for g in self._gen.values():
                if g.fed < len(g.prompt):
                    part = g.prompt[g.fed:g.fed + self.chunk]
                    g.fed += len(part)
                    entries.append((g.key, part, [len(part) - 1] if g.fed == len(g.prompt) else []))
                    if g.fed == len(g.prompt):
                        order.append(g)
                else:
                    entries.append((g.key, [g.out[-1]], [0]))
                    order.append(g)
            logits = self.run_step(entries)
            done = []
            if order:
                nxt = lib.argmax(logits).tolist()          # greedy: lowest index on ties
                for g, t in zip(order, nxt):
                    g.out.append(int(t))
                    if (g.eos is not None and t == g.eos) or len(g.out) >= g.max_new:
                        done.append(g)
            for g in done:
                self.results[g.rid] = g.out
                del self._gen[g.key]
                self.release(g.key)
        return self.results
