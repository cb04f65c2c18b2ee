"""Serving engine of layer-list models: request queue, scheduler, cache / state manager, sampling.

One `Engine.step()` is one forward pass over a flat mixed batch: every running request contributes its one decoded token, and
prompts that are not yet in the cache contribute their next portion (chunked prefill under a token budget), as the reference's
batch engine does (src/engine/batch_engine.rs:172-272 chunked prefill, src/engine/batch_decode.rs:35-209 decode batches).
Requests take a state slot and KV pages from `CacheManager` (blazr_b200/cache.py) on admission / growth and give them back when
they finish; pages and slots are reused.

`Engine.run_entries()` is the same step with the batch given from outside (which request brings which tokens): trace replay and
the tests drive it; `step()` builds the same entries from its own queues.  Both go through `_forward`, the only place that
touches the model.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import seqops
from .batch import StepEntry, build_step
from .cache import CacheFull, CacheManager
from .layered import LayeredModel


@dataclass
class SamplingParams:
    """temperature 0 = greedy (arg-max kernel); otherwise soft-max sampling, optionally among the top_k / top_p tokens"""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: Optional[int] = None
    max_new_tokens: int = 16
    stop_tokens: Tuple[int, ...] = ()


@dataclass
class Request:
    rid: str
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    fed: int = 0                 # prompt tokens already in the cache
    finished: bool = False
    _gen: Optional[torch.Generator] = None


class Engine:
    def __init__(self, model: LayeredModel, max_tokens: int, max_seqs: int = 4, block_size: int = 16, max_step_tokens: int = 2048,
                 prefill_chunk: int = 512):
        """max_tokens: tokens all live requests may hold together (the KV pool is made for this many, rounded up to pages);
        max_seqs: state slots = most requests live at a time"""
        self.model = model
        self.cache = CacheManager(max_tokens, max_seqs, block_size)
        model.allocate(self.cache.pages.num_blocks, block_size, max_seqs, self.cache.pages.num_blocks * block_size)
        self.max_step_tokens, self.prefill_chunk = max_step_tokens, prefill_chunk
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[str, Request] = {}
        self.steps = 0

    # ---- the one place that runs the model -----------------------------------------------------------------------------------
    def _forward(self, batch: Sequence[Tuple[str, Sequence[int], Sequence[int]]], sample: bool = False) -> torch.Tensor:
        """batch: (request id, next tokens, wanted places) per entry.  Admits unseen ids, reserves pages, runs the step, advances
        the token counts.  Returns the f32 logits [wanted, vocab] (device; valid until the next step)."""
        entries: List[StepEntry] = []
        seen = set()
        for rid, toks, want in batch:
            if rid in seen:
                raise ValueError(f"request {rid} appears twice in one step")
            seen.add(rid)
            seq = self.cache.live.get(rid) or self.cache.admit(rid)
            self.cache.reserve(seq, len(toks))
            entries.append(StepEntry(tokens=toks, pos0=seq.n_tokens, slot=seq.slot, block_table=seq.blocks, want=want, prev=seq.last_token))
        sa = build_step(entries, self.cache.block_size)
        logits = self.model.forward(sa, sample=sample)
        for rid, toks, _ in batch:
            self.cache.live[rid].n_tokens += len(toks)
            self.cache.live[rid].last_token = int(toks[-1])
        self.steps += 1
        return logits

    def release(self, rid: str) -> None:
        if rid in self.cache.live:
            self.cache.release(rid)

    # ---- externally scheduled steps (trace replay) ----------------------------------------------------------------------------
    def run_entries(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        """entries: [{"id", "tokens", "want"}]; end: requests whose pages and slot are given back after the step.
        Returns the logits of the wanted places as a host array, or None when nothing was wanted."""
        out = None
        entries = [e for e in entries if len(e.get("tokens", ()))]      # an entry that brings no token has nothing to run
        if entries:
            logits = self._forward([(str(e["id"]), list(e["tokens"]), list(e.get("want", ()))) for e in entries])
            if logits.shape[0]:
                out = logits.cpu().numpy()
        for rid in end:
            self.release(str(rid))
        return out

    # ---- own scheduler ---------------------------------------------------------------------------------------------------------
    def add_request(self, rid: str, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        if rid in self.requests:
            raise ValueError(f"request id {rid} is in use")
        if not len(prompt):
            raise ValueError("empty prompt")
        r = Request(str(rid), [int(t) for t in prompt], params or SamplingParams())
        if r.params.temperature > 0:
            r._gen = torch.Generator(device=self.model.dev)
            r._gen.manual_seed(r.params.seed if r.params.seed is not None else 0)
        self.requests[r.rid] = r
        self.waiting.append(r)
        return r

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _schedule(self) -> List[Tuple[Request, List[int], List[int]]]:
        """decoded tokens of running requests first, then prompt portions while the token budget, the slots and the pages last"""
        plan: List[Tuple[Request, List[int], List[int]]] = []
        budget = self.max_step_tokens
        free_pages = self.cache.pages.free_blocks
        free_slots = self.cache.slots.free_slots
        for r in self.running:
            if r.fed < len(r.prompt):
                continue
            seq = self.cache.live[r.rid]
            need = self.cache.pages_needed(seq, 1)
            if budget < 1 or need > free_pages:
                continue
            plan.append((r, [r.output[-1]], [0]))
            budget -= 1
            free_pages -= need
        prefilling = [r for r in self.running if r.fed < len(r.prompt)]
        for r in prefilling + list(self.waiting):
            if budget < 1:
                break
            seq = self.cache.live.get(r.rid)
            if seq is None:
                if free_slots < 1:
                    break
                free_slots -= 1
            n = min(len(r.prompt) - r.fed, self.prefill_chunk, budget)
            have = len(seq.blocks) if seq else 0
            held = seq.n_tokens if seq else 0
            room = (have + free_pages) * self.cache.block_size - held
            n = min(n, room)
            if n < 1:
                if seq is None:
                    free_slots += 1
                break
            need = max(0, -(-(held + n) // self.cache.block_size) - have)
            free_pages -= need
            budget -= n
            last = r.fed + n == len(r.prompt)
            plan.append((r, r.prompt[r.fed:r.fed + n], [n - 1] if last else []))
        return plan

    def step(self) -> List[Request]:
        """one forward pass over what the scheduler picked; returns the requests that finished in it"""
        plan = self._schedule()
        if not plan:
            if self.has_work():
                raise CacheFull("no request can make progress: the KV pool is too small for the live requests")
            return []
        for r, _, _ in plan:
            if r in self.waiting:
                self.waiting.remove(r)
                self.running.append(r)
        greedy = all(r.params.temperature <= 0 for r, _, w in plan if w)
        logits = self._forward([(r.rid, toks, want) for r, toks, want in plan], sample=greedy)
        sampled = [r for r, _, w in plan if w]
        ids = self.model.last_ids.cpu().tolist() if (greedy and sampled) else None
        for r, toks, _ in plan:
            if r.fed < len(r.prompt):
                r.fed += len(toks)
        done: List[Request] = []
        for row, r in enumerate(sampled):
            tok = ids[row] if ids is not None else self._sample(logits[row], r)
            r.output.append(int(tok))
            if len(r.output) >= r.params.max_new_tokens or int(tok) in r.params.stop_tokens:
                r.finished = True
                done.append(r)
        for r in done:
            self.running.remove(r)
            self.release(r.rid)
        return done

    def _sample(self, logits: torch.Tensor, r: Request) -> int:
        p = r.params
        if p.temperature <= 0:
            ids = torch.empty(1, dtype=torch.int32, device=logits.device)
            seqops.argmax(logits.reshape(1, -1).contiguous(), ids)
            return int(ids.item())
        z = logits.float() / p.temperature
        if p.top_k and p.top_k < z.numel():
            kth = torch.topk(z, p.top_k).values[-1]
            z = torch.where(z < kth, torch.full_like(z, float("-inf")), z)
        pr = torch.softmax(z, 0)
        if p.top_p < 1.0:
            sp, si = torch.sort(pr, descending=True)
            keep = torch.cumsum(sp, 0) - sp < p.top_p
            pr = torch.zeros_like(pr).scatter(0, si[keep], sp[keep])
            pr = pr / pr.sum()
        return int(torch.multinomial(pr, 1, generator=r._gen).item())

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        """runs the prompts to completion through the scheduler (more prompts than slots queue up); returns the new tokens of each"""
        reqs = [self.add_request(f"g{self.steps}_{i}", p, params) for i, p in enumerate(prompts)]
        while any(not r.finished for r in reqs):
            self.step()
        flags = seqops.error_flags()
        if flags:
            raise RuntimeError(f"device error flags {flags:#x} (1: KV position outside its block table, 2: a bounded wait ran out, 4: expert table entry out of range)")
        for r in reqs:
            del self.requests[r.rid]
        return [r.output for r in reqs]
