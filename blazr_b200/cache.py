"""Cache and state bookkeeping of the serving engine (host side, no GPU): KV pages and recurrent-state slots.

The reference keeps a block allocator + per-sequence block tables for paged attention (src/engine/batch_engine.rs, block_size 16,
src/config/inference.rs:94-98).  Layer-list models with recurrent layers need a second resource: one state slot per live request
(convolution tails, state-space matrices, element-wise recurrent states), handed out on admission and returned on release; the
request's last token is kept beside it for embeddings that hash neighbouring tokens.  Pages and slots are reused; a new
request never sees what the previous owner left because a sequence at position 0 reads its carried state as zero and its pages
are written before they are read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List


class CacheFull(RuntimeError):
    pass


class PagePool:
    """free list of KV pages (last freed, first reused: recycled pages turn up early and out of order)"""

    def __init__(self, num_blocks: int, block_size: int):
        assert num_blocks >= 0 and block_size >= 1
        self.num_blocks, self.block_size = num_blocks, block_size
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} KV pages wanted, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        return out

    def free(self, blocks: List[int]) -> None:
        for b in blocks:
            assert 0 <= b < self.num_blocks and b not in self._free
            self._free.append(b)


class SlotPool:
    def __init__(self, n: int):
        self.n = n
        self._free: List[int] = list(range(n - 1, -1, -1))

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n} state slots are in use")
        return self._free.pop()

    def free(self, s: int) -> None:
        assert 0 <= s < self.n and s not in self._free
        self._free.append(s)


@dataclass
class SeqState:
    """what one live request holds"""
    rid: str
    slot: int
    blocks: List[int] = field(default_factory=list)
    n_tokens: int = 0          # tokens already in the cache / folded into the state
    last_token: int = -1       # the last token fed (state of embeddings that hash the previous token with the current one)


class CacheManager:
    """pages for `max_tokens` tokens in all and `max_seqs` state slots"""

    def __init__(self, max_tokens: int, max_seqs: int, block_size: int = 16):
        self.block_size = block_size
        # every live request may hold one partly filled page
        self.pages = PagePool(-(-max_tokens // block_size) + max_seqs, block_size)
        self.slots = SlotPool(max_seqs)
        self.live: Dict[str, SeqState] = {}

    def admit(self, rid: str) -> SeqState:
        if rid in self.live:
            raise ValueError(f"request {rid} is already live")
        s = SeqState(rid, self.slots.alloc())
        self.live[rid] = s
        return s

    def can_admit(self) -> bool:
        return self.slots.free_slots > 0

    def pages_needed(self, seq: SeqState, n_new: int) -> int:
        return max(0, -(-(seq.n_tokens + n_new) // self.block_size) - len(seq.blocks))

    def reserve(self, seq: SeqState, n_new: int) -> None:
        """make room for n_new more tokens of this request"""
        seq.blocks += self.pages.alloc(self.pages_needed(seq, n_new))

    def release(self, rid: str) -> None:
        s = self.live.pop(rid)
        self.pages.free(s.blocks)
        self.slots.free(s.slot)
        s.blocks = []
