"""Host-side builders of the batched-decode inputs and of flat mixed steps (pure Python, no GPU).

Mirror of reference src/engine/batch_decode.rs:59-131 (`process_decode_batch`): for every decoding sequence the
last token, the KV slot of the new token (`block * block_size + offset`, -1 when the block table is too short) and its
block table; the batch pads block tables with 0 to the longest one and reports the largest sequence length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np


@dataclass
class DecodeSeqData:
    """reference batch_decode.rs DecodeSeqData"""
    seq_id: int
    last_token: int
    slot: int
    block_table: List[int]
    seq_len: int


@dataclass
class DecodeBatch:
    seq_ids: List[int]
    input_ids: np.ndarray      # int64 [N, 1]
    slot_mapping: np.ndarray   # int32 [N]
    block_table: np.ndarray    # int32 [N, max_num_blocks], shorter tables padded with 0
    max_seq_len: int

    @property
    def position(self) -> int:
        """the `max_seq_len - 1` position argument of forward_with_paged_kv_cache (batch_decode.rs:146)"""
        return self.max_seq_len - 1


def decode_seq_data(seq_id: int, token_history: Sequence[int], blocks: Sequence[int], block_size: int) -> DecodeSeqData:
    """batch_decode.rs:76-98"""
    seq_len = len(token_history)
    last_token = token_history[-1] if seq_len else 0
    token_pos = seq_len - 1
    block_idx, block_offset = divmod(token_pos, block_size) if seq_len else (0, 0)
    slot = int(blocks[block_idx]) * block_size + block_offset if 0 <= block_idx < len(blocks) and seq_len else -1
    return DecodeSeqData(seq_id, int(last_token), int(slot), [int(b) for b in blocks], seq_len)


def build_decode_batch(decode_seqs: Sequence[int], token_histories: Dict[int, Sequence[int]], block_tables: Dict[int, Sequence[int]],
                       block_size: int, serviceable: Optional[Dict[int, bool]] = None) -> Optional[DecodeBatch]:
    """batch_decode.rs:59-131: sequences missing a token history, a block table or a generation config are skipped;
    returns None when nothing is left (the reference returns Ok(()) without a forward pass)."""
    data: List[DecodeSeqData] = []
    for sid in decode_seqs:
        hist = token_histories.get(sid)
        blocks = block_tables.get(sid)
        if hist is None or blocks is None:
            continue
        if serviceable is not None and not serviceable.get(sid, False):
            continue
        data.append(decode_seq_data(sid, hist, blocks, block_size))
    if not data:
        return None
    n = len(data)
    max_blocks = max(len(s.block_table) for s in data)
    bt = np.zeros((n, max_blocks), dtype=np.int32)
    for i, s in enumerate(data):
        bt[i, :len(s.block_table)] = s.block_table
    return DecodeBatch([s.seq_id for s in data], np.asarray([[s.last_token] for s in data], dtype=np.int64),
                       np.asarray([s.slot for s in data], dtype=np.int32), bt, max(s.seq_len for s in data))


# ------------------------------------------------------------------------------------------------------------------------------
# flat mixed steps: prompt portions beside single decoded tokens (the chunked-prefill batches of reference
# src/engine/batch_engine.rs:172-272 and the decode batches above, as one token list)
# ------------------------------------------------------------------------------------------------------------------------------
@dataclass
class StepEntry:
    """the next tokens of one request"""
    tokens: Sequence[int]
    pos0: int                   # position of tokens[0] in its sequence
    slot: int                   # recurrent-state slot of the request
    block_table: Sequence[int]  # KV pages of the request (must cover pos0 + len(tokens) positions)
    want: Sequence[int] = ()    # indices into `tokens` whose logits are wanted
    prev: int = -1              # the request's last token before this portion (-1: none yet); models with a bigram embedding read it


@dataclass
class StepArrays:
    """int32 arrays of one step (include/b200seq.h: b200seq_step), host side"""
    tok_ids: np.ndarray
    tok_ent: np.ndarray
    tok_pos: np.ndarray
    ent_start: np.ndarray
    ent_slot: np.ndarray
    ent_pos0: np.ndarray
    block_table: np.ndarray    # [B, max_blocks]
    want_rows: np.ndarray      # token rows whose logits are wanted, in entry order
    T: int
    B: int
    ent_prev: Optional[np.ndarray] = None   # the token before each entry's first one (carried per request; unused at position 0)

    @property
    def decode_only(self) -> bool:
        return self.T == self.B


def build_step(entries: Sequence[StepEntry], block_size: int, max_blocks: Optional[int] = None) -> StepArrays:
    B = len(entries)
    lens = [len(e.tokens) for e in entries]
    if any(n < 1 for n in lens):
        raise ValueError("an entry without tokens")
    T = int(sum(lens))
    need = [-(-(e.pos0 + n) // block_size) for e, n in zip(entries, lens)]
    for e, nb in zip(entries, need):
        if len(e.block_table) < nb:
            raise ValueError(f"block table of {len(e.block_table)} pages does not cover {nb} pages")
    mb = max(need) if max_blocks is None else max_blocks
    if mb < max(need):
        raise ValueError("max_blocks too small for this step")
    start = np.zeros(B + 1, dtype=np.int32)
    start[1:] = np.cumsum(lens)
    bt = np.zeros((B, mb), dtype=np.int32)
    want: List[int] = []
    for i, (e, nb) in enumerate(zip(entries, need)):
        bt[i, :nb] = np.asarray(e.block_table[:nb], dtype=np.int32)
        for w in e.want:
            if not 0 <= w < lens[i]:
                raise ValueError("a wanted place outside its entry")
            want.append(int(start[i]) + int(w))
    return StepArrays(
        tok_ids=np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries]) if B else np.zeros(0, np.int32),
        tok_ent=np.repeat(np.arange(B, dtype=np.int32), lens),
        tok_pos=np.concatenate([np.arange(e.pos0, e.pos0 + n, dtype=np.int32) for e, n in zip(entries, lens)]) if B else np.zeros(0, np.int32),
        ent_start=start, ent_slot=np.asarray([e.slot for e in entries], dtype=np.int32),
        ent_pos0=np.asarray([e.pos0 for e in entries], dtype=np.int32), block_table=bt, want_rows=np.asarray(want, dtype=np.int32), T=T, B=B,
        ent_prev=np.asarray([max(int(e.prev), 0) for e in entries], dtype=np.int32))
