"""CPU ORACLE for the integer side of the verify path — test infrastructure, not product code.

A plain-Python restatement of the reference's bookkeeping, each piece citing the code it follows
(paths inside ikematta/kiln). PINNED: the known-answer tests the reference keeps next to this code
(block.rs:428-688, drafter.rs:149-198, engine.rs:2798-2853) are ported in tests/test_bookkeeping.py and
run against both this module and the C++ host library.

  BlockManager / BlockTable     crates/kiln-engine/src/block.rs:88-426
  spec_gamma_at_width           crates/kiln-engine/src/drafter.rs:62-70
  canonical_prefill_len         crates/kiln-engine/src/engine.rs:167-179
  settle_walk                   crates/kiln-engine/src/engine.rs:2336-2366
  write_runs                    crates/kiln-engine/src/engine.rs:2757-2769
  round_gamma                   crates/kiln-engine/src/engine.rs:1515-1547
  should_stand_down             crates/kiln-engine/src/engine.rs:1616-1623
  gamma_bound                   crates/kiln-models/src/model.rs:239-252
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple


class BlockError(Exception):
    def __init__(self, kind: str, **info):
        super().__init__(f"{kind} {info}")
        self.kind = kind
        self.info = info

    def __eq__(self, other):
        return isinstance(other, BlockError) and (self.kind, self.info) == (other.kind, other.info)

    __hash__ = None


class BlockManager:
    """Fixed pool of KV blocks: allocation, refcounting, copy-on-write (block.rs:88-203)."""

    def __init__(self, capacity: int, block_size: int):
        if block_size == 0 or (block_size & (block_size - 1)) != 0:
            raise BlockError("InvalidBlockSize", size=block_size)          # block.rs:99-101
        if capacity == 0 or capacity > 0xFFFFFFFF:
            raise BlockError("InvalidCapacity", capacity=capacity)         # block.rs:102-106
        self.block_size = block_size
        self.refcounts = [0] * capacity
        self.free = list(range(capacity - 1, -1, -1))   # reversed so blocks are first issued 0, 1, 2, ... (block.rs:110-111)

    @property
    def capacity(self) -> int:
        return len(self.refcounts)

    @property
    def num_free(self) -> int:
        return len(self.free)

    def refcount(self, bid: int) -> Optional[int]:
        return self.refcounts[bid] if 0 <= bid < len(self.refcounts) else None

    def allocate(self) -> int:
        if not self.free:
            raise BlockError("OutOfBlocks", capacity=self.capacity, needed=1)
        bid = self.free.pop()
        self.refcounts[bid] = 1
        return bid

    def retain(self, bid: int) -> None:
        if self.refcount(bid) is None or self.refcounts[bid] == 0:
            raise BlockError("NotAllocated", id=bid)
        if self.refcounts[bid] == 0xFFFFFFFF:
            raise BlockError("RefcountOverflow", id=bid)
        self.refcounts[bid] += 1

    def release(self, bid: int) -> None:
        if self.refcount(bid) is None or self.refcounts[bid] == 0:
            raise BlockError("NotAllocated", id=bid)
        self.refcounts[bid] -= 1
        if self.refcounts[bid] == 0:
            self.free.append(bid)                        # LIFO (block.rs:167-169)

    def copy_on_write(self, bid: int) -> Tuple[str, int, int]:
        """('writable', id, id) or ('copied', src, dst) (block.rs:181-196)."""
        rc = self.refcount(bid)
        if rc is None or rc == 0:
            raise BlockError("NotAllocated", id=bid)
        if rc == 1:
            return ("writable", bid, bid)
        dst = self.allocate()            # first, so exhaustion leaves the pool untouched
        self.release(bid)
        return ("copied", bid, dst)


@dataclass
class AppendPlan:
    cow: Optional[Tuple[int, int]] = None     # (src, dst)
    appended: List[int] = field(default_factory=list)


class BlockTable:
    """Per-request map from token positions to pool blocks (block.rs:223-426)."""

    def __init__(self):
        self.blocks: List[int] = []
        self.num_tokens = 0

    def append_tokens(self, mgr: BlockManager, n: int) -> AppendPlan:
        if n == 0:
            return AppendPlan()
        bs = mgr.block_size
        new_total = self.num_tokens + n
        cow_src = None
        if self.num_tokens % bs != 0 and self.blocks:
            tail = self.blocks[-1]
            rc = mgr.refcount(tail)
            if rc is not None and rc > 1:
                cow_src = tail
        fresh = max(0, -(-new_total // bs) - len(self.blocks))
        needed = fresh + (1 if cow_src is not None else 0)
        if mgr.num_free < needed:                                         # atomic on failure (block.rs:282-287)
            raise BlockError("OutOfBlocks", capacity=mgr.capacity, needed=needed)
        plan = AppendPlan()
        if cow_src is not None:
            kind, src, dst = mgr.copy_on_write(cow_src)
            if kind == "copied":
                self.blocks[-1] = dst
                plan.cow = (src, dst)
        for _ in range(fresh):
            bid = mgr.allocate()
            self.blocks.append(bid)
            plan.appended.append(bid)
        self.num_tokens = new_total
        return plan

    def push_full_block(self, bid: int, block_size: int) -> None:
        if self.num_tokens % block_size != 0:
            raise BlockError("MisalignedAdoption")
        self.num_tokens += block_size
        self.blocks.append(bid)

    def push_partial_block(self, bid: int, rows: int, block_size: int) -> None:
        if rows == 0 or rows >= block_size or self.num_tokens % block_size != 0:
            raise BlockError("MisalignedAdoption")
        self.num_tokens += rows
        self.blocks.append(bid)

    def truncate(self, mgr: BlockManager, keep_tokens: int) -> None:
        """The speculative rollback (block.rs:381-396): release blocks past the kept tail, in table order."""
        if keep_tokens > self.num_tokens:
            raise BlockError("TokenCountOverflow")
        keep_blocks = -(-keep_tokens // mgr.block_size)
        for bid in self.blocks[min(keep_blocks, len(self.blocks)):]:
            mgr.release(bid)
        del self.blocks[keep_blocks:]
        self.num_tokens = keep_tokens

    def fork(self, mgr: BlockManager) -> "BlockTable":
        done = []
        try:
            for bid in self.blocks:
                mgr.retain(bid)
                done.append(bid)
        except BlockError:
            for bid in done:
                mgr.release(bid)
            raise
        t = BlockTable()
        t.blocks = list(self.blocks)
        t.num_tokens = self.num_tokens
        return t

    def release(self, mgr: BlockManager) -> None:
        for bid in self.blocks:
            mgr.release(bid)
        self.blocks = []
        self.num_tokens = 0


def spec_gamma_at_width(gamma: int, spec_max_batch: int, width: int) -> int:
    """drafter.rs:62-70."""
    width = max(width, 1)
    if gamma == 0 or width > spec_max_batch:
        return 0
    return -(-(gamma * (spec_max_batch + 1 - width)) // spec_max_batch)


def canonical_prefill_len(at: int, limit: int, prefill_chunk: int, fine: int) -> int:
    """engine.rs:167-179."""
    assert at < limit
    fine = min(max(fine, 1), prefill_chunk)
    tail_start = limit // prefill_chunk * prefill_chunk
    if at < tail_start:
        return prefill_chunk - at % prefill_chunk
    return min(fine - at % fine, limit - at)


def settle_walk(rows: List[int], draft: List[int]) -> Tuple[List[int], int]:
    """The verify settle walk without stop/length handling (engine.rs:2340-2366): (committed tokens, accepted)."""
    committed, accepted = [], 0
    for j, token in enumerate(rows):
        agrees = j < len(draft) and token == draft[j]
        if agrees:
            accepted += 1
        committed.append(token)
        if not agrees:
            break
    return committed, accepted


def write_runs(blocks: List[int], offset: int, length: int, block_size: int):
    """WriteRun derivation (engine.rs:2757-2769): (block, row_start, src_start, len)."""
    runs, pos = [], offset
    while pos < offset + length:
        run = min(block_size - pos % block_size, offset + length - pos)
        runs.append((blocks[pos // block_size], pos % block_size, pos - offset, run))
        pos += run
    return runs


def round_gamma(cfg_gamma: int, spec_max_batch: int, running: int, det_width: int, remaining: int, offset: int,
                max_key_len: int) -> int:
    """Per-round gamma (engine.rs:1515-1547). max_key_len = 0 means the backend has no key-length bound."""
    g = spec_gamma_at_width(cfg_gamma, spec_max_batch, running)
    if g == 0:
        return 0
    g = min(g, max(det_width - 1, 0), max(remaining - 1, 0))
    if max_key_len > 0:
        g = min(g, max(max_key_len - (offset + 1), 0))
    return g


def should_stand_down(min_acceptance: float, proposed: int, accepted: int, warmup: int = 16) -> bool:
    """engine.rs:1616-1623."""
    if min_acceptance <= 0.0 or proposed < warmup:
        return False
    return float(accepted) < min_acceptance * float(proposed)


def gamma_bound(heads: int, kv_heads: int, head_dim: int, quantized: bool = True, fused: bool = True) -> Optional[int]:
    """AnyModel::speculative_gamma_bound under the REFERENCE's MLX envelope (model.rs:239-252)."""
    if not quantized or not fused or kv_heads == 0 or head_dim not in (64, 96, 128, 256):
        return None
    gqa = heads // kv_heads
    if gqa == 0:
        return None
    rows = min(32 // gqa, 8)
    return rows - 1 if rows >= 2 else None
