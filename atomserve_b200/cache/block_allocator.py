"""Which pages of one cache pool are free, which are in use, and which hold a reusable prefix.

Bookkeeping over page ids only (no tensors), so policy is testable without a device. A page is
in use (reference count > 0), free and still holding a hashed prefix (found again by lookup
until the memory is needed), or free and empty. Free pages are handed out oldest first, which
evicts the least recently freed prefix first. Full pages are named by a chained hash of their
tokens and everything before them, so equal hashes mean equal keys and values. The rules are
the reference's (atomserve/block_allocator.py:33-129).
"""

from __future__ import annotations

import hashlib
from array import array
from collections import OrderedDict


def blocks_for_tokens(num_tokens: int, block_size: int) -> int:
    return -(-num_tokens // block_size)


def block_hash(parent: bytes, tokens: list[int]) -> bytes:
    """sha256(parent hash || tokens as uint32): commits to the page and all before it."""
    return hashlib.sha256(parent + array("I", tokens).tobytes()).digest()


class OutOfBlocksError(RuntimeError):
    """More pages were asked for than are free; none was taken."""


class BlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._refcount = [0] * num_blocks
        self._free: OrderedDict[int, None] = OrderedDict.fromkeys(range(num_blocks))
        self._hash_of: dict[int, bytes] = {}
        self._block_of: dict[bytes, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_cached(self) -> int:
        return len(self._block_of)

    def refcount(self, block: int) -> int:
        return self._refcount[block]

    def allocate(self, n: int) -> list[int]:
        """Take n free pages, oldest first; all or none."""
        if n > len(self._free):
            raise OutOfBlocksError(f"need {n} cache pages, only {len(self._free)} free")
        taken = []
        for _ in range(n):
            block, _ = self._free.popitem(last=False)
            old = self._hash_of.pop(block, None)
            if old is not None:  # about to be overwritten: its prefix must no longer be found
                del self._block_of[old]
            self._refcount[block] = 1
            taken.append(block)
        return taken

    def free(self, blocks: list[int]) -> None:
        """Drop one reference to each page, last page first, so that a prefix's later pages
        are evicted before its earlier, more widely shared ones."""
        for block in reversed(blocks):
            if not 0 <= block < self.num_blocks or self._refcount[block] == 0:
                raise ValueError(f"page {block} is not allocated")
            self._refcount[block] -= 1
            if self._refcount[block] == 0:
                self._free[block] = None

    def lookup(self, h: bytes) -> int | None:
        return self._block_of.get(h)

    def acquire(self, block: int) -> None:
        """Add a reference to a page found by lookup, reviving it if it was free."""
        if self._refcount[block] == 0:
            del self._free[block]
        self._refcount[block] += 1

    def register(self, block: int, h: bytes) -> None:
        """Record that `block` (full, computed) holds the prefix `h`; the first copy wins."""
        if h not in self._block_of and block not in self._hash_of:
            self._block_of[h] = block
            self._hash_of[block] = h
