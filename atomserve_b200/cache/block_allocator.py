"""The page ledger of one cache pool: which pages requests hold, which are idle, and which idle
or held pages still carry a prefix that a later request may pick up.

No tensors, so the policy is testable without a device. Every page is in one of three
conditions: held (one or more requests count on it), idle but remembered (its contents are
still named by a content key and `lookup` finds it until the memory is needed), or idle and
blank. Idle pages wait in a queue threaded through two index arrays (`_toward_old`,
`_toward_new`): a page joins at the young end when its last holder lets go and leaves from the
old end when pages are handed out, so the prefix that has been idle longest is the first one
overwritten; a remembered page that is picked up again is unhooked from the middle in O(1).

A full page is named by sha256 over the name of the page before it and its own token ids, so
equal names mean equal tokens all the way back to position 0 and therefore equal keys and
values. The rules (oldest idle first, all-or-nothing hand-out, last page let go first, the
first copy of a prefix wins) are the reference's (atomserve/block_allocator.py:33-129).
"""

from __future__ import annotations

import hashlib
from array import array

_NONE = -1  # end of the idle queue / not queued


def blocks_for_tokens(num_tokens: int, block_size: int) -> int:
    """Pages needed to hold `num_tokens` positions."""
    return (num_tokens + block_size - 1) // block_size


def block_hash(parent: bytes, tokens: list[int]) -> bytes:
    """Content key of a full page: the key of the page before it, then its tokens as uint32."""
    digest = hashlib.sha256(parent)
    digest.update(array("I", tokens).tobytes())
    return digest.digest()


class OutOfBlocksError(RuntimeError):
    """A hand-out asked for more pages than are idle; nothing was taken."""


class BlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._holders = array("i", bytes(4 * num_blocks))  # how many requests count on each page
        # the idle queue, oldest first: page p's neighbours are _toward_old[p] and _toward_new[p]
        self._toward_old = array("i", range(-1, num_blocks - 1))
        self._toward_new = array("i", range(1, num_blocks + 1))
        if num_blocks:
            self._toward_new[num_blocks - 1] = _NONE
        self._oldest = 0 if num_blocks else _NONE
        self._youngest = num_blocks - 1
        self._idle = num_blocks
        self._key_of_page: list[bytes | None] = [None] * num_blocks
        self._page_of_key: dict[bytes, int] = {}

    # ---- counts --------------------------------------------------------------------------------

    @property
    def num_free(self) -> int:
        return self._idle

    @property
    def num_cached(self) -> int:
        return len(self._page_of_key)

    def refcount(self, block: int) -> int:
        return self._holders[block]

    # ---- the idle queue ------------------------------------------------------------------------

    def _unhook(self, page: int) -> None:
        older, younger = self._toward_old[page], self._toward_new[page]
        if older == _NONE:
            self._oldest = younger
        else:
            self._toward_new[older] = younger
        if younger == _NONE:
            self._youngest = older
        else:
            self._toward_old[younger] = older
        self._idle -= 1

    def _hook_youngest(self, page: int) -> None:
        self._toward_old[page], self._toward_new[page] = self._youngest, _NONE
        if self._youngest == _NONE:
            self._oldest = page
        else:
            self._toward_new[self._youngest] = page
        self._youngest = page
        self._idle += 1

    # ---- handing out and taking back -----------------------------------------------------------

    def allocate(self, n: int) -> list[int]:
        """The n pages that have been idle longest, each now held once; all of them or an error."""
        if n > self._idle:
            raise OutOfBlocksError(f"need {n} cache pages, only {self._idle} free")
        pages = []
        page = self._oldest
        for _ in range(n):
            pages.append(page)
            page = self._toward_new[page]
        for page in pages:
            self._unhook(page)
            stale = self._key_of_page[page]
            if stale is not None:  # the page is about to be overwritten: forget what it held
                self._key_of_page[page] = None
                del self._page_of_key[stale]
            self._holders[page] = 1
        return pages

    def free(self, blocks: list[int]) -> None:
        """One holder fewer on each page. Pages are let go from the back of the list, so the tail
        of a prefix becomes older in the idle queue than its head and is overwritten first (the
        head is what most requests share)."""
        for page in blocks[::-1]:
            if not 0 <= page < self.num_blocks or self._holders[page] == 0:
                raise ValueError(f"page {page} is not allocated")
            self._holders[page] -= 1
            if self._holders[page] == 0:
                self._hook_youngest(page)

    # ---- prefixes ------------------------------------------------------------------------------

    def lookup(self, h: bytes) -> int | None:
        """The page remembered under content key `h`, held or idle, if any."""
        return self._page_of_key.get(h)

    def acquire(self, block: int) -> None:
        """Count one more holder on a page that `lookup` returned (an idle one leaves the queue)."""
        if self._holders[block] == 0:
            self._unhook(block)
        self._holders[block] += 1

    def register(self, block: int, h: bytes) -> None:
        """Remember that `block` (full and computed) holds the prefix named `h`. A prefix that is
        already remembered elsewhere keeps its first page, and a page keeps its first name."""
        if self._key_of_page[block] is None and h not in self._page_of_key:
            self._key_of_page[block] = h
            self._page_of_key[h] = block
