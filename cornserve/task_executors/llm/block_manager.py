"""Page allocator for the paged KV cache (128-token pages; page 0 is reserved as a scratch page so
that padded block-table entries always point at valid memory)."""

from __future__ import annotations

from collections import deque

PAGE = 128


class OutOfPages(RuntimeError):
    pass


class BlockManager:
    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("need at least two pages")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(1, num_pages))
        self._owned: dict[str, list[int]] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def capacity(self) -> int:
        """Pages a single sequence could ever own (page 0 is the scratch page)."""
        return self.num_pages - 1

    def pages_of(self, seq_id: str) -> list[int]:
        return self._owned.get(seq_id, [])

    def can_allocate(self, num_tokens: int, seq_id: str | None = None) -> bool:
        have = len(self._owned.get(seq_id, [])) if seq_id else 0
        need = -(-num_tokens // PAGE) - have
        return need <= len(self._free)

    def ensure(self, seq_id: str, num_tokens: int) -> list[int]:
        """Grow the page list of ``seq_id`` to cover ``num_tokens`` tokens."""
        pages = self._owned.setdefault(seq_id, [])
        need = -(-num_tokens // PAGE) - len(pages)
        if need > len(self._free):
            raise OutOfPages(f"{need} pages needed, {len(self._free)} free")
        for _ in range(max(need, 0)):
            pages.append(self._free.popleft())
        return pages

    def free(self, seq_id: str) -> None:
        for p in self._owned.pop(seq_id, []):
            self._free.append(p)

    def detach(self, seq_id: str) -> list[int]:
        """Give up the bookkeeping of ``seq_id`` without freeing its pages (they are held for a remote reader)."""
        return self._owned.pop(seq_id, [])

    def release(self, pages: list[int]) -> None:
        """Return detached pages to the pool."""
        self._free.extend(pages)

    def adopt(self, seq_id: str, pages: list[int]) -> None:
        """Take ownership of pages filled by someone else (prefill/decode disaggregation)."""
        for p in pages:
            self._free.remove(p)
        self._owned[seq_id] = list(pages)
