"""First-fit allocator of contiguous slot runs inside a slab (reference:
python/cornserve/services/sidecar/shm_manager.py:105-174).  Offsets are in elements of the slab dtype;
runs are aligned to ``align`` elements so that every region starts on a 256-byte boundary."""

from __future__ import annotations

from bisect import insort


class OutOfSlots(Exception):
    pass


class SlotAllocator:
    def __init__(self, total_numel: int, slot_numel: int, align: int = 128):
        self.align = max(1, align)
        self.slot_numel = max(1, slot_numel)
        self.total = total_numel
        self._free: list[tuple[int, int]] = [(0, total_numel)]  # sorted (offset, length)
        self._used: dict[int, int] = {}

    def _round(self, n: int) -> int:
        return (n + self.align - 1) // self.align * self.align

    def allocate(self, numel: int) -> int:
        """Offset of a free run of at least ``numel`` elements (whole slots, aligned)."""
        slots = max(1, -(-numel // self.slot_numel))
        need = self._round(slots * self.slot_numel)
        for i, (off, length) in enumerate(self._free):
            if length >= need:
                if length == need:
                    self._free.pop(i)
                else:
                    self._free[i] = (off + need, length - need)
                self._used[off] = need
                return off
        raise OutOfSlots(f"no free run of {need} elements ({self.free_numel()} free in {len(self._free)} runs)")

    def free(self, offset: int) -> None:
        length = self._used.pop(offset)
        insort(self._free, (offset, length))
        merged: list[tuple[int, int]] = []
        for off, ln in self._free:
            if merged and merged[-1][0] + merged[-1][1] == off:
                merged[-1] = (merged[-1][0], merged[-1][1] + ln)
            else:
                merged.append((off, ln))
        self._free = merged

    def free_numel(self) -> int:
        return sum(ln for _, ln in self._free)

    def used_runs(self) -> int:
        return len(self._used)
