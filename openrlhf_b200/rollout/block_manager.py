"""KV page pool with reference counts (prefix sharing between the n samples of one prompt)."""
from __future__ import annotations


class BlockManager:
    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free_list = list(range(num_pages - 1, -1, -1))
        self.ref = [0] * num_pages

    def num_free(self) -> int:
        return len(self.free_list)

    def alloc(self) -> int:
        if not self.free_list:
            raise MemoryError("KV page pool exhausted")
        p = self.free_list.pop()
        self.ref[p] = 1
        return p

    def share(self, page: int) -> int:
        assert self.ref[page] > 0
        self.ref[page] += 1
        return page

    def free(self, page: int) -> None:
        assert self.ref[page] > 0, "double free of a KV page"
        self.ref[page] -= 1
        if self.ref[page] == 0:
            self.free_list.append(page)
