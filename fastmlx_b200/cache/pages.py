"""Host-side book-keeping of pages: a pool with a free list, and block tables."""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """The pool cannot give the pages a step needs.  Nothing was taken."""


class PagePool:
    """`num_pages` pages of `page_size` tokens.  The free list is last-in first-out, so a
    page that was just given back is the next one handed out: stale contents are met
    early, in tests as in service."""

    def __init__(self, num_pages: int, page_size: int):
        if num_pages <= 0 or page_size <= 0:
            raise ValueError("a pool needs a positive number of pages and a positive page size")
        self.num_pages, self.page_size = int(num_pages), int(page_size)
        self._free = list(range(self.num_pages - 1, -1, -1))
        self._held = [False] * self.num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} of {self.num_pages} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise RuntimeError(f"page {p} is given back but is not held")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """No page lost and none both free and held."""
        assert len(set(self._free)) == len(self._free), "a page is on the free list twice"
        assert all(not self._held[p] for p in self._free), "a free page is marked held"
        assert sum(self._held) + len(self._free) == self.num_pages, "a page is lost"


class BlockTable:
    """Pages of one request in one group: entry i holds tokens [i*page_size, (i+1)*page_size).
    An entry is -1 once a window has passed it and its page was given back."""

    def __init__(self):
        self.pages: list[int] = []
        self.first_live = 0          # entries before this one are -1

    def live(self) -> list[int]:
        return self.pages[self.first_live:]
