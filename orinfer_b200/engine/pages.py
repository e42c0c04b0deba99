"""Reference-counted KV page pool and the page-granular prefix index.

Pages hold 128 tokens of INT8 K/V for every attention layer.  A full page can be
shared read-only by many requests (prefix reuse); the partially filled last page
of a request is always private, so no copy-on-write is needed.  Sharing is
charged once, like the reference's ``Resident`` bank accounting
(crates/orinfer-engine/src/prefix.rs:146-201).  Page 0 is reserved as the
target of padded rows.
"""

from __future__ import annotations

from typing import Dict, List, Optional


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, pages: int):
        if pages < 2:
            raise ValueError("need at least one usable page besides the dummy page 0")
        self.pages = pages
        self.free: List[int] = list(range(pages - 1, 0, -1))
        self.refs: List[int] = [0] * pages

    @property
    def available(self) -> int:
        return len(self.free)

    def take(self, n: int) -> List[int]:
        if n > len(self.free):
            raise OutOfPages(f"need {n} pages, {len(self.free)} free")
        out = [self.free.pop() for _ in range(n)]
        for p in out:
            self.refs[p] = 1
        return out

    def share(self, page: int) -> None:
        if self.refs[page] <= 0:
            raise ValueError("sharing a free page")
        self.refs[page] += 1

    def release(self, pages) -> None:
        for p in pages:
            if p == 0:
                continue
            self.refs[p] -= 1
            if self.refs[p] < 0:
                raise ValueError("page released twice")
            if self.refs[p] == 0:
                self.free.append(p)
