"""Host-side model of how the balanced persistent kernel shares the work out (test support).

The kernel (csrc/paged_decode_balanced.cuh: ``Chunking``, ``PairList::boundary``, ``chunk_range``),
its plan kernel and its merge kernel all derive the partition from ``seq_lens`` alone; this module
restates that arithmetic in Python so that the partition can be inspected (which warp group
attends which pages, where the pieces of a cut sequence land in the workspace) and its invariants
tested without a GPU.

Cost is counted in pages: sequence ``b`` owns the cost range that starts at
``2 * pairs_before(b) + piece_cost * b``; its first ``piece_cost`` units stand for taking the
sequence up, then comes one unit per page, two per page pair (the second unit of a last pair
that holds one page stands for nothing).  The cost axis is cut into ``groups`` contiguous chunks
whose lengths differ by at most one unit, and a page belongs to the chunk that holds its unit: a
boundary may fall between the two pages of a pair, which both neighbours then step through.
"""

from __future__ import annotations

from dataclasses import dataclass

PAGE = 16
WARPS_PER_SM = 8
PIECE_COST = 2
MIN_CHUNK_COST = 8


def pages_of(seq_len: int, kv_start: int = 0) -> int:
    return -(-seq_len // PAGE) - kv_start // PAGE if seq_len > kv_start else 0


def pairs_of(seq_len: int, kv_start: int = 0) -> int:
    return (pages_of(seq_len, kv_start) + 1) // 2


@dataclass(frozen=True)
class Piece:
    sequence: int
    group: int        # warp group (chunk) that attends it
    first_page: int   # page range inside the sequence (relative to the first attended page)
    last_page: int
    slot: int | None  # workspace slot 2 * group + which, None when the sequence is whole


@dataclass(frozen=True)
class Range:
    first_pair: int   # pairs of the flattened list the chunk steps through: [first_pair, end_pair)
    end_pair: int
    head_split: bool  # the first pair's first page is the previous chunk's
    tail_split: bool  # the last pair's second page is the next chunk's


class ChunkPlan:
    def __init__(self, seq_lens, num_kv_heads: int, sm_count: int = 148, *, kv_start: int = 0,
                 piece_cost: int = PIECE_COST, warps_per_sm: int = WARPS_PER_SM):
        self.pages = [pages_of(int(n), kv_start) for n in seq_lens]
        self.pairs = [(p + 1) // 2 for p in self.pages]
        self.batch = len(self.pairs)
        self.piece_cost = piece_cost
        self.prefix = [0]
        for n in self.pairs:
            self.prefix.append(self.prefix[-1] + n)
        total = 2 * self.prefix[-1] + piece_cost * self.batch
        max_groups = max(sm_count * warps_per_sm // num_kv_heads, 1)
        self.groups = max(min(max_groups, total // MIN_CHUNK_COST), 1)
        self.base, self.rem = divmod(total, self.groups)
        self.total_cost = total

    # ---- the device functions, one to one
    def start_of(self, chunk: int) -> int:
        return chunk * self.base + min(chunk, self.rem)

    def chunk_of(self, unit: int) -> int:
        wide = self.rem * (self.base + 1)
        return unit // (self.base + 1) if unit < wide else self.rem + (unit - wide) // max(self.base, 1)

    def first_unit(self, sequence: int) -> int:
        return 2 * self.prefix[sequence] + self.piece_cost * (sequence + 1)

    def boundary(self, cost: int) -> tuple[int, bool]:
        """(pairs whose first unit lies before ``cost``, the boundary falls inside the last of them)."""
        if cost >= self.total_cost:
            return self.prefix[-1], False
        b = max(i for i in range(self.batch) if 2 * self.prefix[i] + self.piece_cost * i <= cost)
        off = cost - self.first_unit(b)
        split = off > 0 and off % 2 == 1 and off < self.pages[b]
        return self.prefix[b] + min(max((off + 1) // 2, 0), self.pairs[b]), split

    # ---- derived views
    def chunk_range(self, chunk: int) -> Range:
        if chunk >= self.groups:
            return Range(self.prefix[-1], self.prefix[-1], False, False)
        before, head = self.boundary(self.start_of(chunk))
        end, tail = self.boundary(self.start_of(chunk + 1))
        return Range(before - (1 if head else 0), end, head, tail)

    def pages_of_chunk(self, chunk: int) -> list[tuple[int, int]]:
        """(sequence, page) of every page the chunk attends, in order."""
        r = self.chunk_range(chunk)
        out = []
        for g in range(r.first_pair, r.end_pair):
            b = max(i for i in range(self.batch) if self.prefix[i] <= g and self.pairs[i] > 0)
            q = g - self.prefix[b]
            for u in (0, 1):
                page = 2 * q + u
                if page >= self.pages[b]:
                    continue
                if (r.head_split and g == r.first_pair and u == 0) or (r.tail_split and g == r.end_pair - 1 and u == 1):
                    continue
                out.append((b, page))
        return out

    def pieces_of(self, sequence: int) -> list[Piece]:
        """What the merge derives for one sequence: its pieces and their slots."""
        n = self.pages[sequence]
        if n == 0:
            return []
        s0 = self.first_unit(sequence)
        first, last = self.chunk_of(s0), self.chunk_of(s0 + n - 1)
        out = []
        for c in range(first, last + 1):
            a = max(self.start_of(c), s0) - s0
            e = min(self.start_of(c + 1), s0 + n) - s0
            which = 1 if s0 > self.start_of(c) else 0
            out.append(Piece(sequence, c, a, e - 1, None if first == last else 2 * c + which))
        return out
